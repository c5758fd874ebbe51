"""Helpers shared by the tests: seeded synthetic tensors and torch<->numpy plumbing."""
import numpy as np


def bf16_round(x):
    """fp32 array rounded to the nearest bf16 value (ties to even), kept as fp32."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32)


def bf16_bits(x):
    """fp32 array -> uint16 bf16 bit patterns (round to nearest even)."""
    return (bf16_round(x).view(np.uint32) >> 16).astype(np.uint16)


def from_bf16_bits(h):
    return (np.ascontiguousarray(h, np.uint16).astype(np.uint32) << 16).view(np.float32)


def nvfp4_divisor(x):
    """Per-tensor NVFP4 global divisor 6*448/amax (docs/CHECKPOINT_FORMAT.md:87-95)."""
    return float(np.float32(6.0 * 448.0) / np.float32(np.abs(x).max()))


def to_dev(a, dev):
    import torch
    a = np.ascontiguousarray(a)
    if a.dtype == np.uint16:
        return torch.from_numpy(a.view(np.int16)).to(dev)
    return torch.from_numpy(a).to(dev)


def to_np(t, dtype=None):
    a = t.detach().cpu().numpy()
    if dtype is not None:
        a = a.view(dtype)
    return a


def rel_fro(a, b):
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-300))
