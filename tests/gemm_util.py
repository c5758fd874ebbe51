"""Shared set-up for the prefill GEMM tests: seeded operands quantised on the GPU by the
(separately parity-tested) quantizers, in both scale layouts."""
import numpy as np
import torch

from tests.util import to_np


def nvfp4_operand(lib, dev, rows, k, std, seed):
    """Returns dict with packed bytes, compact + interleaved scales (device) and the divisor."""
    g = torch.Generator(device=dev)
    g.manual_seed(seed)
    x = (torch.randn((rows, k), device=dev, generator=g) * std).to(torch.bfloat16)
    div = float(np.float32(6.0 * 448.0) / np.float32(x.abs().max().item()))
    packed = torch.empty((rows, k // 2), dtype=torch.uint8, device=dev)
    compact = torch.empty((rows, k // 16), dtype=torch.uint8, device=dev)
    lib.gemb_nvfp4_quantize(x.view(torch.int16), 1, packed, compact, rows, k, div, 0, 0, None)
    inter = torch.empty((lib.cdll.gemb_interleaved_scale_bytes(rows, k),), dtype=torch.uint8, device=dev)
    lib.gemb_nvfp4_interleave_scales(compact, inter, rows, k, None)
    return {"x": x, "packed": packed, "compact": compact, "inter": inter, "div": div}


def fp8_operand(lib, dev, rows, k, std, seed):
    g = torch.Generator(device=dev)
    g.manual_seed(seed)
    x = (torch.randn((rows, k), device=dev, generator=g) * std).to(torch.bfloat16)
    q = torch.empty((rows, k), dtype=torch.uint8, device=dev)
    s = torch.empty((rows,), dtype=torch.float32, device=dev)
    lib.gemb_fp8_quantize(x.view(torch.int16), 1, q, s, rows, k, None)
    return {"x": x, "q": q, "scales": s, "scales_bf16": s.to(torch.bfloat16).view(torch.int16)}


def bf16_tensor_to_f32(t):
    return t.view(torch.bfloat16).float().cpu().numpy()


def error_stats(got_bf16_f32, want_f64):
    """Relative Frobenius error and friends of a bf16 result against the bf16-rounded oracle."""
    from tests.util import bf16_round
    want = bf16_round(want_f64.astype(np.float32)).astype(np.float64)
    got = got_bf16_f32.astype(np.float64)
    diff = got - want
    return {
        "rel_fro": float(np.linalg.norm(diff) / max(np.linalg.norm(want), 1e-300)),
        "max_abs": float(np.abs(diff).max()),
        "mismatch": float((got != want).mean()),
        "cos": float((got * want).sum() / max(np.linalg.norm(got) * np.linalg.norm(want), 1e-300)),
    }
