"""Checkpoint bytes -> library layouts (host-side harness, like moe.py; the kernels never see files).

gem16 loads a compressed-tensors safetensors checkpoint and re-tiles every NVFP4 weight on the host
into its SM120 Row8/K64 layout (src/cuda/engine/target_model.cu:88-143,211-248,345-388,
src/cuda/nvfp4/sm120_layout.cpp:58-145; format in docs/CHECKPOINT_FORMAT.md:62-95).  With this
library the payload is uploaded unchanged and only the block scales are rewritten, once, into the
128x4 interleave the block-scaled MMA reads (gemb_nvfp4_interleave_scales); the decode GEMV reads
the compact scales as stored.  FP8 tensors need no change at all.

Tensor names per linear module `<prefix>`:
  NVFP4   <prefix>.weight_packed        U8      [rows, K/2]   (or [experts, rows, K/2])
          <prefix>.weight_scale         F8_E4M3 [rows, K/16]  (or [experts, rows, K/16])
          <prefix>.weight_global_scale  F32     scalar        (or [experts]) -- stored as a DIVISOR
          <prefix>.input_global_scale   F32     scalar        (or [experts]) -- stored as a DIVISOR
  FP8     <prefix>.weight               F8_E4M3 [rows, K]
          <prefix>.weight_scale         BF16    [rows] or [rows, 1]

The safetensors container is read directly (8-byte little-endian header length, JSON header, raw
bytes); nothing outside numpy is needed.
"""
from __future__ import annotations

import json
import struct
from dataclasses import dataclass

import numpy as np

_DTYPES = {"U8": (np.uint8, 1), "I8": (np.int8, 1), "F8_E4M3": (np.uint8, 1), "F8_E5M2": (np.uint8, 1),
           "BF16": (np.uint16, 2), "F16": (np.float16, 2), "F32": (np.float32, 4), "I32": (np.int32, 4),
           "I64": (np.int64, 8), "F64": (np.float64, 8), "BOOL": (np.uint8, 1)}


class CheckpointError(ValueError):
    pass


class SafetensorsFile:
    """Read-only view of one .safetensors file; tensors come back as numpy views of a memory map
    (F8 and BF16 as their raw bytes / 16-bit patterns)."""

    def __init__(self, path: str):
        self.path = path
        with open(path, "rb") as f:
            head = f.read(8)
            if len(head) != 8:
                raise CheckpointError(f"{path}: truncated header length")
            (n,) = struct.unpack("<Q", head)
            if n == 0 or n > 100 << 20:
                raise CheckpointError(f"{path}: implausible header size {n}")
            raw = f.read(n)
            if len(raw) != n:
                raise CheckpointError(f"{path}: truncated header")
        try:
            self.header = json.loads(raw.decode("utf-8"))
        except Exception as exc:
            raise CheckpointError(f"{path}: header is not JSON: {exc}") from None
        self.metadata = self.header.pop("__metadata__", {})
        self._base = 8 + n
        self._map = np.memmap(path, dtype=np.uint8, mode="r")
        size = self._map.size - self._base
        for name, info in self.header.items():
            if info.get("dtype") not in _DTYPES:
                raise CheckpointError(f"{path}: tensor {name} has unsupported dtype {info.get('dtype')}")
            b, e = info["data_offsets"]
            want = int(np.prod(info["shape"], dtype=np.int64)) * _DTYPES[info["dtype"]][1]
            if not (0 <= b <= e <= size) or e - b != want:
                raise CheckpointError(f"{path}: tensor {name} has inconsistent shape / offsets")

    def names(self):
        return list(self.header)

    def __contains__(self, name):
        return name in self.header

    def dtype(self, name):
        return self.header[name]["dtype"]

    def tensor(self, name) -> np.ndarray:
        if name not in self.header:
            raise CheckpointError(f"{self.path}: tensor {name} is missing")
        info = self.header[name]
        b, e = info["data_offsets"]
        np_dtype, _ = _DTYPES[info["dtype"]]
        return self._map[self._base + b:self._base + e].view(np_dtype).reshape(info["shape"])


def write_safetensors(path: str, tensors: dict, metadata: dict | None = None) -> None:
    """tensors: name -> (dtype string, numpy array holding the raw representation).  For fixtures."""
    header, blobs, off = {}, [], 0
    for name, (dtype, arr) in tensors.items():
        np_dtype, size = _DTYPES[dtype]
        a = np.array(arr, dtype=np_dtype, order="C")   # keeps 0-d scalars 0-d
        data = a.tobytes()
        header[name] = {"dtype": dtype, "shape": list(a.shape), "data_offsets": [off, off + len(data)]}
        blobs.append(data)
        off += len(data)
    if metadata:
        header["__metadata__"] = metadata
    raw = json.dumps(header, separators=(",", ":")).encode("utf-8")
    raw += b" " * (-len(raw) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(raw)))
        f.write(raw)
        for b in blobs:
            f.write(b)


@dataclass
class Nvfp4Linear:
    """One NVFP4 weight (or a stack of expert weights) in the library's layouts, on the device."""
    packed: object            # uint8 [rows, K/2] or [experts, rows, K/2]
    compact_scales: object    # uint8 [rows, K/16] (decode GEMV)
    interleaved_scales: object  # uint8, 128x4 interleave per matrix, experts back to back (prefill / grouped GEMM)
    weight_divisor: object    # float, or list of floats per expert
    input_divisor: object     # float, or list of floats per expert
    rows: int
    k: int
    experts: int              # 0 for a plain linear


@dataclass
class Fp8Linear:
    weight: object            # uint8 [rows, K] E4M3
    scales_bf16: object       # int16 [rows] bf16 bits
    rows: int
    k: int


def _global_divisor(st, name, experts):
    """A per-tensor global divisor: present, stored as F32, shape [1] ([experts] for a stack), positive
    and finite -- the reference returns kDataLoss otherwise (src/model/manifest.cpp:346-365)."""
    what = name
    if name not in st:
        raise CheckpointError(f"{what}: NVFP4 module is missing this required scale tensor")
    if st.dtype(name) != "F32":
        raise CheckpointError(f"{what}: global scales must be stored as F32, found {st.dtype(name)}")
    arr = st.tensor(name)
    if tuple(arr.shape) != (max(experts, 1),):
        raise CheckpointError(f"{what}: expected shape [{max(experts, 1)}], found {list(arr.shape)}")
    a = np.asarray(arr, dtype=np.float32).reshape(-1)
    if not np.all(np.isfinite(a)) or np.any(a <= 0):
        raise CheckpointError(f"{what}: global divisors must be positive and finite")
    return [float(v) for v in a] if experts else float(a[0])


def load_nvfp4_linear(st: SafetensorsFile, prefix: str, dev, lib=None) -> Nvfp4Linear:
    """Validates the four tensors of an NVFP4 module the way the reference's loader does (exact
    dtypes and shapes, no NaN scale bytes: src/cuda/engine/target_model.cu:211-248) and uploads them."""
    import torch
    from .lib import load
    lib = lib or load()
    packed, scale = st.tensor(prefix + ".weight_packed"), st.tensor(prefix + ".weight_scale")
    if st.dtype(prefix + ".weight_packed") != "U8" or st.dtype(prefix + ".weight_scale") != "F8_E4M3":
        raise CheckpointError(f"{prefix}: weight_packed must be U8 and weight_scale F8_E4M3")
    if packed.ndim not in (2, 3) or scale.ndim != packed.ndim:
        raise CheckpointError(f"{prefix}: weight_packed / weight_scale must both be 2-D (or 3-D expert stacks)")
    experts = packed.shape[0] if packed.ndim == 3 else 0
    rows, half_k = packed.shape[-2:]
    k = 2 * half_k
    if k % 64 or rows % 8:
        raise CheckpointError(f"{prefix}: K must be a multiple of 64 and rows of 8 (got rows={rows}, K={k})")
    if tuple(scale.shape[-2:]) != (rows, k // 16) or (experts and scale.shape[0] != experts):
        raise CheckpointError(f"{prefix}: weight_scale shape {tuple(scale.shape)} does not match weight_packed")
    if np.any((scale & 0x7F) == 0x7F):
        raise CheckpointError(f"{prefix}: weight_scale holds an E4M3FN NaN encoding")
    gw = _global_divisor(st, prefix + ".weight_global_scale", experts)
    ga = _global_divisor(st, prefix + ".input_global_scale", experts)
    d_packed = torch.from_numpy(np.array(packed)).to(dev)   # a copy: the map is read-only
    d_compact = torch.from_numpy(np.array(scale)).to(dev)
    per = lib.cdll.gemb_interleaved_scale_bytes(rows, k)
    d_inter = torch.zeros((max(experts, 1) * per,), dtype=torch.uint8, device=dev)
    for e in range(max(experts, 1)):
        src = d_compact[e] if experts else d_compact
        lib.gemb_nvfp4_interleave_scales(src, d_inter[e * per:(e + 1) * per], rows, k, None)
    return Nvfp4Linear(d_packed, d_compact, d_inter, gw, ga, rows, k, experts)


def load_fp8_linear(st: SafetensorsFile, prefix: str, dev) -> Fp8Linear:
    import torch
    w, s = st.tensor(prefix + ".weight"), st.tensor(prefix + ".weight_scale")
    if st.dtype(prefix + ".weight") != "F8_E4M3" or st.dtype(prefix + ".weight_scale") != "BF16":
        raise CheckpointError(f"{prefix}: weight must be F8_E4M3 and weight_scale BF16")
    if w.ndim != 2 or s.size != w.shape[0] or s.ndim not in (1, 2):
        raise CheckpointError(f"{prefix}: weight must be [rows, K] with one scale per row")
    rows, k = w.shape
    if k % 16:
        raise CheckpointError(f"{prefix}: K must be a multiple of 16")
    if np.any((w & 0x7F) == 0x7F):
        raise CheckpointError(f"{prefix}: weight holds an E4M3FN NaN encoding")
    return Fp8Linear(torch.from_numpy(np.array(w)).to(dev),
                     torch.from_numpy(np.array(s).reshape(-1).view(np.int16)).to(dev), rows, k)
