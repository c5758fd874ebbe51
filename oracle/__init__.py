"""ctypes bindings for the CPU oracle.  TEST INFRASTRUCTURE ONLY.

Only tests/, the smoke check and the benchmark's CPU-baseline leg may import this package; the
product package (gem16_b200) never does.  `Oracle()` wraps our restatement; `Oracle(ref=True)`
wraps the reference's own numeric sources compiled by oracle/build.py (linear path only).
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import build as _build

_u8p = np.ctypeslib.ndpointer(np.uint8, flags="C_CONTIGUOUS")
_u16p = np.ctypeslib.ndpointer(np.uint16, flags="C_CONTIGUOUS")
_i32p = np.ctypeslib.ndpointer(np.int32, flags="C_CONTIGUOUS")
_f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
_f64p = np.ctypeslib.ndpointer(np.float64, flags="C_CONTIGUOUS")


def default_threads() -> int:
    return max(1, len(os.sched_getaffinity(0)))


def ref_available() -> bool:
    return _build.build_ref() is not None


class Oracle:
    def __init__(self, ref: bool = False):
        self.ref = ref
        if ref:
            path = _build.build_ref()
            if path is None:
                raise RuntimeError("reference oracle not built and reference tree absent")
            self.p = "ref_"
        else:
            path = _build.build_oracle()
            self.p = "orc_"
        self.lib = C.CDLL(path)
        L, p = self.lib, self.p
        for name, res, args in [
            ("e2m1_decode", C.c_float, [C.c_uint8]),
            ("e2m1_encode", C.c_int if ref else C.c_uint8, [C.c_float]),
            ("e4m3_decode", C.c_float, [C.c_uint8]),
            ("e4m3_encode", C.c_int if ref else C.c_uint8, [C.c_float]),
            ("nvfp4_quantize", C.c_int, [_f32p, C.c_uint64, C.c_uint64, C.c_float, _u8p, _u8p, C.c_int]),
            ("fp8_quantize", C.c_int, [_f32p, C.c_uint64, C.c_uint64, _u8p, _f32p, C.c_int]),
            ("nvfp4_matmul", C.c_int, [_u8p, _u8p, _u8p, _u8p, C.c_uint64, C.c_uint64, C.c_uint64,
                                       C.c_float, C.c_float, _f64p, C.c_int]),
            ("fp8_matmul", C.c_int, [_u8p, _f32p, _u8p, _u16p, C.c_uint64, C.c_uint64, C.c_uint64,
                                     _f64p, C.c_int]),
        ]:
            fn = getattr(L, p + name)
            fn.restype, fn.argtypes = res, args
        if ref:
            L.ref_rmsnorm.restype = C.c_int
            L.ref_rmsnorm.argtypes = [_f32p, C.c_void_p, C.c_uint64, C.c_uint64, C.c_float, _f32p]
        if not ref:
            L.orc_det_exp.restype, L.orc_det_exp.argtypes = C.c_float, [C.c_float]
            L.orc_f32_to_bf16_array.argtypes = [_f32p, _u16p, C.c_uint64]
            L.orc_bf16_to_f32_array.argtypes = [_u16p, _f32p, C.c_uint64]
            L.orc_rmsnorm_bf16.argtypes = [_f32p, C.c_void_p, C.c_uint64, C.c_uint64, C.c_float, _f32p]
            L.orc_gated_gelu.argtypes = [_f32p, _f32p, C.c_uint64, _f32p]
            L.orc_interleaved_scale_bytes.restype = C.c_uint64
            L.orc_interleaved_scale_bytes.argtypes = [C.c_uint64, C.c_uint64]
            L.orc_interleave_scales.argtypes = [_u8p, _u8p, C.c_uint64, C.c_uint64]
            L.orc_moe_router_logits.argtypes = [_u16p, _f32p, C.c_void_p, C.c_uint64, C.c_uint64,
                                                C.c_uint64, _f32p, C.c_int]
            L.orc_moe_router_input.argtypes = [_u16p, _u16p, C.c_uint64, C.c_uint64, C.c_float, _u16p]
            L.orc_moe_route.restype = C.c_int
            L.orc_moe_route.argtypes = [_f32p, C.c_uint64, C.c_uint64, C.c_uint64, C.c_void_p, _i32p,
                                        _f32p, C.c_void_p]
            L.orc_moe_permute.restype = C.c_int
            L.orc_moe_permute.argtypes = [_i32p, C.c_uint64, C.c_uint64, C.c_uint64, _i32p, _i32p, _i32p]
            L.orc_moe_combine.argtypes = [_u16p, _f32p, C.c_void_p, C.c_uint64, C.c_uint64, C.c_uint64,
                                          _u16p]
            L.orc_output_head.restype = C.c_int
            L.orc_output_head.argtypes = [_u16p, _f32p, C.c_uint64, C.c_uint64, C.c_uint64, C.c_void_p, C.c_uint64,
                                          _f32p, C.c_void_p, C.c_int]

    # ---- codecs ----
    def e2m1_decode(self, nib): return getattr(self.lib, self.p + "e2m1_decode")(nib)
    def e2m1_encode(self, v): return int(getattr(self.lib, self.p + "e2m1_encode")(v))
    def e4m3_decode(self, b): return getattr(self.lib, self.p + "e4m3_decode")(b)
    def e4m3_encode(self, v): return int(getattr(self.lib, self.p + "e4m3_encode")(v))

    # ---- quantizers ----
    def nvfp4_quantize(self, x, g, threads=None):
        x = np.ascontiguousarray(x, np.float32)
        x2 = x.reshape(-1, x.shape[-1])
        t, k = x2.shape
        packed = np.zeros((t, k // 2), np.uint8)
        scales = np.zeros((t, k // 16), np.uint8)
        rc = getattr(self.lib, self.p + "nvfp4_quantize")(x2, t, k, g, packed, scales,
                                                         threads or default_threads())
        if rc:
            raise ValueError(f"nvfp4_quantize rejected its input (status {rc})")
        return packed.reshape(*x.shape[:-1], k // 2), scales.reshape(*x.shape[:-1], k // 16)

    def fp8_quantize(self, x, threads=None):
        x = np.ascontiguousarray(x, np.float32)
        x2 = x.reshape(-1, x.shape[-1])
        t, k = x2.shape
        q = np.zeros((t, k), np.uint8)
        s = np.zeros((t,), np.float32)
        rc = getattr(self.lib, self.p + "fp8_quantize")(x2, t, k, q, s, threads or default_threads())
        if rc:
            raise ValueError(f"fp8_quantize rejected its input (status {rc})")
        return q.reshape(x.shape), s.reshape(x.shape[:-1])

    def nvfp4_matmul(self, a_packed, a_scales, w_packed, w_scales, ga, gw, threads=None):
        a_packed = np.ascontiguousarray(a_packed); a_scales = np.ascontiguousarray(a_scales)
        w_packed = np.ascontiguousarray(w_packed); w_scales = np.ascontiguousarray(w_scales)
        t, kb = a_packed.shape
        rows = w_packed.shape[0]
        out = np.zeros((t, rows), np.float64)
        rc = getattr(self.lib, self.p + "nvfp4_matmul")(a_packed, a_scales, w_packed, w_scales, t, rows,
                                                       kb * 2, ga, gw, out, threads or default_threads())
        if rc:
            raise ValueError(f"nvfp4_matmul rejected its input (status {rc})")
        return out

    def fp8_matmul(self, a, a_scales, w, w_scales_bf16, threads=None):
        a = np.ascontiguousarray(a); w = np.ascontiguousarray(w)
        a_scales = np.ascontiguousarray(a_scales, np.float32).reshape(-1)
        w_scales_bf16 = np.ascontiguousarray(w_scales_bf16, np.uint16)
        t, k = a.shape
        rows = w.shape[0]
        out = np.zeros((t, rows), np.float64)
        rc = getattr(self.lib, self.p + "fp8_matmul")(a, a_scales, w, w_scales_bf16, t, rows, k, out,
                                                     threads or default_threads())
        if rc:
            raise ValueError(f"fp8_matmul rejected its input (status {rc})")
        return out

    # ---- helpers only in the restatement ----
    def to_bf16(self, x):
        x = np.ascontiguousarray(x, np.float32)
        out = np.zeros(x.shape, np.uint16)
        self.lib.orc_f32_to_bf16_array(x.reshape(-1), out.reshape(-1), x.size)
        return out

    def from_bf16(self, h):
        h = np.ascontiguousarray(h, np.uint16)
        out = np.zeros(h.shape, np.float32)
        self.lib.orc_bf16_to_f32_array(h.reshape(-1), out.reshape(-1), h.size)
        return out

    def det_exp(self, x): return self.lib.orc_det_exp(x)

    def ref_rmsnorm(self, x, weight, eps):
        """gem16::layer::RmsNorm of the compiled reference (binary64 sums, fp32 out, no bf16 boundary)."""
        assert self.ref
        x = np.ascontiguousarray(x, np.float32)
        t, k = x.shape
        out = np.zeros_like(x)
        wv = None if weight is None else np.ascontiguousarray(weight, np.float32)
        rc = self.lib.ref_rmsnorm(x, None if wv is None else wv.ctypes.data, t, k, eps, out)
        if rc:
            raise ValueError(f"reference RmsNorm rejected its input (status {rc})")
        return out

    def rmsnorm_bf16(self, x, w_bf16, eps):
        x = np.ascontiguousarray(x, np.float32)
        t, k = x.shape
        out = np.zeros_like(x)
        wp = None if w_bf16 is None else np.ascontiguousarray(w_bf16, np.uint16).ctypes.data
        self.lib.orc_rmsnorm_bf16(x, wp, t, k, eps, out)
        return out

    def gated_gelu(self, gate, up):
        gate = np.ascontiguousarray(gate, np.float32); up = np.ascontiguousarray(up, np.float32)
        out = np.zeros_like(gate)
        self.lib.orc_gated_gelu(gate.reshape(-1), up.reshape(-1), gate.size, out.reshape(-1))
        return out

    def interleave_scales(self, compact, k):
        compact = np.ascontiguousarray(compact, np.uint8)
        rows = compact.shape[0]
        out = np.zeros(self.lib.orc_interleaved_scale_bytes(rows, k), np.uint8)
        self.lib.orc_interleave_scales(compact, out, rows, k)
        return out

    def moe_router_logits(self, x_bf16, w, bias, threads=None):
        x_bf16 = np.ascontiguousarray(x_bf16, np.uint16); w = np.ascontiguousarray(w, np.float32)
        t, h = x_bf16.shape
        e = w.shape[0]
        out = np.zeros((t, e), np.float32)
        bp = None if bias is None else np.ascontiguousarray(bias, np.float32)
        self._keep = bp
        self.lib.orc_moe_router_logits(x_bf16, w, None if bp is None else bp.ctypes.data, t, h, e, out,
                                       threads or default_threads())
        return out

    def moe_router_input(self, x_bf16, scale_bf16, eps):
        x_bf16 = np.ascontiguousarray(x_bf16, np.uint16)
        out = np.zeros_like(x_bf16)
        self.lib.orc_moe_router_input(x_bf16, np.ascontiguousarray(scale_bf16, np.uint16),
                                      x_bf16.shape[0], x_bf16.shape[1], eps, out)
        return out

    def moe_route(self, logits, topk, per_expert_scale=None, want_probs=False):
        logits = np.ascontiguousarray(logits, np.float32)
        t, e = logits.shape
        ids = np.zeros((t, topk), np.int32)
        w = np.zeros((t, topk), np.float32)
        probs = np.zeros((t, e), np.float32) if want_probs else None
        pes = None if per_expert_scale is None else np.ascontiguousarray(per_expert_scale, np.float32)
        rc = self.lib.orc_moe_route(logits, t, e, topk, None if pes is None else pes.ctypes.data, ids, w,
                                    None if probs is None else probs.ctypes.data)
        if rc:
            raise ValueError(f"moe_route rejected its input (status {rc})")
        return (ids, w, probs) if want_probs else (ids, w)

    def moe_permute(self, ids, experts):
        ids = np.ascontiguousarray(ids, np.int32)
        t, k = ids.shape
        counts = np.zeros(experts, np.int32)
        offsets = np.zeros(experts + 1, np.int32)
        perm = np.zeros(t * k, np.int32)
        rc = self.lib.orc_moe_permute(ids, t, k, experts, counts, offsets, perm)
        if rc:
            raise ValueError("moe_permute: expert id out of range")
        return counts, offsets, perm

    def output_head(self, weights_bf16, hidden_rows, suppressed=()):
        """(capped logits [rows, vocabulary] fp32, selected [rows] uint32); weights as bf16 bits."""
        w = np.ascontiguousarray(weights_bf16, np.uint16)
        h = np.ascontiguousarray(hidden_rows, np.float32)
        vocab, hidden = w.shape
        rows = h.shape[0]
        sup = np.ascontiguousarray(np.asarray(suppressed, np.uint32))
        logits = np.zeros((rows, vocab), np.float32)
        selected = np.zeros((rows,), np.uint32)
        rc = self.lib.orc_output_head(w, h, rows, vocab, hidden, sup.ctypes.data if sup.size else None, sup.size, logits,
                                      selected.ctypes.data, default_threads())
        assert rc == 0
        return logits, selected

    def moe_combine(self, y_slots_bf16, weights, shared_bf16):
        y = np.ascontiguousarray(y_slots_bf16, np.uint16)
        w = np.ascontiguousarray(weights, np.float32)
        t, k = w.shape
        h = y.shape[-1]
        out = np.zeros((t, h), np.uint16)
        sp = None if shared_bf16 is None else np.ascontiguousarray(shared_bf16, np.uint16)
        self._keep = sp
        self.lib.orc_moe_combine(y.reshape(-1, h), w, None if sp is None else sp.ctypes.data, t, k, h, out)
        return out
