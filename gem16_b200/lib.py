"""ctypes loader for libgemb200.so.

Prototypes are derived from include/gemb200.h itself, so the binding cannot drift from the
header.  Every call checks the returned gemb_status and raises GembError carrying the status
name and gemb_last_error().  A missing library is a hard error: nothing here falls back to
another implementation.
"""
from __future__ import annotations

import ctypes as C
import os
import re

HERE = os.path.dirname(os.path.abspath(__file__))
HEADER = os.path.join(os.path.dirname(HERE), "include", "gemb200.h")
LIB_PATH = os.path.join(HERE, "libgemb200.so")

STATUS_NAMES = ["kOk", "kInvalidArgument", "kNotFound", "kIoError", "kDataLoss", "kUnsupported",
                "kResourceExhausted", "kCancelled", "kInternal"]


class GembError(RuntimeError):
    def __init__(self, status: int, message: str):
        self.status = status
        self.status_name = STATUS_NAMES[status] if 0 <= status < len(STATUS_NAMES) else str(status)
        super().__init__(f"{self.status_name}: {message}")


_SCALARS = {"uint64_t": C.c_uint64, "int32_t": C.c_int32, "float": C.c_float, "size_t": C.c_size_t,
            "int64_t": C.c_int64, "uint32_t": C.c_uint32}


class Fp8Binding(C.Structure):
    """gemb_fp8_binding of include/gemb200.h."""
    _fields_ = [("weight", C.c_void_p), ("scales", C.c_void_p), ("rows", C.c_uint64), ("contracting", C.c_uint64)]


class Nvfp4Binding(C.Structure):
    """gemb_nvfp4_binding of include/gemb200.h."""
    _fields_ = [("packed_weight", C.c_void_p), ("scales", C.c_void_p), ("input_divisor_device", C.c_void_p),
                ("input_divisor", C.c_float), ("weight_divisor", C.c_float), ("rows", C.c_uint64),
                ("contracting", C.c_uint64), ("scales_interleaved", C.c_void_p),
                ("weight_divisors_device", C.c_void_p), ("experts", C.c_uint64)]


class MoeLayerWeights(C.Structure):
    """gemb_moe_layer_weights of include/gemb200.h."""
    _fields_ = [("hidden", C.c_uint64), ("experts", C.c_uint64), ("topk", C.c_uint64), ("intermediate", C.c_uint64),
                ("shared_intermediate", C.c_uint64), ("router_weight", C.c_void_p), ("router_bias", C.c_void_p),
                ("per_expert_scale", C.c_void_p), ("router_input_scale", C.c_void_p), ("router_epsilon", C.c_float),
                ("gate_up", Nvfp4Binding), ("down", Nvfp4Binding), ("shared_gate_up", Nvfp4Binding),
                ("shared_down", Nvfp4Binding), ("gate_up_fused", C.c_void_p), ("gate_up_fused_scales", C.c_void_p),
                ("shared_gate_up_fused", C.c_void_p), ("shared_gate_up_fused_scales", C.c_void_p)]


class MoeRecords(C.Structure):
    """gemb_moe_records of include/gemb200.h."""
    _fields_ = [(n, C.c_void_p) for n in ("logits", "top_ids", "top_weights", "counts", "offsets", "perm", "slot_rows",
                                           "plan", "expert_rows")] + [("padded_rows_max", C.c_uint64),
                                                                      ("counts_all", C.c_void_p)]


class MoeEpComm(C.Structure):
    """gemb_moe_ep_comm of include/gemb200.h."""
    _fields_ = [("ranks", C.c_uint64), ("rank", C.c_uint64), ("send_buffers_host", C.c_void_p),
                ("recv_buffers_host", C.c_void_p), ("count_buffers_host", C.c_void_p), ("flag_arrays_host", C.c_void_p),
                ("local_epochs", C.c_void_p)]


STRUCTS = [Fp8Binding, Nvfp4Binding, MoeLayerWeights, MoeRecords, MoeEpComm]   # order of gemb_struct_bytes


def parse_header(path: str = HEADER) -> dict[str, tuple[str, list[tuple[str, str]]]]:
    """name -> (return type, [(ctype, param name)]) for every function the header declares."""
    text = open(path).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    text = re.sub(r"//[^\n]*", "", text)
    out = {}
    for m in re.finditer(r"\b(const char\*|int32_t|uint64_t|void)\s+(gemb_\w+)\s*\(([^)]*)\)\s*;", text):
        ret, name, params = m.group(1), m.group(2), m.group(3).strip()
        plist = []
        if params and params != "void":
            for prm in params.split(","):
                prm = " ".join(prm.split())
                pname = prm.split()[-1].lstrip("*")
                ptype = prm[: prm.rfind(pname)].strip()
                plist.append((ptype, pname))
        out[name] = (ret, plist)
    return out


def _ctype(t: str):
    if "*" in t or t == "gemb_stream_t":
        return C.c_void_p
    return _SCALARS[t.replace("const ", "")]


def _as_arg(v):
    if v is None:
        return None
    if hasattr(v, "data_ptr"):
        return v.data_ptr()
    if hasattr(v, "cuda_stream"):
        return v.cuda_stream
    if isinstance(v, C.Structure):
        return C.addressof(v)
    if isinstance(v, C.Array):
        return C.addressof(v)
    return v


class Lib:
    def __init__(self, path: str = LIB_PATH):
        if not os.path.exists(path):
            raise RuntimeError(
                f"{path} is missing: build it with `python -m gem16_b200.build` (no fallback exists)")
        self.path = path
        self.cdll = C.CDLL(path)
        self.protos = parse_header()
        for name, (ret, params) in self.protos.items():
            fn = getattr(self.cdll, name)
            fn.argtypes = [_ctype(t) for t, _ in params]
            fn.restype = {"const char*": C.c_char_p, "int32_t": C.c_int32, "uint64_t": C.c_uint64,
                          "void": None}[ret]

    def last_error(self) -> str:
        return self.cdll.gemb_last_error().decode()

    def raw(self, name: str, *args) -> int:
        """Calls `name` and returns the raw status without raising."""
        return getattr(self.cdll, name)(*[_as_arg(a) for a in args])

    def __getattr__(self, name: str):
        if not name.startswith("gemb_"):
            raise AttributeError(name)
        ret = self.protos[name][0]
        fn = getattr(self.cdll, name)

        def call(*args):
            rc = fn(*[_as_arg(a) for a in args])
            if ret == "int32_t" and rc != 0:
                raise GembError(rc, self.last_error())
            return rc

        return call


_LIB: Lib | None = None


def load() -> Lib:
    global _LIB
    if _LIB is None:
        _LIB = Lib()
    return _LIB
