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
