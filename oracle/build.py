"""Build recipe for the CPU oracle (test infrastructure, never a product path).

Two shared objects:
  oracle/libgemb_oracle.so   -- gemb_oracle.cpp, our restatement of the reference contract.
  oracle/_ref/libgem16_ref.so -- the UNMODIFIED gem16 sources src/numeric/{nvfp4,fp8,layer}.cpp
                                 compiled where they lie under $GEM16_REFERENCE (a checkout of
                                 gem16; without the variable, a `reference` directory beside this
                                 repository) plus ref_wrap.cpp.  Only built when that tree is
                                 present; the prebuilt file is used otherwise.
Nothing from the reference tree is copied into this repository.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF_ROOT = os.environ.get("GEM16_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
ORACLE_SO = os.path.join(HERE, "libgemb_oracle.so")
REF_DIR = os.path.join(HERE, "_ref")
REF_SO = os.path.join(REF_DIR, "libgem16_ref.so")


def _stale(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def build_oracle(force: bool = False) -> str:
    src = os.path.join(HERE, "gemb_oracle.cpp")
    if force or _stale(ORACLE_SO, [src]):
        cmd = ["g++", "-std=c++17", "-O2", "-mfma", "-ffp-contract=off", "-fPIC", "-shared",
               "-pthread", src, "-o", ORACLE_SO]
        subprocess.check_call(cmd)
    return ORACLE_SO


def reference_available() -> bool:
    return os.path.isfile(os.path.join(REF_ROOT, "src", "numeric", "nvfp4.cpp"))


def build_ref(force: bool = False) -> str | None:
    """Compile the reference's own numeric sources into oracle/_ref/. Returns the path, or the
    prebuilt file when the reference tree is absent, or None when neither exists."""
    if not reference_available():
        return REF_SO if os.path.exists(REF_SO) else None
    srcs = [os.path.join(REF_ROOT, "src", "numeric", "nvfp4.cpp"),
            os.path.join(REF_ROOT, "src", "numeric", "fp8.cpp"),
            os.path.join(REF_ROOT, "src", "numeric", "layer.cpp"),
            os.path.join(HERE, "ref_wrap.cpp")]
    if force or _stale(REF_SO, srcs):
        os.makedirs(REF_DIR, exist_ok=True)
        cmd = ["g++", "-std=c++20", "-O2", "-fPIC", "-shared", "-pthread",
               "-I", os.path.join(REF_ROOT, "include"), *srcs, "-o", REF_SO]
        subprocess.check_call(cmd)
    return REF_SO


if __name__ == "__main__":
    print(build_oracle(force="--force" in sys.argv))
    print(build_ref(force="--force" in sys.argv))
