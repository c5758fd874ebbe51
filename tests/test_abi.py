"""CPU tests of the C-ABI boundary: the library loads, exports every symbol the header declares,
validates arguments like the reference launchers do, and refuses to compute without a B200."""
import ctypes

import pytest

from gem16_b200.lib import GembError, parse_header


def test_exports_every_declared_symbol(lib):
    protos = parse_header()
    assert len(protos) >= 18
    for name in protos:
        assert hasattr(lib.cdll, name), name


def test_status_names_mirror_reference(lib):
    # include/gem16/status.h:9-19
    names = ["kOk", "kInvalidArgument", "kNotFound", "kIoError", "kDataLoss", "kUnsupported",
             "kResourceExhausted", "kCancelled", "kInternal"]
    for code, name in enumerate(names):
        assert lib.cdll.gemb_status_name(code).decode() == name


def test_interleaved_bytes(lib):
    assert lib.cdll.gemb_interleaved_scale_bytes(129, 3840) == 256 * 240
    assert lib.cdll.gemb_interleaved_scale_bytes(128, 704) == 128 * 44
    assert lib.cdll.gemb_interleaved_scale_bytes(1, 16) == 128 * 4


def test_invalid_arguments_are_rejected_before_any_launch(lib):
    p = 0x1000  # never dereferenced: validation fails first
    cases = [
        ("gemb_nvfp4_quantize", (None, 0, p, p, 1, 16, 1.0, 0, 0, None)),        # null input
        ("gemb_nvfp4_quantize", (p, 0, p, p, 1, 15, 1.0, 0, 0, None)),           # K % 16
        ("gemb_nvfp4_quantize", (p, 0, p, p, 1, 16, 0.0, 0, 0, None)),           # divisor 0
        ("gemb_nvfp4_quantize", (p, 0, p, p, 1, 16, float("inf"), 0, 0, None)),  # divisor inf
        ("gemb_nvfp4_quantize", (p, 7, p, p, 1, 16, 1.0, 0, 0, None)),           # dtype
        ("gemb_fp8_quantize", (p, 0, p, p, 0, 16, None)),                         # empty
        ("gemb_fp8_gemv", (p, p, p, p, p, 8, 24, None)),                          # K % 16
        ("gemb_nvfp4_gemv", (p, p, p, p, p, 12, 64, 1.0, 1.0, None)),             # rows % 8
        ("gemb_nvfp4_gemv", (p, p, p, p, p, 8, 48, 1.0, 1.0, None)),              # K % 64
        ("gemb_nvfp4_gemv", (p, p, p, p, p, 8, 64, -1.0, 1.0, None)),             # divisor
        ("gemb_nvfp4_reference_projection", (p, p, p, p, p, 1, 8, 8, 1.0, 1.0, None)),
    ]
    for name, args in cases:
        assert lib.raw(name, *args) == 1, name
        assert name in lib.last_error()
    with pytest.raises(GembError) as e:
        lib.gemb_nvfp4_quantize(None, 0, p, p, 1, 16, 1.0, 0, 0, None)
    assert e.value.status_name == "kInvalidArgument"


def test_no_cpu_fallback(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    p = 0x1000
    assert lib.raw("gemb_device_check") == 5
    assert lib.raw("gemb_nvfp4_quantize", p, 0, p, p, 1, 16, 1.0, 0, 0, None) == 5
    assert lib.raw("gemb_fp8_gemv", p, p, p, p, p, 8, 32, None) == 5


def test_missing_library_fails_loudly(tmp_path):
    from gem16_b200.lib import Lib
    with pytest.raises(RuntimeError):
        Lib(str(tmp_path / "libgemb200.so"))


def test_shim_compiles_against_the_reference_headers():
    # The drop-in shim must match the reference's own launcher declarations: compile it against
    # the gem16 headers where the reference tree is present; -Wmissing-declarations turns a
    # definition whose signature matches no reference declaration into an error.
    import os
    import subprocess
    from oracle.build import REF_ROOT as ref      # $GEM16_REFERENCE, or `reference` beside this repository
    if not os.path.isfile(os.path.join(ref, "src", "cuda", "nvfp4", "sm120.h")):
        pytest.skip("reference tree not present")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cuda_inc = "/usr/local/cuda/include"
    cmd = ["g++", "-std=c++20", "-fsyntax-only", "-Wall", "-Wmissing-declarations", "-Werror", "-I", os.path.join(ref, "include"),
           "-I", os.path.join(ref, "src"), "-I", os.path.join(root, "include"), "-I", cuda_inc,
           os.path.join(root, "gem16_b200", "shim", "gem16_internal_shim.cpp")]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]


def test_shim_defines_every_launcher_of_the_operator_headers():
    # The shim replaces gem16's operator sources at link time only if it defines every launcher the
    # operator headers of this path declare (and the RMSNorm + residual forms of layer/reference.h).
    import os
    import re
    from oracle.build import REF_ROOT as ref
    if not os.path.isfile(os.path.join(ref, "src", "cuda", "nvfp4", "sm120.h")):
        pytest.skip("reference tree not present")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    shim = open(os.path.join(root, "gem16_b200", "shim", "gem16_internal_shim.cpp")).read()
    defined = set(re.findall(r"^Status (Launch\w+)\(", shim, flags=re.M))
    declared = set()
    for h in ("nvfp4/reference", "nvfp4/sm120", "nvfp4/cutlass_sm120", "nvfp4/gemv", "nvfp4/mlp", "fp8/reference", "fp8/sm120",
              "fp8/cutlass_sm120", "output_head"):
        declared |= set(re.findall(r"Status (Launch\w+)\(", open(os.path.join(ref, "src", "cuda", h + ".h")).read()))
    assert declared and not (declared - defined), sorted(declared - defined)
    assert {"LaunchRmsNormResidualBf16", "LaunchRmsNormResidualBf16Input", "LaunchRmsNormResidualPhysicalBf16"} <= defined
