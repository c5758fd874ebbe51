"""GPU parity of the tcgen05 prefill GEMMs against the binary64 CPU oracle.

Gate (bf16 output against the bf16-rounded oracle, both consuming the same quantised bytes):
relative Frobenius error <= 1e-3, plus the budgets the reference's CUDA tests use at real shapes
(tests/cuda/nvfp4_reference_test.cu:782, :1247-1248): max_abs < 0.125, cosine > 0.9999 / 0.99999.
"""
import numpy as np
import pytest
import torch

from tests.gemm_util import bf16_tensor_to_f32, error_stats, fp8_operand, nvfp4_operand
from tests.util import to_np

pytestmark = pytest.mark.gpu

REL_FRO = 1e-3
SHAPES = [
    # tokens, rows, K                      origin
    (1, 8, 64),                            # minimum geometry
    (17, 136, 704),                        # token / row / K tails together (expert down K)
    (128, 3840, 15360),                    # tests/cuda/nvfp4_reference_test.cu: Down
    (129, 15360, 3840),                    # ... Gate with a one-row token tail
    (2048, 128, 3840),                     # ... many token tiles, one row tile
    (300, 2112, 2816),                     # shared FFN: rows not a multiple of 128
    (257, 2816, 2112),                     # shared FFN down: K = 33 * 64
]


def sample_tokens(m, n=24):
    return np.unique(np.concatenate([np.arange(min(m, 3)), np.linspace(0, m - 1, min(m, n)).astype(int)]))


@pytest.mark.parametrize("bn", [128, 256])
@pytest.mark.parametrize("tokens,rows,k", SHAPES)
def test_nvfp4_gemm(lib, dev, orc, tokens, rows, k, bn):
    lib.gemb_set_tuning(3, bn)
    try:
        a = nvfp4_operand(lib, dev, tokens, k, 1.0, 11 + tokens)
        w = nvfp4_operand(lib, dev, rows, k, 0.02, 23 + rows)
        out = torch.full((tokens, rows), 0x7FC0, dtype=torch.int16, device=dev)  # NaN canary
        lib.gemb_nvfp4_gemm_bf16(a["packed"], a["inter"], w["packed"], w["inter"], out, tokens, rows, k,
                                 a["div"], w["div"], None)
        lib.gemb_check_device_status()
    finally:
        lib.gemb_set_tuning(3, 0)
    idx = sample_tokens(tokens)
    want = orc.nvfp4_matmul(to_np(a["packed"])[idx], to_np(a["compact"])[idx], to_np(w["packed"]),
                            to_np(w["compact"]), a["div"], w["div"])
    got_all = bf16_tensor_to_f32(out)
    assert np.isfinite(got_all).all()
    st = error_stats(got_all[idx], want)
    assert st["rel_fro"] <= REL_FRO and st["max_abs"] < 0.125 and st["cos"] > 0.9999, st
    # every output (not just the sampled tokens) against the scalar GPU cross-check
    ref = torch.zeros((tokens, rows), device=dev)
    lib.gemb_nvfp4_reference_projection(a["packed"], a["compact"], w["packed"], w["compact"], ref, tokens, rows, k,
                                        a["div"], w["div"], None)
    st = error_stats(got_all, ref.cpu().numpy().astype(np.float64))
    assert st["rel_fro"] <= REL_FRO, st


@pytest.mark.parametrize("bn", [128, 256])
@pytest.mark.parametrize("tokens,rows,k", [(1, 8, 32), (17, 136, 96), (128, 4096, 3840), (129, 3840, 4096), (512, 8192, 3840)])
def test_fp8_gemm(lib, dev, orc, tokens, rows, k, bn):
    lib.gemb_set_tuning(3, bn)
    try:
        a = fp8_operand(lib, dev, tokens, k, 1.0, 5 + tokens)
        w = fp8_operand(lib, dev, rows, k, 0.02, 7 + rows)
        out = torch.full((tokens, rows), 0x7FC0, dtype=torch.int16, device=dev)
        lib.gemb_fp8_gemm_bf16(a["q"], a["scales"], w["q"], w["scales_bf16"], out, tokens, rows, k, None)
        lib.gemb_check_device_status()
    finally:
        lib.gemb_set_tuning(3, 0)
    idx = sample_tokens(tokens)
    want = orc.fp8_matmul(to_np(a["q"])[idx], to_np(a["scales"])[idx], to_np(w["q"]), to_np(w["scales_bf16"], np.uint16))
    got_all = bf16_tensor_to_f32(out)
    assert np.isfinite(got_all).all()
    st = error_stats(got_all[idx], want)
    assert st["rel_fro"] <= REL_FRO and st["max_abs"] < 0.125 and st["cos"] > 0.99999, st
    ref = torch.zeros((tokens, rows), device=dev)
    lib.gemb_fp8_reference_projection(a["q"], a["scales"], w["q"], w["scales_bf16"], ref, tokens, rows, k, None)
    st = error_stats(got_all, ref.cpu().numpy().astype(np.float64))
    assert st["rel_fro"] <= REL_FRO, st


def test_nvfp4_linear_config0_full(lib, dev, orc):
    # The full single-linear configuration: X[512, 3840] ~ N(0,1), W[15360, 3840] ~ N(0, 0.02),
    # every one of the 7,864,320 outputs against the binary64 oracle.
    tokens, rows, k = 512, 15360, 3840
    a = nvfp4_operand(lib, dev, tokens, k, 1.0, 20261125)
    w = nvfp4_operand(lib, dev, rows, k, 0.02, 20261126)
    out = torch.zeros((tokens, rows), dtype=torch.int16, device=dev)
    lib.gemb_nvfp4_gemm_bf16(a["packed"], a["inter"], w["packed"], w["inter"], out, tokens, rows, k, a["div"],
                             w["div"], None)
    lib.gemb_check_device_status()
    want = orc.nvfp4_matmul(to_np(a["packed"]), to_np(a["compact"]), to_np(w["packed"]), to_np(w["compact"]),
                            a["div"], w["div"])
    st = error_stats(bf16_tensor_to_f32(out), want)
    print("config-0 full parity:", st)
    assert st["rel_fro"] <= REL_FRO and st["max_abs"] < 0.125 and st["cos"] > 0.9999, st
    # determinism: a second run is bit-identical
    out2 = torch.zeros_like(out)
    lib.gemb_nvfp4_gemm_bf16(a["packed"], a["inter"], w["packed"], w["inter"], out2, tokens, rows, k, a["div"],
                             w["div"], None)
    assert torch.equal(out, out2)


def test_gemm_agrees_with_gemv(lib, dev):
    # One token through the prefill GEMM equals the decode GEMV rounded to bf16 (up to rare
    # 1-ulp flips from accumulation order).
    rows, k = 3840, 15360
    a = nvfp4_operand(lib, dev, 1, k, 1.0, 1)
    w = nvfp4_operand(lib, dev, rows, k, 0.02, 2)
    out = torch.zeros((1, rows), dtype=torch.int16, device=dev)
    lib.gemb_nvfp4_gemm_bf16(a["packed"], a["inter"], w["packed"], w["inter"], out, 1, rows, k, a["div"], w["div"], None)
    y = torch.zeros((rows,), device=dev)
    lib.gemb_nvfp4_gemv(a["packed"], a["compact"], w["packed"], w["compact"], y, rows, k, a["div"], w["div"], None)
    st = error_stats(bf16_tensor_to_f32(out)[0], y.cpu().numpy().astype(np.float64))
    assert st["rel_fro"] <= REL_FRO and st["mismatch"] < 0.01, st


def test_prefill_property_at_full_size(lib, dev):
    # 16,384-token prefill shape without the CPU oracle: permuting tokens permutes outputs
    # bit-exactly (tile placement must not change a token's result), sampled rows match the
    # scalar GPU cross-check.
    tokens, rows, k = 16384, 3840, 3840
    a = nvfp4_operand(lib, dev, tokens, k, 1.0, 3)
    w = nvfp4_operand(lib, dev, rows, k, 0.02, 4)
    out = torch.zeros((tokens, rows), dtype=torch.int16, device=dev)
    lib.gemb_nvfp4_gemm_bf16(a["packed"], a["inter"], w["packed"], w["inter"], out, tokens, rows, k, a["div"], w["div"], None)
    perm = torch.randperm(tokens, device=dev)
    packed_p = a["packed"][perm].contiguous()
    compact_p = a["compact"][perm].contiguous()
    inter_p = torch.empty_like(a["inter"])
    lib.gemb_nvfp4_interleave_scales(compact_p, inter_p, tokens, k, None)
    out_p = torch.zeros_like(out)
    lib.gemb_nvfp4_gemm_bf16(packed_p, inter_p, w["packed"], w["inter"], out_p, tokens, rows, k, a["div"], w["div"], None)
    lib.gemb_check_device_status()
    assert torch.equal(out[perm], out_p)
    sel = torch.arange(0, tokens, 331, device=dev)
    ref = torch.zeros((sel.numel(), rows), device=dev)
    lib.gemb_nvfp4_reference_projection(a["packed"][sel].contiguous(), a["compact"][sel].contiguous(), w["packed"],
                                        w["compact"], ref, sel.numel(), rows, k, a["div"], w["div"], None)
    st = error_stats(bf16_tensor_to_f32(out[sel]), ref.cpu().numpy().astype(np.float64))
    assert st["rel_fro"] <= REL_FRO, st


def test_nvfp4_gemm_f32_output(lib, dev, orc):
    # fp32 epilogue (row-split partial sums): against the binary64 oracle without bf16 rounding.
    tokens, rows, k = 77, 328, 704
    a = nvfp4_operand(lib, dev, tokens, k, 1.0, 5)
    w = nvfp4_operand(lib, dev, rows, k, 0.02, 6)
    out = torch.full((tokens, rows), float("nan"), device=dev)
    lib.gemb_nvfp4_gemm_f32(a["packed"], a["inter"], w["packed"], w["inter"], out, tokens, rows, k, a["div"], w["div"], None)
    lib.gemb_check_device_status()
    want = orc.nvfp4_matmul(to_np(a["packed"]), to_np(a["compact"]), to_np(w["packed"]), to_np(w["compact"]), a["div"], w["div"])
    got = out.cpu().numpy().astype(np.float64)
    assert np.isfinite(got).all()
    assert np.linalg.norm(got - want) / np.linalg.norm(want) < 1e-6


@pytest.mark.parametrize("tokens,rows,k", [(128, 256, 64), (300, 1000, 704), (4096, 4096, 512), (1153, 2816, 2112)])
def test_cta_pair_and_single_cta_tiles_agree_bit_for_bit(lib, dev, tokens, rows, k):
    """The dense GEMMs run on CTA pairs by default; GEMB_TUNE_GEMM_PAIR = 1 runs the 256-wide tile on one
    CTA, GEMB_TUNE_GEMM_BN = 128 with pairs forced the 256 x 128 pair tile.  Same accumulation order along
    K in all of them: the outputs must be identical.
    Shapes cover an odd number of 128-row tiles (the odd CTA of the last pair has no rows), ragged
    rows / columns, a K tail, and several tiles per cluster."""
    a = nvfp4_operand(lib, dev, tokens, k, 1.0, 3)
    w = nvfp4_operand(lib, dev, rows, k, 0.02, 4)
    a8 = fp8_operand(lib, dev, tokens, k, 1.0, 5)
    w8 = fp8_operand(lib, dev, rows, k, 0.02, 6)
    outs = {}
    try:
        for mode in (1, 2, 3):          # 3: pairs on 256 x 128 tiles with two accumulators (NVFP4)
            lib.gemb_set_tuning(5, min(mode, 2))
            lib.gemb_set_tuning(3, 128 if mode == 3 else 0)
            o4 = torch.full((tokens, rows), 0x7FC0, dtype=torch.int16, device=dev)
            o8 = torch.full((tokens, rows), 0x7FC0, dtype=torch.int16, device=dev)
            o32 = torch.full((tokens, rows), float("nan"), device=dev)
            lib.gemb_nvfp4_gemm_bf16(a["packed"], a["inter"], w["packed"], w["inter"], o4, tokens, rows, k,
                                     a["div"], w["div"], None)
            lib.gemb_nvfp4_gemm_f32(a["packed"], a["inter"], w["packed"], w["inter"], o32, tokens, rows, k,
                                    a["div"], w["div"], None)
            lib.gemb_fp8_gemm_bf16(a8["q"], a8["scales"], w8["q"], w8["scales_bf16"], o8, tokens, rows, k, None)
            torch.cuda.synchronize()
            lib.gemb_check_device_status()
            outs[mode] = (o4, o32, o8)
    finally:
        lib.gemb_set_tuning(5, 0)
        lib.gemb_set_tuning(3, 0)
    for x, y, z, name in zip(outs[1], outs[2], outs[3], ("nvfp4 bf16", "nvfp4 f32", "fp8 bf16")):
        assert torch.equal(x, y), name
        assert torch.equal(x, z), name + " (256 x 128 pair tiles)"
        assert not torch.isnan(y.float() if y.dtype == torch.float32 else y.view(torch.bfloat16).float()).any(), name
