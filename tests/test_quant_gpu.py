"""GPU parity of the activation quantizers against the CPU oracle (bit-exact bytes)."""
import numpy as np
import pytest
import torch

from tests.util import bf16_bits, bf16_round, from_bf16_bits, nvfp4_divisor, to_dev, to_np

pytestmark = pytest.mark.gpu

F32, BF16 = 0, 1
COMPACT, INTERLEAVED = 0, 1
EXACT, RCP = 0, 1


def run_nvfp4(lib, dev, x, g, dtype=F32, layout=COMPACT, mode=EXACT):
    t, k = x.shape
    xin = to_dev(bf16_bits(x) if dtype == BF16 else x.astype(np.float32), dev)
    packed = torch.full((t, k // 2), 0xA5, dtype=torch.uint8, device=dev)
    nsc = lib.cdll.gemb_interleaved_scale_bytes(t, k) if layout == INTERLEAVED else t * (k // 16)
    scales = torch.full((nsc,), 0xA5, dtype=torch.uint8, device=dev)
    lib.gemb_nvfp4_quantize(xin, dtype, packed, scales, t, k, g, layout, mode, None)
    torch.cuda.synchronize()
    return to_np(packed), to_np(scales)


def test_reference_kat(lib, dev, orc):
    # tests/cuda/nvfp4_reference_test.cu:128-206 (GPU bytes == CPU oracle bytes on the KAT).
    act = np.array([orc.e2m1_decode(i) / 2.0 for i in range(16)], np.float32)[None]
    p, s = run_nvfp4(lib, dev, act, 2.0)
    assert p.tobytes() == bytes([0x10, 0x32, 0x54, 0x76, 0x98, 0xBA, 0xDC, 0xFE]) and s.tobytes() == b"\x38"
    p, s = run_nvfp4(lib, dev, np.zeros((1, 16), np.float32), 11.0)
    assert not p.any() and not s.any()


def test_vllm_boundary_fixture_rcp_mode(lib, dev):
    # tests/cuda/nvfp4_reference_test.cu:208-255: pins the device (rcp.approx) contract.
    act = np.array([[-0.1708984375, 0.5703125, -0.4375, 2.777576446533203e-05, -3.46875,
                     -0.000461578369140625, 0.6015625, -0.0830078125, 0.10009765625, 0.06884765625,
                     0.69921875, -0.000652313232421875, -0.875, 6.866455078125e-05,
                     -2.682209014892578e-05, 0.8359375]], np.float32)
    p, s = run_nvfp4(lib, dev, act, 0.375, mode=RCP)
    assert p.tobytes() == bytes([0x29, 0x09, 0x8F, 0x82, 0x00, 0x82, 0x0B, 0x38])
    assert s.tobytes() == b"\x26"


def test_golden_vectors(lib, dev, golden):
    x = golden["nvfp4_x"]
    for dtype in (F32, BF16):
        p, s = run_nvfp4(lib, dev, x, float(golden["nvfp4_ga"]), dtype=dtype)
        assert np.array_equal(p, golden["nvfp4_packed"])
        assert np.array_equal(s.reshape(golden["nvfp4_scales"].shape), golden["nvfp4_scales"])
    p, s = run_nvfp4(lib, dev, x, 300.0)
    assert np.array_equal(p, golden["nvfp4_packed_g300"])
    assert np.array_equal(s.reshape(golden["nvfp4_scales_g300"].shape), golden["nvfp4_scales_g300"])
    w = golden["nvfp4_w"]
    p, s = run_nvfp4(lib, dev, w, float(golden["nvfp4_gw"]))
    assert np.array_equal(p, golden["nvfp4_wp"]) and np.array_equal(s.reshape(-1), golden["nvfp4_ws"].reshape(-1))


@pytest.mark.parametrize("tokens,k", [(1, 16), (1, 3840), (17, 704), (129, 2816), (512, 3840), (3, 48), (64, 15360)])
@pytest.mark.parametrize("dtype", [F32, BF16])
def test_seeded_parity(lib, dev, orc, tokens, k, dtype):
    rng = np.random.default_rng(1000 + tokens * 7 + k)
    x = bf16_round(rng.standard_normal((tokens, k)).astype(np.float32))
    if dtype == F32:
        x = (x * rng.uniform(0.5, 1.5, size=x.shape)).astype(np.float32)  # values off the bf16 grid
    g = nvfp4_divisor(x)
    p, s = run_nvfp4(lib, dev, x, g, dtype=dtype)
    xo = bf16_round(x) if dtype == BF16 else x
    po, so = orc.nvfp4_quantize(xo, g)
    assert np.array_equal(p, po)
    assert np.array_equal(s.reshape(so.shape), so)


@pytest.mark.parametrize("tokens,k", [(1, 64), (129, 3840), (300, 704), (5, 48)])
def test_interleaved_scales(lib, dev, orc, tokens, k):
    rng = np.random.default_rng(tokens + k)
    x = bf16_round(rng.standard_normal((tokens, k)).astype(np.float32))
    g = nvfp4_divisor(x)
    p, s = run_nvfp4(lib, dev, x, g, dtype=BF16, layout=INTERLEAVED)
    po, so = orc.nvfp4_quantize(x, g)
    assert np.array_equal(p, po)
    assert np.array_equal(s, orc.interleave_scales(so, k))
    # standalone shuffle
    out = torch.full((s.size,), 0x5A, dtype=torch.uint8, device=dev)
    lib.gemb_nvfp4_interleave_scales(to_dev(so, dev), out, tokens, k, None)
    assert np.array_equal(to_np(out), s)


def test_rcp_mode_close_to_exact(lib, dev, orc):
    # The two contracts differ by at most a few nibbles per thousand (one nibble on the 16-value vLLM
    # fixture of tests/cuda/nvfp4_reference_test.cu:208-255); scales are identical except at rounding boundaries.
    rng = np.random.default_rng(5)
    x = bf16_round(rng.standard_normal((64, 3840)).astype(np.float32))
    g = nvfp4_divisor(x)
    p0, s0 = run_nvfp4(lib, dev, x, g, dtype=BF16, mode=EXACT)
    p1, s1 = run_nvfp4(lib, dev, x, g, dtype=BF16, mode=RCP)
    lo = ((p0 & 15) != (p1 & 15)).mean()
    hi = ((p0 >> 4) != (p1 >> 4)).mean()
    assert (s0 != s1).mean() < 0.01 and lo < 0.01 and hi < 0.01


def test_gated_gelu_quantize(lib, dev, orc):
    # Boundaries of src/cuda/nvfp4/reference.cu:177-217.  tanhf differs by an ulp between the
    # device and the host libm, which can flip a bf16 rounding; allow 0.2 % nibble mismatches.
    rng = np.random.default_rng(11)
    t, k = 37, 704
    gate = rng.standard_normal((t, k)).astype(np.float32) * 2
    up = rng.standard_normal((t, k)).astype(np.float32)
    prod = orc.gated_gelu(gate, up)
    g = nvfp4_divisor(prod)
    po, so = orc.nvfp4_quantize(prod, g)
    for dtype in (F32, BF16):
        a = to_dev(bf16_bits(gate) if dtype == BF16 else gate, dev)
        b = to_dev(bf16_bits(up) if dtype == BF16 else up, dev)
        packed = torch.zeros((t, k // 2), dtype=torch.uint8, device=dev)
        scales = torch.zeros((t, k // 16), dtype=torch.uint8, device=dev)
        lib.gemb_nvfp4_gated_gelu_quantize(a, b, dtype, packed, scales, t, k, g, COMPACT, EXACT, None)
        p, s = to_np(packed), to_np(scales)
        mism = (((p & 15) != (po & 15)).sum() + ((p >> 4) != (po >> 4)).sum()) / (t * k)
        assert mism < 2e-3 and (s != so).mean() < 2e-3


def test_rmsnorm_quantize(lib, dev, orc):
    # src/cuda/nvfp4/reference.cu:92-153; rsqrtf is approximate on the device, so a few bf16
    # roundings may flip: allow 0.5 % nibble mismatches, scales nearly identical.
    rng = np.random.default_rng(13)
    t, k = 9, 3840
    x = rng.standard_normal((t, k)).astype(np.float32) * 3
    w = bf16_bits(1.0 + 0.1 * rng.standard_normal(k).astype(np.float32))
    normed = orc.rmsnorm_bf16(x, w, 1e-6)
    g = nvfp4_divisor(normed)
    po, so = orc.nvfp4_quantize(normed, g)
    packed = torch.zeros((t, k // 2), dtype=torch.uint8, device=dev)
    scales = torch.zeros((t, k // 16), dtype=torch.uint8, device=dev)
    lib.gemb_nvfp4_rmsnorm_quantize(to_dev(x, dev), F32, to_dev(w, dev), packed, scales, t, k, 1e-6, g, COMPACT, EXACT, None)
    p, s = to_np(packed), to_np(scales)
    mism = (((p & 15) != (po & 15)).sum() + ((p >> 4) != (po >> 4)).sum()) / (t * k)
    assert mism < 5e-3 and (s != so).mean() < 5e-3
    # FP8 flavour: src/cuda/fp8/reference.cu:71-136
    qo, sco = orc.fp8_quantize(normed)
    q = torch.zeros((t, k), dtype=torch.uint8, device=dev)
    sc = torch.zeros((t,), dtype=torch.float32, device=dev)
    lib.gemb_fp8_rmsnorm_quantize(to_dev(x, dev), F32, to_dev(w, dev), q, sc, t, k, 1e-6, None)
    assert (to_np(q) != qo).mean() < 5e-3
    assert np.allclose(to_np(sc), sco, rtol=1e-2)


@pytest.mark.parametrize("tokens,k", [(1, 16), (1, 3840), (1, 15360), (33, 4096), (512, 3840)])
@pytest.mark.parametrize("dtype", [F32, BF16])
def test_fp8_quantize_parity(lib, dev, orc, tokens, k, dtype):
    rng = np.random.default_rng(tokens * 31 + k)
    x = bf16_round(rng.standard_normal((tokens, k)).astype(np.float32))
    if dtype == F32:
        x = (x * rng.uniform(0.5, 1.5, size=x.shape)).astype(np.float32)
    if tokens > 2:
        x[1] = 0.0
    q = torch.full((tokens, k), 0xA5, dtype=torch.uint8, device=dev)
    sc = torch.zeros((tokens,), dtype=torch.float32, device=dev)
    lib.gemb_fp8_quantize(to_dev(bf16_bits(x) if dtype == BF16 else x, dev), dtype, q, sc, tokens, k, None)
    qo, so = orc.fp8_quantize(x)
    assert np.array_equal(to_np(q), qo)
    assert np.array_equal(to_np(sc), so)


def test_fp8_golden(lib, dev, golden):
    x = golden["fp8_x"]
    t, k = x.shape
    q = torch.zeros((t, k), dtype=torch.uint8, device=dev)
    sc = torch.zeros((t,), dtype=torch.float32, device=dev)
    lib.gemb_fp8_quantize(to_dev(x, dev), F32, q, sc, t, k, None)
    assert np.array_equal(to_np(q), golden["fp8_q"]) and np.array_equal(to_np(sc), golden["fp8_scales"])


def test_quantizer_properties_at_full_size(lib, dev):
    # Size-independent checks at the 16,384-token prefill shape: idempotence on the dequantised
    # grid and determinism across two runs.
    torch.manual_seed(0)
    t, k = 16384, 3840
    x = torch.randn((t, k), device=dev, dtype=torch.bfloat16)
    g = float(6 * 448 / x.abs().max().item())
    outs = []
    for _ in range(2):
        p = torch.zeros((t, k // 2), dtype=torch.uint8, device=dev)
        s = torch.zeros((t, k // 16), dtype=torch.uint8, device=dev)
        lib.gemb_nvfp4_quantize(x.view(torch.int16), BF16, p, s, t, k, g, COMPACT, EXACT, None)
        outs.append((p, s))
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
    p, s = outs[0]
    assert int(s.max()) <= 0x7E
    # scale bytes are monotone in block amax: the block holding the global amax gets 448.
    assert int(s.max()) == 0x7E
