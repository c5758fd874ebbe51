"""GPU parity of the batch-1 decode projections against the binary64 CPU oracle."""
import numpy as np
import pytest
import torch

from tests.util import bf16_bits, bf16_round, nvfp4_divisor, rel_fro, to_dev, to_np

pytestmark = pytest.mark.gpu


def make_fp8_problem(orc, rows, k, seed):
    rng = np.random.default_rng(seed)
    x = bf16_round(rng.standard_normal((1, k)).astype(np.float32))
    w = (rng.standard_normal((rows, k)) * 0.02).astype(np.float32)
    wq, wsc = orc.fp8_quantize(w)
    xq, xsc = orc.fp8_quantize(x)
    return x, xq, xsc, wq, bf16_bits(wsc)


# Budget: the reference accepts < 1e-5 absolute for T=1 native vs binary64 on its fixture
# (tests/cuda/nvfp4_reference_test.cu:488); on N(0,1) data we bound the relative error.
@pytest.mark.parametrize("rows,k", [(8, 16), (40, 528), (3840, 4096), (8192, 3840), (3840, 15360), (30720, 3840), (13, 3840)])
def test_fp8_gemv(lib, dev, orc, rows, k):
    x, xq, xsc, wq, wsb = make_fp8_problem(orc, rows, k, rows + k)
    want = orc.fp8_matmul(xq, xsc, wq, wsb)[0]
    out = torch.full((rows,), float("nan"), device=dev)
    lib.gemb_fp8_gemv(to_dev(xq, dev), to_dev(xsc, dev), to_dev(wq, dev), to_dev(wsb, dev), out, rows, k, None)
    got = to_np(out)
    assert rel_fro(got, want) < 1e-6
    assert np.abs(got - want).max() <= 1e-5 * max(1.0, np.abs(want).max())
    # scalar GPU cross-check agrees as well
    ref = torch.zeros((rows,), device=dev)
    lib.gemb_fp8_reference_projection(to_dev(xq, dev), to_dev(xsc, dev), to_dev(wq, dev), to_dev(wsb, dev), ref, 1, rows, k, None)
    assert rel_fro(to_np(ref), want) < 1e-6
    # fused bf16 -> FP8 quantisation inside the GEMV is bit-identical to the two-step form
    for odt in (0, 1):
        o2 = torch.zeros((rows,), device=dev, dtype=torch.float32 if odt == 0 else torch.int16)
        lib.gemb_fp8_gemv_bf16in(to_dev(bf16_bits(x), dev), to_dev(wq, dev), to_dev(wsb, dev), o2, odt, rows, k, None)
        if odt == 0:
            assert np.array_equal(to_np(o2), got)
        else:
            assert np.array_equal(to_np(o2, np.uint16), bf16_bits(got))


def test_fp8_gemv_grouped_qkv(lib, dev, orc):
    k = 3840
    x, xq, xsc, _, _ = make_fp8_problem(orc, 8, k, 1)
    mats = [make_fp8_problem(orc, r, k, 100 + r)[3:] for r in (4096, 2048, 2048)]
    outs = [torch.zeros((r,), device=dev) for r in (4096, 2048, 2048)]
    d = [(to_dev(w, dev), to_dev(s, dev)) for w, s in mats]
    lib.gemb_fp8_gemv_qkv(to_dev(xq, dev), to_dev(xsc, dev), d[0][0], d[0][1], outs[0], 4096, d[1][0], d[1][1],
                          outs[1], 2048, d[2][0], d[2][1], outs[2], 2048, k, None)
    for (w, s), o in zip(mats, outs):
        assert rel_fro(to_np(o), orc.fp8_matmul(xq, xsc, w, s)[0]) < 1e-6
    # null V: global-attention layers reuse K (src/cuda/fp8/sm120.h:66-68)
    o0, o1 = torch.zeros((4096,), device=dev), torch.zeros((2048,), device=dev)
    lib.gemb_fp8_gemv_qkv(to_dev(xq, dev), to_dev(xsc, dev), d[0][0], d[0][1], o0, 4096, d[1][0], d[1][1], o1,
                          2048, None, None, None, 0, k, None)
    assert torch.equal(o0, outs[0]) and torch.equal(o1, outs[1])


def make_fp4_problem(orc, rows, k, seed):
    rng = np.random.default_rng(seed)
    x = bf16_round(rng.standard_normal((1, k)).astype(np.float32))
    ga = nvfp4_divisor(x)
    xp, xs = orc.nvfp4_quantize(x, ga)
    w = (rng.standard_normal((rows, k)) * 0.02).astype(np.float32)
    gw = nvfp4_divisor(w)
    wp, ws = orc.nvfp4_quantize(w, gw)
    return xp, xs, ga, wp, ws, gw


@pytest.mark.parametrize("rows,k", [(8, 64), (24, 704), (15360, 3840), (3840, 15360), (2816, 704), (1408, 2816)])
def test_nvfp4_gemv(lib, dev, orc, rows, k):
    xp, xs, ga, wp, ws, gw = make_fp4_problem(orc, rows, k, rows * 3 + k)
    want = orc.nvfp4_matmul(xp, xs, wp, ws, ga, gw)[0]
    out = torch.full((rows,), float("nan"), device=dev)
    lib.gemb_nvfp4_gemv(to_dev(xp, dev), to_dev(xs, dev), to_dev(wp, dev), to_dev(ws, dev), out, rows, k, ga, gw, None)
    got = to_np(out)
    assert rel_fro(got, want) < 1e-6
    ref = torch.zeros((rows,), device=dev)
    lib.gemb_nvfp4_reference_projection(to_dev(xp, dev), to_dev(xs, dev), to_dev(wp, dev), to_dev(ws, dev), ref, 1, rows, k, ga, gw, None)
    assert rel_fro(to_np(ref), want) < 1e-6


def test_nvfp4_reference_kat(lib, dev):
    # tests/unit/nvfp4_test.cpp:70-102 through the GPU projections: 17.125 exactly.
    packed = torch.tensor([0x10, 0x32, 0x54, 0x76, 0x98, 0xBA, 0xDC, 0xFE], dtype=torch.uint8, device=dev)
    sc = torch.tensor([0x38], dtype=torch.uint8, device=dev)
    out = torch.zeros((1,), device=dev)
    lib.gemb_nvfp4_reference_projection(packed, sc, packed, sc, out, 1, 1, 16, 2.0, 4.0, None)
    assert out.item() == 17.125


def test_nvfp4_gemv_gate_up(lib, dev, orc):
    rows, k = 15360, 3840
    xp, xs, ga, gp, gs, ggw = make_fp4_problem(orc, rows, k, 1)
    _, _, _, up, us, ugw = make_fp4_problem(orc, rows, k, 2)
    gate = orc.nvfp4_matmul(xp, xs, gp, gs, ga, ggw)[0]
    upv = orc.nvfp4_matmul(xp, xs, up, us, ga, ugw)[0]
    want = orc.gated_gelu(gate.astype(np.float32), upv.astype(np.float32))
    og, ou, op = (torch.zeros((rows,), device=dev) for _ in range(3))
    args = [to_dev(a, dev) for a in (xp, xs, gp, gs, up, us)]
    lib.gemb_nvfp4_gemv_gate_up(*args, og, ou, op, rows, k, ga, ggw, ga, ugw, None)
    assert rel_fro(to_np(og), gate) < 1e-6 and rel_fro(to_np(ou), upv) < 1e-6
    # bf16 boundaries: allow rare 1-ulp flips
    got = to_np(op)
    assert (got != want).mean() < 5e-3 and rel_fro(got, want) < 2e-3
    op2 = torch.zeros((rows,), device=dev)
    lib.gemb_nvfp4_gemv_gate_up(*args, None, None, op2, rows, k, ga, ggw, ga, ugw, None)
    assert torch.equal(op, op2)


def test_decode_set_round_trip_property(lib, dev):
    # Linearity at full decode size without the CPU oracle: W(2x) == 2 W(x) exactly, because
    # doubling a bf16 vector doubles the token scale and leaves the E4M3 bytes unchanged.
    torch.manual_seed(1)
    rows, k = 30720, 3840
    w = torch.randint(0, 256, (rows, k), dtype=torch.uint8, device=dev)
    w[(w & 0x7F) == 0x7F] = 0
    ws = torch.full((rows,), 0x3C00, dtype=torch.int16, device=dev)
    x = torch.randn((k,), device=dev, dtype=torch.bfloat16)
    y1, y2 = torch.zeros((rows,), device=dev), torch.zeros((rows,), device=dev)
    lib.gemb_fp8_gemv_bf16in(x.view(torch.int16), w, ws, y1, 0, rows, k, None)
    lib.gemb_fp8_gemv_bf16in((x * 2).view(torch.int16), w, ws, y2, 0, rows, k, None)
    assert torch.equal(y1 * 2, y2)


def test_fused_quantisation_at_rounding_boundaries(lib, dev, orc):
    # The fused GEMV replaces x/scale by x*(1/scale) away from E4M3 rounding boundaries; feed it
    # values whose quotients sit exactly on (and next to) midpoints and in the subnormal range.
    rows, k = 64, 2048
    tab = np.array([orc.e4m3_decode(i) for i in range(127)], np.float32)
    mids = (tab[:-1] + tab[1:]) / 2
    vals = np.concatenate([mids * 3, -mids * 3, tab * 3, np.nextafter(mids * 3, np.float32(1e9)),
                           mids * 3 * (1 + 2.0 ** -8), mids * 3 * (1 - 2.0 ** -8)]).astype(np.float32)
    rng = np.random.default_rng(0)
    x = bf16_round(np.resize(vals, k)).reshape(1, k)
    x[0, 0] = 448.0 * 3  # amax -> scale exactly 3
    xq, xsc = orc.fp8_quantize(x)
    assert xsc[0] == 3.0
    w = (rng.standard_normal((rows, k)) * 0.02).astype(np.float32)
    wq, wsc = orc.fp8_quantize(w)
    wsb = bf16_bits(wsc)
    y_plain, y_fused = torch.zeros((rows,), device=dev), torch.zeros((rows,), device=dev)
    lib.gemb_fp8_gemv(to_dev(xq, dev), to_dev(xsc, dev), to_dev(wq, dev), to_dev(wsb, dev), y_plain, rows, k, None)
    lib.gemb_fp8_gemv_bf16in(to_dev(bf16_bits(x), dev), to_dev(wq, dev), to_dev(wsb, dev), y_fused, 0, rows, k, None)
    assert torch.equal(y_plain, y_fused)
    # a scale that is not a power-of-two multiple: amax 5.0 -> scale 5/448
    x2 = bf16_round(rng.standard_normal((1, k)).astype(np.float32))
    x2[0, 1] = 5.0
    x2 = np.clip(x2, -5, 5)
    xq2, xsc2 = orc.fp8_quantize(x2)
    lib.gemb_fp8_gemv(to_dev(xq2, dev), to_dev(xsc2, dev), to_dev(wq, dev), to_dev(wsb, dev), y_plain, rows, k, None)
    lib.gemb_fp8_gemv_bf16in(to_dev(bf16_bits(x2), dev), to_dev(wq, dev), to_dev(wsb, dev), y_fused, 0, rows, k, None)
    assert torch.equal(y_plain, y_fused)


@pytest.mark.parametrize("tokens,rows,k", [(2, 40, 528), (3, 8192, 3840), (5, 3840, 15360), (8, 1000, 4096), (7, 13, 16),
                                           (4, 3841, 2816), (6, 30720, 3840), (3, 64, 8192), (6, 200, 12288)])
def test_fp8_gemv_small_batch(lib, dev, orc, tokens, rows, k):
    """The verifier-sized batch (src/cuda/fp8/sm120.h:45-55): one pass over the weights for all tokens on
    the warp-level tensor-core path, within the GEMV budget of the binary64 oracle; the SIMT form behind
    the tuning knob stays bit-identical per token to the single-token GEMV."""
    rng = np.random.default_rng(tokens * 1000 + rows)
    x = bf16_round(rng.standard_normal((tokens, k)).astype(np.float32) * np.arange(1, tokens + 1, dtype=np.float32)[:, None])
    w = (rng.standard_normal((rows, k)) * 0.02).astype(np.float32)
    wq, wsc = orc.fp8_quantize(w)
    wsb = bf16_bits(wsc)
    xq, xsc = orc.fp8_quantize(x)
    want = orc.fp8_matmul(xq, xsc, wq, wsb)
    out = torch.full((tokens, rows), float("nan"), device=dev)
    xd, sd, wd, wsd = to_dev(xq, dev), to_dev(xsc, dev), to_dev(wq, dev), to_dev(wsb, dev)
    lib.gemb_fp8_gemv_batch(xd, sd, wd, wsd, out, tokens, rows, k, None)
    got = to_np(out)
    assert rel_fro(got, want) < 1e-6, rel_fro(got, want)
    assert np.abs(got - want).max() <= 1e-5 * max(1.0, np.abs(want).max())
    lib.gemb_set_tuning(4, 1)           # GEMB_TUNE_GEMV_IMPL: the SIMT form
    try:
        simt = torch.full((tokens, rows), float("nan"), device=dev)
        lib.gemb_fp8_gemv_batch(xd, sd, wd, wsd, simt, tokens, rows, k, None)
        for t in range(tokens):
            one = torch.zeros((rows,), device=dev)
            lib.gemb_fp8_gemv(xd[t], sd[t:t + 1], wd, wsd, one, rows, k, None)
            assert np.array_equal(to_np(one), to_np(simt[t])), t
    finally:
        lib.gemb_set_tuning(4, 0)
    assert rel_fro(to_np(simt), want) < 1e-6


def test_fp8_gemv_small_batch_is_exact_on_representable_sums(lib, dev):
    """The reference holds its tensor-core batch kernel to equality with its scalar one on values whose
    partial sums are all representable (tests/cuda/nvfp4_reference_test.cu:1131-1140; seven E4M3 codes of
    magnitude 0.5 .. 2 and power-of-two scales).  The same here: both forms and the single-token kernel
    return the same bits."""
    codes = np.array([0x00, 0x30, 0x38, 0x40, 0xB0, 0xB8, 0xC0], np.uint8)
    tokens, rows, k = 8, 1030, 4096
    idx = np.arange(tokens * k, dtype=np.int64)
    x = codes[(idx * 5 + idx // k) % 7].reshape(tokens, k)
    idx = np.arange(rows * k, dtype=np.int64)
    w = codes[(idx * 3 + idx // k) % 7].reshape(rows, k)
    xs = np.array([0.125, 0.25, 0.5, 1.0], np.float32)[np.arange(tokens) % 4]
    ws = np.array([0x3E00, 0x3E80, 0x3F00, 0x3F80], np.uint16)[np.arange(rows) % 4]
    xd, sd, wd, wsd = (to_dev(a, dev) for a in (x, xs, w, ws))
    mma = torch.zeros((tokens, rows), device=dev)
    lib.gemb_fp8_gemv_batch(xd, sd, wd, wsd, mma, tokens, rows, k, None)
    for t in range(tokens):
        one = torch.zeros((rows,), device=dev)
        lib.gemb_fp8_gemv(xd[t], sd[t:t + 1], wd, wsd, one, rows, k, None)
        assert torch.equal(one, mma[t]), t
    assert float(mma.abs().max()) > 0


def test_fp8_gemv_small_batch_grouped_and_limits(lib, dev, orc):
    from gem16_b200.lib import GembError
    tokens, k = 3, 3840
    rng = np.random.default_rng(5)
    x = bf16_round(rng.standard_normal((tokens, k)).astype(np.float32))
    xq, xsc = orc.fp8_quantize(x)
    mats = [make_fp8_problem(orc, r, k, 200 + r)[3:] for r in (4096, 2048, 2048)]
    outs = [torch.full((tokens, r), float("nan"), device=dev) for r in (4096, 2048, 2048)]
    d = [(to_dev(w, dev), to_dev(s, dev)) for w, s in mats]
    xd, sd = to_dev(xq, dev), to_dev(xsc, dev)
    lib.gemb_fp8_gemv_qkv_batch(xd, sd, d[0][0], d[0][1], outs[0], 4096, d[1][0], d[1][1], outs[1], 2048, d[2][0], d[2][1],
                                outs[2], 2048, tokens, k, None)
    for (w, s), o in zip(mats, outs):
        assert rel_fro(to_np(o), orc.fp8_matmul(xq, xsc, w, s)) < 1e-6
    o0, o1 = torch.zeros((tokens, 4096), device=dev), torch.zeros((tokens, 2048), device=dev)
    lib.gemb_fp8_gemv_qkv_batch(xd, sd, d[0][0], d[0][1], o0, 4096, d[1][0], d[1][1], o1, 2048, None, None, None, 0,
                                tokens, k, None)
    assert torch.equal(o0, outs[0]) and torch.equal(o1, outs[1])
    with pytest.raises(GembError):
        lib.gemb_fp8_gemv_batch(xd, sd, d[0][0], d[0][1], o0, 9, 4096, k, None)          # more than 8 tokens
    with pytest.raises(GembError):
        lib.gemb_fp8_gemv_batch(xd, sd, d[0][0], d[0][1], o0, 8, 4096, 15360, None)      # 8 x 15360 does not fit


@pytest.mark.parametrize("tokens,rows,k", [(2, 8, 64), (3, 3840, 15360), (5, 15360, 3840), (8, 1000, 4096)])
def test_nvfp4_gemv_small_batch(lib, dev, orc, tokens, rows, k):
    """src/cuda/nvfp4/sm120.h:26-37 at verifier batch sizes: one pass over the weights, every token
    bit-identical to the single-token GEMV and within its budget of the binary64 oracle."""
    rng = np.random.default_rng(tokens * 7 + rows)
    x = bf16_round(rng.standard_normal((tokens, k)).astype(np.float32))
    ga = nvfp4_divisor(x)
    xp, xs = orc.nvfp4_quantize(x, ga)
    w = (rng.standard_normal((rows, k)) * 0.02).astype(np.float32)
    gw = nvfp4_divisor(w)
    wp, ws = orc.nvfp4_quantize(w, gw)
    want = orc.nvfp4_matmul(xp, xs, wp, ws, ga, gw)
    d = [to_dev(a, dev) for a in (xp, xs, wp, ws)]
    out = torch.full((tokens, rows), float("nan"), device=dev)
    lib.gemb_nvfp4_gemv_batch(d[0], d[1], d[2], d[3], out, tokens, rows, k, ga, gw, None)
    got = to_np(out)
    assert rel_fro(got, want) < 1e-6
    for t in range(tokens):
        one = torch.zeros((rows,), device=dev)
        lib.gemb_nvfp4_gemv(d[0][t], d[1][t], d[2], d[3], one, rows, k, ga, gw, None)
        assert np.array_equal(to_np(one), got[t]), t
    from gem16_b200.lib import GembError
    with pytest.raises(GembError):
        lib.gemb_nvfp4_gemv_batch(d[0], d[1], d[2], d[3], out, 9, rows, k, ga, gw, None)
