"""GPU parity of the operators beside the projections: the Up projection with a materialised gate,
the batch gate/up GEMV, RMSNorm + residual, the fp32 GELU product and residual add, the arg-max over
materialised logits and the bf16-weight GEMV."""
import numpy as np
import pytest
import torch

from tests.util import bf16_bits, bf16_round, from_bf16_bits, to_dev, to_np

pytestmark = pytest.mark.gpu


def interleaved(lib, dev, compact, rows, k):
    out = torch.zeros((lib.cdll.gemb_interleaved_scale_bytes(rows, k),), dtype=torch.uint8, device=dev)
    lib.gemb_nvfp4_interleave_scales(to_dev(compact, dev), out, rows, k, None)
    return out


@pytest.mark.parametrize("tokens,rows,k", [(300, 1408, 512), (64, 128, 2816), (1000, 704, 256)])
def test_up_projection_with_materialised_gate_is_byte_identical(lib, dev, orc, tokens, rows, k):
    """gemb_nvfp4_gemm_up_gated_quant against up GEMM + gemb_nvfp4_gated_gelu_quantize: same payload and
    same scale bytes on every real row."""
    rng = np.random.default_rng(tokens)
    x = bf16_round(rng.standard_normal((tokens, k)).astype(np.float32))
    ga = float(np.float32(2688.0) / np.abs(x).max())
    xp, xs = orc.nvfp4_quantize(x, ga)
    w = (rng.standard_normal((rows, k)) * 0.05).astype(np.float32)
    gw = float(np.float32(2688.0) / np.abs(w).max())
    wp, ws = orc.nvfp4_quantize(w, gw)
    gate = to_dev(bf16_bits(rng.standard_normal((tokens, rows)).astype(np.float32) * 1.5), dev)
    d_xp, d_xs = to_dev(xp, dev), interleaved(lib, dev, xs, tokens, k)
    d_wp, d_ws = to_dev(wp, dev), interleaved(lib, dev, ws, rows, k)
    g_dn = 2688.0 / 6.0
    up = torch.zeros((tokens, rows), dtype=torch.int16, device=dev)
    lib.gemb_nvfp4_gemm_bf16(d_xp, d_xs, d_wp, d_ws, up, tokens, rows, k, ga, gw, None)
    nb = lib.cdll.gemb_interleaved_scale_bytes(tokens, rows)
    want_p = torch.zeros((tokens, rows // 2), dtype=torch.uint8, device=dev)
    want_s = torch.zeros((nb,), dtype=torch.uint8, device=dev)
    lib.gemb_nvfp4_gated_gelu_quantize(gate, up, 1, want_p, want_s, tokens, rows, g_dn, 1, 0, None)
    got_p = torch.zeros_like(want_p)
    got_s = torch.zeros_like(want_s)
    lib.gemb_nvfp4_gemm_up_gated_quant(d_xp, d_xs, d_wp, d_ws, gate, got_p, got_s, tokens, rows, k, ga, gw, g_dn, None)
    torch.cuda.synchronize()
    lib.gemb_check_device_status()
    assert torch.equal(got_p, want_p)
    r = torch.arange(tokens, device=dev)[:, None]
    c = torch.arange(rows // 16, device=dev)[None, :]
    c_pad = (rows // 16 + 3) // 4 * 4
    off = ((r // 128) * (c_pad // 4) + c // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + c % 4
    assert torch.equal(got_s[off], want_s[off])


def test_batch_gate_up_gemv_equals_the_single_token_operator(lib, dev, orc):
    rng = np.random.default_rng(4)
    tokens, rows, k = 5, 256, 1024
    x = bf16_round(rng.standard_normal((tokens, k)).astype(np.float32))
    xp, xs = orc.nvfp4_quantize(x, 500.0)
    wg, sg = orc.nvfp4_quantize((rng.standard_normal((rows, k)) * 0.03).astype(np.float32), 9000.0)
    wu, su = orc.nvfp4_quantize((rng.standard_normal((rows, k)) * 0.03).astype(np.float32), 8000.0)
    d = [to_dev(a, dev) for a in (xp, xs, wg, sg, wu, su)]
    outs = [torch.zeros((tokens, rows), device=dev) for _ in range(3)]
    lib.gemb_nvfp4_gemv_gate_up_batch(*d, outs[0], outs[1], outs[2], tokens, rows, k, 500.0, 9000.0, 500.0, 8000.0, None)
    for t in range(tokens):
        one = [torch.zeros((rows,), device=dev) for _ in range(3)]
        lib.gemb_nvfp4_gemv_gate_up(d[0][t], d[1][t], d[2], d[3], d[4], d[5], one[0], one[1], one[2], rows, k, 500.0, 9000.0,
                                    500.0, 8000.0, None)
        for a, b in zip(outs, one):
            assert torch.equal(a[t], b)
    want_gate = orc.nvfp4_matmul(xp, xs, wg, sg, 500.0, 9000.0)
    assert np.linalg.norm(to_np(outs[0]) - want_gate) <= 1e-6 * np.linalg.norm(want_gate)


def rmsnorm_residual_ref(x, w, res, eps, scalar):
    """numpy restatement of src/cuda/norm/reference.cu:66-110 (binary64 sum instead of the fp32 tree)."""
    inv = 1.0 / np.sqrt((x.astype(np.float64) ** 2).mean(axis=1, keepdims=True) + eps)
    n = bf16_round((x * inv.astype(np.float32) * (1.0 if w is None else w)).astype(np.float32))
    v = bf16_round(n + res)
    if scalar is not None:
        v = bf16_round(v * scalar)
    return n, v


@pytest.mark.parametrize("physical", [False, True])
def test_rmsnorm_residual(lib, dev, physical):
    rng = np.random.default_rng(8)
    vectors, width = 37, 3840
    x = bf16_round(rng.standard_normal((vectors, width)).astype(np.float32) * 2)
    w = bf16_round((1 + 0.1 * rng.standard_normal(width)).astype(np.float32))
    res = bf16_round(rng.standard_normal((vectors, width)).astype(np.float32))
    scalar = bf16_round(np.array([0.75], np.float32))
    for use_w, use_s in ((True, True), (False, False)):
        n_ref, v_ref = rmsnorm_residual_ref(x, w if use_w else None, res, 1e-6, scalar[0] if use_s else None)
        d_w = to_dev(bf16_bits(w), dev) if use_w else None
        d_s = to_dev(bf16_bits(scalar), dev) if use_s else None
        if physical:
            out = torch.zeros((vectors, width), dtype=torch.int16, device=dev)
            lib.gemb_rmsnorm_residual(to_dev(bf16_bits(x), dev), 1, d_w, to_dev(bf16_bits(res), dev), None, out, 1, vectors, width,
                                      1e-6, d_s, None)
            got = from_bf16_bits(to_np(out, np.uint16))
        else:
            norm = torch.zeros((vectors, width), device=dev)
            out = torch.zeros((vectors, width), device=dev)
            lib.gemb_rmsnorm_residual(to_dev(x, dev), 0, d_w, to_dev(res, dev), norm, out, 0, vectors, width, 1e-6, d_s, None)
            got = to_np(out)
            nb = bf16_bits(to_np(norm)).astype(np.int64) - bf16_bits(n_ref).astype(np.int64)
            assert np.abs(nb).max() <= 1 and (nb != 0).mean() < 5e-3
        # the device's rsqrtf and fp32 tree against binary64: a result may sit one bf16 step away
        diff = bf16_bits(got).astype(np.int64) - bf16_bits(v_ref).astype(np.int64)
        assert np.abs(diff).max() <= 1 and (diff != 0).mean() < 5e-3, (diff != 0).mean()


def test_elementwise_bridges_and_logit_argmax(lib, dev, orc):
    rng = np.random.default_rng(15)
    n = 100_003
    gate = (rng.standard_normal(n) * 2).astype(np.float32)
    up = rng.standard_normal(n).astype(np.float32)
    out = torch.zeros((n,), device=dev)
    lib.gemb_gelu_tanh_product_f32(to_dev(gate, dev), to_dev(up, dev), out, n, None)
    inner = np.float32(0.7978845608028654) * (gate + np.float32(0.044715) * gate * gate * gate)
    th = np.tanh(inner.astype(np.float64)).astype(np.float32)          # a correctly rounded fp32 tanh
    gelu = bf16_round((np.float32(0.5) * gate * (np.float32(1) + th)).astype(np.float32))
    want = gelu * up
    got = to_np(out)
    # "1 + tanh" cancels for negative gates: below about -3 the formula itself (with a perfect fp32 tanh) is
    # several per cent away from the exact value, and every implementation -- the reference's tanhf, numpy's,
    # this library's -- lands on its own neighbour there.  Those values are of the order 1e-5; they are held to
    # an absolute bound, everything else to one bf16 step on a small fraction of the elements.
    main = gate >= -3.0
    rel = np.abs(got - want)[main] / np.maximum(np.abs(want[main]), 1e-30)
    assert (got != want)[main].mean() < 2e-3 and rel.max() <= 2.0 ** -7
    assert np.all(np.abs(got - want)[~main] <= 4e-5 * np.abs(up[~main]))      # one bf16 step of a GELU value below 5e-3
    lib.gemb_add_residual_f32(to_dev(gate, dev), to_dev(up, dev), out, n, None)
    assert np.array_equal(to_np(out), gate + up)
    logits = rng.standard_normal(262144).astype(np.float32)
    logits[[7, 1000, 200000]] = 9.5       # a three-way tie above everything else
    sel = torch.zeros((1,), dtype=torch.int32, device=dev)
    lib.gemb_logit_argmax(to_dev(logits, dev), None, 0, sel, logits.size, None)
    assert int(sel.item()) == 7
    sup = torch.tensor([7, 3], dtype=torch.int32, device=dev)
    lib.gemb_logit_argmax(to_dev(logits, dev), sup, 2, sel, logits.size, None)
    assert int(sel.item()) == 1000


def test_bf16_gemv(lib, dev):
    rng = np.random.default_rng(16)
    for rows, k in ((1000, 1024), (4096, 2048), (7, 264)):
        x = rng.standard_normal(k).astype(np.float32)
        w = bf16_round((rng.standard_normal((rows, k)) * 0.05).astype(np.float32))
        y = torch.zeros((rows,), device=dev)
        lib.gemb_bf16_gemv(to_dev(x, dev), to_dev(bf16_bits(w), dev), y, rows, k, None)
        want = bf16_round((w.astype(np.float64) @ x.astype(np.float64)).astype(np.float32))
        diff = bf16_bits(to_np(y)).astype(np.int64) - bf16_bits(want).astype(np.int64)
        assert np.abs(diff).max() <= 1 and (diff != 0).mean() < 1e-2


def test_output_head_logits_without_candidates(lib, dev, orc):
    rng = np.random.default_rng(17)
    vocab, hidden = 5000, 256
    w = bf16_bits((rng.standard_normal((vocab, hidden)) * 0.2).astype(np.float32))
    h = rng.standard_normal((1, hidden)).astype(np.float32)
    logits = torch.zeros((1, vocab), device=dev)
    lib.gemb_output_head_candidates(to_dev(w, dev), to_dev(h, dev), 1, None, 0, None, None, logits, vocab, hidden, None)
    want, sel = orc.output_head(w, h)
    assert np.abs(to_np(logits) - want).max() < 1e-4
    out = torch.zeros((1,), dtype=torch.int32, device=dev)
    lib.gemb_logit_argmax(logits, None, 0, out, vocab, None)
    assert int(out.item()) == int(np.argmax(to_np(logits)[0]))
