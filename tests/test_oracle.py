"""CPU tests of the oracle itself: the reference's known-answer tests, the committed golden
vectors (generated from the compiled reference by tests/golden/make_golden.py) and, when the
compiled reference is present, a direct comparison on fresh seeded inputs."""
import numpy as np
import pytest

from tests.util import bf16_bits, bf16_round, from_bf16_bits


def test_e2m1_codec_kat(orc):
    # tests/unit/nvfp4_test.cpp:15-41
    mags = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]
    for i in range(16):
        v = orc.e2m1_decode(i)
        assert v == (-mags[i & 7] if i & 8 else mags[i & 7])
        if i != 8:
            assert orc.e2m1_encode(v) == i
    for value, want in [(0.25, 0.0), (0.75, 1.0), (1.75, 2.0), (3.5, 4.0), (100.0, 6.0), (2.5, 2.0), (5.0, 4.0)]:
        assert orc.e2m1_decode(orc.e2m1_encode(value)) == want
    assert orc.e2m1_encode(-0.0) == 8


def test_e4m3_codec_kat(orc):
    # tests/unit/nvfp4_test.cpp:43-68
    assert orc.e4m3_decode(0x38) == 1.0
    assert orc.e4m3_decode(0x7E) == 448.0
    assert orc.e4m3_decode(0x01) == 2.0 ** -9
    assert orc.e4m3_decode(0x61) == 36.0
    assert np.isnan(orc.e4m3_decode(0x7F)) and np.isnan(orc.e4m3_decode(0xFF))
    for b in range(256):
        if b & 0x7F == 0x7F:
            continue
        assert orc.e4m3_encode(orc.e4m3_decode(b)) == b or b == 0x80
    assert orc.e4m3_encode(1000.0) == 0x7E


def test_nvfp4_quantize_kat(orc):
    # tests/unit/nvfp4_test.cpp:70-102
    act = np.array([orc.e2m1_decode(i) / 2.0 for i in range(16)], np.float32)[None]
    packed, scales = orc.nvfp4_quantize(act, 2.0)
    assert packed.tobytes() == bytes([0x10, 0x32, 0x54, 0x76, 0x98, 0xBA, 0xDC, 0xFE])
    assert scales.tobytes() == b"\x38"
    y = orc.nvfp4_matmul(packed, scales, packed, np.array([[0x38]], np.uint8), 2.0, 4.0)
    assert y[0, 0] == 17.125
    packed, scales = orc.nvfp4_quantize(np.zeros((1, 16), np.float32), 11.0)
    assert not packed.any() and not scales.any()


def test_nvfp4_checkpoint_bytes_kat(orc):
    # tests/unit/nvfp4_test.cpp:104-134: pinned checkpoint bytes, scale 0x61 = 36, divisor 9600.
    w = np.array([[0x37, 0xC1, 0x53, 0xA0, 0xFB, 0x5D, 0xAD, 0xFE]], np.uint8)
    nibbles = [7, 3, 1, 12, 3, 5, 0, 10, 11, 15, 13, 5, 13, 10, 14, 15]
    for sel in range(16):
        a = np.zeros((1, 8), np.uint8)
        a[0, sel // 2] = 2 << (4 if sel % 2 else 0)
        y = orc.nvfp4_matmul(a, np.array([[0x38]], np.uint8), w, np.array([[0x61]], np.uint8), 1.0, 9600.0)
        assert abs(y[0, 0] - orc.e2m1_decode(nibbles[sel]) * 36.0 / 9600.0) < 1e-12


def test_nvfp4_invalid_inputs(orc):
    # tests/unit/nvfp4_test.cpp:136-153
    with pytest.raises(ValueError):
        orc.nvfp4_quantize(np.zeros((1, 15), np.float32), 1.0)
    with pytest.raises(ValueError):
        orc.nvfp4_quantize(np.zeros((1, 16), np.float32), 0.0)
    x = np.zeros((1, 16), np.float32)
    x[0, 3] = np.nan
    with pytest.raises(ValueError):
        orc.nvfp4_quantize(x, 1.0)
    with pytest.raises(ValueError):
        orc.nvfp4_matmul(np.zeros((1, 8), np.uint8), np.array([[0x7F]], np.uint8), np.zeros((1, 8), np.uint8),
                         np.array([[0x38]], np.uint8), 1.0, 1.0)


def test_fp8_kat(orc):
    # tests/unit/fp8_test.cpp:13-67
    assert from_bf16_bits(np.array([0x3F80, 0xC020], np.uint16)).tolist() == [1.0, -2.5]
    act = np.array([[-4.0, -2.0, -1.0, -0.5, 0.0, 0.5, 2.0, 4.0]], np.float32)
    q, s = orc.fp8_quantize(act)
    assert s[0] == np.float32(4.0) / np.float32(448.0)
    assert q[0, 0] == 0xFE and q[0, -1] == 0x7E
    q0, s0 = orc.fp8_quantize(np.zeros((1, 4), np.float32))
    assert s0[0] == 1.0 and not q0.any()
    act = np.array([[1.0, -2.0, 3.0, -4.0]], np.float32)
    q, s = orc.fp8_quantize(act)
    w = np.array([[0x38, 0xB8, 0x40, 0xC0]], np.uint8)
    y = orc.fp8_matmul(q, s, w, np.array([0x3F00], np.uint16))
    want = sum(float(orc.e4m3_decode(int(a))) * float(orc.e4m3_decode(int(b))) for a, b in zip(q[0], w[0]))
    assert y[0, 0] == want * float(s[0]) * 0.5


def test_golden_codecs(orc, golden):
    assert [orc.e2m1_decode(i) for i in range(16)] == golden["e2m1_table"].tolist()
    tab = golden["e4m3_table"]
    for i in range(256):
        v = orc.e4m3_decode(i)
        assert (np.isnan(v) and np.isnan(tab[i])) or v == tab[i]
    probes = golden["codec_probes"]
    assert [orc.e4m3_encode(float(v)) for v in probes] == golden["codec_e4m3"].tolist()
    assert [orc.e2m1_encode(float(v)) for v in probes] == golden["codec_e2m1"].tolist()


def test_golden_nvfp4(orc, golden):
    p, s = orc.nvfp4_quantize(golden["nvfp4_x"], float(golden["nvfp4_ga"]))
    assert np.array_equal(p, golden["nvfp4_packed"]) and np.array_equal(s, golden["nvfp4_scales"])
    p2, s2 = orc.nvfp4_quantize(golden["nvfp4_x"], 300.0)
    assert np.array_equal(p2, golden["nvfp4_packed_g300"]) and np.array_equal(s2, golden["nvfp4_scales_g300"])
    wp, ws = orc.nvfp4_quantize(golden["nvfp4_w"], float(golden["nvfp4_gw"]))
    assert np.array_equal(wp, golden["nvfp4_wp"]) and np.array_equal(ws, golden["nvfp4_ws"])
    y = orc.nvfp4_matmul(p, s, wp, ws, float(golden["nvfp4_ga"]), float(golden["nvfp4_gw"]))
    assert np.array_equal(y, golden["nvfp4_y"])


def test_golden_fp8(orc, golden):
    q, s = orc.fp8_quantize(golden["fp8_x"])
    assert np.array_equal(q, golden["fp8_q"]) and np.array_equal(s, golden["fp8_scales"])
    y = orc.fp8_matmul(q, s, golden["fp8_wq"], golden["fp8_wscales_bf16"])
    assert np.array_equal(y, golden["fp8_y"])


def test_against_compiled_reference(orc):
    from oracle import Oracle, ref_available
    if not ref_available():
        pytest.skip("compiled reference (oracle/_ref) not present")
    ref = Oracle(ref=True)
    rng = np.random.default_rng(7)
    x = bf16_round(rng.standard_normal((16, 704)).astype(np.float32))
    g = float(np.float32(2688.0) / np.abs(x).max())
    a, b = orc.nvfp4_quantize(x, g), ref.nvfp4_quantize(x, g)
    assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])
    w = (rng.standard_normal((32, 704)) * 0.02).astype(np.float32)
    gw = float(np.float32(2688.0) / np.abs(w).max())
    wp, ws = orc.nvfp4_quantize(w, gw)
    assert np.array_equal(orc.nvfp4_matmul(a[0], a[1], wp, ws, g, gw), ref.nvfp4_matmul(a[0], a[1], wp, ws, g, gw))
    q1, q2 = orc.fp8_quantize(x), ref.fp8_quantize(x)
    assert np.array_equal(q1[0], q2[0]) and np.array_equal(q1[1], q2[1])
    wq, wsc = orc.fp8_quantize(w)
    assert np.array_equal(orc.fp8_matmul(q1[0], q1[1], wq, bf16_bits(wsc)), ref.fp8_matmul(q1[0], q1[1], wq, bf16_bits(wsc)))


def test_rmsnorm_restatement_against_reference_vectors(orc, golden):
    """orc.rmsnorm_bf16 restates the DEVICE contract (fp32 partial sums folded by a tree, fp32 1/sqrt,
    bf16 result: src/cuda/nvfp4/reference.cu:92-135); the vectors are gem16::layer::RmsNorm
    (src/numeric/layer.cpp:27-63: binary64 sums, fp32 result).  After the same bf16 rounding the two may
    differ only where the fp32 arithmetic moved a value across a rounding boundary: at most one bf16
    step, on well under 2 % of the elements."""
    x, w, eps = golden["rms_x"], golden["rms_w"], float(golden["rms_eps"])
    for weight, want in ((bf16_bits(w), golden["rms_y"]), (None, golden["rms_y_noweight"])):
        got = bf16_bits(orc.rmsnorm_bf16(x, weight, eps)).astype(np.int64)
        ref_bits = bf16_bits(want).astype(np.int64)
        assert np.abs(got - ref_bits).max() <= 1
        assert (got != ref_bits).mean() < 0.02, (got != ref_bits).mean()
    from oracle import Oracle, ref_available
    if ref_available():       # and the compiled reference still gives the committed vectors
        ref = Oracle(ref=True)
        assert np.array_equal(ref.ref_rmsnorm(x, w, eps), golden["rms_y"])
        assert np.array_equal(ref.ref_rmsnorm(x, None, eps), golden["rms_y_noweight"])


def test_interleave_layout(orc):
    # src/cuda/nvfp4/cutlass_sm120.cu:160-194
    rows, k = 130, 16 * 6
    compact = np.arange(rows * 6, dtype=np.uint32).astype(np.uint8).reshape(rows, 6) | 1
    out = orc.interleave_scales(compact, k)
    assert out.size == 256 * 8
    for r, c in [(0, 0), (1, 0), (31, 3), (32, 0), (127, 5), (128, 1), (129, 4)]:
        off = ((r // 128) * 2 + c // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + c % 4
        assert out[off] == compact[r, c]
    assert np.count_nonzero(out) == rows * 6


def test_bf16_helpers(orc):
    rng = np.random.default_rng(3)
    x = rng.standard_normal(4096).astype(np.float32)
    assert np.array_equal(orc.to_bf16(x), bf16_bits(x))
    assert np.array_equal(orc.from_bf16(bf16_bits(x)), bf16_round(x))


def test_division_by_reciprocal_and_residual_is_correctly_rounded():
    """The device quantisers compute (x * g) / scale as q0 = RN(t * r), q = RN(q0 + (t - scale * q0) * r)
    with r = RN(1 / scale) -- one division per 16-block instead of sixteen.  Exact rational arithmetic
    shows that for every value an E4M3 scale can take this equals the correctly rounded quotient, in
    particular on and next to every E2M1 rounding boundary, so the bytes stay those of
    src/numeric/nvfp4.cpp:145-150."""
    from fractions import Fraction
    import random

    def rn32(fr):
        if fr == 0:
            return Fraction(0)
        a = abs(fr)
        e = a.numerator.bit_length() - a.denominator.bit_length()
        if Fraction(2) ** e > a:
            e -= 1
        if Fraction(2) ** (e + 1) <= a:
            e += 1
        ulp = Fraction(2) ** (e - 23)
        q = a / ulp
        n = q.numerator // q.denominator
        rem = q - n
        if rem > Fraction(1, 2) or (rem == Fraction(1, 2) and n % 2 == 1):
            n += 1
        return (n if fr > 0 else -n) * ulp

    def step(x, k):
        a = np.float32(float(x))
        for _ in range(abs(k)):
            a = np.nextafter(a, np.float32(np.inf if k > 0 else -np.inf))
        return Fraction(float(a))

    random.seed(1)
    mids = [Fraction(1, 4), Fraction(3, 4), Fraction(5, 4), Fraction(7, 4), Fraction(5, 2), Fraction(7, 2), Fraction(5)]
    checked = 0
    for bits in range(1, 127):
        ex, m = (bits >> 3) & 15, bits & 7
        ds = Fraction(m, 8) * Fraction(2) ** -6 if ex == 0 else (1 + Fraction(m, 8)) * Fraction(2) ** (ex - 7)
        r = rn32(1 / ds)
        cands = [step(rn32(mid * ds), k) for mid in mids for k in range(-2, 3)]
        cands += [Fraction(float(np.float32(random.uniform(0, 7) * float(ds)))) for _ in range(10)]
        for t in cands:
            if t <= 0:
                continue
            q0 = rn32(t * r)
            q = rn32(q0 + rn32(t - ds * q0) * r)
            assert q == rn32(t / ds), (bits, float(t))
            checked += 1
    assert checked > 5000
