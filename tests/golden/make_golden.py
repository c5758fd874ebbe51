"""Generates tests/golden/linear_path.npz from the gem16 reference itself.

Run where a checkout of gem16 is present ($GEM16_REFERENCE, or a `reference` directory beside this
repository):

    python tests/golden/make_golden.py

Inputs are seeded numpy arrays; outputs come from the UNMODIFIED reference functions
gem16::nvfp4::QuantizeActivation / ReferenceDotProduct and gem16::fp8::QuantizeToken /
ReferenceDotProduct and gem16::layer::RmsNorm (src/numeric/nvfp4.cpp, src/numeric/fp8.cpp,
src/numeric/layer.cpp) compiled by oracle/build.py.
The GPU box has no reference tree; it only reads the committed .npz.
"""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))
from oracle import Oracle  # noqa: E402


def bf16_round(x):
    u = x.astype(np.float32).view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32)


def main():
    ref = Oracle(ref=True)
    rng = np.random.default_rng(20261125)
    out = {}

    # NVFP4 activations: N(0,1) rows rounded to bf16, plus edge rows.
    k = 512
    x = bf16_round(rng.standard_normal((12, k)).astype(np.float32))
    x[1] = 0.0                                   # all-zero token -> zero scales and nibbles
    x[2, :16] = 0.0                              # one zero block
    x[3] *= 1e-4                                 # scale underflow region
    x[4, ::7] *= 40.0                            # outliers -> saturation of neighbours
    x[5, :32] = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0] * 4, np.float32)  # E2M1 ties
    x[5, 32:64] = -x[5, :32]
    x[6] = bf16_round(rng.standard_normal(k).astype(np.float32) * 30.0)
    ga = np.float32(6.0 * 448.0 / np.abs(x).max())
    packed, scales = ref.nvfp4_quantize(x, float(ga), threads=1)
    out.update(nvfp4_x=x, nvfp4_ga=ga, nvfp4_packed=packed, nvfp4_scales=scales)
    # Same inputs with a divisor that does not come from amax (exercises scale saturation).
    p2, s2 = ref.nvfp4_quantize(x, 300.0, threads=1)
    out.update(nvfp4_packed_g300=p2, nvfp4_scales_g300=s2)

    # NVFP4 weights: N(0, 0.02) quantised row-wise with the same reference function.
    w = (rng.standard_normal((24, k)) * 0.02).astype(np.float32)
    gw = np.float32(6.0 * 448.0 / np.abs(w).max())
    wp, ws = ref.nvfp4_quantize(w, float(gw), threads=1)
    y = ref.nvfp4_matmul(packed, scales, wp, ws, float(ga), float(gw), threads=1)
    out.update(nvfp4_w=w, nvfp4_gw=gw, nvfp4_wp=wp, nvfp4_ws=ws, nvfp4_y=y)

    # FP8 path.
    xf = bf16_round(rng.standard_normal((10, 384)).astype(np.float32))
    xf[1] = 0.0
    xf[2] *= 1e-3
    xf[3, 5] = 300.0
    q, sc = ref.fp8_quantize(xf, threads=1)
    wf = (rng.standard_normal((20, 384)) * 0.02).astype(np.float32)
    wq, wsc = ref.fp8_quantize(wf, threads=1)
    wsc_bf16 = (bf16_round(wsc).view(np.uint32) >> 16).astype(np.uint16)
    yf = ref.fp8_matmul(q, sc, wq, wsc_bf16, threads=1)
    out.update(fp8_x=xf, fp8_q=q, fp8_scales=sc, fp8_w=wf, fp8_wq=wq, fp8_wscales_bf16=wsc_bf16, fp8_y=yf)

    # Codec tables.
    out["e2m1_table"] = np.array([ref.e2m1_decode(i) for i in range(16)], np.float32)
    out["e4m3_table"] = np.array([ref.e4m3_decode(i) for i in range(256)], np.float32)
    probes = np.concatenate([
        rng.standard_normal(2000).astype(np.float32) * s for s in (1e-3, 0.05, 1.0, 8.0, 200.0)])
    tab = out["e4m3_table"][:127]
    mids = ((tab[:-1].astype(np.float64) + tab[1:]) / 2).astype(np.float32)
    probes = np.concatenate([probes, tab, mids, np.nextafter(mids, np.float32(1e9)),
                             np.nextafter(mids, np.float32(-1e9)), -mids,
                             np.array([0.0, -0.0, 448, 449, 464, 480, 1000, 5, 2.5, 0.25, 0.75, 1.75, 3.5, 7, -7],
                                      np.float32)]).astype(np.float32)
    out["codec_probes"] = probes
    out["codec_e4m3"] = np.array([ref.e4m3_encode(float(v)) for v in probes], np.uint8)
    out["codec_e2m1"] = np.array([ref.e2m1_encode(float(v)) for v in probes], np.uint8)

    # RMSNorm (gem16::layer::RmsNorm: binary64 sums, fp32 result) with and without a learned weight;
    # the weight is bf16-representable because the device kernels take it as bf16.
    xn = bf16_round(rng.standard_normal((9, 704)).astype(np.float32) * 3.0)
    xn[1] *= 1e-3
    xn[2] *= 200.0
    xn[3, 1:] = 0.0
    wn = bf16_round((1.0 + 0.2 * rng.standard_normal(704)).astype(np.float32))
    out.update(rms_x=xn, rms_w=wn, rms_eps=np.float32(1e-6), rms_y=ref.ref_rmsnorm(xn, wn, 1e-6),
               rms_y_noweight=ref.ref_rmsnorm(xn, None, 1e-6))

    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "linear_path.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
