// Scalar cross-check projections: one thread per (token, row), fp32 fma over k in ascending
// order, the arithmetic of ProjectionReferenceKernel in src/cuda/nvfp4/reference.cu:220-256 and
// src/cuda/fp8/reference.cu:138-164.  Deliberately simple and slow; used to check the fast
// kernels on shapes too large for the CPU oracle.
#include "common.cuh"

namespace gemb {
namespace {

__global__ void __launch_bounds__(128)
nvfp4_reference_projection_kernel(const uint8_t* __restrict__ a, const uint8_t* __restrict__ as,
                                  const uint8_t* __restrict__ w, const uint8_t* __restrict__ ws,
                                  float* __restrict__ out, uint64_t tokens, uint64_t rows,
                                  uint64_t k, float divisor) {
  const uint64_t token = blockIdx.y;
  const uint64_t row = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (token >= tokens || row >= rows) return;
  const uint8_t* ap = a + token * (k / 2);
  const uint8_t* asp = as + token * (k / 16);
  const uint8_t* wp = w + row * (k / 2);
  const uint8_t* wsp = ws + row * (k / 16);
  float acc = 0.0f;
  for (uint64_t b = 0; b < k / 16; ++b) {
    const float sa = e4m3_decode(asp[b]), sw = e4m3_decode(wsp[b]);
    for (int i = 0; i < 8; ++i) {
      const float2 av = __half22float2(e2m1x2_decode(ap[b * 8 + i]));
      const float2 wv = __half22float2(e2m1x2_decode(wp[b * 8 + i]));
      acc = fmaf(av.x * sa, wv.x * sw, acc);
      acc = fmaf(av.y * sa, wv.y * sw, acc);
    }
  }
  out[token * rows + row] = __fdiv_rn(acc, divisor);
}

__global__ void __launch_bounds__(128)
fp8_reference_projection_kernel(const uint8_t* __restrict__ a, const float* __restrict__ as,
                                const uint8_t* __restrict__ w, const uint16_t* __restrict__ ws,
                                float* __restrict__ out, uint64_t tokens, uint64_t rows, uint64_t k) {
  const uint64_t token = blockIdx.y;
  const uint64_t row = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (token >= tokens || row >= rows) return;
  const uint8_t* ap = a + token * k;
  const uint8_t* wp = w + row * k;
  float acc = 0.0f;
  for (uint64_t i = 0; i < k; ++i) acc = fmaf(e4m3_decode(ap[i]), e4m3_decode(wp[i]), acc);
  out[token * rows + row] = __fmul_rn(__fmul_rn(acc, as[token]), bf16_bits_to_float(ws[row]));
}

}  // namespace
}  // namespace gemb

using namespace gemb;

extern "C" {

int32_t gemb_nvfp4_reference_projection(const uint8_t* a, const uint8_t* as, const uint8_t* w,
                                        const uint8_t* ws, float* out, uint64_t tokens, uint64_t rows,
                                        uint64_t k, float ga, float gw, gemb_stream_t stream) {
  const char* op = "gemb_nvfp4_reference_projection";
  GEMB_REQUIRE(a && as && w && ws && out, "%s: pointers must be nonnull", op);
  GEMB_REQUIRE(tokens > 0 && rows > 0 && k > 0 && k % 16 == 0,
               "%s: contracting extent must be a nonzero multiple of 16", op);
  GEMB_REQUIRE(tokens <= 65535, "%s: at most 65535 tokens per launch", op);
  GEMB_REQUIRE(positive_finite(ga) && positive_finite(gw) && std::isfinite(ga * gw),
               "%s: global divisors must be positive and finite", op);
  GEMB_ENTER(op);
  dim3 grid(static_cast<unsigned>((rows + 127) / 128), static_cast<unsigned>(tokens));
  nvfp4_reference_projection_kernel<<<grid, 128, 0, stream>>>(a, as, w, ws, out, tokens, rows, k, ga * gw);
  return check_launch(op);
}

int32_t gemb_fp8_reference_projection(const uint8_t* a, const float* as, const uint8_t* w,
                                      const uint16_t* ws, float* out, uint64_t tokens, uint64_t rows,
                                      uint64_t k, gemb_stream_t stream) {
  const char* op = "gemb_fp8_reference_projection";
  GEMB_REQUIRE(a && as && w && ws && out, "%s: pointers must be nonnull", op);
  GEMB_REQUIRE(tokens > 0 && rows > 0 && k > 0, "%s: geometry must be nonzero", op);
  GEMB_REQUIRE(tokens <= 65535, "%s: at most 65535 tokens per launch", op);
  GEMB_ENTER(op);
  dim3 grid(static_cast<unsigned>((rows + 127) / 128), static_cast<unsigned>(tokens));
  fp8_reference_projection_kernel<<<grid, 128, 0, stream>>>(a, as, w, ws, out, tokens, rows, k);
  return check_launch(op);
}

}  // extern "C"
