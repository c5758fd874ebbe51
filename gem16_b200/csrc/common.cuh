// Shared host/device helpers for the gemb200 operator library.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp4.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdint>

#include "gemb200.h"

#ifdef GEMB_NVTX
#include <nvtx3/nvToolsExt.h>
namespace gemb {
struct OpRange {
  explicit OpRange(const char* name) { nvtxRangePushA(name); }
  ~OpRange() { nvtxRangePop(); }
};
}  // namespace gemb
#endif

namespace gemb {

// Records `message` (printf style) as the calling thread's last error and returns `code`.
int32_t fail(int32_t code, const char* fmt, ...);
// cudaGetLastError() after a launch: GEMB_OK, or GEMB_INTERNAL with "op: cudaErrorName: string"
// (the format of CudaFailure at src/cuda/nvfp4/reference.cu:27-31).
int32_t check_launch(const char* op);
// GEMB_OK when the current device is sm_100-class; cached per device.
int32_t require_sm100(const char* op);
// Number of SMs of the current device (cached).
int sm_count();
// Tuning knobs owned by the GEMM translation unit (see gemb_set_tuning).
int32_t gemm_set_tuning(int32_t knob, int32_t value);
int32_t ep_set_tuning(int32_t knob, int32_t value);
int32_t moe_set_tuning(int32_t knob, int32_t value);
// Decode-size FP8 token quantizer (bf16 input, K <= 16384, K % 8 == 0); bit-identical to the
// general kernel, one global round trip, programmatic-dependent-launch aware.
int32_t launch_fp8_quantize_decode(const char* op, const uint16_t* x, uint8_t* out, float* scales, uint64_t tokens,
                                   uint64_t k, cudaStream_t stream);
// Reads and clears the decode GEMV's bounded-wait flag (0 = clean, -1 = could not read).
int gemv_take_device_error();
int ep_take_device_error();
int moe_take_device_error();

inline bool positive_finite(float v) { return std::isfinite(v) && v > 0.0f; }

#define GEMB_REQUIRE(cond, ...)                                           \
  do {                                                                    \
    if (!(cond)) return ::gemb::fail(GEMB_INVALID_ARGUMENT, __VA_ARGS__); \
  } while (0)

// Device gate plus, when the library is built with -DGEMB_NVTX, an NVTX range named after the entry
// point for the rest of the call (gem16 brackets its operators the same way,
// src/cuda/engine/inference_engine.cu:81-87).  Off by default: a range costs a few hundred
// nanoseconds per launch.
#ifdef GEMB_NVTX
#define GEMB_ENTER(op)                     \
  GEMB_TRY(::gemb::require_sm100(op));     \
  ::gemb::OpRange gemb_op_range_(op)
#else
#define GEMB_ENTER(op) GEMB_TRY(::gemb::require_sm100(op))
#endif

#define GEMB_TRY(expr)                   \
  do {                                   \
    int32_t gemb_rc_ = (expr);           \
    if (gemb_rc_ != GEMB_OK) return gemb_rc_; \
  } while (0)

// ---------------------------------------------------------------------------------------------
// Device-side codecs.  E2M1/E4M3 conversions use the hardware cvt instructions, which round to
// nearest with ties to the even code and saturate to the largest finite value: the same rule
// as ChooseNearestE2M1 / ChooseNearestPositiveE4M3Fn in src/numeric/nvfp4.cpp:26-56.
// ---------------------------------------------------------------------------------------------
#ifdef __CUDACC__

__device__ __forceinline__ float bf16_bits_to_float(uint16_t bits) {
  return __uint_as_float(static_cast<uint32_t>(bits) << 16);
}
__device__ __forceinline__ uint16_t float_to_bf16_bits(float v) {
  return __bfloat16_as_ushort(__float2bfloat16_rn(v));
}
__device__ __forceinline__ float bf16_round(float v) {
  return __bfloat162float(__float2bfloat16_rn(v));
}

__device__ __forceinline__ uint8_t e4m3_encode(float v) {
  return static_cast<uint8_t>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3));
}
__device__ __forceinline__ float e4m3_decode(uint8_t bits) {
  __half_raw h = __nv_cvt_fp8_to_halfraw(bits, __NV_E4M3);
  return __half2float(__half(h));
}
// Two floats -> one byte, `lo` in the low nibble.
__device__ __forceinline__ uint8_t e2m1x2_encode(float lo, float hi) {
  return static_cast<uint8_t>(
      __nv_cvt_float2_to_fp4x2(make_float2(lo, hi), __NV_E2M1, cudaRoundNearest));
}
// One byte -> half2, low nibble in .x.
__device__ __forceinline__ __half2 e2m1x2_decode(uint8_t byte) {
  __half2_raw r = __nv_cvt_fp4x2_to_halfraw2(byte, __NV_E2M1);
  return __half2(r);
}
__device__ __forceinline__ float rcp_approx_ftz(float v) {
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(v));
  return r;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
  return v;
}

// Byte offset of block scale (row r, scale column c) in the 128x4 interleaved layout with
// `c_pad` = K/16 rounded up to 4  (src/cuda/nvfp4/cutlass_sm120.cu:160-172).
__host__ __device__ __forceinline__ uint64_t interleaved_scale_offset(uint64_t r, uint64_t c,
                                                                       uint64_t c_pad) {
  return ((r / 128) * (c_pad / 4) + c / 4) * 512 + (r % 32) * 16 + ((r % 128) / 32) * 4 + c % 4;
}

// tanh for the GELU boundary: 1 - 2 / (exp(2x) + 1) with ex2.approx, rcp.approx and one Newton step
// on the reciprocal (two MUFU operations and five arithmetic ones, against the two dozen of tanhf).
// Absolute error about 1e-7, i.e. one or two ulps of the "1 + tanh" the GELU formula adds it to --
// the same class as tanhf's own deviation from a correctly rounded tanh.  Every kernel that
// applies the GELU uses this one function, so their results agree byte for byte with one another.
__device__ __forceinline__ float tanh_gelu(float x) {
  float e;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(fminf(__fmul_rn(x, 2.8853900817779268f), 126.0f)));   // exp(2x), finite
  const float d = __fadd_rn(e, 1.0f);
  const float y0 = rcp_approx_ftz(d);
  const float y = fmaf(fmaf(-d, y0, 1.0f), y0, y0);
  return fmaf(-2.0f, y, 1.0f);
}
// bf16(gelu_tanh(g)) * u with the bf16 boundaries of src/cuda/nvfp4/reference.cu:177-190
// (g and u already bf16 values): gelu = bf16(0.5 g (1 + tanh(0.79788456 (g + 0.044715 g^3)))),
// product = bf16(gelu * u).
__device__ __forceinline__ float gelu_tanh_product(float g, float u) {
  const float inner = 0.7978845608028654f * (g + 0.044715f * g * g * g);
  const float gelu = bf16_round(0.5f * g * (1.0f + tanh_gelu(inner)));
  return bf16_round(gelu * u);
}

constexpr float kInvSix = 1.0f / 6.0f;  // kE2M1MaxReciprocal, src/numeric/nvfp4.cpp:16

// Quantizes 16 values into 8 packed bytes (returned as two 32-bit words) and one scale byte.
// EXACT follows src/numeric/nvfp4.cpp:139-150, RCP_APPROX follows
// src/cuda/nvfp4/reference.cu:60-78.  Explicit _rn intrinsics keep the compiler from fusing
// the multiplies into fma, which would change the rounding.
template <bool kRcp>
__device__ __forceinline__ void quantize_block16(const float (&v)[16], float g, uint32_t& lo,
                                                 uint32_t& hi, uint8_t& scale_bits) {
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
  float n[16];
  bool zero_scale = false;
  if constexpr (kRcp) {
    scale_bits = e4m3_encode(__fmul_rn(__fmul_rn(amax, rcp_approx_ftz(6.0f)), g));
    const float ds = e4m3_decode(scale_bits);
    const float os = ds == 0.0f ? 0.0f : rcp_approx_ftz(__fmul_rn(ds, rcp_approx_ftz(g)));
#pragma unroll
    for (int i = 0; i < 16; ++i) n[i] = __fmul_rn(v[i], os);
  } else {
    scale_bits = e4m3_encode(__fmul_rn(__fmul_rn(amax, kInvSix), g));
    const float ds = e4m3_decode(scale_bits);
    // (x * g) / ds, correctly rounded, with ONE division per block: r = RN(1 / ds), then per element
    // q0 = RN(t * r), e = t - ds * q0 (exact in one fma), q = RN(q0 + e * r).  With a correctly rounded
    // reciprocal this residual correction yields the correctly rounded quotient (Markstein); for the
    // 126 values an E4M3 scale can take it is also checked exhaustively around every E2M1 rounding
    // boundary in tests/test_oracle.py.  Sixteen IEEE divisions per block kept the conversion pipe of
    // the fused GEMM epilogue busier than the tensor pipe.
    // Two elements per instruction (packed fp32 multiply and fma: one IEEE operation per half, so the
    // rounding of every step is that of the scalar form).  A zero scale gives sixteen +0 codes, set after
    // the packing below.
    const float r = ds == 0.0f ? 0.0f : __fdiv_rn(1.0f, ds);
    const float2 g2 = make_float2(g, g), r2 = make_float2(r, r), nds2 = make_float2(-ds, -ds);
#pragma unroll
    for (int i = 0; i < 16; i += 2) {
      const float2 t = __fmul2_rn(make_float2(v[i], v[i + 1]), g2);
      const float2 q0 = __fmul2_rn(t, r2);
      const float2 q = __ffma2_rn(__ffma2_rn(nds2, q0, t), r2, q0);
      // (the quotient has the sign of t, also when it is zero: -0 keeps its sign bit in E2M1, and the
      // residual correction alone would turn -0 into +0)
      n[i] = copysignf(q.x, t.x);
      n[i + 1] = copysignf(q.y, t.y);
    }
    zero_scale = ds == 0.0f;
  }
  lo = hi = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    lo |= static_cast<uint32_t>(e2m1x2_encode(n[2 * i], n[2 * i + 1])) << (8 * i);
    hi |= static_cast<uint32_t>(e2m1x2_encode(n[8 + 2 * i], n[8 + 2 * i + 1])) << (8 * i);
  }
  if (zero_scale) lo = hi = 0;
}

#endif  // __CUDACC__

}  // namespace gemb
