// Activation quantizers: NVFP4 block quantizer (plain, RMSNorm-fused, gated-GELU-fused), the
// compact->interleaved scale shuffle, and the FP8 per-token quantizer (plain, RMSNorm-fused).
//
// All of them are HBM-streaming kernels: every input element is read once with 128-bit loads,
// every output byte written once.  Algorithmic bytes per element (bf16 input): NVFP4
// 2 + 0.5 + 1/16 = 2.5625 B, FP8 2 + 2 (second pass hits L2 or L1) + 1 = 3 B (+4 B per token).
#include "common.cuh"

namespace gemb {
namespace {


__device__ __forceinline__ void load16(const float* p, float (&v)[16]) {
  const float4* q = reinterpret_cast<const float4*>(p);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float4 t = __ldg(q + i);
    v[4 * i] = t.x; v[4 * i + 1] = t.y; v[4 * i + 2] = t.z; v[4 * i + 3] = t.w;
  }
}
__device__ __forceinline__ void load16(const uint16_t* p, float (&v)[16]) {
  const uint4* q = reinterpret_cast<const uint4*>(p);
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    uint4 t = __ldg(q + i);
    const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      v[8 * i + 2 * j] = __uint_as_float(w[j] << 16);
      v[8 * i + 2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
    }
  }
}

template <typename In>
struct PlainLoader {
  const In* x;
  __device__ __forceinline__ void operator()(uint64_t offset, float (&v)[16]) const {
    load16(x + offset, v);
  }
};

// src/cuda/nvfp4/reference.cu:177-190.  For fp32 inputs gate/up are first rounded to bf16.
template <typename In>
struct GatedGeluLoader {
  const In* gate;
  const In* up;
  __device__ __forceinline__ void operator()(uint64_t offset, float (&v)[16]) const {
    float g[16], u[16];
    load16(gate + offset, g);
    load16(up + offset, u);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float gv = sizeof(In) == 4 ? bf16_round(g[i]) : g[i];
      const float uv = sizeof(In) == 4 ? bf16_round(u[i]) : u[i];
      v[i] = gelu_tanh_product(gv, uv);
    }
  }
};

// One thread per group of four consecutive 16-blocks ("quad", 64 elements): it writes 32 packed
// bytes and one 32-bit word of scales.  The thread grid covers rows_out x quads where, for the
// interleaved layout, rows_out is `tokens` rounded up to 128 and padded cells get zero scales.
template <class Loader, bool kRcp, bool kInterleaved>
__global__ void __launch_bounds__(256)
nvfp4_quantize_kernel(Loader loader, uint8_t* __restrict__ packed, uint8_t* __restrict__ scales,
                      uint64_t tokens, uint64_t k, uint64_t rows_out, uint64_t quads, float g) {
  const uint64_t idx = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= rows_out * quads) return;
  const uint64_t r = idx / quads, q = idx % quads;
  const uint64_t c_real = k / 16;
  uint32_t scale_word = 0;
  if (r < tokens) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint64_t c = q * 4 + j;
      if (c < c_real) {
        float v[16];
        loader(r * k + c * 16, v);
        uint32_t lo, hi;
        uint8_t sb;
        quantize_block16<kRcp>(v, g, lo, hi, sb);
        *reinterpret_cast<uint2*>(packed + r * (k / 2) + c * 8) = make_uint2(lo, hi);
        scale_word |= static_cast<uint32_t>(sb) << (8 * j);
      }
    }
  }
  if constexpr (kInterleaved) {
    *reinterpret_cast<uint32_t*>(scales + interleaved_scale_offset(r, q * 4, quads * 4)) = scale_word;
  } else {
    if (q * 4 + 4 <= c_real && c_real % 4 == 0) {
      *reinterpret_cast<uint32_t*>(scales + r * c_real + q * 4) = scale_word;
    } else {
      for (int j = 0; j < 4 && q * 4 + j < c_real; ++j)
        scales[r * c_real + q * 4 + j] = static_cast<uint8_t>(scale_word >> (8 * j));
    }
  }
}

template <class Loader>
int32_t launch_nvfp4_quantize(const char* op, Loader loader, uint8_t* packed, uint8_t* scales,
                              uint64_t tokens, uint64_t k, float g, int32_t layout, int32_t mode,
                              cudaStream_t stream) {
  const bool inter = layout == GEMB_SCALES_INTERLEAVED;
  const uint64_t rows_out = inter ? (tokens + 127) / 128 * 128 : tokens;
  const uint64_t quads = (k / 16 + 3) / 4;
  const uint64_t threads = rows_out * quads;
  const unsigned grid = static_cast<unsigned>((threads + 255) / 256);
  const bool rcp = mode == GEMB_QUANT_RCP_APPROX;
  if (inter) {
    if (rcp) nvfp4_quantize_kernel<Loader, true, true><<<grid, 256, 0, stream>>>(loader, packed, scales, tokens, k, rows_out, quads, g);
    else nvfp4_quantize_kernel<Loader, false, true><<<grid, 256, 0, stream>>>(loader, packed, scales, tokens, k, rows_out, quads, g);
  } else {
    if (rcp) nvfp4_quantize_kernel<Loader, true, false><<<grid, 256, 0, stream>>>(loader, packed, scales, tokens, k, rows_out, quads, g);
    else nvfp4_quantize_kernel<Loader, false, false><<<grid, 256, 0, stream>>>(loader, packed, scales, tokens, k, rows_out, quads, g);
  }
  return check_launch(op);
}

int32_t validate_nvfp4_quantize(const char* op, const void* in, const void* packed,
                                const void* scales, int32_t dtype, uint64_t tokens, uint64_t k,
                                float g, int32_t layout, int32_t mode) {
  GEMB_REQUIRE(in && packed && scales, "%s: pointers must be nonnull", op);
  GEMB_REQUIRE(dtype == GEMB_F32 || dtype == GEMB_BF16, "%s: input dtype must be GEMB_F32 or GEMB_BF16", op);
  GEMB_REQUIRE(tokens > 0 && k > 0 && k % 16 == 0,
               "%s: extent must be a nonzero multiple of 16 per token", op);
  GEMB_REQUIRE(tokens <= (1ull << 31) && k <= (1ull << 31), "%s: extent too large", op);
  GEMB_REQUIRE(positive_finite(g), "%s: global divisor must be positive and finite", op);
  GEMB_REQUIRE(layout == GEMB_SCALES_COMPACT || layout == GEMB_SCALES_INTERLEAVED, "%s: unknown scale layout", op);
  GEMB_REQUIRE(mode == GEMB_QUANT_EXACT || mode == GEMB_QUANT_RCP_APPROX, "%s: unknown quantizer mode", op);
  GEMB_REQUIRE(reinterpret_cast<uintptr_t>(in) % 16 == 0 && reinterpret_cast<uintptr_t>(packed) % 8 == 0 &&
                   reinterpret_cast<uintptr_t>(scales) % 4 == 0,
               "%s: input must be 16-byte, payload 8-byte and scales 4-byte aligned", op);
  return require_sm100(op);
}

// ---------------------------------------------------------------------------------------------
// RMSNorm fused quantizers.  One CTA of 256 threads per token.  The sum of squares follows the
// reference exactly: thread t fma-accumulates index t, t+256, ... and a power-of-two tree folds
// the 256 partials (src/cuda/nvfp4/reference.cu:102-118), so the fp32 sum is bit-identical.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float load_scalar(const float* p, uint64_t i) { return __ldg(p + i); }
__device__ __forceinline__ float load_scalar(const uint16_t* p, uint64_t i) {
  return bf16_bits_to_float(__ldg(p + i));
}

template <typename In>
__device__ __forceinline__ float rmsnorm_inverse(const In* row, uint64_t k, float eps, float* red) {
  float ss = 0.0f;
  for (uint64_t i = threadIdx.x; i < k; i += 256) {
    const float v = load_scalar(row, i);
    ss = fmaf(v, v, ss);
  }
  red[threadIdx.x] = ss;
  __syncthreads();
  for (unsigned stride = 128; stride; stride >>= 1) {
    if (threadIdx.x < stride) red[threadIdx.x] += red[threadIdx.x + stride];
    __syncthreads();
  }
  return rsqrtf(red[0] / static_cast<float>(k) + eps);
}

// RMSNorm + residual (+ layer scalar) with the bf16 boundaries of src/cuda/norm/reference.cu:66-160:
// n = bf16(x * inv * w), v = bf16(n + residual), v = bf16(v * scalar) when a scalar is given.
__device__ __forceinline__ void store_scalar(float* p, uint64_t i, float v) { p[i] = v; }
__device__ __forceinline__ void store_scalar(uint16_t* p, uint64_t i, float v) { p[i] = float_to_bf16_bits(v); }

template <typename In, typename Res, typename Out>
__global__ void __launch_bounds__(256)
rmsnorm_residual_kernel(const In* __restrict__ x, const uint16_t* __restrict__ w, const Res* __restrict__ residual,
                        float* __restrict__ normalized, Out* __restrict__ out, uint64_t k, float eps,
                        const uint16_t* __restrict__ scalar) {
  __shared__ float red[256];
  const uint64_t base = static_cast<uint64_t>(blockIdx.x) * k;
  const float inv = rmsnorm_inverse(x + base, k, eps, red);
  const float layer_scale = scalar ? bf16_bits_to_float(__ldg(scalar)) : 1.0f;
  for (uint64_t i = threadIdx.x; i < k; i += 256) {
    const float ws = w ? bf16_bits_to_float(__ldg(w + i)) : 1.0f;
    const float n = bf16_round(__fmul_rn(__fmul_rn(load_scalar(x + base, i), inv), ws));
    if (normalized) normalized[base + i] = n;
    float v = bf16_round(__fadd_rn(n, load_scalar(residual + base, i)));
    if (scalar) v = bf16_round(__fmul_rn(v, layer_scale));
    store_scalar(out, base + i, v);
  }
}

template <typename In, bool kRcp, bool kInterleaved>
__global__ void __launch_bounds__(256)
rmsnorm_nvfp4_quantize_kernel(const In* __restrict__ x, const uint16_t* __restrict__ w,
                              uint8_t* __restrict__ packed, uint8_t* __restrict__ scales,
                              uint64_t k, float eps, float g, uint64_t c_pad) {
  __shared__ float red[256];
  const uint64_t r = blockIdx.x;
  const In* row = x + r * k;
  const float inv = rmsnorm_inverse(row, k, eps, red);
  for (uint64_t c = threadIdx.x; c < k / 16; c += 256) {
    float v[16];
    load16(row + c * 16, v);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float ws = w ? bf16_bits_to_float(__ldg(w + c * 16 + i)) : 1.0f;
      v[i] = bf16_round(__fmul_rn(__fmul_rn(v[i], inv), ws));
    }
    uint32_t lo, hi;
    uint8_t sb;
    quantize_block16<kRcp>(v, g, lo, hi, sb);
    *reinterpret_cast<uint2*>(packed + r * (k / 2) + c * 8) = make_uint2(lo, hi);
    if constexpr (kInterleaved) scales[interleaved_scale_offset(r, c, c_pad)] = sb;
    else scales[r * (k / 16) + c] = sb;
  }
}

// ---------------------------------------------------------------------------------------------
// FP8 per-token quantizer.  One CTA per token; pass 1 finds amax (max is order independent),
// pass 2 divides and converts.  src/numeric/fp8.cpp:41-58, src/cuda/fp8/reference.cu:39-69.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float block_max_256(float v, float* red) {
  v = warp_max(v);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float m = red[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) m = fmaxf(m, red[i]);
  return m;
}

template <typename In, bool kNorm>
__global__ void __launch_bounds__(256)
fp8_quantize_kernel(const In* __restrict__ x, const uint16_t* __restrict__ w,
                    uint8_t* __restrict__ out, float* __restrict__ scales, uint64_t k, float eps) {
  __shared__ float red[256];
  __shared__ float red2[8];
  const uint64_t r = blockIdx.x;
  const In* row = x + r * k;
  float inv = 1.0f;
  if constexpr (kNorm) inv = rmsnorm_inverse(row, k, eps, red);
  auto value = [&](uint64_t i, float raw) {
    if constexpr (kNorm) {
      const float ws = w ? bf16_bits_to_float(__ldg(w + i)) : 1.0f;
      return bf16_round(__fmul_rn(__fmul_rn(raw, inv), ws));
    } else {
      return raw;
    }
  };
  float amax = 0.0f;
  for (uint64_t c = threadIdx.x; c < k / 16; c += 256) {
    float v[16];
    load16(row + c * 16, v);
#pragma unroll
    for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(value(c * 16 + i, v[i])));
  }
  for (uint64_t i = (k / 16) * 16 + threadIdx.x; i < k; i += 256)
    amax = fmaxf(amax, fabsf(value(i, load_scalar(row, i))));
  amax = block_max_256(amax, red2);
  const float scale = amax == 0.0f ? 1.0f : __fdiv_rn(amax, 448.0f);
  if (threadIdx.x == 0) scales[r] = scale;
  uint8_t* orow = out + r * k;
  for (uint64_t c = threadIdx.x; c < k / 16; c += 256) {
    float v[16];
    load16(row + c * 16, v);
    uint32_t words[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint32_t word = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i)
        word |= static_cast<uint32_t>(e4m3_encode(__fdiv_rn(value(c * 16 + 4 * j + i, v[4 * j + i]), scale))) << (8 * i);
      words[j] = word;
    }
    *reinterpret_cast<uint4*>(orow + c * 16) = make_uint4(words[0], words[1], words[2], words[3]);
  }
  for (uint64_t i = (k / 16) * 16 + threadIdx.x; i < k; i += 256)
    orow[i] = e4m3_encode(__fdiv_rn(value(i, load_scalar(row, i)), scale));
}

__global__ void __launch_bounds__(256)
interleave_scales_kernel(const uint8_t* __restrict__ compact, uint8_t* __restrict__ out,
                         uint64_t rows, uint64_t c_real, uint64_t rows_pad, uint64_t quads) {
  const uint64_t idx = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= rows_pad * quads) return;
  const uint64_t r = idx / quads, q = idx % quads;
  uint32_t word = 0;
  if (r < rows)
    for (int j = 0; j < 4; ++j)
      if (q * 4 + j < c_real) word |= static_cast<uint32_t>(__ldg(compact + r * c_real + q * 4 + j)) << (8 * j);
  *reinterpret_cast<uint32_t*>(out + interleaved_scale_offset(r, q * 4, quads * 4)) = word;
}

}  // namespace
}  // namespace gemb

using namespace gemb;

extern "C" {

int32_t gemb_nvfp4_quantize(const void* input, int32_t input_dtype, uint8_t* packed, uint8_t* scales,
                            uint64_t tokens, uint64_t k, float g, int32_t layout, int32_t mode,
                            gemb_stream_t stream) {
  const char* op = "gemb_nvfp4_quantize";
  GEMB_TRY(validate_nvfp4_quantize(op, input, packed, scales, input_dtype, tokens, k, g, layout, mode));
  if (input_dtype == GEMB_F32)
    return launch_nvfp4_quantize(op, PlainLoader<float>{static_cast<const float*>(input)}, packed, scales, tokens, k, g, layout, mode, stream);
  return launch_nvfp4_quantize(op, PlainLoader<uint16_t>{static_cast<const uint16_t*>(input)}, packed, scales, tokens, k, g, layout, mode, stream);
}

int32_t gemb_nvfp4_gated_gelu_quantize(const void* gate, const void* up, int32_t input_dtype,
                                       uint8_t* packed, uint8_t* scales, uint64_t tokens, uint64_t k,
                                       float g, int32_t layout, int32_t mode, gemb_stream_t stream) {
  const char* op = "gemb_nvfp4_gated_gelu_quantize";
  GEMB_REQUIRE(up != nullptr && reinterpret_cast<uintptr_t>(up) % 16 == 0, "%s: up must be nonnull and 16-byte aligned", op);
  GEMB_TRY(validate_nvfp4_quantize(op, gate, packed, scales, input_dtype, tokens, k, g, layout, mode));
  if (input_dtype == GEMB_F32)
    return launch_nvfp4_quantize(op, GatedGeluLoader<float>{static_cast<const float*>(gate), static_cast<const float*>(up)}, packed, scales, tokens, k, g, layout, mode, stream);
  return launch_nvfp4_quantize(op, GatedGeluLoader<uint16_t>{static_cast<const uint16_t*>(gate), static_cast<const uint16_t*>(up)}, packed, scales, tokens, k, g, layout, mode, stream);
}

int32_t gemb_nvfp4_rmsnorm_quantize(const void* input, int32_t input_dtype, const uint16_t* weight,
                                    uint8_t* packed, uint8_t* scales, uint64_t tokens, uint64_t k,
                                    float eps, float g, int32_t layout, int32_t mode,
                                    gemb_stream_t stream) {
  const char* op = "gemb_nvfp4_rmsnorm_quantize";
  GEMB_TRY(validate_nvfp4_quantize(op, input, packed, scales, input_dtype, tokens, k, g, layout, mode));
  GEMB_REQUIRE(std::isfinite(eps) && eps >= 0.0f, "%s: epsilon must be finite and nonnegative", op);
  const bool inter = layout == GEMB_SCALES_INTERLEAVED;
  const uint64_t c_pad = (k / 16 + 3) / 4 * 4;
  if (inter) {
    // Padded rows / columns of the interleaved buffer must read as zero.
    cudaError_t e = cudaMemsetAsync(scales, 0, gemb_interleaved_scale_bytes(tokens, k), stream);
    if (e != cudaSuccess) return fail(GEMB_INTERNAL, "%s: %s: %s", op, cudaGetErrorName(e), cudaGetErrorString(e));
  }
  const unsigned grid = static_cast<unsigned>(tokens);
  const bool rcp = mode == GEMB_QUANT_RCP_APPROX;
#define GEMB_LAUNCH_RMS(T, RCP, INTER)                                                         \
  rmsnorm_nvfp4_quantize_kernel<T, RCP, INTER><<<grid, 256, 0, stream>>>(                      \
      static_cast<const T*>(input), weight, packed, scales, k, eps, g, c_pad)
  if (input_dtype == GEMB_F32) {
    if (inter) { if (rcp) GEMB_LAUNCH_RMS(float, true, true); else GEMB_LAUNCH_RMS(float, false, true); }
    else { if (rcp) GEMB_LAUNCH_RMS(float, true, false); else GEMB_LAUNCH_RMS(float, false, false); }
  } else {
    if (inter) { if (rcp) GEMB_LAUNCH_RMS(uint16_t, true, true); else GEMB_LAUNCH_RMS(uint16_t, false, true); }
    else { if (rcp) GEMB_LAUNCH_RMS(uint16_t, true, false); else GEMB_LAUNCH_RMS(uint16_t, false, false); }
  }
#undef GEMB_LAUNCH_RMS
  return check_launch(op);
}

int32_t gemb_nvfp4_interleave_scales(const uint8_t* compact, uint8_t* interleaved, uint64_t rows,
                                     uint64_t k, gemb_stream_t stream) {
  const char* op = "gemb_nvfp4_interleave_scales";
  GEMB_REQUIRE(compact && interleaved, "%s: pointers must be nonnull", op);
  GEMB_REQUIRE(rows > 0 && k > 0 && k % 16 == 0, "%s: geometry must be nonzero with K a multiple of 16", op);
  GEMB_REQUIRE(reinterpret_cast<uintptr_t>(interleaved) % 4 == 0, "%s: output must be 4-byte aligned", op);
  GEMB_ENTER(op);
  const uint64_t rows_pad = (rows + 127) / 128 * 128, quads = (k / 16 + 3) / 4;
  const unsigned grid = static_cast<unsigned>((rows_pad * quads + 255) / 256);
  interleave_scales_kernel<<<grid, 256, 0, stream>>>(compact, interleaved, rows, k / 16, rows_pad, quads);
  return check_launch(op);
}

static int32_t validate_fp8_quantize(const char* op, const void* in, const void* out, const void* scales,
                                     int32_t dtype, uint64_t tokens, uint64_t k) {
  GEMB_REQUIRE(in && out && scales, "%s: pointers must be nonnull", op);
  GEMB_REQUIRE(dtype == GEMB_F32 || dtype == GEMB_BF16, "%s: input dtype must be GEMB_F32 or GEMB_BF16", op);
  GEMB_REQUIRE(tokens > 0 && k > 0, "%s: token activation must be nonempty", op);
  GEMB_REQUIRE(tokens <= (1ull << 31) - 1 && k <= (1ull << 31), "%s: extent too large", op);
  GEMB_REQUIRE(k % 16 == 0, "%s: elements per token must be a multiple of 16", op);
  GEMB_REQUIRE(reinterpret_cast<uintptr_t>(in) % 16 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0,
               "%s: input and output must be 16-byte aligned", op);
  return require_sm100(op);
}

int32_t gemb_fp8_quantize(const void* input, int32_t input_dtype, uint8_t* out, float* scales,
                          uint64_t tokens, uint64_t k, gemb_stream_t stream) {
  const char* op = "gemb_fp8_quantize";
  GEMB_TRY(validate_fp8_quantize(op, input, out, scales, input_dtype, tokens, k));
  const unsigned grid = static_cast<unsigned>(tokens);
  if (input_dtype == GEMB_BF16 && tokens <= 16 && k <= 16384)   // decode batches: latency-optimised kernel
    return launch_fp8_quantize_decode(op, static_cast<const uint16_t*>(input), out, scales, tokens, k, stream);
  if (input_dtype == GEMB_F32)
    fp8_quantize_kernel<float, false><<<grid, 256, 0, stream>>>(static_cast<const float*>(input), nullptr, out, scales, k, 0.0f);
  else
    fp8_quantize_kernel<uint16_t, false><<<grid, 256, 0, stream>>>(static_cast<const uint16_t*>(input), nullptr, out, scales, k, 0.0f);
  return check_launch(op);
}

int32_t gemb_fp8_rmsnorm_quantize(const void* input, int32_t input_dtype, const uint16_t* weight,
                                  uint8_t* out, float* scales, uint64_t tokens, uint64_t k, float eps,
                                  gemb_stream_t stream) {
  const char* op = "gemb_fp8_rmsnorm_quantize";
  GEMB_TRY(validate_fp8_quantize(op, input, out, scales, input_dtype, tokens, k));
  GEMB_REQUIRE(std::isfinite(eps) && eps >= 0.0f, "%s: epsilon must be finite and nonnegative", op);
  const unsigned grid = static_cast<unsigned>(tokens);
  if (input_dtype == GEMB_F32)
    fp8_quantize_kernel<float, true><<<grid, 256, 0, stream>>>(static_cast<const float*>(input), weight, out, scales, k, eps);
  else
    fp8_quantize_kernel<uint16_t, true><<<grid, 256, 0, stream>>>(static_cast<const uint16_t*>(input), weight, out, scales, k, eps);
  return check_launch(op);
}

int32_t gemb_rmsnorm_residual(const void* input, int32_t input_dtype, const uint16_t* weight_bf16, const void* residual,
                              float* normalized_output, void* output, int32_t residual_output_dtype, uint64_t vectors,
                              uint64_t width, float epsilon, const uint16_t* scalar_bf16, gemb_stream_t stream) {
  const char* op = "gemb_rmsnorm_residual";
  GEMB_REQUIRE(input && residual && output, "%s: input, residual and output must be nonnull", op);
  GEMB_REQUIRE((input_dtype == GEMB_F32 || input_dtype == GEMB_BF16) &&
                   (residual_output_dtype == GEMB_F32 || residual_output_dtype == GEMB_BF16), "%s: unknown dtype", op);
  GEMB_REQUIRE(vectors > 0 && vectors < (1ull << 31) && width > 0 && width < (1ull << 31), "%s: bad geometry", op);
  GEMB_REQUIRE(positive_finite(epsilon), "%s: epsilon must be positive and finite", op);
  GEMB_REQUIRE(residual_output_dtype == GEMB_F32 || (input_dtype == GEMB_BF16 && normalized_output == nullptr),
               "%s: bf16 residual and output go with a bf16 input and no separate normalised output", op);
  GEMB_ENTER(op);
  const unsigned grid = static_cast<unsigned>(vectors);
  if (residual_output_dtype == GEMB_BF16)
    rmsnorm_residual_kernel<<<grid, 256, 0, stream>>>(static_cast<const uint16_t*>(input), weight_bf16,
                                                      static_cast<const uint16_t*>(residual), normalized_output,
                                                      static_cast<uint16_t*>(output), width, epsilon, scalar_bf16);
  else if (input_dtype == GEMB_BF16)
    rmsnorm_residual_kernel<<<grid, 256, 0, stream>>>(static_cast<const uint16_t*>(input), weight_bf16,
                                                      static_cast<const float*>(residual), normalized_output,
                                                      static_cast<float*>(output), width, epsilon, scalar_bf16);
  else
    rmsnorm_residual_kernel<<<grid, 256, 0, stream>>>(static_cast<const float*>(input), weight_bf16,
                                                      static_cast<const float*>(residual), normalized_output,
                                                      static_cast<float*>(output), width, epsilon, scalar_bf16);
  return check_launch(op);
}

}  // extern "C"
