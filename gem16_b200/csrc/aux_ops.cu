// Small operators beside the contraction path that gem16's engine calls between projections and
// that a drop-in operator library therefore has to define too: the fp32 GELU-tanh product and the
// residual add of the MLP (src/cuda/nvfp4/mlp.cu:27-43), the arg-max over materialised logits
// (src/cuda/output_head.cu:414-422) and the assistant's bf16-weight GEMV (src/cuda/mtp/assistant.cu:99-122).
#include <algorithm>
#include <cfloat>

#include "common.cuh"

namespace gemb {
namespace {

// out = bf16(gelu_tanh(gate)) * up in fp32: gate and up enter unrounded, only the GELU value is
// rounded to bf16 (src/cuda/nvfp4/mlp.cu:27-36).
__global__ void __launch_bounds__(256)
gelu_tanh_product_kernel(const float* __restrict__ gate, const float* __restrict__ up, float* __restrict__ out, uint64_t n) {
  const uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float g = __ldg(gate + i);
  const float inner = 0.7978845608028654f * (g + 0.044715f * g * g * g);
  const float gelu = bf16_round(0.5f * g * (1.0f + tanh_gelu(inner)));
  out[i] = gelu * __ldg(up + i);
}

__global__ void __launch_bounds__(256)
add_residual_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ out, uint64_t n) {
  const uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) out[i] = __fadd_rn(__ldg(a + i), __ldg(b + i));
}

struct Best {
  float value;
  uint32_t token;
};
__device__ __forceinline__ bool better(Best a, Best b) {   // larger value, then lower token id
  return a.value > b.value || (a.value == b.value && a.token < b.token);
}

// One CTA: the largest logit that is not on the suppression list; ties go to the lower token id.
__global__ void __launch_bounds__(1024)
logit_argmax_kernel(const float* __restrict__ logits, const uint32_t* __restrict__ suppressed, uint32_t suppressed_count,
                    uint32_t vocabulary, uint32_t* __restrict__ selected) {
  __shared__ Best warp_best[32];
  Best best{-FLT_MAX, 0xFFFFFFFFu};
  for (uint32_t t = threadIdx.x; t < vocabulary; t += blockDim.x) {
    bool skip = false;
    for (uint32_t s = 0; s < suppressed_count; ++s) skip |= __ldg(suppressed + s) == t;
    const Best c{__ldg(logits + t), t};
    if (!skip && better(c, best)) best = c;
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) {
    const Best other{__shfl_xor_sync(0xFFFFFFFFu, best.value, o), __shfl_xor_sync(0xFFFFFFFFu, best.token, o)};
    if (better(other, best)) best = other;
  }
  if ((threadIdx.x & 31) == 0) warp_best[threadIdx.x >> 5] = best;
  __syncthreads();
  if (threadIdx.x < 32) {
    best = threadIdx.x < (blockDim.x >> 5) ? warp_best[threadIdx.x] : Best{-FLT_MAX, 0xFFFFFFFFu};
#pragma unroll
    for (int o = 16; o; o >>= 1) {
      const Best other{__shfl_xor_sync(0xFFFFFFFFu, best.value, o), __shfl_xor_sync(0xFFFFFFFFu, best.token, o)};
      if (better(other, best)) best = other;
    }
    if (threadIdx.x == 0) *selected = best.token;
  }
}

// y[row] = bf16(sum_k x[k] * W[row][k]), fp32 x, bf16 W, fp32 accumulation.  HBM-streaming: one warp
// per row, every lane keeps four 16-byte weight loads in flight, the activation sits in shared
// memory as fp32.  Within a row lane l sums its elements in ascending k, the lanes combine through
// an xor butterfly.
constexpr int kBgThreads = 256;
__global__ void __launch_bounds__(kBgThreads)
bf16_gemv_kernel(const float* __restrict__ x, const uint16_t* __restrict__ w, float* __restrict__ y, uint32_t rows, uint32_t k) {
  extern __shared__ __align__(16) float xs[];
  for (uint32_t i = threadIdx.x; i < k; i += kBgThreads) xs[i] = __ldg(x + i);
  __syncthreads();
  const uint32_t lane = threadIdx.x & 31, warps = gridDim.x * (kBgThreads / 32);
  const uint32_t vecs = k / 8;   // 16-byte pieces per row
  for (uint32_t row = blockIdx.x * (kBgThreads / 32) + (threadIdx.x >> 5); row < rows; row += warps) {
    const uint4* wr = reinterpret_cast<const uint4*>(w + static_cast<uint64_t>(row) * k);
    float acc = 0.0f;
    for (uint32_t v0 = lane; v0 < vecs; v0 += 128) {
      uint4 q[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t v = v0 + 32 * j;
        q[j] = make_uint4(0u, 0u, 0u, 0u);
        if (v < vecs) asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                                   : "=r"(q[j].x), "=r"(q[j].y), "=r"(q[j].z), "=r"(q[j].w) : "l"(wr + v));
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t v = v0 + 32 * j;
        if (v >= vecs) continue;
        const uint32_t ww[4] = {q[j].x, q[j].y, q[j].z, q[j].w};
        const float4 xa = *reinterpret_cast<const float4*>(xs + v * 8), xb = *reinterpret_cast<const float4*>(xs + v * 8 + 4);
        const float xv[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          acc = fmaf(xv[2 * i], __uint_as_float(ww[i] << 16), acc);
          acc = fmaf(xv[2 * i + 1], __uint_as_float(ww[i] & 0xFFFF0000u), acc);
        }
      }
    }
    acc = warp_sum(acc);
    if (lane == 0) y[row] = bf16_round(acc);
  }
}

}  // namespace
}  // namespace gemb

using namespace gemb;

extern "C" {

int32_t gemb_gelu_tanh_product_f32(const float* gate, const float* up, float* output, uint64_t elements, gemb_stream_t stream) {
  const char* op = "gemb_gelu_tanh_product_f32";
  GEMB_REQUIRE(gate && up && output, "%s: pointers must be nonnull", op);
  GEMB_REQUIRE(elements > 0 && elements < (1ull << 40), "%s: extent must be nonzero", op);
  GEMB_ENTER(op);
  gelu_tanh_product_kernel<<<static_cast<unsigned>((elements + 255) / 256), 256, 0, stream>>>(gate, up, output, elements);
  return check_launch(op);
}

int32_t gemb_add_residual_f32(const float* values, const float* residual, float* output, uint64_t elements, gemb_stream_t stream) {
  const char* op = "gemb_add_residual_f32";
  GEMB_REQUIRE(values && residual && output, "%s: pointers must be nonnull", op);
  GEMB_REQUIRE(elements > 0 && elements < (1ull << 40), "%s: extent must be nonzero", op);
  GEMB_ENTER(op);
  add_residual_kernel<<<static_cast<unsigned>((elements + 255) / 256), 256, 0, stream>>>(values, residual, output, elements);
  return check_launch(op);
}

int32_t gemb_logit_argmax(const float* logits, const uint32_t* suppressed, uint64_t suppressed_count, uint32_t* selected,
                          uint64_t vocabulary, gemb_stream_t stream) {
  const char* op = "gemb_logit_argmax";
  GEMB_REQUIRE(logits && selected, "%s: pointers must be nonnull", op);
  GEMB_REQUIRE(suppressed_count == 0 || suppressed != nullptr, "%s: a nonempty suppression list needs a pointer", op);
  GEMB_REQUIRE(suppressed_count < 4096 && vocabulary > 0 && vocabulary < (1ull << 31), "%s: bad geometry", op);
  GEMB_ENTER(op);
  logit_argmax_kernel<<<1, 1024, 0, stream>>>(logits, suppressed, static_cast<uint32_t>(suppressed_count),
                                             static_cast<uint32_t>(vocabulary), selected);
  return check_launch(op);
}

int32_t gemb_bf16_gemv(const float* input, const uint16_t* weight_bf16, float* output, uint64_t rows,
                       uint64_t contracting_elements, gemb_stream_t stream) {
  const char* op = "gemb_bf16_gemv";
  GEMB_REQUIRE(input && weight_bf16 && output, "%s: pointers must be nonnull", op);
  GEMB_REQUIRE(rows > 0 && rows < (1ull << 31), "%s: bad row count", op);
  GEMB_REQUIRE(contracting_elements > 0 && contracting_elements % 8 == 0 && contracting_elements <= 48 * 1024 / 4,
               "%s: the contracting extent must be a nonzero multiple of 8, at most 12,288", op);
  GEMB_REQUIRE(reinterpret_cast<uintptr_t>(weight_bf16) % 16 == 0, "%s: weights must be 16-byte aligned", op);
  GEMB_ENTER(op);
  const uint64_t ctas = std::min<uint64_t>((rows + 7) / 8, static_cast<uint64_t>(sm_count()) * 8);
  bf16_gemv_kernel<<<static_cast<unsigned>(ctas), kBgThreads, contracting_elements * 4, stream>>>(
      input, weight_bf16, output, static_cast<uint32_t>(rows), static_cast<uint32_t>(contracting_elements));
  return check_launch(op);
}

}  // extern "C"
