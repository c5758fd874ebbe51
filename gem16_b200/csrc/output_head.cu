// Tied bf16 output head of the decode step: logits = softcap(W_bf16 . h), fused with the
// suppression list and the first stage of the arg-max, then a second small launch that reduces the
// per-block candidates.  One token reads the whole 262,144 x 3,840 bf16 matrix (2.0 GB): the kernel
// is an HBM stream, organised like the decode GEMVs (warp per vocabulary row, 16-byte loads, all of
// a row's loads in flight before the first fma, activations staged once per CTA in shared memory).
//
// Contract of src/cuda/output_head.cu:55-110,337-414 of the reference: per vocabulary row the fp32 dot
// product of the bf16 weights with the fp32 hidden vector, soft cap tanhf(sum / 30) * 30, rows on
// the suppression list never win, ties go to the lower token id; the launch writes one candidate per
// block (4,096 of them per hidden row, like the reference) and, if asked, every capped logit.  Up
// to kMaxRows hidden rows (the reference's speculative-decoding verifier uses up to five) share
// one pass over the weights.  The order in which a row's partial sums are added differs from the
// reference's, as it does between the reference's own kernels; values agree to fp32 rounding.
#include <cfloat>

#include "common.cuh"

namespace gemb {
namespace {

constexpr int kOhThreads = 256, kOhWarps = kOhThreads / 32;
constexpr int kOhBlocks = 4096;   // candidates per hidden row, as kOutputHeadCandidateBlocks
constexpr int kOhMaxRows = 8;

struct Candidate {
  float value;
  uint32_t token;
};

__device__ __forceinline__ bool better(float v, uint32_t t, const Candidate& c) {
  return v > c.value || (v == c.value && t < c.token);
}

__device__ __forceinline__ bool is_suppressed(uint32_t token, const uint32_t* __restrict__ list, uint32_t n) {
  for (uint32_t i = 0; i < n; ++i)
    if (__ldg(list + i) == token) return true;
  return false;
}

// kRows hidden vectors share one pass over the weights.  A warp takes kTok vocabulary rows at a time
// (kTok * kU 16-byte loads per lane in flight before any arithmetic) so that each shared-memory read
// of the activations serves kTok weight rows: with five hidden rows and one weight row at a time the
// kernel is bound by shared-memory bandwidth, not by HBM.
template <int kRows>
__global__ void __launch_bounds__(kOhThreads)
output_head_kernel(const uint16_t* __restrict__ weights, const float* __restrict__ hidden_rows,
                   const uint32_t* __restrict__ suppressed, uint32_t suppressed_count,
                   const uint32_t* __restrict__ dynamic_suppressed_count, Candidate* __restrict__ candidates,
                   float* __restrict__ logits_out, uint32_t vocab, uint32_t hidden) {
  constexpr int kTok = kRows >= 3 ? 4 : kRows;   // weight rows per warp iteration
  constexpr int kU = 8 / kTok;                   // 16-byte pieces per lane, weight row and pass
  // Activations as float4 [kRows][2][hidden / 8]: piece p of a weight row (8 bf16) meets elements
  // 8p .. 8p+3 in half 0 and 8p+4 .. 8p+7 in half 1, so consecutive lanes read consecutive 16 bytes.
  extern __shared__ __align__(16) float4 hs[];
  __shared__ Candidate warp_best[kRows][kOhWarps];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t pieces = hidden / 8;   // 16-byte pieces per weight row
  for (uint32_t i = threadIdx.x; i < kRows * hidden / 4; i += kOhThreads) {
    const uint32_t r = i / (hidden / 4), q = i % (hidden / 4);
    hs[(r * 2 + (q & 1)) * pieces + (q >> 1)] = __ldg(reinterpret_cast<const float4*>(hidden_rows) + i);
  }
  __syncthreads();
  const uint32_t n_sup = dynamic_suppressed_count != nullptr ? __ldg(dynamic_suppressed_count) : suppressed_count;
  Candidate best[kRows];
#pragma unroll
  for (int r = 0; r < kRows; ++r) best[r] = {-FLT_MAX, 0u};
  // Same assignment of vocabulary rows to warps as the reference (row = block * 8 + warp, then
  // steps of gridDim * 8), taken kTok steps at a time.
  const uint32_t stride = gridDim.x * kOhWarps;
  for (uint32_t token0 = blockIdx.x * kOhWarps + warp; token0 < vocab; token0 += stride * kTok) {
    const uint4* wrow[kTok];
    bool live[kTok];
#pragma unroll
    for (int j = 0; j < kTok; ++j) {
      const uint64_t token = static_cast<uint64_t>(token0) + static_cast<uint64_t>(j) * stride;
      live[j] = token < vocab;
      wrow[j] = reinterpret_cast<const uint4*>(weights + (live[j] ? token : token0) * hidden);
    }
    float sum[kTok][kRows];
#pragma unroll
    for (int j = 0; j < kTok; ++j)
#pragma unroll
      for (int r = 0; r < kRows; ++r) sum[j][r] = 0.0f;
    for (uint32_t p0 = 0; p0 < pieces; p0 += 32 * kU) {
      uint4 wv[kTok][kU];
#pragma unroll
      for (int j = 0; j < kTok; ++j)
#pragma unroll
        for (int u = 0; u < kU; ++u) {
          const uint32_t p = p0 + u * 32 + lane;
          wv[j][u] = (p < pieces && live[j]) ? __ldcs(wrow[j] + p) : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        const uint32_t p = p0 + u * 32 + lane;
        if (p >= pieces) continue;
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
          const float4 ha = hs[(r * 2) * pieces + p];
          const float4 hb = hs[(r * 2 + 1) * pieces + p];
#pragma unroll
          for (int j = 0; j < kTok; ++j) {
            const uint32_t ww[4] = {wv[j][u].x, wv[j][u].y, wv[j][u].z, wv[j][u].w};
            float a = sum[j][r];
            a = fmaf(__uint_as_float(ww[0] << 16), ha.x, a);
            a = fmaf(__uint_as_float(ww[0] & 0xFFFF0000u), ha.y, a);
            a = fmaf(__uint_as_float(ww[1] << 16), ha.z, a);
            a = fmaf(__uint_as_float(ww[1] & 0xFFFF0000u), ha.w, a);
            a = fmaf(__uint_as_float(ww[2] << 16), hb.x, a);
            a = fmaf(__uint_as_float(ww[2] & 0xFFFF0000u), hb.y, a);
            a = fmaf(__uint_as_float(ww[3] << 16), hb.z, a);
            a = fmaf(__uint_as_float(ww[3] & 0xFFFF0000u), hb.w, a);
            sum[j][r] = a;
          }
        }
      }
    }
#pragma unroll
    for (int j = 0; j < kTok; ++j)
#pragma unroll
      for (int r = 0; r < kRows; ++r) {
#pragma unroll
        for (int off = 16; off != 0; off >>= 1) sum[j][r] += __shfl_xor_sync(0xFFFFFFFFu, sum[j][r], off);
      }
    if (lane == 0) {
#pragma unroll
      for (int j = 0; j < kTok; ++j) {
        if (!live[j]) continue;
        const uint32_t token = token0 + j * stride;
        const bool allowed = !is_suppressed(token, suppressed, n_sup);
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
          const float capped = tanhf(sum[j][r] / 30.0f) * 30.0f;   // src/cuda/output_head.cu:53,88
          if (logits_out != nullptr) logits_out[static_cast<uint64_t>(r) * vocab + token] = capped;
          if (allowed && better(capped, token, best[r])) best[r] = {capped, token};
        }
      }
    }
  }
  if (lane == 0) {
#pragma unroll
    for (int r = 0; r < kRows; ++r) warp_best[r][warp] = best[r];
  }
  __syncthreads();
  if (warp == 0) {
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
      Candidate c = lane < kOhWarps ? warp_best[r][lane] : Candidate{-FLT_MAX, 0u};
#pragma unroll
      for (int off = 16; off != 0; off >>= 1) {
        const float ov = __shfl_down_sync(0xFFFFFFFFu, c.value, off);
        const uint32_t ot = __shfl_down_sync(0xFFFFFFFFu, c.token, off);
        if (better(ov, ot, c)) c = {ov, ot};
      }
      if (lane == 0 && candidates != nullptr) candidates[static_cast<uint64_t>(r) * kOhBlocks + blockIdx.x] = c;
    }
  }
}

// One CTA per hidden row: best of its 4,096 candidates.
__global__ void __launch_bounds__(kOhThreads)
output_head_argmax_kernel(const Candidate* __restrict__ candidates, uint32_t* __restrict__ selected) {
  __shared__ Candidate scratch[kOhWarps];
  const Candidate* row = candidates + static_cast<uint64_t>(blockIdx.x) * kOhBlocks;
  Candidate c{-FLT_MAX, 0u};
  for (uint32_t i = threadIdx.x; i < kOhBlocks; i += kOhThreads) {
    const Candidate o = row[i];
    if (better(o.value, o.token, c)) c = o;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
  for (int off = 16; off != 0; off >>= 1) {
    const float ov = __shfl_down_sync(0xFFFFFFFFu, c.value, off);
    const uint32_t ot = __shfl_down_sync(0xFFFFFFFFu, c.token, off);
    if (better(ov, ot, c)) c = {ov, ot};
  }
  if (lane == 0) scratch[warp] = c;
  __syncthreads();
  if (warp == 0) {
    c = lane < kOhWarps ? scratch[lane] : Candidate{-FLT_MAX, 0u};
#pragma unroll
    for (int off = 16; off != 0; off >>= 1) {
      const float ov = __shfl_down_sync(0xFFFFFFFFu, c.value, off);
      const uint32_t ot = __shfl_down_sync(0xFFFFFFFFu, c.token, off);
      if (better(ov, ot, c)) c = {ov, ot};
    }
    if (lane == 0) selected[blockIdx.x] = c.token;
  }
}

template <int kRows>
int32_t launch_output_head(const char* op, const uint16_t* weights, const float* hidden_rows, const uint32_t* suppressed,
                           uint32_t suppressed_count, const uint32_t* dynamic_count, Candidate* candidates,
                           float* logits, uint32_t vocab, uint32_t hidden, cudaStream_t stream) {
  const size_t smem = static_cast<size_t>(kRows) * hidden * sizeof(float);
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  dev &= 63;
  if (!configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(output_head_kernel<kRows>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return fail(GEMB_INTERNAL, "%s: %s: %s", op, cudaGetErrorName(e), cudaGetErrorString(e));
    configured[dev] = true;
  }
  output_head_kernel<kRows><<<kOhBlocks, kOhThreads, smem, stream>>>(weights, hidden_rows, suppressed, suppressed_count,
                                                                    dynamic_count, candidates, logits, vocab, hidden);
  return check_launch(op);
}

}  // namespace
}  // namespace gemb

using namespace gemb;

extern "C" {

uint64_t gemb_output_head_candidate_blocks(void) { return kOhBlocks; }

int32_t gemb_output_head_candidates(const uint16_t* weights_bf16, const float* hidden_rows, uint64_t rows,
                                    const uint32_t* suppressed, uint64_t suppressed_count,
                                    const uint32_t* dynamic_suppressed_count, void* candidates,
                                    float* diagnostic_logits, uint64_t vocabulary, uint64_t hidden,
                                    gemb_stream_t stream) {
  const char* op = "gemb_output_head_candidates";
  GEMB_REQUIRE(weights_bf16 && hidden_rows && (candidates || diagnostic_logits),
               "%s: weights, hidden rows and at least one of candidates / logits must be nonnull", op);
  GEMB_REQUIRE(rows >= 1 && rows <= kOhMaxRows, "%s: between 1 and %d hidden rows", op, kOhMaxRows);
  GEMB_REQUIRE(suppressed_count == 0 || suppressed != nullptr, "%s: a nonempty suppression list needs a pointer", op);
  GEMB_REQUIRE(suppressed_count < (1ull << 20), "%s: suppression list too long", op);
  GEMB_REQUIRE(vocabulary > 0 && vocabulary < (1ull << 31), "%s: bad vocabulary size", op);
  GEMB_REQUIRE(hidden > 0 && hidden % 8 == 0 && rows * hidden * 4 <= 200 * 1024,
               "%s: hidden must be a nonzero multiple of 8 and rows * hidden * 4 bytes must fit 200 KB of shared memory", op);
  GEMB_REQUIRE(reinterpret_cast<uintptr_t>(weights_bf16) % 16 == 0 && reinterpret_cast<uintptr_t>(hidden_rows) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(candidates) % 8 == 0,
               "%s: weights and hidden must be 16-byte, candidates 8-byte aligned", op);
  GEMB_ENTER(op);
  Candidate* c = static_cast<Candidate*>(candidates);
  const uint32_t sc = static_cast<uint32_t>(suppressed_count), v = static_cast<uint32_t>(vocabulary),
                 h = static_cast<uint32_t>(hidden);
  switch (rows) {
    case 1: return launch_output_head<1>(op, weights_bf16, hidden_rows, suppressed, sc, dynamic_suppressed_count, c, diagnostic_logits, v, h, stream);
    case 2: return launch_output_head<2>(op, weights_bf16, hidden_rows, suppressed, sc, dynamic_suppressed_count, c, diagnostic_logits, v, h, stream);
    case 3: return launch_output_head<3>(op, weights_bf16, hidden_rows, suppressed, sc, dynamic_suppressed_count, c, diagnostic_logits, v, h, stream);
    case 4: return launch_output_head<4>(op, weights_bf16, hidden_rows, suppressed, sc, dynamic_suppressed_count, c, diagnostic_logits, v, h, stream);
    case 5: return launch_output_head<5>(op, weights_bf16, hidden_rows, suppressed, sc, dynamic_suppressed_count, c, diagnostic_logits, v, h, stream);
    case 6: return launch_output_head<6>(op, weights_bf16, hidden_rows, suppressed, sc, dynamic_suppressed_count, c, diagnostic_logits, v, h, stream);
    case 7: return launch_output_head<7>(op, weights_bf16, hidden_rows, suppressed, sc, dynamic_suppressed_count, c, diagnostic_logits, v, h, stream);
    default: return launch_output_head<8>(op, weights_bf16, hidden_rows, suppressed, sc, dynamic_suppressed_count, c, diagnostic_logits, v, h, stream);
  }
}

int32_t gemb_output_head_argmax(const void* candidates, uint64_t rows, uint32_t* selected, gemb_stream_t stream) {
  const char* op = "gemb_output_head_argmax";
  GEMB_REQUIRE(candidates && selected, "%s: pointers must be nonnull", op);
  GEMB_REQUIRE(rows >= 1 && rows <= kOhMaxRows, "%s: between 1 and %d rows", op, kOhMaxRows);
  GEMB_ENTER(op);
  output_head_argmax_kernel<<<static_cast<unsigned>(rows), kOhThreads, 0, stream>>>(static_cast<const Candidate*>(candidates), selected);
  return check_launch(op);
}

}  // extern "C"
