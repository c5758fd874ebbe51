// Mixture-of-experts routing path: router logits, softmax / top-k / renormalise, histogram +
// exclusive prefix + stable permutation of the (token, slot) assignments, quantise-and-dispatch
// of expert inputs into the padded per-expert row layout the grouped GEMM consumes, and the
// deterministic weighted combine.
//
// gem16 holds no MoE code; these kernels implement the record layouts and ordering rules of
// docs/plans/gemma4-26b/specs/MOE_ROUTER_SPEC.md and MOE_PREFILL_KERNEL_SPEC.md.  Everything
// that decides routing is computed with a fixed operation order out of IEEE add / mul / fma /
// div only, so expert ids, weights, counts and the permutation are reproducible bit for bit.
#include <algorithm>
#include <atomic>

#include "common.cuh"

namespace gemb {

// Set by the routing kernels when they meet a state the router specification calls impossible
// (MOE_ROUTER_SPEC.md:117-130): 1 = a non-finite router logit, 2 = an expert id outside
// [0, experts) reached the permutation.  The offending access is skipped or replaced by an
// in-range value, never dereferenced; gemb_check_device_status() reports and clears the word.
__device__ int g_moe_error = 0;

// Benchmark hook (GEMB_TUNE_ROUTER_TILE): 0 = automatic, 1 = expert-per-thread kernels wherever they
// apply, 8 / 16 / 32 = the tiled kernel with that many tokens per CTA.  All give the same bits.
int g_router_tile = 0;

int moe_take_device_error() {
  int code = 0;
  if (cudaMemcpyFromSymbol(&code, g_moe_error, sizeof code) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  if (code != 0) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_moe_error, &zero, sizeof zero);
  }
  return code;
}

namespace {

// ---------------------------------------------------------------------------------------------
// Router logits: logits[t][e] = fma(x[t][H-1], w[e][H-1], ... fma(x[t][0], w[e][0], bias[e])),
// one fp32 fma per k in ascending k (the order is the contract; it rules out tensor cores and
// K-splitting).  CTA = 32 tokens x 128 experts, 128 threads, thread = 8 tokens x 4 experts
// (32 independent fma chains).  K is walked in shared-memory tiles of 32; the next tile's global
// loads are issued into registers before the current tile is consumed.
// ---------------------------------------------------------------------------------------------
constexpr int kRtExp = 128, kRtK = 32, kRtThreads = 128;

// kTok = tokens per CTA (64, 56 or 32 for prefill batches -- 64 halves the weight reads from shared memory per
// fma, at 64 accumulators per thread; 56 is the same with 14 tokens per thread, for batches that 64-token
// CTAs would spread unevenly over the SMs -- 8 for decode batches so that a few dozen tokens
// still spread over many SMs).  Shared tiles are stored k-major with an xor swizzle of the column
// (multiples of 4 / 8 keep each thread's float4 groups intact) so that both the transposing
// stores and the float4 loads are bank-conflict free.
template <int kTok>
__global__ void __launch_bounds__(kRtThreads, kTok >= 56 ? 3 : 4)
router_logits_kernel(const uint16_t* __restrict__ x, const float* __restrict__ w,
                     const float* __restrict__ bias, float* __restrict__ logits, uint32_t tokens,
                     uint32_t hidden, uint32_t experts) {
  constexpr int kPerThread = kTok / 4;  // tokens per thread: 16, 14, 8, 4 or 2
  // A warp's tokens occupy a slot of kSlot columns of the shared tile (kSlot = kPerThread rounded up to a
  // multiple of four, so that the float4 reads stay aligned: 16 columns for the 14 tokens of the 56-token tile).
  constexpr int kSlot = kPerThread >= 4 ? (kPerThread + 3) / 4 * 4 : kPerThread;
  constexpr int kXCols = 4 * kSlot > 32 ? 4 * kSlot : 32;
  constexpr int kXLoads = kTok > 32 ? (kTok + 31) / 32 : 1;   // staged 16-byte pieces of the token tile per thread
  __shared__ __align__(16) float xs[kRtK][kXCols];
  __shared__ __align__(16) float ws[kRtK][kRtExp];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // experts tx*4.., tokens ty*kPerThread..
  const uint32_t tok0 = blockIdx.x * kTok, exp0 = blockIdx.y * kRtExp;
  float acc[kPerThread][4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint32_t e = exp0 + tx * 4 + j;
    const float b = (bias != nullptr && e < experts) ? __ldg(bias + e) : 0.0f;
#pragma unroll
    for (int i = 0; i < kPerThread; ++i) acc[i][j] = b;
  }
  // Global -> register staging: X tile kTok tokens x 32 k bf16 = one uint4 per thread (token
  // tid/4, k chunk (tid%4)*8); W tile 128 experts x 32 k fp32 = eight float4 per thread
  // (expert tid/8 + 16 i, k chunk (tid%8)*4).
  const int xt = threadIdx.x >> 2, xq = threadIdx.x & 3, xk = xq * 8;
  const int we = threadIdx.x >> 3, wm = threadIdx.x & 7, wk = wm * 4;
  uint4 xr[kXLoads];
  float4 wr[8];
  auto load_tile = [&](uint32_t k0) {
#pragma unroll
    for (int l = 0; l < kXLoads; ++l) {
      xr[l] = make_uint4(0, 0, 0, 0);
      const int tk = xt + 32 * l;   // token of the tile
      if (tk < kTok && tok0 + tk < tokens) {
        const uint16_t* src = x + static_cast<uint64_t>(tok0 + tk) * hidden + k0 + xk;
        if (k0 + xk + 8 <= hidden) {
          if ((reinterpret_cast<uintptr_t>(src) & 15) == 0) {
            xr[l] = __ldg(reinterpret_cast<const uint4*>(src));
          } else {
            const uint2 a = __ldg(reinterpret_cast<const uint2*>(src)), b2 = __ldg(reinterpret_cast<const uint2*>(src) + 1);
            xr[l] = make_uint4(a.x, a.y, b2.x, b2.y);
          }
        } else if (k0 + xk + 4 <= hidden) {
          const uint2 a = __ldg(reinterpret_cast<const uint2*>(src));
          xr[l] = make_uint4(a.x, a.y, 0, 0);
        }
      }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      wr[i] = make_float4(0.f, 0.f, 0.f, 0.f);
      const uint32_t e = exp0 + we + 16 * i;
      if (e < experts && k0 + wk < hidden)
        wr[i] = __ldg(reinterpret_cast<const float4*>(w + static_cast<uint64_t>(e) * hidden + k0 + wk));
    }
  };
  auto store_tile = [&]() {
#pragma unroll
    for (int l = 0; l < kXLoads; ++l) {
      const uint32_t xw[4] = {xr[l].x, xr[l].y, xr[l].z, xr[l].w};
      const int tk = xt + 32 * l;
      if (tk >= kTok) continue;
      const int xcol = ((tk / kPerThread) * kSlot + tk % kPerThread) ^ (8 * xq);  // rows xk..xk+7 all have (k / 8) & 3 == xq
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        xs[xk + 2 * i][xcol] = __uint_as_float(xw[i] << 16);
        xs[xk + 2 * i + 1][xcol] = __uint_as_float(xw[i] & 0xFFFF0000u);
      }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int col = (we + 16 * i) ^ (4 * wm);  // rows wk..wk+3 all have k / 4 == wm
      ws[wk + 0][col] = wr[i].x;
      ws[wk + 1][col] = wr[i].y;
      ws[wk + 2][col] = wr[i].z;
      ws[wk + 3][col] = wr[i].w;
    }
  };
  load_tile(0);
  for (uint32_t k0 = 0; k0 < hidden; k0 += kRtK) {
    store_tile();
    __syncthreads();
    if (k0 + kRtK < hidden) load_tile(k0 + kRtK);
    const uint32_t kmax = min(static_cast<uint32_t>(kRtK), hidden - k0);
    // One k: four weights, kPerThread activations, kPerThread x 4 fma.  With four or eight tokens per
    // thread two tokens share an instruction: the packed fp32 fma is one IEEE fma per half, so every
    // chain keeps its order and rounding while the issue slots carry half the instructions.
    auto step = [&](uint32_t k) {
      const float4 wv4 = *reinterpret_cast<const float4*>(&ws[k][(tx * 4) ^ (4 * (k >> 2))]);
      const float wv[4] = {wv4.x, wv4.y, wv4.z, wv4.w};
      const int col = (ty * kPerThread) ^ (8 * ((k >> 3) & 3));
      if constexpr (kPerThread >= 4) {
        float2 xp[kPerThread / 2];
#pragma unroll
        for (int q = 0; q < kSlot / 4; ++q) {   // the swizzle moves groups of eight columns: a group of four stays whole
          const float4 xa = *reinterpret_cast<const float4*>(&xs[k][(ty * kSlot + 4 * q) ^ (8 * ((k >> 3) & 3))]);
          xp[2 * q] = make_float2(xa.x, xa.y);
          if (2 * q + 1 < kPerThread / 2) xp[2 * q + 1] = make_float2(xa.z, xa.w);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 wp = make_float2(wv[j], wv[j]);
#pragma unroll
          for (int i = 0; i < kPerThread / 2; ++i) {
            const float2 r = __ffma2_rn(xp[i], wp, make_float2(acc[2 * i][j], acc[2 * i + 1][j]));
            acc[2 * i][j] = r.x;
            acc[2 * i + 1][j] = r.y;
          }
        }
      } else {
        const float2 xa = *reinterpret_cast<const float2*>(&xs[k][col]);
        const float xv[2] = {xa.x, xa.y};
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(xv[i], wv[j], acc[i][j]);
      }
    };
    if (kmax == kRtK) {
#pragma unroll
      for (uint32_t k = 0; k < kRtK; ++k) step(k);
    } else {
#pragma unroll 4
      for (uint32_t k = 0; k < kmax; ++k) step(k);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < kPerThread; ++i) {
    const uint32_t t = tok0 + ty * kPerThread + i;
    if (t >= tokens) continue;
    float* dst = logits + static_cast<uint64_t>(t) * experts + exp0 + tx * 4;
    if (exp0 + tx * 4 + 4 <= experts && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
      *reinterpret_cast<float4*>(dst) = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (exp0 + tx * 4 + j < experts) dst[j] = acc[i][j];
    }
  }
}

// Decode-size and small-batch form of the same contract.  With few tokens the tile above leaves
// most SMs idle (one CTA per 8 or 32 tokens, each walking all of K).  Here a thread owns ONE
// expert and kTpt tokens (kTpt independent fma chains), a warp 32 experts, a CTA of two warps
// 2 * kTpt tokens of the same 32 experts.  K is walked in tiles of 128.  The chain over k is
// serial, so a tile's arithmetic (about 600 clocks) is all there is to hide a load behind, and
// an L2 round trip takes longer than that: the CTA's weight tiles (32 experts x 128 k, fetched
// as coalesced 16-byte cp.async pieces) and the tokens' raw bf16 activations therefore run
// through a ring of kRsDepth shared-memory buffers, three tiles ahead of the arithmetic.  Same
// chain, same order: bias, then one fma per k ascending.
constexpr int kRsK = 128, kRsThreads = 64, kRsPad = 4, kRsDepth = 4;

__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* src, bool valid) {
  const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst));
  const uint32_t n = valid ? 16u : 0u;   // 0 source bytes: the destination is zero filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_8(void* smem_dst, const void* src, bool valid) {
  const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst));
  const uint32_t n = valid ? 8u : 0u;
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;" ::"r"(d), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int kPending>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(kPending) : "memory"); }

template <int kTpt>
struct RouterSmallSmem {
  static constexpr int kTokCta = 2 * kTpt;
  float ws[kRsDepth][32][kRsK + kRsPad];     // row stride 132 words: float4 reads of one k by 32 rows are conflict free
  uint16_t xraw[kRsDepth][kTokCta][kRsK];    // bf16 as loaded
  float xs[kTokCta][kRsK];                   // the current tile's activations as fp32
};

template <int kTpt>
__global__ void __launch_bounds__(kRsThreads)
router_logits_small_kernel(const uint16_t* __restrict__ x, const float* __restrict__ w,
                           const float* __restrict__ bias, float* __restrict__ logits, uint32_t tokens,
                           uint32_t hidden, uint32_t experts) {
  constexpr int kTokCta = 2 * kTpt;
  extern __shared__ __align__(16) uint8_t router_small_smem[];
  auto& sm = *reinterpret_cast<RouterSmallSmem<kTpt>*>(router_small_smem);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t tok0 = blockIdx.x * kTokCta, exp0 = blockIdx.y * 32;
  const uint32_t e = exp0 + lane;
  const bool live = e < experts;
  float acc[kTpt];
  const float b = (bias != nullptr && live) ? __ldg(bias + e) : 0.0f;
#pragma unroll
  for (int i = 0; i < kTpt; ++i) acc[i] = b;
  const uint32_t tiles = (hidden + kRsK - 1) / kRsK;
  // Warp `warp` fetches rows warp*16 .. warp*16+15 of the weight tile (lane = 16-byte piece of the
  // row); the activation tile is kTokCta rows of 32 eight-byte pieces shared out over the CTA.
  auto issue_tile = [&](uint32_t t) {
    if (t < tiles) {
      const uint32_t k0 = t * kRsK, buf = t % kRsDepth;
      const uint32_t kmax = min(static_cast<uint32_t>(kRsK), hidden - k0);   // a multiple of 4
#pragma unroll
      for (int r = 0; r < 16; ++r) {
        const uint32_t row = exp0 + warp * 16 + r;
        const bool ok = row < experts && static_cast<uint32_t>(lane) * 4 < kmax;
        const float* src = w + static_cast<uint64_t>(ok ? row : 0) * hidden + (ok ? k0 + lane * 4 : 0);
        cp_async_16(&sm.ws[buf][warp * 16 + r][lane * 4], src, ok);
      }
#pragma unroll
      for (int q = 0; q < kTokCta * 32 / kRsThreads; ++q) {
        const uint32_t idx = threadIdx.x + q * kRsThreads;
        const uint32_t tk = idx / 32, c = (idx % 32) * 4;
        const bool ok = tok0 + tk < tokens && c < kmax;
        const uint16_t* src = x + static_cast<uint64_t>(ok ? tok0 + tk : 0) * hidden + (ok ? k0 + c : 0);
        cp_async_8(&sm.xraw[buf][tk][c], src, ok);
      }
    }
    cp_async_commit();   // one group per call, empty past the last tile, so the counting stays uniform
  };
#pragma unroll
  for (int t = 0; t < kRsDepth - 1; ++t) issue_tile(t);
  for (uint32_t t = 0; t < tiles; ++t) {
    const uint32_t buf = t % kRsDepth;
    const uint32_t groups = min(static_cast<uint32_t>(kRsK), hidden - t * kRsK) / 4;
    cp_async_wait<kRsDepth - 2>();   // this thread's pieces of tile t have landed
    __syncthreads();                 // everyone's have; and tile t-1 has been consumed
    issue_tile(t + kRsDepth - 1);    // refills the buffer tile t-1 used
    for (uint32_t idx = threadIdx.x; idx < kTokCta * (kRsK / 4); idx += kRsThreads) {
      const uint32_t tk = idx / (kRsK / 4), c = (idx % (kRsK / 4)) * 4;
      const uint2 raw = *reinterpret_cast<const uint2*>(&sm.xraw[buf][tk][c]);
      *reinterpret_cast<float4*>(&sm.xs[tk][c]) =
          make_float4(__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xFFFF0000u),
                      __uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xFFFF0000u));
    }
    __syncthreads();
#pragma unroll 8
    for (uint32_t g = 0; g < groups; ++g) {
      const float4 wv = *reinterpret_cast<const float4*>(&sm.ws[buf][lane][g * 4]);
      float4 xv[kTpt];
#pragma unroll
      for (int i = 0; i < kTpt; ++i) xv[i] = *reinterpret_cast<const float4*>(&sm.xs[warp * kTpt + i][g * 4]);
      // k-major: the kTpt chains advance together, so consecutive instructions are independent
      // (a chain's own steps are four clocks apart at best).
#pragma unroll
      for (int i = 0; i < kTpt; ++i) acc[i] = fmaf(xv[i].x, wv.x, acc[i]);
#pragma unroll
      for (int i = 0; i < kTpt; ++i) acc[i] = fmaf(xv[i].y, wv.y, acc[i]);
#pragma unroll
      for (int i = 0; i < kTpt; ++i) acc[i] = fmaf(xv[i].z, wv.z, acc[i]);
#pragma unroll
      for (int i = 0; i < kTpt; ++i) acc[i] = fmaf(xv[i].w, wv.w, acc[i]);
    }
  }
  cp_async_wait<0>();
  if (!live) return;
#pragma unroll
  for (int i = 0; i < kTpt; ++i) {
    const uint32_t t = tok0 + warp * kTpt + i;
    if (t < tokens) logits[static_cast<uint64_t>(t) * experts + e] = acc[i];
  }
}

// ---------------------------------------------------------------------------------------------
// Softmax over all experts, top-k with the lower id winning ties, renormalise, optional
// per-expert scale (MOE_ROUTER_SPEC.md:27-63).  One warp per token; lane l owns experts
// l, l+32, ...  Reduction orders are part of the contract:
//   max / sum: lane-local over the owned experts in ascending order, then an xor butterfly with
//   strides 16, 8, 4, 2, 1; exp is the fma polynomial below; p = exp / sum; the selected sum
//   adds the k probabilities in slot order; weight = p / selected_sum (* per_expert_scale).
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float det_exp(float x) {
  if (x < -87.0f) return 0.0f;
  const float nf = rintf(__fmul_rn(x, 1.4426950408889634f));
  float r = fmaf(nf, -0.693145751953125f, x);
  r = fmaf(nf, -1.428606765330187e-06f, r);
  float p = 1.9875691500e-4f;
  p = fmaf(p, r, 1.3981999507e-3f);
  p = fmaf(p, r, 8.3334519073e-3f);
  p = fmaf(p, r, 4.1665795894e-2f);
  p = fmaf(p, r, 1.6666665459e-1f);
  p = fmaf(p, r, 5.0000001201e-1f);
  const float r2 = __fmul_rn(r, r);
  const float y = __fadd_rn(fmaf(p, r2, r), 1.0f);
  const float scale = __uint_as_float(static_cast<uint32_t>(static_cast<int>(nf) + 127) << 23);
  return __fmul_rn(y, scale);
}

constexpr int kMaxPerLane = 8;  // up to 256 experts

__global__ void __launch_bounds__(128)
route_kernel(const float* __restrict__ logits, const float* __restrict__ per_expert_scale,
             int32_t* __restrict__ ids, float* __restrict__ weights, float* __restrict__ probs,
             uint32_t tokens, uint32_t experts, uint32_t topk) {
  const uint32_t t = blockIdx.x * 4 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (t >= tokens) return;
  const int per_lane = static_cast<int>(experts / 32);
  const float* lg = logits + static_cast<uint64_t>(t) * experts;
  float p[kMaxPerLane];
  float m = __ldg(lg + lane);
  p[0] = m;
  bool finite = isfinite(m);
#pragma unroll
  for (int j = 1; j < kMaxPerLane; ++j) {
    if (j < per_lane) {
      p[j] = __ldg(lg + lane + 32 * j);
      finite = finite && isfinite(p[j]);
      m = fmaxf(m, p[j]);
    }
  }
  if (!__all_sync(0xFFFFFFFFu, finite)) {
    // A NaN or infinite logit makes every probability of the token meaningless.  The state is
    // recorded, and the token still gets in-range ids (its slot numbers) with zero weights so
    // that nothing downstream indexes with garbage.
    if (lane == 0) atomicCAS(&g_moe_error, 0, 1);
    if (static_cast<uint32_t>(lane) < topk) {
      ids[static_cast<uint64_t>(t) * topk + lane] = lane;
      weights[static_cast<uint64_t>(t) * topk + lane] = 0.0f;
    }
    if (probs)
      for (int j = 0; j < per_lane; ++j) probs[static_cast<uint64_t>(t) * experts + lane + 32 * j] = 0.0f;
    return;
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
  float s = 0.0f;
#pragma unroll
  for (int j = 0; j < kMaxPerLane; ++j) {
    if (j < per_lane) {
      p[j] = det_exp(__fsub_rn(p[j], m));
      s = j == 0 ? p[0] : __fadd_rn(s, p[j]);
    }
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) s = __fadd_rn(s, __shfl_xor_sync(0xFFFFFFFFu, s, o));
#pragma unroll
  for (int j = 0; j < kMaxPerLane; ++j) {
    if (j < per_lane) {
      p[j] = __fdiv_rn(p[j], s);
      if (probs) probs[static_cast<uint64_t>(t) * experts + lane + 32 * j] = p[j];
    }
  }
  // k rounds of arg-max.  Taken entries are marked with -1 (probabilities are >= 0).
  float sel_sum = 0.0f, my_w = 0.0f;
  int my_id = 0;
  for (uint32_t slot = 0; slot < topk; ++slot) {
    float best = -1.0f;
    int best_id = 0x7FFFFFFF;
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j) {
      if (j < per_lane && p[j] > best) {  // ascending id, strict '>' keeps the lower id
        best = p[j];
        best_id = lane + 32 * j;
      }
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) {
      const float ob = __shfl_xor_sync(0xFFFFFFFFu, best, o);
      const int oi = __shfl_xor_sync(0xFFFFFFFFu, best_id, o);
      if (ob > best || (ob == best && oi < best_id)) {
        best = ob;
        best_id = oi;
      }
    }
    if ((best_id & 31) == lane) {
#pragma unroll
      for (int j = 0; j < kMaxPerLane; ++j)
        if (j == (best_id >> 5)) p[j] = -1.0f;
    }
    sel_sum = slot == 0 ? best : __fadd_rn(sel_sum, best);
    if (static_cast<uint32_t>(lane) == slot) {
      my_w = best;
      my_id = best_id;
    }
  }
  if (static_cast<uint32_t>(lane) < topk) {
    float wv = __fdiv_rn(my_w, sel_sum);
    if (per_expert_scale) wv = __fmul_rn(wv, __ldg(per_expert_scale + my_id));
    ids[static_cast<uint64_t>(t) * topk + lane] = my_id;
    weights[static_cast<uint64_t>(t) * topk + lane] = wv;
  }
}

// ---------------------------------------------------------------------------------------------
// Histogram, exclusive prefix and stable permutation (MOE_PREFILL_KERNEL_SPEC.md:34-58).
// Assignment i = token * topk + slot.  Inside an expert the order is i ascending (token, then
// slot).  Three launches, no atomics on global memory, no host readback:
//   1. per segment of 1024 assignments: per-expert counts (block_counts[segment][expert]);
//   2. one CTA: exclusive scan over segments per expert, counts, offsets, and the padded plan
//      (every expert's rows start on a multiple of 256, so neither a 128-row GEMM tile nor the
//      256-row tile of a CTA pair ever mixes experts; a 128-row tile that holds padding only is
//      marked -1 and costs the GEMM nothing);
//   3. per segment: stable ranks from warp match masks, scatter perm[] and slot_rows[].
// ---------------------------------------------------------------------------------------------
constexpr int kSegment = 1024;  // assignments per CTA: 4 warps x 8 chunks x 32
constexpr int kRowAlign = 256;  // every expert's padded rows start on a multiple of this

__global__ void __launch_bounds__(128)
permute_count_kernel(const int32_t* __restrict__ ids, int32_t* __restrict__ block_counts,
                     uint32_t total, uint32_t experts) {
  extern __shared__ int smem_counts[];
  for (uint32_t e = threadIdx.x; e < experts; e += 128) smem_counts[e] = 0;
  __syncthreads();
  const uint32_t base = blockIdx.x * kSegment;
  for (uint32_t i = threadIdx.x; i < kSegment; i += 128) {
    if (base + i >= total) continue;
    uint32_t e = static_cast<uint32_t>(__ldg(ids + base + i));
    if (e >= experts) {   // recorded, and counted under the last expert so that every position stays in range
      atomicCAS(&g_moe_error, 0, 2);
      e = experts - 1;
    }
    atomicAdd(&smem_counts[e], 1);
  }
  __syncthreads();
  for (uint32_t e = threadIdx.x; e < experts; e += 128)
    block_counts[static_cast<uint64_t>(blockIdx.x) * experts + e] = smem_counts[e];
}

// plan layout (int32): [0] number T of 128-row tiles, [1] padded rows in total, [2 .. 2+E] padded
// offset of every expert (+ the end), then T pairs {expert of tile i (-1: padding only), i-th tile
// that holds real rows (what a single-CTA grouped GEMM walks)}, then the number of such tiles.
__global__ void __launch_bounds__(256)
permute_scan_kernel(int32_t* __restrict__ block_counts, int32_t* __restrict__ counts,
                    int32_t* __restrict__ offsets, int32_t* __restrict__ plan, uint32_t segments,
                    uint32_t experts, uint32_t max_tiles) {
  extern __shared__ int sm[];
  int* cnt = sm;                 // [experts]
  int* off = sm + experts;       // [experts + 1]
  int* poff = off + experts + 1; // [experts + 1]
  int* loff = poff + experts + 1; // [experts + 1] first entry of the expert in the list of real tiles
  for (uint32_t e = threadIdx.x; e < experts; e += blockDim.x) {
    int run = 0;
    // sixteen loads in flight at a time: a thread that consumes each count before it asks for the
    // next one waits a full memory round trip per segment
    for (uint32_t b0 = 0; b0 < segments; b0 += 16) {
      int c[16];
#pragma unroll
      for (int j = 0; j < 16; ++j)
        c[j] = b0 + j < segments ? block_counts[static_cast<uint64_t>(b0 + j) * experts + e] : 0;
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        if (b0 + j < segments) block_counts[static_cast<uint64_t>(b0 + j) * experts + e] = run;  // exclusive prefix over segments
        run += c[j];
      }
    }
    cnt[e] = run;
    counts[e] = run;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int o = 0, po = 0, lo = 0;
    for (uint32_t e0 = 0; e0 < experts; e0 += 8) {   // eight counts at a time: one add per expert instead of one shared-memory round trip
      int c[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) c[j] = e0 + j < experts ? cnt[e0 + j] : 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (e0 + j >= experts) break;
        off[e0 + j] = o;
        poff[e0 + j] = po;
        loff[e0 + j] = lo;
        o += c[j];
        po += (c[j] + kRowAlign - 1) / kRowAlign * kRowAlign;
        lo += (c[j] + 127) / 128;
      }
    }
    off[experts] = o;
    poff[experts] = po;
    plan[0] = po / 128;
    plan[1] = po;
    plan[3 + experts + 2 * (po / 128)] = lo;
  }
  __syncthreads();
  for (uint32_t e = threadIdx.x; e <= experts; e += blockDim.x) {
    offsets[e] = off[e];
    plan[2 + e] = poff[e];
  }
  int32_t* info = plan + 3 + experts;
  for (uint32_t e = threadIdx.x; e < experts; e += blockDim.x)
    for (int tile = poff[e] / 128, j = 0; tile < poff[e + 1] / 128; ++tile, ++j) {
      const bool real = tile * 128 - poff[e] < cnt[e];
      info[2 * tile] = real ? static_cast<int32_t>(e) : -1;
      if (real) info[2 * (loff[e] + j) + 1] = tile;
    }
}

__global__ void __launch_bounds__(128)
permute_scatter_kernel(const int32_t* __restrict__ ids, const int32_t* __restrict__ block_prefix,
                       const int32_t* __restrict__ offsets, const int32_t* __restrict__ plan,
                       int32_t* __restrict__ perm, int32_t* __restrict__ slot_rows, uint32_t total,
                       uint32_t experts) {
  extern __shared__ int sm[];
  int* warp_counts = sm;  // [4][experts], becomes each warp's running base
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (uint32_t i = threadIdx.x; i < 4 * experts; i += 128) warp_counts[i] = 0;
  __syncthreads();
  const uint32_t base = blockIdx.x * kSegment + warp * 256;
  int my_ids[8];
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    const uint32_t i = base + c * 32 + lane;
    my_ids[c] = i < total ? __ldg(ids + i) : -1;
    if (i < total && static_cast<uint32_t>(my_ids[c]) >= experts)
      my_ids[c] = static_cast<int>(experts) - 1;   // same clamp as the count kernel, which recorded it
    if (my_ids[c] >= 0) atomicAdd(&warp_counts[warp * experts + my_ids[c]], 1);
  }
  __syncthreads();
  // exclusive prefix over the four warps, plus the segment's own prefix
  for (uint32_t e = threadIdx.x; e < experts; e += 128) {
    int run = block_prefix[static_cast<uint64_t>(blockIdx.x) * experts + e];
    for (int wq = 0; wq < 4; ++wq) {
      const int c = warp_counts[wq * experts + e];
      warp_counts[wq * experts + e] = run;
      run += c;
    }
  }
  __syncthreads();
  int* running = warp_counts + warp * experts;
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    const int e = my_ids[c];
    const unsigned active = __ballot_sync(0xFFFFFFFFu, e >= 0);
    if (e >= 0) {
      const unsigned peers = __match_any_sync(active, e);
      const int rank = __popc(peers & ((1u << lane) - 1));
      const int within = running[e] + rank;  // position inside the expert
      const uint32_t i = base + c * 32 + lane;
      perm[__ldg(offsets + e) + within] = static_cast<int32_t>(i);
      slot_rows[i] = __ldg(plan + 2 + e) + within;
      __syncwarp(active);
      if (rank == 0) running[e] += __popc(peers);
    }
    __syncwarp();
  }
}

// The three steps above in ONE launch of one CTA, for batches of at most kSegment assignments (the
// decode-size layer, where three launches cost more than the work): same records, same order.
__global__ void __launch_bounds__(128)
permute_small_kernel(const int32_t* __restrict__ ids, int32_t* __restrict__ counts, int32_t* __restrict__ offsets,
                     int32_t* __restrict__ plan, int32_t* __restrict__ perm, int32_t* __restrict__ slot_rows,
                     uint32_t total, uint32_t experts, uint32_t max_tiles) {
  extern __shared__ int sm[];
  int* cnt = sm;                        // [experts]
  int* off = cnt + experts;             // [experts + 1]
  int* poff = off + experts + 1;        // [experts + 1]
  int* loff = poff + experts + 1;       // [experts + 1]
  int* warp_counts = loff + experts + 1;  // [4][experts]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (uint32_t i = threadIdx.x; i < 5 * experts; i += 128) (i < experts ? cnt[i] : warp_counts[i - experts]) = 0;
  __syncthreads();
  int my_ids[8];
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    const uint32_t i = warp * 256 + c * 32 + lane;
    my_ids[c] = i < total ? __ldg(ids + i) : -1;
    if (i < total && static_cast<uint32_t>(my_ids[c]) >= experts) {
      atomicCAS(&g_moe_error, 0, 2);
      my_ids[c] = static_cast<int>(experts) - 1;
    }
    if (my_ids[c] >= 0) {
      atomicAdd(&cnt[my_ids[c]], 1);
      atomicAdd(&warp_counts[warp * experts + my_ids[c]], 1);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int o = 0, po = 0, lo = 0;
    for (uint32_t e0 = 0; e0 < experts; e0 += 8) {   // eight counts at a time, as in permute_scan_kernel
      int c[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) c[j] = e0 + j < experts ? cnt[e0 + j] : 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (e0 + j >= experts) break;
        off[e0 + j] = o;
        poff[e0 + j] = po;
        loff[e0 + j] = lo;
        o += c[j];
        po += (c[j] + kRowAlign - 1) / kRowAlign * kRowAlign;
        lo += (c[j] + 127) / 128;
      }
    }
    off[experts] = o;
    poff[experts] = po;
    plan[0] = po / 128;
    plan[1] = po;
    plan[3 + experts + 2 * (po / 128)] = lo;
  }
  __syncthreads();
  int32_t* info = plan + 3 + experts;
  for (uint32_t e = threadIdx.x; e <= experts; e += 128) {
    offsets[e] = off[e];
    plan[2 + e] = poff[e];
    if (e == experts) break;
    counts[e] = cnt[e];
    for (int tile = poff[e] / 128, j = 0; tile < poff[e + 1] / 128; ++tile, ++j) {
      const bool real = tile * 128 - poff[e] < cnt[e];
      info[2 * tile] = real ? static_cast<int32_t>(e) : -1;
      if (real) info[2 * (loff[e] + j) + 1] = tile;
    }
    int run = 0;   // exclusive prefix of the expert over the four warps
    for (int wq = 0; wq < 4; ++wq) {
      const int c = warp_counts[wq * experts + e];
      warp_counts[wq * experts + e] = run;
      run += c;
    }
  }
  __syncthreads();
  int* running = warp_counts + warp * experts;
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    const int e = my_ids[c];
    const unsigned active = __ballot_sync(0xFFFFFFFFu, e >= 0);
    if (e >= 0) {
      const unsigned peers = __match_any_sync(active, e);
      const int rank = __popc(peers & ((1u << lane) - 1));
      const int within = running[e] + rank;
      const uint32_t i = warp * 256 + c * 32 + lane;
      perm[off[e] + within] = static_cast<int32_t>(i);
      slot_rows[i] = poff[e] + within;
      __syncwarp(active);
      if (rank == 0) running[e] += __popc(peers);
    }
    __syncwarp();
  }
}

// ---------------------------------------------------------------------------------------------
// Quantise each token's expert input to NVFP4 once and write it to the padded row of every one
// of its topk assignments, block scales in the interleaved layout of the padded row space.
// One CTA per token, one thread per 16-element block.
// ---------------------------------------------------------------------------------------------
constexpr uint32_t kDispatchMaxBlocks = 1024;   // 16-element blocks of a token whose scales are staged in shared memory
__global__ void __launch_bounds__(256)
dispatch_quantize_kernel(const uint16_t* __restrict__ x, const int32_t* __restrict__ slot_rows,
                         uint8_t* __restrict__ packed, uint8_t* __restrict__ scales, uint32_t hidden,
                         uint32_t topk, float g, uint32_t c_pad) {
  const uint32_t t = blockIdx.x;
  __shared__ int rows[32];
  // The token's scale bytes meet here, so that they leave as 4-byte words (four consecutive K blocks are
  // contiguous in the interleaved layout) instead of one byte store per block and assignment.
  __shared__ __align__(4) uint8_t token_scales[kDispatchMaxBlocks];
  const bool words = hidden / 16 <= kDispatchMaxBlocks && (hidden / 16) % 4 == 0;
  if (threadIdx.x < topk) rows[threadIdx.x] = __ldg(slot_rows + static_cast<uint64_t>(t) * topk + threadIdx.x);
  __syncthreads();
  for (uint32_t c = threadIdx.x; c < hidden / 16; c += blockDim.x) {
    const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<uint64_t>(t) * hidden + c * 16);
    const uint4 a = __ldg(src), b = __ldg(src + 1);
    const uint32_t ww[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    float v[16];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      v[2 * i] = __uint_as_float(ww[i] << 16);
      v[2 * i + 1] = __uint_as_float(ww[i] & 0xFFFF0000u);
    }
    // Same arithmetic as the standalone NVFP4 quantizer (src/numeric/nvfp4.cpp:139-150).
    uint32_t lo, hi;
    uint8_t sb;
    quantize_block16<false>(v, g, lo, hi, sb);
    if (words) token_scales[c] = sb;
    for (uint32_t s = 0; s < topk; ++s) {
      const uint64_t r = static_cast<uint64_t>(rows[s]);
      *reinterpret_cast<uint2*>(packed + r * (hidden / 2) + c * 8) = make_uint2(lo, hi);
      if (!words) scales[interleaved_scale_offset(r, c, c_pad)] = sb;
    }
  }
  if (!words) return;
  __syncthreads();
  const uint32_t quads = hidden / 64;
  for (uint32_t idx = threadIdx.x; idx < quads * topk; idx += blockDim.x) {
    const uint32_t s = idx / quads, q = idx % quads;
    *reinterpret_cast<uint32_t*>(scales + interleaved_scale_offset(static_cast<uint64_t>(rows[s]), 4 * q, c_pad)) =
        *reinterpret_cast<const uint32_t*>(token_scales + 4 * q);
  }
}

// ---------------------------------------------------------------------------------------------
// Expert activation boundary on the padded rows: gate_up is bf16 [rows, 2*inter] with the gate
// in the first `inter` columns (the fused gate_up projection's chunk(2) order); product =
// bf16(bf16(gelu_tanh(gate)) * up) is NVFP4-quantised with the down projection's input divisor
// (boundaries of src/cuda/nvfp4/reference.cu:177-217).  Rows at or past plan[1] are skipped.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
expert_gelu_quantize_kernel(const uint16_t* __restrict__ gate_up, const int32_t* __restrict__ plan,
                            uint8_t* __restrict__ packed, uint8_t* __restrict__ scales, uint32_t rows_max,
                            uint32_t inter, float g, uint32_t c_pad) {
  const uint32_t blocks_per_row = inter / 16;
  const uint32_t rows = plan ? min(rows_max, static_cast<uint32_t>(__ldg(plan + 1))) : rows_max;
  const uint64_t work = static_cast<uint64_t>(rows) * blocks_per_row;
  // Grid-stride: the grid is sized for a bounded number of CTAs, not for rows_max, which with a
  // device-side plan can be far larger than the rows in use.
  for (uint64_t idx = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < work;
       idx += static_cast<uint64_t>(gridDim.x) * blockDim.x) {
  const uint32_t r = static_cast<uint32_t>(idx / blocks_per_row), c = static_cast<uint32_t>(idx % blocks_per_row);
  const uint16_t* gp = gate_up + static_cast<uint64_t>(r) * 2 * inter + c * 16;
  const uint4 ga = __ldg(reinterpret_cast<const uint4*>(gp)), gb = __ldg(reinterpret_cast<const uint4*>(gp) + 1);
  const uint4 ua = __ldg(reinterpret_cast<const uint4*>(gp + inter)), ub = __ldg(reinterpret_cast<const uint4*>(gp + inter) + 1);
  const uint32_t gw[8] = {ga.x, ga.y, ga.z, ga.w, gb.x, gb.y, gb.z, gb.w};
  const uint32_t uw[8] = {ua.x, ua.y, ua.z, ua.w, ub.x, ub.y, ub.z, ub.w};
  float v[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const float gv = __uint_as_float((i & 1) ? (gw[i >> 1] & 0xFFFF0000u) : (gw[i >> 1] << 16));
    const float uv = __uint_as_float((i & 1) ? (uw[i >> 1] & 0xFFFF0000u) : (uw[i >> 1] << 16));
    v[i] = gelu_tanh_product(gv, uv);
  }
  uint32_t lo, hi;
  uint8_t sb;
  quantize_block16<false>(v, g, lo, hi, sb);
  *reinterpret_cast<uint2*>(packed + static_cast<uint64_t>(r) * (inter / 2) + c * 8) = make_uint2(lo, hi);
  scales[interleaved_scale_offset(r, c, c_pad)] = sb;
  }
}

// ---------------------------------------------------------------------------------------------
// Expert-parallel plumbing: row gather (pack assignments in permutation order for the all-to-all,
// and expert outputs back into arrival order) and the scatter of already quantised rows into the
// padded row space with interleaved scales.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
gather_rows_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, const int32_t* __restrict__ index,
                   uint32_t divisor, uint64_t rows, uint32_t chunks_per_row, uint32_t src_stride_chunks,
                   uint32_t dst_stride_chunks) {
  const uint64_t idx = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= rows * chunks_per_row) return;
  const uint64_t r = idx / chunks_per_row, c = idx % chunks_per_row;
  const uint64_t s = static_cast<uint64_t>(__ldg(index + r)) / divisor;
  dst[r * dst_stride_chunks + c] = __ldg(src + s * src_stride_chunks + c);
}

__global__ void __launch_bounds__(256)
scatter_quantized_kernel(const uint8_t* __restrict__ payload, const uint8_t* __restrict__ compact_scales,
                         const int32_t* __restrict__ slot_rows, uint8_t* __restrict__ packed,
                         uint8_t* __restrict__ scales, uint64_t rows, uint32_t hidden, uint32_t c_pad,
                         uint64_t src_row_stride) {
  const uint32_t blocks = hidden / 16;
  const uint64_t idx = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= rows * blocks) return;
  const uint64_t r = idx / blocks;
  const uint32_t c = static_cast<uint32_t>(idx % blocks);
  const uint64_t d = static_cast<uint64_t>(__ldg(slot_rows + r));
  *reinterpret_cast<uint2*>(packed + d * (hidden / 2) + c * 8) =
      __ldg(reinterpret_cast<const uint2*>(payload + r * src_row_stride + c * 8));
  scales[interleaved_scale_offset(d, c, c_pad)] = __ldg(compact_scales + r * src_row_stride + c);
}

// ---------------------------------------------------------------------------------------------
// Deterministic combine (MOE_SEMANTICS_SPEC.md:74-83): acc = 0; for slot 0..k-1:
// acc = fma(weight[slot], y[row(slot)], acc); + shared branch; round to bf16.
// One thread per 8 output columns.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
combine_kernel(const uint16_t* __restrict__ y, const int32_t* __restrict__ slot_rows,
               const float* __restrict__ weights, const uint16_t* __restrict__ shared_out,
               uint16_t* __restrict__ out, uint32_t tokens, uint32_t hidden, uint32_t topk) {
  const uint32_t chunks = hidden / 8;
  const uint64_t idx = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<uint64_t>(tokens) * chunks) return;
  const uint32_t t = static_cast<uint32_t>(idx / chunks), c = static_cast<uint32_t>(idx % chunks);
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
  for (uint32_t s = 0; s < topk; ++s) {
    const float wv = __ldg(weights + static_cast<uint64_t>(t) * topk + s);
    const int64_t r = slot_rows ? static_cast<int64_t>(__ldg(slot_rows + static_cast<uint64_t>(t) * topk + s))
                                : static_cast<int64_t>(t) * topk + s;
    const uint4 v = __ldg(reinterpret_cast<const uint4*>(y + r * hidden) + c);
    const uint32_t ww[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      acc[2 * i] = fmaf(wv, __uint_as_float(ww[i] << 16), acc[2 * i]);
      acc[2 * i + 1] = fmaf(wv, __uint_as_float(ww[i] & 0xFFFF0000u), acc[2 * i + 1]);
    }
  }
  if (shared_out) {
    const uint4 v = __ldg(reinterpret_cast<const uint4*>(shared_out + static_cast<uint64_t>(t) * hidden) + c);
    const uint32_t ww[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      acc[2 * i] = __fadd_rn(acc[2 * i], __uint_as_float(ww[i] << 16));
      acc[2 * i + 1] = __fadd_rn(acc[2 * i + 1], __uint_as_float(ww[i] & 0xFFFF0000u));
    }
  }
  uint32_t o[4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
    o[i] = static_cast<uint32_t>(float_to_bf16_bits(acc[2 * i])) |
           (static_cast<uint32_t>(float_to_bf16_bits(acc[2 * i + 1])) << 16);
  reinterpret_cast<uint4*>(out + static_cast<uint64_t>(t) * hidden)[c] = make_uint4(o[0], o[1], o[2], o[3]);
}

}  // namespace
}  // namespace gemb

using namespace gemb;

namespace {
uint64_t moe_segments(uint64_t tokens, uint64_t topk) { return (tokens * topk + kSegment - 1) / kSegment; }
// sum over experts of ceil(c_e / 256) * 2 tiles of 128 rows <= assignments / 128 + 2 * experts
uint64_t moe_max_tiles(uint64_t tokens, uint64_t experts, uint64_t topk) { return tokens * topk / 128 + 2 * experts; }

// The permutation itself has no warp-shape constraint on the expert count (the expert-parallel
// receiver sorts by a handful of local experts).
int32_t validate_permute_geometry(const char* op, uint64_t tokens, uint64_t experts, uint64_t topk) {
  GEMB_REQUIRE(tokens > 0 && tokens * topk < (1ull << 31), "%s: token count must be nonzero and fit 31 bits", op);
  GEMB_REQUIRE(experts >= 1 && experts <= 1024, "%s: experts must be in [1, 1024]", op);
  GEMB_REQUIRE(topk >= 1 && topk <= 32, "%s: top-k must be in [1, 32]", op);
  return GEMB_OK;
}

// The small-batch router kernel's ring needs more than the 48 KB a kernel gets without opting in.
template <int kTpt>
int32_t router_small_configure(const char* op) {
  static std::atomic<bool> configured[64];   // racing first calls both set the (idempotent) attribute
  int dev = 0;
  cudaGetDevice(&dev);
  dev &= 63;
  if (!configured[dev].load(std::memory_order_acquire)) {
    cudaError_t e = cudaFuncSetAttribute(router_logits_small_kernel<kTpt>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(sizeof(RouterSmallSmem<kTpt>)));
    if (e != cudaSuccess) return fail(GEMB_INTERNAL, "%s: %s: %s", op, cudaGetErrorName(e), cudaGetErrorString(e));
    configured[dev].store(true, std::memory_order_release);
  }
  return GEMB_OK;
}

int32_t validate_moe_geometry(const char* op, uint64_t tokens, uint64_t experts, uint64_t topk) {
  GEMB_REQUIRE(tokens > 0 && tokens * topk < (1ull << 31), "%s: token count must be nonzero and fit 31 bits", op);
  GEMB_REQUIRE(experts >= 32 && experts % 32 == 0 && experts <= 256, "%s: experts must be a multiple of 32 in [32, 256]", op);
  GEMB_REQUIRE(topk >= 1 && topk <= 32 && topk <= experts, "%s: top-k must be in [1, 32] and at most the expert count", op);
  return GEMB_OK;
}
}  // namespace

extern "C" {

int32_t gemb_moe_router_logits(const uint16_t* x_bf16, const float* router_weight, const float* bias,
                               float* logits, uint64_t tokens, uint64_t hidden, uint64_t experts,
                               gemb_stream_t stream) {
  const char* op = "gemb_moe_router_logits";
  GEMB_REQUIRE(x_bf16 && router_weight && logits, "%s: pointers must be nonnull", op);
  GEMB_REQUIRE(tokens > 0 && tokens < (1ull << 31) && experts > 0 && experts < (1ull << 20), "%s: bad geometry", op);
  GEMB_REQUIRE(hidden > 0 && hidden % 4 == 0 && hidden < (1ull << 31), "%s: hidden must be a nonzero multiple of 4", op);
  GEMB_REQUIRE(reinterpret_cast<uintptr_t>(x_bf16) % 8 == 0 && reinterpret_cast<uintptr_t>(router_weight) % 16 == 0,
               "%s: activations must be 8-byte and router weights 16-byte aligned", op);
  GEMB_ENTER(op);
  // Up to a thousand tokens: one expert per thread, weight rows streamed from L2 (the tiled kernel
  // would occupy a fraction of the SMs).  Its L2 traffic grows with the token count (one pass over
  // the router weight per 2 * kTpt tokens), so larger batches use the tiled kernel.  Measured on
  // 2,816 x 128: 25 / 31 / 43 / 56 us at 64 / 256 / 512 / 1,024 tokens here, against 64 us for the
  // tiled kernel; at 2,048 tokens 105 us against 72 us for the 16-token tile.
  if ((tokens <= 1024 && g_router_tile == 0) || (tokens <= 2048 && g_router_tile == 1)) {
    if (tokens <= 256) {
      dim3 g(static_cast<unsigned>((tokens + 3) / 4), static_cast<unsigned>((experts + 31) / 32));
      GEMB_TRY(router_small_configure<2>(op));
      router_logits_small_kernel<2><<<g, kRsThreads, sizeof(RouterSmallSmem<2>), stream>>>(x_bf16, router_weight, bias, logits,
                                                                   static_cast<uint32_t>(tokens), static_cast<uint32_t>(hidden),
                                                                   static_cast<uint32_t>(experts));
    } else if (tokens <= 512) {
      dim3 g(static_cast<unsigned>((tokens + 7) / 8), static_cast<unsigned>((experts + 31) / 32));
      GEMB_TRY(router_small_configure<4>(op));
      router_logits_small_kernel<4><<<g, kRsThreads, sizeof(RouterSmallSmem<4>), stream>>>(x_bf16, router_weight, bias, logits,
                                                                   static_cast<uint32_t>(tokens), static_cast<uint32_t>(hidden),
                                                                   static_cast<uint32_t>(experts));
    } else {
      dim3 g(static_cast<unsigned>((tokens + 15) / 16), static_cast<unsigned>((experts + 31) / 32));
      GEMB_TRY(router_small_configure<8>(op));
      router_logits_small_kernel<8><<<g, kRsThreads, sizeof(RouterSmallSmem<8>), stream>>>(x_bf16, router_weight, bias, logits,
                                                                   static_cast<uint32_t>(tokens), static_cast<uint32_t>(hidden),
                                                                   static_cast<uint32_t>(experts));
    }
    return check_launch(op);
  }
  // 8- and 16-token CTAs only while they do not outnumber the SMs; beyond that the larger tiles do more
  // arithmetic per shared-memory load: 32 tokens, and 64 once there is a 64-token CTA for most SMs
  // (measured on 2,816 x 128: 303 / 268 us at 16,384 tokens, 166 / 158 us at 8,192, 114 / 158 us at 4,096).
  const uint64_t expert_tiles = (experts + kRtExp - 1) / kRtExp;
  unsigned tile = 32;
  if ((tokens + 7) / 8 * expert_tiles <= static_cast<uint64_t>(sm_count())) tile = 8;
  else if ((tokens + 15) / 16 * expert_tiles <= static_cast<uint64_t>(sm_count())) tile = 16;
  else if ((tokens + 63) / 64 * expert_tiles * 8 >= static_cast<uint64_t>(sm_count()) * 6) tile = 64;
  // 56-token CTAs where they even out the load: with up to two of the large CTAs per SM, an SM's time goes with
  // the tokens it holds (16,384 tokens: 256 CTAs of 64 leave 40 SMs with one CTA and 108 with two, 293 CTAs
  // of 56 give every SM two).
  if (tile == 64) {
    const uint64_t sms = static_cast<uint64_t>(sm_count());
    const uint64_t c64 = (tokens + 63) / 64 * expert_tiles, c56 = (tokens + 55) / 56 * expert_tiles;
    if ((c56 + sms - 1) / sms * 56 < (c64 + sms - 1) / sms * 64) tile = 56;
  }
  if (g_router_tile == 8 || g_router_tile == 16 || g_router_tile == 32 || g_router_tile == 56 || g_router_tile == 64)
    tile = static_cast<unsigned>(g_router_tile);
  dim3 grid(static_cast<unsigned>((tokens + tile - 1) / tile), static_cast<unsigned>((experts + kRtExp - 1) / kRtExp));
  if (tile == 8)
    router_logits_kernel<8><<<grid, kRtThreads, 0, stream>>>(x_bf16, router_weight, bias, logits,
                                                            static_cast<uint32_t>(tokens), static_cast<uint32_t>(hidden),
                                                            static_cast<uint32_t>(experts));
  else if (tile == 16)
    router_logits_kernel<16><<<grid, kRtThreads, 0, stream>>>(x_bf16, router_weight, bias, logits,
                                                             static_cast<uint32_t>(tokens), static_cast<uint32_t>(hidden),
                                                             static_cast<uint32_t>(experts));
  else if (tile == 56)
    router_logits_kernel<56><<<grid, kRtThreads, 0, stream>>>(x_bf16, router_weight, bias, logits,
                                                             static_cast<uint32_t>(tokens), static_cast<uint32_t>(hidden),
                                                             static_cast<uint32_t>(experts));
  else if (tile == 64)
    router_logits_kernel<64><<<grid, kRtThreads, 0, stream>>>(x_bf16, router_weight, bias, logits,
                                                             static_cast<uint32_t>(tokens), static_cast<uint32_t>(hidden),
                                                             static_cast<uint32_t>(experts));
  else
    router_logits_kernel<32><<<grid, kRtThreads, 0, stream>>>(x_bf16, router_weight, bias, logits,
                                                             static_cast<uint32_t>(tokens), static_cast<uint32_t>(hidden),
                                                             static_cast<uint32_t>(experts));
  return check_launch(op);
}

int32_t gemb_moe_route(const float* logits, const float* per_expert_scale, int32_t* top_ids, float* top_weights,
                       float* probabilities, uint64_t tokens, uint64_t experts, uint64_t topk,
                       gemb_stream_t stream) {
  const char* op = "gemb_moe_route";
  GEMB_REQUIRE(logits && top_ids && top_weights, "%s: pointers must be nonnull", op);
  GEMB_TRY(validate_moe_geometry(op, tokens, experts, topk));
  GEMB_ENTER(op);
  route_kernel<<<static_cast<unsigned>((tokens + 3) / 4), 128, 0, stream>>>(
      logits, per_expert_scale, top_ids, top_weights, probabilities, static_cast<uint32_t>(tokens),
      static_cast<uint32_t>(experts), static_cast<uint32_t>(topk));
  return check_launch(op);
}

uint64_t gemb_moe_permute_workspace_bytes(uint64_t tokens, uint64_t experts, uint64_t topk) {
  return moe_segments(tokens, topk) * experts * sizeof(int32_t);
}
uint64_t gemb_moe_plan_ints(uint64_t tokens, uint64_t experts, uint64_t topk) {
  return 2 + experts + 1 + 2 * moe_max_tiles(tokens, experts, topk) + 1;
}
uint64_t gemb_moe_padded_rows_max(uint64_t tokens, uint64_t experts, uint64_t topk) {
  return moe_max_tiles(tokens, experts, topk) * 128;
}

int32_t gemb_moe_permute(const int32_t* top_ids, int32_t* counts, int32_t* offsets, int32_t* perm,
                         int32_t* slot_rows, int32_t* plan, void* workspace, uint64_t workspace_bytes,
                         uint64_t tokens, uint64_t experts, uint64_t topk, gemb_stream_t stream) {
  const char* op = "gemb_moe_permute";
  GEMB_REQUIRE(top_ids && counts && offsets && perm && slot_rows && plan && workspace, "%s: pointers must be nonnull", op);
  GEMB_TRY(validate_permute_geometry(op, tokens, experts, topk));
  GEMB_REQUIRE(workspace_bytes >= gemb_moe_permute_workspace_bytes(tokens, experts, topk),
               "%s: workspace too small (%llu bytes needed)", op,
               static_cast<unsigned long long>(gemb_moe_permute_workspace_bytes(tokens, experts, topk)));
  GEMB_ENTER(op);
  const uint32_t total = static_cast<uint32_t>(tokens * topk), e = static_cast<uint32_t>(experts);
  const uint32_t segments = static_cast<uint32_t>(moe_segments(tokens, topk));
  if (segments == 1) {   // decode-size batch: count, scan and scatter in one launch
    permute_small_kernel<<<1, 128, (8 * e + 3) * sizeof(int), stream>>>(
        top_ids, counts, offsets, plan, perm, slot_rows, total, e, static_cast<uint32_t>(moe_max_tiles(tokens, experts, topk)));
    return check_launch(op);
  }
  int32_t* block_counts = static_cast<int32_t*>(workspace);
  permute_count_kernel<<<segments, 128, e * sizeof(int), stream>>>(top_ids, block_counts, total, e);
  GEMB_TRY(check_launch(op));
  permute_scan_kernel<<<1, 256, (4 * e + 3) * sizeof(int), stream>>>(block_counts, counts, offsets, plan, segments, e,
                                                                     static_cast<uint32_t>(moe_max_tiles(tokens, experts, topk)));
  GEMB_TRY(check_launch(op));
  permute_scatter_kernel<<<segments, 128, 4 * e * sizeof(int), stream>>>(top_ids, block_counts, offsets, plan, perm,
                                                                        slot_rows, total, e);
  return check_launch(op);
}

// ---------------------------------------------------------------------------------------------
// Allocation-free variant of gemb_moe_permute.
//
// gemb_moe_permute needs a few kilobytes of scratch for the per-segment expert counts and asks
// the caller for it.  Some hosts cannot supply one: an engine that carves a single arena at
// model load and forbids the allocator afterwards may have no region left for a workspace it
// did not plan for, and code running inside a latency-critical or capture-only section must not
// call cudaMalloc (it synchronises the device and is illegal while a stream is capturing).  For
// them the scratch lives in the file-scope array below, which every GPU that loads the library
// holds until the process exits.  Its size is fixed, so the problem size is capped.
// ---------------------------------------------------------------------------------------------
constexpr uint64_t kStaticMaxSegments = 128;   // 128 segments x 1024 = 131,072 assignments
constexpr uint64_t kStaticMaxExperts = 256;
static __device__ __align__(256) int32_t g_permute_scratch[kStaticMaxSegments * kStaticMaxExperts];  // 128 KiB

// The array's name is only a host-side handle; kernels need its device address.  It is looked
// up once per device, with that device current, and cached.
// (Two host threads racing on a device's first call both store the same address.)
static std::atomic<int32_t*> g_permute_scratch_ptr[64];

static int32_t permute_scratch_address(const char* op, int32_t** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64) {
    cudaGetLastError();
    return fail(GEMB_UNSUPPORTED, "%s: no usable CUDA device", op);
  }
  if (g_permute_scratch_ptr[dev].load(std::memory_order_acquire) == nullptr) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_permute_scratch);
    if (e != cudaSuccess || ptr == nullptr) {
      cudaGetLastError();
      return fail(GEMB_INTERNAL, "%s: cudaGetSymbolAddress: %s: %s", op, cudaGetErrorName(e), cudaGetErrorString(e));
    }
    g_permute_scratch_ptr[dev].store(static_cast<int32_t*>(ptr), std::memory_order_release);
  }
  *out = g_permute_scratch_ptr[dev].load(std::memory_order_acquire);
  return GEMB_OK;
}

int32_t gemb_moe_permute_static(const int32_t* top_ids, int32_t* counts, int32_t* offsets, int32_t* perm,
                                int32_t* slot_rows, int32_t* plan, uint64_t tokens, uint64_t experts,
                                uint64_t topk, gemb_stream_t stream) {
  const char* op = "gemb_moe_permute_static";
  GEMB_REQUIRE(top_ids && counts && offsets && perm && slot_rows && plan, "%s: pointers must be nonnull", op);
  GEMB_TRY(validate_permute_geometry(op, tokens, experts, topk));   // the same rules as gemb_moe_permute
  const uint64_t segments64 = moe_segments(tokens, topk);
  GEMB_REQUIRE(segments64 <= kStaticMaxSegments && experts <= kStaticMaxExperts,
               "%s: %llu assignments over %llu experts exceed the built-in scratch (at most %llu assignments, %llu "
               "experts); use gemb_moe_permute with a caller workspace",
               op, static_cast<unsigned long long>(tokens * topk), static_cast<unsigned long long>(experts),
               static_cast<unsigned long long>(kStaticMaxSegments * kSegment),
               static_cast<unsigned long long>(kStaticMaxExperts));
  GEMB_ENTER(op);
  int32_t* block_counts = nullptr;
  GEMB_TRY(permute_scratch_address(op, &block_counts));
  const uint32_t total = static_cast<uint32_t>(tokens * topk), e = static_cast<uint32_t>(experts);
  const uint32_t segments = static_cast<uint32_t>(segments64);
  // The count kernel overwrites every (segment, expert) cell this call reads, so nothing has to
  // be cleared even though the array still holds the previous call's values.
  permute_count_kernel<<<segments, 128, e * sizeof(int), stream>>>(top_ids, block_counts, total, e);
  GEMB_TRY(check_launch(op));
  permute_scan_kernel<<<1, 256, (4 * e + 3) * sizeof(int), stream>>>(block_counts, counts, offsets, plan, segments, e,
                                                                     static_cast<uint32_t>(moe_max_tiles(tokens, experts, topk)));
  GEMB_TRY(check_launch(op));
  permute_scatter_kernel<<<segments, 128, 4 * e * sizeof(int), stream>>>(top_ids, block_counts, offsets, plan, perm,
                                                                        slot_rows, total, e);
  return check_launch(op);
}

int32_t gemb_moe_dispatch_quantize(const uint16_t* x_bf16, const int32_t* slot_rows, uint8_t* packed_e2m1,
                                   uint8_t* interleaved_scales, uint64_t tokens, uint64_t hidden, uint64_t topk,
                                   float global_divisor, gemb_stream_t stream) {
  const char* op = "gemb_moe_dispatch_quantize";
  GEMB_REQUIRE(x_bf16 && slot_rows && packed_e2m1 && interleaved_scales, "%s: pointers must be nonnull", op);
  GEMB_REQUIRE(tokens > 0 && tokens < (1ull << 31) && topk >= 1 && topk <= 32, "%s: bad geometry", op);
  GEMB_REQUIRE(hidden > 0 && hidden % 16 == 0 && hidden < (1ull << 31), "%s: hidden must be a nonzero multiple of 16", op);
  GEMB_REQUIRE(positive_finite(global_divisor), "%s: global divisor must be positive and finite", op);
  GEMB_REQUIRE(reinterpret_cast<uintptr_t>(x_bf16) % 16 == 0 && reinterpret_cast<uintptr_t>(packed_e2m1) % 8 == 0,
               "%s: input must be 16-byte and payload 8-byte aligned", op);
  GEMB_ENTER(op);
  const uint32_t c_pad = static_cast<uint32_t>((hidden / 16 + 3) / 4 * 4);
  const unsigned threads = static_cast<unsigned>(std::min<uint64_t>(256, (hidden / 16 + 31) / 32 * 32));
  dispatch_quantize_kernel<<<static_cast<unsigned>(tokens), threads, 0, stream>>>(
      x_bf16, slot_rows, packed_e2m1, interleaved_scales, static_cast<uint32_t>(hidden), static_cast<uint32_t>(topk),
      global_divisor, c_pad);
  return check_launch(op);
}

int32_t gemb_moe_gather_rows(const void* src, void* dst, const int32_t* index, uint64_t index_divisor,
                             uint64_t rows, uint64_t row_bytes, uint64_t src_row_stride, uint64_t dst_row_stride,
                             gemb_stream_t stream) {
  const char* op = "gemb_moe_gather_rows";
  GEMB_REQUIRE(src && dst && index, "%s: pointers must be nonnull", op);
  GEMB_REQUIRE(rows > 0 && rows < (1ull << 31) && index_divisor >= 1 && index_divisor < (1ull << 31), "%s: bad geometry", op);
  GEMB_REQUIRE(row_bytes > 0 && row_bytes % 16 == 0 && row_bytes < (1ull << 24), "%s: row size must be a nonzero multiple of 16 bytes", op);
  GEMB_REQUIRE(reinterpret_cast<uintptr_t>(src) % 16 == 0 && reinterpret_cast<uintptr_t>(dst) % 16 == 0,
               "%s: buffers must be 16-byte aligned", op);
  GEMB_REQUIRE(src_row_stride >= row_bytes && dst_row_stride >= row_bytes && src_row_stride % 16 == 0 &&
                   dst_row_stride % 16 == 0 && src_row_stride < (1ull << 30) && dst_row_stride < (1ull << 30),
               "%s: row strides must be multiples of 16 bytes no smaller than the row", op);
  GEMB_ENTER(op);
  const uint32_t chunks = static_cast<uint32_t>(row_bytes / 16);
  gather_rows_kernel<<<static_cast<unsigned>((rows * chunks + 255) / 256), 256, 0, stream>>>(
      static_cast<const uint4*>(src), static_cast<uint4*>(dst), index, static_cast<uint32_t>(index_divisor), rows, chunks,
      static_cast<uint32_t>(src_row_stride / 16), static_cast<uint32_t>(dst_row_stride / 16));
  return check_launch(op);
}

int32_t gemb_moe_scatter_quantized(const uint8_t* packed_rows, const uint8_t* compact_scales, const int32_t* slot_rows,
                                   uint8_t* packed_e2m1, uint8_t* interleaved_scales, uint64_t rows, uint64_t hidden,
                                   uint64_t src_row_stride, gemb_stream_t stream) {
  const char* op = "gemb_moe_scatter_quantized";
  GEMB_REQUIRE(packed_rows && compact_scales && slot_rows && packed_e2m1 && interleaved_scales, "%s: pointers must be nonnull", op);
  GEMB_REQUIRE(rows > 0 && rows < (1ull << 31), "%s: bad row count", op);
  GEMB_REQUIRE(hidden > 0 && hidden % 16 == 0 && hidden < (1ull << 31), "%s: hidden must be a nonzero multiple of 16", op);
  GEMB_REQUIRE(reinterpret_cast<uintptr_t>(packed_rows) % 8 == 0 && reinterpret_cast<uintptr_t>(packed_e2m1) % 8 == 0,
               "%s: payload buffers must be 8-byte aligned", op);
  GEMB_REQUIRE(src_row_stride >= hidden / 2 && src_row_stride % 8 == 0 && src_row_stride < (1ull << 30),
               "%s: source row stride must be a multiple of 8 bytes no smaller than the payload row", op);
  GEMB_ENTER(op);
  const uint32_t c_pad = static_cast<uint32_t>((hidden / 16 + 3) / 4 * 4);
  const uint64_t work = rows * (hidden / 16);
  scatter_quantized_kernel<<<static_cast<unsigned>((work + 255) / 256), 256, 0, stream>>>(
      packed_rows, compact_scales, slot_rows, packed_e2m1, interleaved_scales, rows, static_cast<uint32_t>(hidden), c_pad,
      src_row_stride);
  return check_launch(op);
}

int32_t gemb_moe_expert_gelu_quantize(const uint16_t* gate_up_bf16, const int32_t* plan, uint8_t* packed_e2m1,
                                      uint8_t* interleaved_scales, uint64_t rows_max, uint64_t intermediate,
                                      float global_divisor, gemb_stream_t stream) {
  const char* op = "gemb_moe_expert_gelu_quantize";
  GEMB_REQUIRE(gate_up_bf16 && packed_e2m1 && interleaved_scales, "%s: pointers must be nonnull", op);
  GEMB_REQUIRE(rows_max > 0 && rows_max < (1ull << 31), "%s: bad row count", op);
  GEMB_REQUIRE(intermediate > 0 && intermediate % 16 == 0 && intermediate < (1ull << 30),
               "%s: intermediate size must be a nonzero multiple of 16", op);
  GEMB_REQUIRE(positive_finite(global_divisor), "%s: global divisor must be positive and finite", op);
  GEMB_REQUIRE(reinterpret_cast<uintptr_t>(gate_up_bf16) % 16 == 0 && reinterpret_cast<uintptr_t>(packed_e2m1) % 8 == 0,
               "%s: input must be 16-byte and payload 8-byte aligned", op);
  GEMB_ENTER(op);
  const uint64_t work = rows_max * (intermediate / 16);
  const uint32_t c_pad = static_cast<uint32_t>((intermediate / 16 + 3) / 4 * 4);
  const uint64_t ctas = std::min<uint64_t>((work + 255) / 256, static_cast<uint64_t>(sm_count()) * 32);
  expert_gelu_quantize_kernel<<<static_cast<unsigned>(ctas), 256, 0, stream>>>(
      gate_up_bf16, plan, packed_e2m1, interleaved_scales, static_cast<uint32_t>(rows_max),
      static_cast<uint32_t>(intermediate), global_divisor, c_pad);
  return check_launch(op);
}

int32_t gemb_moe_combine(const uint16_t* y_bf16, const int32_t* slot_rows, const float* top_weights,
                         const uint16_t* shared_bf16, uint16_t* out_bf16, uint64_t tokens, uint64_t hidden,
                         uint64_t topk, gemb_stream_t stream) {
  const char* op = "gemb_moe_combine";
  GEMB_REQUIRE(y_bf16 && top_weights && out_bf16, "%s: pointers must be nonnull", op);
  GEMB_REQUIRE(tokens > 0 && tokens < (1ull << 31) && topk >= 1 && topk <= 32, "%s: bad geometry", op);
  GEMB_REQUIRE(hidden > 0 && hidden % 8 == 0 && hidden < (1ull << 31), "%s: hidden must be a nonzero multiple of 8", op);
  GEMB_REQUIRE(reinterpret_cast<uintptr_t>(y_bf16) % 16 == 0 && reinterpret_cast<uintptr_t>(out_bf16) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(shared_bf16) % 16 == 0,
               "%s: buffers must be 16-byte aligned", op);
  GEMB_ENTER(op);
  const uint64_t work = tokens * (hidden / 8);
  combine_kernel<<<static_cast<unsigned>((work + 255) / 256), 256, 0, stream>>>(
      y_bf16, slot_rows, top_weights, shared_bf16, out_bf16, static_cast<uint32_t>(tokens),
      static_cast<uint32_t>(hidden), static_cast<uint32_t>(topk));
  return check_launch(op);
}

}  // extern "C"
