// Batch-1 decode projections: HBM-streaming, warp-reduced GEMV kernels for FP8 (W8A8) and NVFP4
// (W4A4) weights in the checkpoint's row-major source layout.
//
// Shape of every kernel: a CTA of 8 warps stages the activation vector once in shared memory
// (decoded to fp16, which holds every E4M3 and E2M1 value exactly), then each warp streams
// kRows weight rows with coalesced 128-bit loads (lane l reads bytes [16 l, 16 l + 16) of each
// 512-byte row segment, `no_allocate` so the stream does not evict the activation from L1),
// accumulates in fp32 and folds the 32 lanes with an xor butterfly.  Weights are read exactly
// once: algorithmic bytes per output row are K (FP8) or K/2 + K/16 (NVFP4) plus the scale and
// the 4-byte result; the activation (K bytes or less) is re-read per CTA from L2.
#include <algorithm>
#include <mutex>

#include "common.cuh"
#include "ptx.cuh"

namespace gemb {

__device__ int g_gemv_error = 0;

namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;

int g_rows_override = 0;  // 0 = automatic; set through gemb_set_tuning(GEMB_TUNE_GEMV_ROWS, n)
int g_gemv_impl = 0;  // single token: 0 = bulk-copy ring when it fits, 1 = direct global loads; batch: 1 = SIMT form
int g_pdl = 1;            // programmatic dependent launch; gemb_set_tuning(GEMB_TUNE_GEMV_PDL, 0/1)

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// Two E4M3 bytes (low half of `pair`) -> two fp16 values.
__device__ __forceinline__ uint32_t e4m3x2_to_half2(uint16_t pair) {
  uint32_t r;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(r) : "h"(pair));
  return r;
}
// acc += a * b with fp16 inputs and an fp32 accumulator, one rounding (sm_100 mixed fma).
__device__ __forceinline__ void fma_f16(float& acc, uint16_t a, uint16_t b) {
  asm("fma.rn.f32.f16 %0, %1, %2, %0;" : "+f"(acc) : "h"(a), "h"(b));
}
__device__ __forceinline__ void dot16_fp8(float& acc, const uint4& w, const uint4& xa, const uint4& xb) {
  const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
  const uint32_t xx[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t h0 = e4m3x2_to_half2(static_cast<uint16_t>(ww[i] & 0xFFFFu));
    const uint32_t h1 = e4m3x2_to_half2(static_cast<uint16_t>(ww[i] >> 16));
    fma_f16(acc, static_cast<uint16_t>(h0 & 0xFFFFu), static_cast<uint16_t>(xx[2 * i] & 0xFFFFu));
    fma_f16(acc, static_cast<uint16_t>(h0 >> 16), static_cast<uint16_t>(xx[2 * i] >> 16));
    fma_f16(acc, static_cast<uint16_t>(h1 & 0xFFFFu), static_cast<uint16_t>(xx[2 * i + 1] & 0xFFFFu));
    fma_f16(acc, static_cast<uint16_t>(h1 >> 16), static_cast<uint16_t>(xx[2 * i + 1] >> 16));
  }
}

struct Fp8Problem {
  const uint8_t* w;
  const uint16_t* w_scales;
  void* out;
  uint64_t rows;
};
// Up to three projections that share one activation (grouped Q/K/V).  Their rows form one
// virtual row space; row_start[i] is the first virtual row of problem i, row_start[n] the total.
struct Fp8Group {
  Fp8Problem p[3];
  uint64_t row_start[4];
  int n;
};

// Shared-memory layout of the staged activation: per 512-element segment, lane l's sixteen
// values are split into two 8-value halves stored at [l*8, l*8+8) and [256 + l*8, 256 + l*8 + 8)
// so that each 128-bit shared load of a warp touches 512 contiguous bytes (no bank conflicts).
//
// The staging buffer is padded to a whole 512-element segment; lanes past K multiply zero
// weights with whatever the padding holds, so it must hold finite values: zero it.
template <int kW>
__device__ __forceinline__ void zero_fp8_staging_tail(uint64_t k, __half* xs) {
  const uint64_t chunks = k / 16, chunks_pad = (k + 511) / 512 * 32;
  for (uint64_t c = chunks + threadIdx.x; c < chunks_pad; c += kW * 32) {
    __half* dst = xs + (c / 32) * 512 + (c % 32) * 8;
    *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
    *reinterpret_cast<uint4*>(dst + 256) = make_uint4(0, 0, 0, 0);
  }
}

// Stages an already quantized activation (E4M3 bytes) as fp16 in shared memory.
template <int kW>
__device__ __forceinline__ void stage_fp8_activation(const uint8_t* act, uint64_t k, __half* xs) {
  for (uint64_t c = threadIdx.x; c < k / 16; c += kW * 32) {
    const uint4 v = __ldg(reinterpret_cast<const uint4*>(act) + c);
    const uint32_t ww[4] = {v.x, v.y, v.z, v.w};
    uint32_t h[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      h[2 * i] = e4m3x2_to_half2(static_cast<uint16_t>(ww[i] & 0xFFFFu));
      h[2 * i + 1] = e4m3x2_to_half2(static_cast<uint16_t>(ww[i] >> 16));
    }
    __half* dst = xs + (c / 32) * 512 + (c % 32) * 8;
    *reinterpret_cast<uint4*>(dst) = make_uint4(h[0], h[1], h[2], h[3]);
    *reinterpret_cast<uint4*>(dst + 256) = make_uint4(h[4], h[5], h[6], h[7]);
  }
  zero_fp8_staging_tail<kW>(k, xs);
}

// A value y with E4M3(y) == E4M3(x / scale) for the IEEE quotient x / scale.  x * (1/scale) is
// within two ulp of the quotient, so both round to the same E4M3 code unless y sits within a
// few ulp of a rounding boundary of the 3-bit mantissa (fraction bits 0x80000) or in E4M3's
// subnormal range (below 2^-6), where the true division is used.
__device__ __forceinline__ float quotient_for_e4m3(float x, float scale, float inv_scale) {
  const float y = __fmul_rn(x, inv_scale);
  const uint32_t bits = __float_as_uint(y);
  const uint32_t mag = bits & 0x7FFFFFFFu;
  const bool near_boundary = ((bits & 0xFFFFFu) - 0x7FFFCu) <= 8u;
  const bool tiny = mag < 0x3C800000u && mag != 0u;  // |y| < 2^-6 (and not an exact zero)
  if (near_boundary || tiny) return __fdiv_rn(x, scale);
  return y;
}

// Quantizes eight bf16 values (one 16-byte chunk) and stages them as fp16.
__device__ __forceinline__ void stage_bf16_chunk(const uint4& v, uint64_t c, float scale,
                                                 float inv_scale, __half* xs) {
  const uint32_t ww[4] = {v.x, v.y, v.z, v.w};
  uint32_t h[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float lo = quotient_for_e4m3(__uint_as_float(ww[i] << 16), scale, inv_scale);
    const float hi = quotient_for_e4m3(__uint_as_float(ww[i] & 0xFFFF0000u), scale, inv_scale);
    const uint16_t q = static_cast<uint16_t>(
        __nv_cvt_float2_to_fp8x2(make_float2(lo, hi), __NV_SATFINITE, __NV_E4M3));
    h[i] = e4m3x2_to_half2(q);
  }
  const uint64_t c16 = c / 2;
  *reinterpret_cast<uint4*>(xs + (c16 / 32) * 512 + (c % 2) * 256 + (c16 % 32) * 8) =
      make_uint4(h[0], h[1], h[2], h[3]);
}
__device__ __forceinline__ float chunk_amax(const uint4& v) {
  const uint32_t ww[4] = {v.x, v.y, v.z, v.w};
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    amax = fmaxf(amax, fabsf(__uint_as_float(ww[i] << 16)));
    amax = fmaxf(amax, fabsf(__uint_as_float(ww[i] & 0xFFFF0000u)));
  }
  return amax;
}

// Quantizes a bf16 activation per token inside the CTA (same arithmetic as the standalone FP8
// quantizer: scale = amax/448, q = E4M3(x/scale), src/numeric/fp8.cpp:41-58) and stages the
// decoded bytes as fp16.  Returns the token scale.  The first pass keeps up to 16,384 elements
// of loads in flight at once; the second pass re-reads the token from L1.
template <int kW>
__device__ __forceinline__ float stage_bf16_activation(const uint16_t* x, uint64_t k, __half* xs,
                                                       float* red) {
  constexpr int kBatch = 8;  // 8 chunks x 256 threads x 8 elements = 16,384 per batch
  const uint64_t chunks = k / 8;
  const uint4* xp = reinterpret_cast<const uint4*>(x);
  float amax = 0.0f;
  for (uint64_t base = threadIdx.x; base < chunks; base += static_cast<uint64_t>(kBatch) * (kW * 32)) {
    uint4 v[kBatch];
#pragma unroll
    for (int i = 0; i < kBatch; ++i) {
      const uint64_t c = base + static_cast<uint64_t>(i) * (kW * 32);
      v[i] = c < chunks ? __ldg(xp + c) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int i = 0; i < kBatch; ++i) amax = fmaxf(amax, chunk_amax(v[i]));
  }
  amax = warp_max(amax);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = red[0];
#pragma unroll
  for (int i = 1; i < kW; ++i) amax = fmaxf(amax, red[i]);
  const float scale = amax == 0.0f ? 1.0f : __fdiv_rn(amax, 448.0f);
  const float inv_scale = __frcp_rn(scale);
  // Second pass: the token was just read by this CTA, so these loads hit L1.
  for (uint64_t base = threadIdx.x; base < chunks; base += 4ull * (kW * 32)) {
    uint4 v[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint64_t c = base + static_cast<uint64_t>(i) * (kW * 32);
      v[i] = c < chunks ? __ldg(xp + c) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint64_t c = base + static_cast<uint64_t>(i) * (kW * 32);
      if (c < chunks) stage_bf16_chunk(v[i], c, scale, inv_scale, xs);
    }
  }
  zero_fp8_staging_tail<kW>(k, xs);
  return scale;
}

// Persistent FP8 GEMV.  The grid is one wave of CTAs (SM count x resident CTAs per SM); warp
// (cta, w) owns tasks cta*8 + w, + gridDim*8, ...; task t covers virtual rows [t*kRows,
// (t+1)*kRows).  Per task the warp walks K in steps of kUnroll 512-byte segments, issuing all
// kRows*kUnroll 128-bit loads of a step (predicated at the K tail) before it consumes them.
// The first step of the first task is issued before the activation is staged, so the HBM
// pipeline fills while the CTA quantizes / decodes the activation.
// Warps per CTA.  (One 24-warp CTA per SM for the fused-quantisation variant, so that the
// activation is quantised once per SM, measured slower than three 8-warp CTAs: the prologue is
// bound by its dependent global round trips, not by instruction issue.)
template <bool kFusedQuant>
__host__ __device__ constexpr int fp8_gemv_warps() { return kWarps; }

template <int kRows, int kUnroll, bool kFusedQuant, bool kBf16Out>
__global__ void __launch_bounds__(fp8_gemv_warps<kFusedQuant>() * 32, kFusedQuant ? 3 : 4)
fp8_gemv_kernel(const void* __restrict__ act, const float* __restrict__ act_scale,
                const __grid_constant__ Fp8Group grp, uint64_t k) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __half* xs = reinterpret_cast<__half*>(smem_raw);
  constexpr int kW = fp8_gemv_warps<kFusedQuant>();
  __shared__ float red[kW];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint64_t total_rows = grp.row_start[grp.n];
  const uint64_t num_tasks = (total_rows + kRows - 1) / kRows;
  const uint64_t task_stride = static_cast<uint64_t>(gridDim.x) * kW;
  const uint64_t step = 512ull * kUnroll;

  auto row_pointer = [&](uint64_t vrow) -> const uint8_t* {
    if (vrow >= total_rows) vrow = total_rows - 1;
    int pi = 0;
    while (pi + 1 < grp.n && vrow >= grp.row_start[pi + 1]) ++pi;
    return grp.p[pi].w + (vrow - grp.row_start[pi]) * k;
  };
  uint4 wv[kUnroll][kRows];
  auto load_step = [&](uint64_t task, uint64_t kb) {
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
      const uint8_t* wp = row_pointer(task * kRows + r) + kb + lane * 16;
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        if (kb + u * 512 + lane * 16 < k) wv[u][r] = ldg_stream(wp + u * 512);
        else wv[u][r] = make_uint4(0, 0, 0, 0);
      }
    }
  };

  // Programmatic dependent launch: let the next kernel in the stream start its own weight
  // prefetch as soon as SM slots free up; weights are immutable so they may be read before the
  // previous kernel has finished, everything else waits for it.
  asm volatile("griddepcontrol.launch_dependents;");
  uint64_t task = static_cast<uint64_t>(blockIdx.x) * kW + warp;
  bool prefetched = false;
  if (task < num_tasks) {
    load_step(task, 0);
    prefetched = true;
  }
  asm volatile("griddepcontrol.wait;" ::: "memory");

  float a_scale;
  if constexpr (kFusedQuant) {
    a_scale = stage_bf16_activation<kW>(static_cast<const uint16_t*>(act), k, xs, red);
  } else {
    stage_fp8_activation<kW>(static_cast<const uint8_t*>(act), k, xs);
    a_scale = __ldg(act_scale);
  }
  __syncthreads();

  for (; task < num_tasks; task += task_stride) {
    float acc[kRows];
#pragma unroll
    for (int r = 0; r < kRows; ++r) acc[r] = 0.0f;
    for (uint64_t kb = 0; kb < k; kb += step) {
      if (!prefetched) load_step(task, kb);
      prefetched = false;
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        if (kb + u * 512 < k) {  // warp-uniform; lanes past K hold zero weights
          const __half* xp = xs + kb + u * 512 + lane * 8;
          const uint4 xa = *reinterpret_cast<const uint4*>(xp), xb = *reinterpret_cast<const uint4*>(xp + 256);
#pragma unroll
          for (int r = 0; r < kRows; ++r) dot16_fp8(acc[r], wv[u][r], xa, xb);
        }
      }
    }
#pragma unroll
    for (int r = 0; r < kRows; ++r) acc[r] = warp_sum(acc[r]);
    if (lane == 0) {
#pragma unroll
      for (int r = 0; r < kRows; ++r) {
        const uint64_t vrow = task * kRows + r;
        if (vrow < total_rows) {
          int pi = 0;
          while (pi + 1 < grp.n && vrow >= grp.row_start[pi + 1]) ++pi;
          const uint64_t row = vrow - grp.row_start[pi];
          // (acc * a_scale) * w_scale, in that order: src/cuda/fp8/sm120.cu:234-239.
          const float ws = bf16_bits_to_float(__ldg(grp.p[pi].w_scales + row));
          const float y = __fmul_rn(__fmul_rn(acc[r], a_scale), ws);
          if constexpr (kBf16Out) static_cast<uint16_t*>(grp.p[pi].out)[row] = float_to_bf16_bits(y);
          else static_cast<float*>(grp.p[pi].out)[row] = y;
        }
      }
    }
  }
}


// Rows per warp task.  One row per task keeps tasks fine-grained (best balance over the
// persistent grid) and measured fastest on every decode shape; 2 and 4 remain selectable.
int pick_rows_per_warp(uint64_t total_rows, uint64_t k) {
  if (g_rows_override == 1 || g_rows_override == 2 || g_rows_override == 4) return g_rows_override;
  (void)total_rows;
  (void)k;
  return 1;
}

template <int kRows, int kUnroll, bool kFusedQuant, bool kBf16Out>
int32_t launch_fp8_gemv_variant(const char* op, const void* act, const float* act_scale,
                                const Fp8Group& grp, uint64_t k, cudaStream_t stream) {
  constexpr int kW = fp8_gemv_warps<kFusedQuant>();
  auto kern = fp8_gemv_kernel<kRows, kUnroll, kFusedQuant, kBf16Out>;
  const size_t smem = (k + 511) / 512 * 512 * sizeof(__half);
  static int resident[64] = {0};      // CTAs per SM, per device, for the smem size last seen
  static size_t resident_smem[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  dev &= 63;
  if (resident[dev] == 0 || smem != resident_smem[dev]) {
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           static_cast<int>(smem));
      if (e != cudaSuccess)
        return fail(GEMB_INTERNAL, "%s: %s: %s", op, cudaGetErrorName(e), cudaGetErrorString(e));
    }
    int occ = 0;
    cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, kW * 32, smem);
    if (e != cudaSuccess || occ < 1)
      return fail(GEMB_INTERNAL, "%s: occupancy query failed: %s", op, cudaGetErrorName(e));
    resident[dev] = occ;
    resident_smem[dev] = smem;
  }
  const uint64_t tasks = (grp.row_start[grp.n] + kRows - 1) / kRows;
  const uint64_t wave = static_cast<uint64_t>(sm_count()) * resident[dev];
  const unsigned blocks = static_cast<unsigned>(std::min<uint64_t>((tasks + kW - 1) / kW, wave));
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(blocks);
  cfg.blockDim = dim3(kW * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = g_pdl ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t le = cudaLaunchKernelEx(&cfg, kern, act, act_scale, grp, k);
  if (le != cudaSuccess) {
    cudaGetLastError();
    return fail(GEMB_INTERNAL, "%s: %s: %s", op, cudaGetErrorName(le), cudaGetErrorString(le));
  }
  return check_launch(op);
}

// ---------------------------------------------------------------------------------------------
// Small-batch FP8 GEMV (2..8 tokens): the speculative-decoding verifier's projections.  Same
// stream over the weights as the single-token kernel -- the matrix is read once -- with kTok
// staged activations and kTok accumulators per row; a tensor-core tile would be 97 % padding
// at these sizes and the launch is bound by HBM either way.  Output fp32 [tokens, rows] per
// problem, (acc * a_scale[t]) * w_scale in that order like the single-token kernel.
// ---------------------------------------------------------------------------------------------
template <int kTok>
__global__ void __launch_bounds__(kWarps * 32)
fp8_gemv_batch_kernel(const uint8_t* __restrict__ act, const float* __restrict__ act_scales,
                      const __grid_constant__ Fp8Group grp, uint64_t k) {
  constexpr int kUnroll = 8 / (kTok > 4 ? 2 : 1);   // 16-byte loads in flight per lane: 8, or 4 with many tokens (registers)
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __half* xs = reinterpret_cast<__half*>(smem_raw);   // [kTok][k padded to 512]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint64_t k_pad = (k + 511) / 512 * 512;
  const uint64_t total_rows = grp.row_start[grp.n];
  const uint64_t task_stride = static_cast<uint64_t>(gridDim.x) * kWarps;
  const uint64_t step = 512ull * kUnroll;
  auto row_pointer = [&](uint64_t vrow) -> const uint8_t* {
    if (vrow >= total_rows) vrow = total_rows - 1;
    int pi = 0;
    while (pi + 1 < grp.n && vrow >= grp.row_start[pi + 1]) ++pi;
    return grp.p[pi].w + (vrow - grp.row_start[pi]) * k;
  };
  uint4 wv[kUnroll];
  auto load_step = [&](uint64_t task, uint64_t kb) {
    const uint8_t* wp = row_pointer(task) + kb + lane * 16;
#pragma unroll
    for (int u = 0; u < kUnroll; ++u)
      wv[u] = kb + u * 512 + lane * 16 < k ? ldg_stream(wp + u * 512) : make_uint4(0, 0, 0, 0);
  };
  asm volatile("griddepcontrol.launch_dependents;");
  uint64_t task = static_cast<uint64_t>(blockIdx.x) * kWarps + warp;
  bool prefetched = false;
  if (task < total_rows) {
    load_step(task, 0);
    prefetched = true;
  }
  asm volatile("griddepcontrol.wait;" ::: "memory");
#pragma unroll 1
  for (int t = 0; t < kTok; ++t) stage_fp8_activation<kWarps>(act + static_cast<uint64_t>(t) * k, k, xs + t * k_pad);
  float a_scale[kTok];
#pragma unroll
  for (int t = 0; t < kTok; ++t) a_scale[t] = __ldg(act_scales + t);
  __syncthreads();
  for (; task < total_rows; task += task_stride) {
    float acc[kTok];
#pragma unroll
    for (int t = 0; t < kTok; ++t) acc[t] = 0.0f;
    for (uint64_t kb = 0; kb < k; kb += step) {
      if (!prefetched) load_step(task, kb);
      prefetched = false;
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        if (kb + u * 512 < k) {  // warp-uniform; lanes past K hold zero weights
#pragma unroll
          for (int t = 0; t < kTok; ++t) {
            const __half* xp = xs + t * k_pad + kb + u * 512 + lane * 8;
            const uint4 xa = *reinterpret_cast<const uint4*>(xp), xb = *reinterpret_cast<const uint4*>(xp + 256);
            dot16_fp8(acc[t], wv[u], xa, xb);
          }
        }
      }
    }
#pragma unroll
    for (int t = 0; t < kTok; ++t) acc[t] = warp_sum(acc[t]);
    if (lane == 0) {
      int pi = 0;
      while (pi + 1 < grp.n && task >= grp.row_start[pi + 1]) ++pi;
      const uint64_t row = task - grp.row_start[pi];
      const uint64_t rows = grp.p[pi].rows;
      const float ws = bf16_bits_to_float(__ldg(grp.p[pi].w_scales + row));
#pragma unroll
      for (int t = 0; t < kTok; ++t)
        static_cast<float*>(grp.p[pi].out)[static_cast<uint64_t>(t) * rows + row] = __fmul_rn(__fmul_rn(acc[t], a_scale[t]), ws);
    }
  }
}

template <int kTok>
int32_t launch_fp8_gemv_batch_variant(const char* op, const uint8_t* act, const float* act_scales, const Fp8Group& grp,
                                      uint64_t k, cudaStream_t stream) {
  auto kern = fp8_gemv_batch_kernel<kTok>;
  const size_t smem = static_cast<size_t>(kTok) * ((k + 511) / 512 * 512) * sizeof(__half);
  static int resident[64] = {0};
  static size_t resident_smem[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  dev &= 63;
  if (resident[dev] == 0 || smem != resident_smem[dev]) {
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
      if (e != cudaSuccess) return fail(GEMB_INTERNAL, "%s: %s: %s", op, cudaGetErrorName(e), cudaGetErrorString(e));
    }
    int occ = 0;
    cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, kWarps * 32, smem);
    if (e != cudaSuccess || occ < 1) return fail(GEMB_INTERNAL, "%s: occupancy query failed: %s", op, cudaGetErrorName(e));
    resident[dev] = occ;
    resident_smem[dev] = smem;
  }
  const uint64_t tasks = grp.row_start[grp.n];
  const uint64_t wave = static_cast<uint64_t>(sm_count()) * resident[dev];
  const unsigned blocks = static_cast<unsigned>(std::min<uint64_t>((tasks + kWarps - 1) / kWarps, wave));
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(blocks);
  cfg.blockDim = dim3(kWarps * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = g_pdl ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t le = cudaLaunchKernelEx(&cfg, kern, act, act_scales, grp, k);
  if (le != cudaSuccess) {
    cudaGetLastError();
    return fail(GEMB_INTERNAL, "%s: %s: %s", op, cudaGetErrorName(le), cudaGetErrorString(le));
  }
  return check_launch(op);
}

// ---------------------------------------------------------------------------------------------
// Small-batch FP8 GEMV on the warp-level tensor-core path (mma.sync m16n8k32, E4M3 x E4M3 -> fp32):
// 2..8 tokens share one pass over the weights at the streaming rate of the single-token kernel.
// With more than two or three tokens the SIMT form above is bound by its dot-product arithmetic
// (one mixed fma per token and weight); here the weights are the M side of the MMA (row-major
// weights are the "row" A operand as they lie in memory) and the tokens its N = 8 columns, so the
// arithmetic is one MMA per 16 rows x 32 k whatever the token count.
//
// A CTA takes 16 weight rows; its eight warps split K in 256-byte spans, round robin, and their
// partial sums meet in shared memory in warp order.  That keeps every warp of the GPU loading even
// when a projection has few rows (3,840 rows are 240 CTAs), which a warp-per-16-rows split does not.
//
// Fragment mapping (lane = 4 g + t): the lane loads 16 contiguous bytes of rows g and g + 8 at k
// offset 16 t of a 64-byte piece -- four lanes cover 64 contiguous bytes of a row, eight rows per
// load instruction.  Those 2 x 16 bytes feed two MMAs: MMA j takes bytes [8 j, 8 j + 4) of each
// load as a0 / a1 and bytes [8 j + 4, 8 j + 8) as a2 / a3.  That permutes k inside the piece
// relative to the instruction's canonical order, which is harmless as long as the B operand uses
// the same permutation: b0 / b1 of the lane are the 8 activation bytes of token g at the same k
// offset (16 t + 8 j), half of one 16-byte load of the token's row (the activations, at most 8 x K
// bytes, stay in L1; the weights stream past it).  Accumulators c0 / c1 belong to row g and tokens
// 2 t, 2 t + 1, c2 / c3 to row g + 8.  The result differs from the single-token kernel's only in the
// order of the fp32 additions.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void mma_e4m3_m16n8k32(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                   uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

constexpr int kMmaPieces = 4;                  // 64-byte pieces per span: eight 16-byte weight loads in flight per lane
constexpr int kMmaSpan = kMmaPieces * 64;      // bytes of K one warp takes per step

__global__ void __launch_bounds__(kWarps * 32, 3)
fp8_gemv_mma_kernel(const uint8_t* __restrict__ act, const float* __restrict__ act_scales,
                    const __grid_constant__ Fp8Group grp, uint64_t k, uint32_t tokens) {
  __shared__ float4 partial[kWarps][32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
  const uint64_t total_rows = grp.row_start[grp.n];
  const uint64_t num_tasks = (total_rows + 15) / 16;
  auto row_pointer = [&](uint64_t vrow) -> const uint8_t* {
    if (vrow >= total_rows) vrow = total_rows - 1;
    int pi = 0;
    while (pi + 1 < grp.n && vrow >= grp.row_start[pi + 1]) ++pi;
    return grp.p[pi].w + (vrow - grp.row_start[pi]) * k;
  };
  uint4 wa[kMmaPieces], wb[kMmaPieces];
  auto load_span = [&](const uint8_t* ra, const uint8_t* rb, uint64_t kb) {
#pragma unroll
    for (int u = 0; u < kMmaPieces; ++u) {
      const uint64_t off = kb + u * 64 + t4 * 16;
      const bool in = off < k;
      wa[u] = in ? ldg_stream(ra + off) : make_uint4(0, 0, 0, 0);
      wb[u] = in ? ldg_stream(rb + off) : make_uint4(0, 0, 0, 0);
    }
  };
  asm volatile("griddepcontrol.launch_dependents;");
  uint64_t task = blockIdx.x;
  const uint64_t first_kb = static_cast<uint64_t>(warp) * kMmaSpan;
  const uint8_t* ra = nullptr;
  const uint8_t* rb = nullptr;
  bool prefetched = false;
  if (task < num_tasks && first_kb < k) {   // the weights do not depend on the kernel before this one
    ra = row_pointer(task * 16 + g);
    rb = row_pointer(task * 16 + g + 8);
    load_span(ra, rb, first_kb);
    prefetched = true;
  }
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const bool token_live = static_cast<uint32_t>(g) < tokens;   // B column g = token g; columns past the batch are zero
  const uint8_t* xrow = act + static_cast<uint64_t>(token_live ? g : 0) * k + t4 * 16;
  const float s0 = 2 * t4 < static_cast<int>(tokens) ? __ldg(act_scales + 2 * t4) : 0.0f;
  const float s1 = 2 * t4 + 1 < static_cast<int>(tokens) ? __ldg(act_scales + 2 * t4 + 1) : 0.0f;
  for (; task < num_tasks; task += gridDim.x) {
    if (!prefetched) {
      ra = row_pointer(task * 16 + g);
      rb = row_pointer(task * 16 + g + 8);
    }
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    for (uint64_t kb = first_kb; kb < k; kb += static_cast<uint64_t>(kWarps) * kMmaSpan) {
      if (!prefetched) load_span(ra, rb, kb);
      prefetched = false;
#pragma unroll
      for (int u = 0; u < kMmaPieces; ++u) {
        if (kb + u * 64 < k) {   // warp-uniform; K is a multiple of 16, lanes past it hold zero weights
          uint4 xv = make_uint4(0, 0, 0, 0);
          if (token_live && kb + u * 64 + t4 * 16 < k) xv = __ldg(reinterpret_cast<const uint4*>(xrow + kb + u * 64));
          mma_e4m3_m16n8k32(acc, wa[u].x, wb[u].x, wa[u].y, wb[u].y, xv.x, xv.y);
          mma_e4m3_m16n8k32(acc, wa[u].z, wb[u].z, wa[u].w, wb[u].w, xv.z, xv.w);
        }
      }
    }
    __syncthreads();   // the previous task's sums have been read
    partial[warp][lane] = make_float4(acc[0], acc[1], acc[2], acc[3]);
    __syncthreads();
    if (warp == 0) {
      float4 sum = partial[0][lane];
#pragma unroll
      for (int w = 1; w < kWarps; ++w) {   // warp order: the same sum on every launch
        const float4 v = partial[w][lane];
        sum.x = __fadd_rn(sum.x, v.x);
        sum.y = __fadd_rn(sum.y, v.y);
        sum.z = __fadd_rn(sum.z, v.z);
        sum.w = __fadd_rn(sum.w, v.w);
      }
      // (acc * a_scale) * w_scale, in that order: src/cuda/fp8/sm120.cu:234-239.
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const uint64_t vrow = task * 16 + g + 8 * half;
        if (vrow >= total_rows) continue;
        int pi = 0;
        while (pi + 1 < grp.n && vrow >= grp.row_start[pi + 1]) ++pi;
        const uint64_t row = vrow - grp.row_start[pi];
        const float ws = bf16_bits_to_float(__ldg(grp.p[pi].w_scales + row));
        float* out = static_cast<float*>(grp.p[pi].out);
        const float c0 = half ? sum.z : sum.x, c1 = half ? sum.w : sum.y;
        if (2 * t4 < static_cast<int>(tokens)) out[static_cast<uint64_t>(2 * t4) * grp.p[pi].rows + row] = __fmul_rn(__fmul_rn(c0, s0), ws);
        if (2 * t4 + 1 < static_cast<int>(tokens))
          out[static_cast<uint64_t>(2 * t4 + 1) * grp.p[pi].rows + row] = __fmul_rn(__fmul_rn(c1, s1), ws);
      }
    }
  }
}

int32_t launch_fp8_gemv_mma(const char* op, const uint8_t* act, const float* act_scales, const Fp8Group& grp,
                            uint64_t tokens, uint64_t k, cudaStream_t stream) {
  const uint64_t tasks = (grp.row_start[grp.n] + 15) / 16;
  const unsigned blocks = static_cast<unsigned>(std::min<uint64_t>(tasks, static_cast<uint64_t>(sm_count()) * 3));
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(blocks);
  cfg.blockDim = dim3(kWarps * 32);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = g_pdl ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t le = cudaLaunchKernelEx(&cfg, fp8_gemv_mma_kernel, act, act_scales, grp, k, static_cast<uint32_t>(tokens));
  if (le != cudaSuccess) {
    cudaGetLastError();
    return fail(GEMB_INTERNAL, "%s: %s: %s", op, cudaGetErrorName(le), cudaGetErrorString(le));
  }
  return check_launch(op);
}

int32_t launch_fp8_gemv_batch(const char* op, const uint8_t* act, const float* act_scales, const Fp8Group& grp,
                              uint64_t tokens, uint64_t k, cudaStream_t stream) {
  // Tensor-core form by default; GEMB_TUNE_GEMV_IMPL = 1 keeps the SIMT form, whose per-token results
  // are bit-identical to the single-token kernel.
  if (g_gemv_impl != 1) return launch_fp8_gemv_mma(op, act, act_scales, grp, tokens, k, stream);
  switch (tokens) {
    case 2: return launch_fp8_gemv_batch_variant<2>(op, act, act_scales, grp, k, stream);
    case 3: return launch_fp8_gemv_batch_variant<3>(op, act, act_scales, grp, k, stream);
    case 4: return launch_fp8_gemv_batch_variant<4>(op, act, act_scales, grp, k, stream);
    case 5: return launch_fp8_gemv_batch_variant<5>(op, act, act_scales, grp, k, stream);
    case 6: return launch_fp8_gemv_batch_variant<6>(op, act, act_scales, grp, k, stream);
    case 7: return launch_fp8_gemv_batch_variant<7>(op, act, act_scales, grp, k, stream);
    default: return launch_fp8_gemv_batch_variant<8>(op, act, act_scales, grp, k, stream);
  }
}

// ---------------------------------------------------------------------------------------------
// FP8 GEMV with a bulk-copy ring.  One persistent CTA per SM: warp 0 is the producer, sixteen
// consumer warps follow.  The weight matrix is cut into chunks of whole rows (about 16 KB); the
// producer streams chunk after chunk into a ring of shared-memory stages with 1-D bulk copies
// (cp.async.bulk, completion on an mbarrier), so the bytes in flight are bounded by shared
// memory (about 190 KB per SM), not by registers, and keep flowing while the consumers quantise
// the activation or wait for the previous kernel (weights are immutable, so the producer starts
// before griddepcontrol.wait).  Consumer warp w owns stage w, i.e. the CTA's chunks w, w+12, ...
// (an mbarrier parity wait may run at most one phase ahead, so a warp must see every phase of
// the stages it waits on): it dots every row of the chunk from shared memory and releases the
// stage.
// ---------------------------------------------------------------------------------------------
constexpr int kRingConsumers = 12;   // also the ring depth: consumer w owns stage w
constexpr int kRingThreads = 32 * (1 + kRingConsumers);
constexpr uint32_t kRingStageBytes = 16384;

struct RingTask {
  const uint8_t* src;
  uint32_t first_vrow, rows;
};

__device__ __forceinline__ void zero_fp8_staging_tail_n(uint64_t k, __half* xs, int tid, int nthreads) {
  const uint64_t chunks = k / 16, chunks_pad = (k + 511) / 512 * 32;
  for (uint64_t c = chunks + tid; c < chunks_pad; c += nthreads) {
    __half* dst = xs + (c / 32) * 512 + (c % 32) * 8;
    *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
    *reinterpret_cast<uint4*>(dst + 256) = make_uint4(0, 0, 0, 0);
  }
}

template <bool kFusedQuant, bool kBf16Out>
__global__ void __launch_bounds__(kRingThreads, 1)
fp8_gemv_ring_kernel(const void* __restrict__ act, const float* __restrict__ act_scale,
                     const __grid_constant__ Fp8Group grp, uint32_t k, uint32_t rows_per_chunk,
                     uint32_t stages) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const uint32_t k_pad = (k + 511) / 512 * 512;
  __half* xs = reinterpret_cast<__half*>(smem_raw);
  unsigned char* ring = smem_raw + ((k_pad * 2 + 127) / 128) * 128;
  uint64_t* full = reinterpret_cast<uint64_t*>(ring + static_cast<size_t>(stages) * kRingStageBytes);
  uint64_t* empty = full + stages;
  float* red = reinterpret_cast<float*>(empty + stages);      // [kRingConsumers]
  volatile int* abort_flag = reinterpret_cast<volatile int*>(red + kRingConsumers);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (uint32_t s = 0; s < stages; ++s) {
      ptx::mbar_init(&full[s], 1);
      ptx::mbar_init(&empty[s], 1);
    }
    *abort_flag = 0;
    ptx::fence_barrier_init();
  }
  __syncthreads();
  asm volatile("griddepcontrol.launch_dependents;");

  // Chunk j of this CTA is global chunk blockIdx.x + j * gridDim.x.  Chunks never straddle two
  // problems of a grouped launch: each problem is cut separately.
  uint32_t chunk_start[4];
  chunk_start[0] = 0;
  for (int i = 0; i < grp.n; ++i)
    chunk_start[i + 1] = chunk_start[i] + static_cast<uint32_t>((grp.p[i].rows + rows_per_chunk - 1) / rows_per_chunk);
  const uint32_t total_chunks = chunk_start[grp.n];
  auto task_of = [&](uint32_t chunk) {
    int pi = 0;
    while (pi + 1 < grp.n && chunk >= chunk_start[pi + 1]) ++pi;
    const uint32_t row0 = (chunk - chunk_start[pi]) * rows_per_chunk;
    RingTask t;
    t.rows = min(rows_per_chunk, static_cast<uint32_t>(grp.p[pi].rows) - row0);
    t.src = grp.p[pi].w + static_cast<uint64_t>(row0) * k;
    t.first_vrow = static_cast<uint32_t>(grp.row_start[pi]) + row0;
    return t;
  };
  const uint32_t my_chunks = blockIdx.x < total_chunks ? (total_chunks - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;

  if (warp == 0) {
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      for (uint32_t j = 0; j < my_chunks && !*abort_flag; ++j) {
        if (!ptx::mbar_wait(&empty[stage], phase ^ 1, 1u << 18)) {
          atomicCAS(&g_gemv_error, 0, 1);
          *abort_flag = 1;
          break;
        }
        const RingTask t = task_of(blockIdx.x + j * gridDim.x);
        const uint32_t bytes = t.rows * k;
        ptx::mbar_expect_tx(&full[stage], bytes);
        ptx::bulk_load_1d(ring + static_cast<size_t>(stage) * kRingStageBytes, t.src, bytes, &full[stage]);
        if (++stage == stages) { stage = 0; phase ^= 1; }
      }
    }
  } else {
    // Everything that is not an immutable weight is read only after the previous kernel is done.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int ctid = threadIdx.x - 32, cthreads = kRingConsumers * 32;
    float a_scale;
    if constexpr (kFusedQuant) {
      const uint16_t* x = static_cast<const uint16_t*>(act);
      const uint4* xp = reinterpret_cast<const uint4*>(x);
      const uint32_t chunks8 = k / 8;
      float amax = 0.0f;
      for (uint32_t base = ctid; base < chunks8; base += 4u * cthreads) {
        uint4 v[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint32_t c = base + i * cthreads;
          v[i] = c < chunks8 ? __ldg(xp + c) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) amax = fmaxf(amax, chunk_amax(v[i]));
      }
      amax = warp_max(amax);
      if (lane == 0) red[warp - 1] = amax;
      asm volatile("bar.sync 1, %0;" ::"n"(kRingConsumers * 32));
      amax = red[0];
#pragma unroll
      for (int i = 1; i < kRingConsumers; ++i) amax = fmaxf(amax, red[i]);
      a_scale = amax == 0.0f ? 1.0f : __fdiv_rn(amax, 448.0f);
      const float inv_scale = __frcp_rn(a_scale);
      for (uint32_t c = ctid; c < chunks8; c += cthreads) stage_bf16_chunk(__ldg(xp + c), c, a_scale, inv_scale, xs);
    } else {
      const uint8_t* a8 = static_cast<const uint8_t*>(act);
      for (uint32_t c = ctid; c < k / 16; c += cthreads) {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(a8) + c);
        const uint32_t ww[4] = {v.x, v.y, v.z, v.w};
        uint32_t h[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          h[2 * i] = e4m3x2_to_half2(static_cast<uint16_t>(ww[i] & 0xFFFFu));
          h[2 * i + 1] = e4m3x2_to_half2(static_cast<uint16_t>(ww[i] >> 16));
        }
        __half* dst = xs + (c / 32) * 512 + (c % 32) * 8;
        *reinterpret_cast<uint4*>(dst) = make_uint4(h[0], h[1], h[2], h[3]);
        *reinterpret_cast<uint4*>(dst + 256) = make_uint4(h[4], h[5], h[6], h[7]);
      }
      a_scale = __ldg(act_scale);
    }
    zero_fp8_staging_tail_n(k, xs, ctid, cthreads);
    asm volatile("bar.sync 1, %0;" ::"n"(kRingConsumers * 32));

    const uint32_t cw = warp - 1;
    for (uint32_t j = cw; j < my_chunks && !*abort_flag; j += kRingConsumers) {
      const uint32_t stage = j % stages, phase = (j / stages) & 1;
      if (!ptx::mbar_wait(&full[stage], phase, 1u << 18)) {
        atomicCAS(&g_gemv_error, 0, 2);
        *abort_flag = 1;
        break;
      }
      const RingTask t = task_of(blockIdx.x + j * gridDim.x);
      const unsigned char* sw = ring + static_cast<size_t>(stage) * kRingStageBytes;
      // Two rows at a time, each with two accumulators (even / odd 512-byte segment): four
      // independent fma chains per lane, and the staged activation is read once per row pair.
      for (uint32_t r = 0; r < t.rows; r += 2) {
        const bool two = r + 1 < t.rows;
        const unsigned char* row0 = sw + static_cast<size_t>(r) * k;
        const unsigned char* row1 = row0 + k;
        float acc[2][2] = {{0.0f, 0.0f}, {0.0f, 0.0f}};
        uint32_t kk = lane * 16;
        for (; kk + 512 < k; kk += 1024) {
          const __half* xp = xs + (kk / 512) * 512 + lane * 8;
          const uint4 xa0 = *reinterpret_cast<const uint4*>(xp), xb0 = *reinterpret_cast<const uint4*>(xp + 256);
          const uint4 xa1 = *reinterpret_cast<const uint4*>(xp + 512), xb1 = *reinterpret_cast<const uint4*>(xp + 768);
          const uint4 w00 = *reinterpret_cast<const uint4*>(row0 + kk), w01 = *reinterpret_cast<const uint4*>(row0 + kk + 512);
          uint4 w10 = w00, w11 = w01;
          if (two) {
            w10 = *reinterpret_cast<const uint4*>(row1 + kk);
            w11 = *reinterpret_cast<const uint4*>(row1 + kk + 512);
          }
          dot16_fp8(acc[0][0], w00, xa0, xb0);
          dot16_fp8(acc[0][1], w01, xa1, xb1);
          if (two) {  // warp-uniform
            dot16_fp8(acc[1][0], w10, xa0, xb0);
            dot16_fp8(acc[1][1], w11, xa1, xb1);
          }
        }
        if (kk < k) {  // odd number of segments (or a ragged last one): one more for this lane
          const __half* xp = xs + (kk / 512) * 512 + lane * 8;
          const uint4 xa0 = *reinterpret_cast<const uint4*>(xp), xb0 = *reinterpret_cast<const uint4*>(xp + 256);
          dot16_fp8(acc[0][0], *reinterpret_cast<const uint4*>(row0 + kk), xa0, xb0);
          if (two) dot16_fp8(acc[1][0], *reinterpret_cast<const uint4*>(row1 + kk), xa0, xb0);
        }
        float y0 = warp_sum(acc[0][0] + acc[0][1]);
        float y1 = warp_sum(acc[1][0] + acc[1][1]);
        if (lane < (two ? 2 : 1)) {
          const uint32_t vrow = t.first_vrow + r + lane;
          int pi = 0;
          while (pi + 1 < grp.n && vrow >= grp.row_start[pi + 1]) ++pi;
          const uint64_t orow = vrow - grp.row_start[pi];
          // (acc * a_scale) * w_scale, in that order: src/cuda/fp8/sm120.cu:234-239.
          const float ws = bf16_bits_to_float(__ldg(grp.p[pi].w_scales + orow));
          const float y = __fmul_rn(__fmul_rn(lane == 0 ? y0 : y1, a_scale), ws);
          if constexpr (kBf16Out) static_cast<uint16_t*>(grp.p[pi].out)[orow] = float_to_bf16_bits(y);
          else static_cast<float*>(grp.p[pi].out)[orow] = y;
        }
      }
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&empty[stage]);
    }
  }
  __syncthreads();
  if (*abort_flag) {
    // give bulk copies still in flight a bounded time to land before the CTA's memory is reused
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
}

template <bool kFusedQuant, bool kBf16Out>
int32_t launch_fp8_gemv_ring(const char* op, const void* act, const float* act_scale, const Fp8Group& grp,
                             uint64_t k, cudaStream_t stream, bool* launched) {
  *launched = false;
  const uint32_t rows_per_chunk = static_cast<uint32_t>(kRingStageBytes / k);
  // Measured: the ring hides the fused-quantisation prologue (it wins for K = 15360 in isolation)
  // but is slower than direct loads on the short-K shapes, and alternating the two in one decode
  // pass costs more than it gains (their shared-memory footprints differ, so consecutive kernels
  // cannot overlap).  The direct kernel is therefore the default; the ring runs on request.
  if (rows_per_chunk == 0 || g_gemv_impl != 2) return GEMB_OK;
  const size_t x_bytes = ((k + 511) / 512 * 512 * 2 + 127) / 128 * 128;
  const size_t fixed = x_bytes + 2 * 16 * 8 + kRingConsumers * 4 + 64;
  const size_t budget = 227 * 1024 - 1024;
  if (fixed + static_cast<size_t>(kRingConsumers) * kRingStageBytes > budget) return GEMB_OK;
  const uint32_t stages = kRingConsumers;
  const size_t smem = x_bytes + static_cast<size_t>(stages) * kRingStageBytes + 2 * stages * 8 + kRingConsumers * 4 + 64;
  auto kern = fp8_gemv_ring_kernel<kFusedQuant, kBf16Out>;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  dev &= 63;
  if (!configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return fail(GEMB_INTERNAL, "%s: %s: %s", op, cudaGetErrorName(e), cudaGetErrorString(e));
    configured[dev] = true;
  }
  uint64_t chunks = 0;
  for (int i = 0; i < grp.n; ++i) chunks += (grp.p[i].rows + rows_per_chunk - 1) / rows_per_chunk;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<unsigned>(std::min<uint64_t>(chunks, static_cast<uint64_t>(sm_count()))));
  cfg.blockDim = dim3(kRingThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = g_pdl ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t le = cudaLaunchKernelEx(&cfg, kern, act, act_scale, grp, static_cast<uint32_t>(k), rows_per_chunk, stages);
  if (le != cudaSuccess) {
    cudaGetLastError();
    return fail(GEMB_INTERNAL, "%s: %s: %s", op, cudaGetErrorName(le), cudaGetErrorString(le));
  }
  *launched = true;
  return check_launch(op);
}

template <bool kFusedQuant, bool kBf16Out>
int32_t launch_fp8_gemv(const char* op, const void* act, const float* act_scale, Fp8Group grp,
                        uint64_t k, cudaStream_t stream) {
  uint64_t total_rows = 0;
  for (int i = 0; i < grp.n; ++i) {
    grp.row_start[i] = total_rows;
    total_rows += grp.p[i].rows;
  }
  grp.row_start[grp.n] = total_rows;
  bool launched = false;
  GEMB_TRY((launch_fp8_gemv_ring<kFusedQuant, kBf16Out>(op, act, act_scale, grp, k, stream, &launched)));
  if (launched) return GEMB_OK;
  const int rpw = pick_rows_per_warp(total_rows, k);
  if (rpw == 4) return launch_fp8_gemv_variant<4, 2, kFusedQuant, kBf16Out>(op, act, act_scale, grp, k, stream);
  if (rpw == 2) return launch_fp8_gemv_variant<2, 4, kFusedQuant, kBf16Out>(op, act, act_scale, grp, k, stream);
  return launch_fp8_gemv_variant<1, 8, kFusedQuant, kBf16Out>(op, act, act_scale, grp, k, stream);
}

int32_t validate_fp8_gemv(const char* op, const void* act, const void* w, const void* ws,
                          const void* out, uint64_t rows, uint64_t k) {
  GEMB_REQUIRE(act && w && ws && out, "%s: pointers must be nonnull", op);
  GEMB_REQUIRE(rows > 0 && k > 0, "%s: geometry must be nonzero", op);
  GEMB_REQUIRE(k % 16 == 0, "%s: contracting extent must be a multiple of 16", op);
  GEMB_REQUIRE(k <= 110 * 1024, "%s: contracting extent exceeds the shared-memory staging limit (112640)", op);
  GEMB_REQUIRE(rows < (1ull << 31), "%s: too many rows", op);
  GEMB_REQUIRE(reinterpret_cast<uintptr_t>(act) % 16 == 0 && reinterpret_cast<uintptr_t>(w) % 16 == 0,
               "%s: activation and weight must be 16-byte aligned", op);
  return GEMB_OK;
}

// ---------------------------------------------------------------------------------------------
// NVFP4 GEMV.  Activation staged as fp16 values (decoded E2M1) plus fp32 decoded block scales.
// A lane's 16-byte weight chunk is two 16-element blocks; within a block the sixteen E2M1
// products are summed in fp16 (exact: each product is a multiple of 1/4 no larger than 36, a
// half2 lane sums eight of them, at most 288), then the block sum is scaled by sa*sw in fp32.
// ---------------------------------------------------------------------------------------------
// All four bytes of a word -> four half2.
__device__ __forceinline__ void e2m1x8_to_half2(uint32_t word, uint32_t (&h)[4]) {
  asm("{ .reg .b8 t0, t1, t2, t3;\n"
      "  mov.b32 {t0, t1, t2, t3}, %4;\n"
      "  cvt.rn.f16x2.e2m1x2 %0, t0;\n"
      "  cvt.rn.f16x2.e2m1x2 %1, t1;\n"
      "  cvt.rn.f16x2.e2m1x2 %2, t2;\n"
      "  cvt.rn.f16x2.e2m1x2 %3, t3; }"
      : "=r"(h[0]), "=r"(h[1]), "=r"(h[2]), "=r"(h[3])
      : "r"(word));
}
__device__ __forceinline__ uint32_t hfma2_bits(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ float half2_sum(uint32_t h) {
  const __half2 v = *reinterpret_cast<const __half2*>(&h);
  return __low2float(v) + __high2float(v);
}
// One 16-element block: w bytes (lo, hi words) against 16 staged fp16 activations.
__device__ __forceinline__ float block_dot_fp4(uint32_t w_lo, uint32_t w_hi, const uint4& xa, const uint4& xb) {
  uint32_t h[4];
  uint32_t acc = 0;
  e2m1x8_to_half2(w_lo, h);
  acc = hfma2_bits(h[0], xa.x, acc);
  acc = hfma2_bits(h[1], xa.y, acc);
  acc = hfma2_bits(h[2], xa.z, acc);
  acc = hfma2_bits(h[3], xa.w, acc);
  e2m1x8_to_half2(w_hi, h);
  acc = hfma2_bits(h[0], xb.x, acc);
  acc = hfma2_bits(h[1], xb.y, acc);
  acc = hfma2_bits(h[2], xb.z, acc);
  acc = hfma2_bits(h[3], xb.w, acc);
  return half2_sum(acc);
}

template <int kRows, bool kGateUp>
__global__ void __launch_bounds__(kThreads)
nvfp4_gemv_kernel(const uint8_t* __restrict__ act, const uint8_t* __restrict__ act_scales,
                  const uint8_t* __restrict__ w0, const uint8_t* __restrict__ ws0,
                  const uint8_t* __restrict__ w1, const uint8_t* __restrict__ ws1,
                  float* __restrict__ out0, float* __restrict__ out1, float* __restrict__ product,
                  uint64_t rows, uint64_t k, float div0, float div1) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  // Staged activation: per 1024-element segment (512 weight bytes), lane l's 32 values are
  // stored as four 8-value parts at [p*256 + l*8, +8), p = 0..3 (conflict-free 128-bit loads).
  const uint64_t k_pad = (k + 1023) / 1024 * 1024;
  __half* xs = reinterpret_cast<__half*>(smem_raw);              // k_pad halves
  float* sa = reinterpret_cast<float*>(smem_raw + k_pad * 2);    // k/16 decoded scales
  for (uint64_t c = threadIdx.x; c < k / 32; c += kThreads) {
    const uint4 v = __ldg(reinterpret_cast<const uint4*>(act) + c);  // 32 elements
    const uint32_t ww[4] = {v.x, v.y, v.z, v.w};
    uint32_t h[16];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint32_t t[4];
      e2m1x8_to_half2(ww[i], t);
      h[4 * i] = t[0]; h[4 * i + 1] = t[1]; h[4 * i + 2] = t[2]; h[4 * i + 3] = t[3];
    }
    __half* dst = xs + (c / 32) * 1024 + (c % 32) * 8;
#pragma unroll
    for (int i = 0; i < 4; ++i)
      *reinterpret_cast<uint4*>(dst + i * 256) = make_uint4(h[4 * i], h[4 * i + 1], h[4 * i + 2], h[4 * i + 3]);
  }
  for (uint64_t c = threadIdx.x; c < k / 16; c += kThreads) sa[c] = e4m3_decode(__ldg(act_scales + c));
  __syncthreads();

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint64_t row0 = (static_cast<uint64_t>(blockIdx.x) * kWarps + warp) * kRows;
  if (row0 >= rows) return;
  constexpr int kMats = kGateUp ? 2 : 1;
  const uint64_t row_bytes = k / 2, srow_bytes = k / 16;
  float acc[kMats][kRows];
#pragma unroll
  for (int m = 0; m < kMats; ++m)
#pragma unroll
    for (int r = 0; r < kRows; ++r) acc[m][r] = 0.0f;

  // A lane owns 16 weight bytes = 32 elements = 2 blocks per 512-byte row segment.
  for (uint64_t kb = lane * 16ull; kb < row_bytes; kb += 512) {
    uint4 wv[kMats][kRows];
    uint16_t sv[kMats][kRows];
#pragma unroll
    for (int m = 0; m < kMats; ++m)
#pragma unroll
      for (int r = 0; r < kRows; ++r) {
        const uint64_t row = row0 + r < rows ? row0 + r : rows - 1;
        const uint8_t* wp = (m == 0 ? w0 : w1) + row * row_bytes + kb;
        const uint8_t* sp = (m == 0 ? ws0 : ws1) + row * srow_bytes + kb / 8;
        wv[m][r] = ldg_stream(wp);
        sv[m][r] = __ldg(reinterpret_cast<const uint16_t*>(sp));
      }
    const __half* xp = xs + (kb / 512) * 1024 + lane * 8;
    const uint4 x0 = *reinterpret_cast<const uint4*>(xp), x1 = *reinterpret_cast<const uint4*>(xp + 256),
                x2 = *reinterpret_cast<const uint4*>(xp + 512), x3 = *reinterpret_cast<const uint4*>(xp + 768);
    const float sa0 = sa[kb / 8], sa1 = sa[kb / 8 + 1];
#pragma unroll
    for (int m = 0; m < kMats; ++m)
#pragma unroll
      for (int r = 0; r < kRows; ++r) {
        const float d0 = block_dot_fp4(wv[m][r].x, wv[m][r].y, x0, x1);
        const float d1 = block_dot_fp4(wv[m][r].z, wv[m][r].w, x2, x3);
        const float sw0 = e4m3_decode(static_cast<uint8_t>(sv[m][r] & 0xFF));
        const float sw1 = e4m3_decode(static_cast<uint8_t>(sv[m][r] >> 8));
        acc[m][r] = fmaf(d0, sa0 * sw0, acc[m][r]);
        acc[m][r] = fmaf(d1, sa1 * sw1, acc[m][r]);
      }
  }
#pragma unroll
  for (int m = 0; m < kMats; ++m)
#pragma unroll
    for (int r = 0; r < kRows; ++r) acc[m][r] = warp_sum(acc[m][r]);
  if (lane == 0) {
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
      if (row0 + r >= rows) continue;
      // Single final division by ga*gw: src/cuda/nvfp4/sm120.cu:243.
      const float y0 = __fdiv_rn(acc[0][r], div0);
      if constexpr (kGateUp) {
        const float y1 = __fdiv_rn(acc[1][r], div1);
        if (out0) out0[row0 + r] = y0;
        if (out1) out1[row0 + r] = y1;
        // bf16 boundaries and GELU-tanh product: src/cuda/nvfp4/sm120.cu:375-386.
        const float g = bf16_round(y0), u = bf16_round(y1);
        product[row0 + r] = gelu_tanh_product(g, u);
      } else {
        out0[row0 + r] = y0;
      }
    }
  }
}

// Small-batch NVFP4 GEMV (2..8 tokens, the verifier's MLP projections): the weight chunk is
// converted to fp16 once and meets kTok staged activations; per token the arithmetic and its
// order are those of the single-token kernel, so each token's result is bit-identical to it.
template <int kTok>
__global__ void __launch_bounds__(kThreads)
nvfp4_gemv_batch_kernel(const uint8_t* __restrict__ act, const uint8_t* __restrict__ act_scales,
                        const uint8_t* __restrict__ w, const uint8_t* __restrict__ ws, float* __restrict__ out,
                        uint64_t rows, uint64_t k, float div) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const uint64_t k_pad = (k + 1023) / 1024 * 1024;
  const uint64_t tok_bytes = k_pad * 2 + (k / 16) * 4;   // staged fp16 values, then fp32 block scales
  for (int t = 0; t < kTok; ++t) {
    __half* xs = reinterpret_cast<__half*>(smem_raw + t * tok_bytes);
    float* sa = reinterpret_cast<float*>(smem_raw + t * tok_bytes + k_pad * 2);
    const uint8_t* a = act + static_cast<uint64_t>(t) * (k / 2);
    for (uint64_t c = threadIdx.x; c < k / 32; c += kThreads) {
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(a) + c);  // 32 elements
      const uint32_t ww[4] = {v.x, v.y, v.z, v.w};
      __half* dst = xs + (c / 32) * 1024 + (c % 32) * 8;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        uint32_t h[4];
        e2m1x8_to_half2(ww[i], h);
        *reinterpret_cast<uint4*>(dst + i * 256) = make_uint4(h[0], h[1], h[2], h[3]);
      }
    }
    for (uint64_t c = threadIdx.x; c < k / 16; c += kThreads)
      sa[c] = e4m3_decode(__ldg(act_scales + static_cast<uint64_t>(t) * (k / 16) + c));
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint64_t row = static_cast<uint64_t>(blockIdx.x) * kWarps + warp;
  if (row >= rows) return;
  const uint64_t row_bytes = k / 2, srow_bytes = k / 16;
  float acc[kTok];
#pragma unroll
  for (int t = 0; t < kTok; ++t) acc[t] = 0.0f;
  for (uint64_t kb = lane * 16ull; kb < row_bytes; kb += 512) {
    const uint4 wv = ldg_stream(w + row * row_bytes + kb);
    const uint16_t sv = __ldg(reinterpret_cast<const uint16_t*>(ws + row * srow_bytes + kb / 8));
    const float sw0 = e4m3_decode(static_cast<uint8_t>(sv & 0xFF)), sw1 = e4m3_decode(static_cast<uint8_t>(sv >> 8));
#pragma unroll
    for (int t = 0; t < kTok; ++t) {
      const __half* xp = reinterpret_cast<const __half*>(smem_raw + t * tok_bytes) + (kb / 512) * 1024 + lane * 8;
      const float* sa = reinterpret_cast<const float*>(smem_raw + t * tok_bytes + k_pad * 2);
      const uint4 x0 = *reinterpret_cast<const uint4*>(xp), x1 = *reinterpret_cast<const uint4*>(xp + 256),
                  x2 = *reinterpret_cast<const uint4*>(xp + 512), x3 = *reinterpret_cast<const uint4*>(xp + 768);
      const float d0 = block_dot_fp4(wv.x, wv.y, x0, x1);
      const float d1 = block_dot_fp4(wv.z, wv.w, x2, x3);
      acc[t] = fmaf(d0, sa[kb / 8] * sw0, acc[t]);
      acc[t] = fmaf(d1, sa[kb / 8 + 1] * sw1, acc[t]);
    }
  }
#pragma unroll
  for (int t = 0; t < kTok; ++t) acc[t] = warp_sum(acc[t]);
  if (lane == 0) {
#pragma unroll
    for (int t = 0; t < kTok; ++t) out[static_cast<uint64_t>(t) * rows + row] = __fdiv_rn(acc[t], div);
  }
}

template <int kTok>
int32_t launch_nvfp4_gemv_batch_variant(const char* op, const uint8_t* act, const uint8_t* act_scales, const uint8_t* w,
                                        const uint8_t* ws, float* out, uint64_t rows, uint64_t k, float div,
                                        cudaStream_t stream) {
  auto kern = nvfp4_gemv_batch_kernel<kTok>;
  const size_t smem = static_cast<size_t>(kTok) * ((k + 1023) / 1024 * 1024 * 2 + (k / 16) * 4);
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return fail(GEMB_INTERNAL, "%s: %s: %s", op, cudaGetErrorName(e), cudaGetErrorString(e));
  }
  const unsigned blocks = static_cast<unsigned>((rows + kWarps - 1) / kWarps);
  kern<<<blocks, kThreads, smem, stream>>>(act, act_scales, w, ws, out, rows, k, div);
  return check_launch(op);
}

template <bool kGateUp>
int32_t launch_nvfp4_gemv(const char* op, const uint8_t* act, const uint8_t* act_scales,
                          const uint8_t* w0, const uint8_t* ws0, const uint8_t* w1,
                          const uint8_t* ws1, float* out0, float* out1, float* product,
                          uint64_t rows, uint64_t k, float div0, float div1, cudaStream_t stream) {
  const int rpw = kGateUp ? (rows / (kWarps * 2) >= 2ull * sm_count() ? 2 : 1)
                          : (rows / (kWarps * 4) >= 2ull * sm_count() ? 4 : rows / (kWarps * 2) >= 2ull * sm_count() ? 2 : 1);
  const unsigned blocks = static_cast<unsigned>((rows + kWarps * rpw - 1) / (kWarps * rpw));
  const size_t smem = (k + 1023) / 1024 * 1024 * 2 + (k / 16) * 4;
#define GEMB_LAUNCH_FP4_GEMV(R)                                                                   \
  do {                                                                                            \
    auto kern = nvfp4_gemv_kernel<R, kGateUp>;                                                    \
    if (smem > 48 * 1024) {                                                                       \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,     \
                                           static_cast<int>(smem));                               \
      if (e != cudaSuccess)                                                                       \
        return fail(GEMB_INTERNAL, "%s: %s: %s", op, cudaGetErrorName(e), cudaGetErrorString(e)); \
    }                                                                                             \
    kern<<<blocks, kThreads, smem, stream>>>(act, act_scales, w0, ws0, w1, ws1, out0, out1,       \
                                             product, rows, k, div0, div1);             \
  } while (0)
  if (rpw == 4) { if constexpr (!kGateUp) GEMB_LAUNCH_FP4_GEMV(4); }
  else if (rpw == 2) GEMB_LAUNCH_FP4_GEMV(2);
  else GEMB_LAUNCH_FP4_GEMV(1);
#undef GEMB_LAUNCH_FP4_GEMV
  return check_launch(op);
}

int32_t validate_nvfp4_gemv(const char* op, uint64_t rows, uint64_t k, float ga, float gw) {
  GEMB_REQUIRE(rows > 0 && k > 0, "%s: geometry must be nonzero", op);
  GEMB_REQUIRE(k % 64 == 0 && rows % 8 == 0,
               "%s: requires K divisible by 64 and rows divisible by 8", op);
  GEMB_REQUIRE(k <= 96 * 1024, "%s: contracting extent exceeds the shared-memory staging limit (98304)", op);
  GEMB_REQUIRE(rows < (1ull << 31), "%s: too many rows", op);
  GEMB_REQUIRE(positive_finite(ga) && positive_finite(gw), "%s: global divisors must be positive and finite", op);
  GEMB_REQUIRE(std::isfinite(ga * gw), "%s: combined global divisor overflowed", op);
  return GEMB_OK;
}

// ---------------------------------------------------------------------------------------------
// Decode-time FP8 token quantizer: one 1024-thread CTA per token, the token held in registers
// between the amax pass and the conversion (one global round trip), quotients through
// quotient_for_e4m3 (bit-identical to the IEEE division of src/numeric/fp8.cpp:41-58).  It
// triggers its dependents at once and waits for its predecessor before touching the
// activation, so under programmatic dependent launch the GEMV that follows can prefetch its
// weights while this kernel runs.  bf16 input, K <= 16384, K % 8 == 0.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(1024)
fp8_quantize_decode_kernel(const uint16_t* __restrict__ x, uint8_t* __restrict__ out,
                           float* __restrict__ scales, uint32_t k) {
  __shared__ float red[32];
  asm volatile("griddepcontrol.launch_dependents;");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const uint64_t t = blockIdx.x;
  const uint4* xp = reinterpret_cast<const uint4*>(x + t * k);
  const uint32_t chunks = k / 8;
  uint4 v[2];
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const uint32_t c = threadIdx.x + i * 1024;
    v[i] = c < chunks ? __ldg(xp + c) : make_uint4(0, 0, 0, 0);
    amax = fmaxf(amax, chunk_amax(v[i]));
  }
  amax = warp_max(amax);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = red[0];
#pragma unroll
  for (int i = 1; i < 32; ++i) amax = fmaxf(amax, red[i]);
  const float scale = amax == 0.0f ? 1.0f : __fdiv_rn(amax, 448.0f);
  const float inv_scale = __frcp_rn(scale);
  if (threadIdx.x == 0) scales[t] = scale;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const uint32_t c = threadIdx.x + i * 1024;
    if (c >= chunks) continue;
    const uint32_t ww[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
    uint32_t q[2] = {0, 0};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float lo = quotient_for_e4m3(__uint_as_float(ww[j] << 16), scale, inv_scale);
      const float hi = quotient_for_e4m3(__uint_as_float(ww[j] & 0xFFFF0000u), scale, inv_scale);
      const uint32_t pair = static_cast<uint16_t>(__nv_cvt_float2_to_fp8x2(make_float2(lo, hi), __NV_SATFINITE, __NV_E4M3));
      q[j >> 1] |= pair << (16 * (j & 1));
    }
    *reinterpret_cast<uint2*>(out + t * k + static_cast<uint64_t>(c) * 8) = make_uint2(q[0], q[1]);
  }
}

}  // namespace

int32_t launch_fp8_quantize_decode(const char* op, const uint16_t* x, uint8_t* out, float* scales, uint64_t tokens,
                                   uint64_t k, cudaStream_t stream) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<unsigned>(tokens));
  cfg.blockDim = dim3(1024);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = g_pdl ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t le = cudaLaunchKernelEx(&cfg, fp8_quantize_decode_kernel, x, out, scales, static_cast<uint32_t>(k));
  if (le != cudaSuccess) {
    cudaGetLastError();
    return fail(GEMB_INTERNAL, "%s: %s: %s", op, cudaGetErrorName(le), cudaGetErrorString(le));
  }
  return check_launch(op);
}

// Reads and clears the GEMV ring's bounded-wait flag (0 = clean).
int gemv_take_device_error() {
  int code = 0;
  if (cudaMemcpyFromSymbol(&code, g_gemv_error, sizeof code) != cudaSuccess) return -1;
  if (code != 0) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_gemv_error, &zero, sizeof zero);
  }
  return code;
}

}  // namespace gemb

using namespace gemb;

extern "C" {

int32_t gemb_set_tuning(int32_t knob, int32_t value) {
  if (knob == GEMB_TUNE_GEMV_ROWS) {
    GEMB_REQUIRE(value == 0 || value == 1 || value == 2 || value == 4,
                 "gemb_set_tuning: rows per warp must be 0 (auto), 1, 2 or 4");
    g_rows_override = value;
    return GEMB_OK;
  }
  if (knob == GEMB_TUNE_GEMV_IMPL) {
    GEMB_REQUIRE(value == 0 || value == 1 || value == 2,
                 "gemb_set_tuning: GEMV implementation must be 0 (automatic), 1 (direct loads) or 2 (ring)");
    g_gemv_impl = value;
    return GEMB_OK;
  }
  if (knob == GEMB_TUNE_GEMV_PDL) {
    g_pdl = value != 0;
    return GEMB_OK;
  }
  return gemm_set_tuning(knob, value);
}

int32_t gemb_fp8_gemv(const uint8_t* act, const float* act_scale, const uint8_t* w,
                      const uint16_t* w_scales, float* out, uint64_t rows, uint64_t k,
                      gemb_stream_t stream) {
  const char* op = "gemb_fp8_gemv";
  GEMB_REQUIRE(act_scale != nullptr, "%s: pointers must be nonnull", op);
  GEMB_TRY(validate_fp8_gemv(op, act, w, w_scales, out, rows, k));
  GEMB_ENTER(op);
  Fp8Group grp{};
  grp.n = 1;
  grp.p[0] = {w, w_scales, out, rows};
  return launch_fp8_gemv<false, false>(op, act, act_scale, grp, k, stream);
}

int32_t gemb_fp8_gemv_qkv(const uint8_t* act, const float* act_scale, const uint8_t* q_w,
                          const uint16_t* q_s, float* q_out, uint64_t q_rows, const uint8_t* k_w,
                          const uint16_t* k_s, float* k_out, uint64_t k_rows, const uint8_t* v_w,
                          const uint16_t* v_s, float* v_out, uint64_t v_rows, uint64_t k,
                          gemb_stream_t stream) {
  const char* op = "gemb_fp8_gemv_qkv";
  GEMB_REQUIRE(act_scale != nullptr, "%s: pointers must be nonnull", op);
  GEMB_TRY(validate_fp8_gemv(op, act, q_w, q_s, q_out, q_rows, k));
  GEMB_TRY(validate_fp8_gemv(op, act, k_w, k_s, k_out, k_rows, k));
  const bool has_v = v_w != nullptr || v_rows != 0;
  if (has_v) GEMB_TRY(validate_fp8_gemv(op, act, v_w, v_s, v_out, v_rows, k));
  GEMB_ENTER(op);
  Fp8Group grp{};
  grp.n = has_v ? 3 : 2;
  grp.p[0] = {q_w, q_s, q_out, q_rows};
  grp.p[1] = {k_w, k_s, k_out, k_rows};
  if (has_v) grp.p[2] = {v_w, v_s, v_out, v_rows};
  return launch_fp8_gemv<false, false>(op, act, act_scale, grp, k, stream);
}

int32_t gemb_fp8_gemv_batch(const uint8_t* act, const float* act_scales, const uint8_t* w, const uint16_t* w_scales,
                            float* out, uint64_t tokens, uint64_t rows, uint64_t k, gemb_stream_t stream) {
  const char* op = "gemb_fp8_gemv_batch";
  GEMB_REQUIRE(act_scales != nullptr, "%s: pointers must be nonnull", op);
  GEMB_TRY(validate_fp8_gemv(op, act, w, w_scales, out, rows, k));
  GEMB_REQUIRE(tokens >= 1 && tokens <= 8, "%s: between 1 and 8 tokens (larger batches go through gemb_fp8_gemm_bf16)", op);
  GEMB_REQUIRE(tokens * ((k + 511) / 512 * 512) * 2 <= 200 * 1024,
               "%s: tokens * K exceeds the shared-memory staging limit (102400 elements)", op);
  GEMB_ENTER(op);
  Fp8Group grp{};
  grp.n = 1;
  grp.p[0] = {w, w_scales, out, rows};
  grp.row_start[1] = rows;
  if (tokens == 1) return launch_fp8_gemv<false, false>(op, act, act_scales, grp, k, stream);
  return launch_fp8_gemv_batch(op, act, act_scales, grp, tokens, k, stream);
}

int32_t gemb_fp8_gemv_qkv_batch(const uint8_t* act, const float* act_scales, const uint8_t* q_w, const uint16_t* q_s,
                                float* q_out, uint64_t q_rows, const uint8_t* k_w, const uint16_t* k_s, float* k_out,
                                uint64_t k_rows, const uint8_t* v_w, const uint16_t* v_s, float* v_out, uint64_t v_rows,
                                uint64_t tokens, uint64_t k, gemb_stream_t stream) {
  const char* op = "gemb_fp8_gemv_qkv_batch";
  GEMB_REQUIRE(act_scales != nullptr, "%s: pointers must be nonnull", op);
  GEMB_TRY(validate_fp8_gemv(op, act, q_w, q_s, q_out, q_rows, k));
  GEMB_TRY(validate_fp8_gemv(op, act, k_w, k_s, k_out, k_rows, k));
  const bool has_v = v_w != nullptr || v_rows != 0;
  if (has_v) GEMB_TRY(validate_fp8_gemv(op, act, v_w, v_s, v_out, v_rows, k));
  GEMB_REQUIRE(tokens >= 1 && tokens <= 8, "%s: between 1 and 8 tokens", op);
  GEMB_REQUIRE(tokens * ((k + 511) / 512 * 512) * 2 <= 200 * 1024,
               "%s: tokens * K exceeds the shared-memory staging limit (102400 elements)", op);
  GEMB_ENTER(op);
  Fp8Group grp{};
  grp.n = has_v ? 3 : 2;
  grp.p[0] = {q_w, q_s, q_out, q_rows};
  grp.p[1] = {k_w, k_s, k_out, k_rows};
  if (has_v) grp.p[2] = {v_w, v_s, v_out, v_rows};
  grp.row_start[1] = q_rows;
  grp.row_start[2] = q_rows + k_rows;
  grp.row_start[3] = q_rows + k_rows + (has_v ? v_rows : 0);
  if (tokens == 1) return launch_fp8_gemv<false, false>(op, act, act_scales, grp, k, stream);
  return launch_fp8_gemv_batch(op, act, act_scales, grp, tokens, k, stream);
}

int32_t gemb_fp8_gemv_bf16in(const uint16_t* act_bf16, const uint8_t* w, const uint16_t* w_scales,
                             void* out, int32_t out_dtype, uint64_t rows, uint64_t k,
                             gemb_stream_t stream) {
  const char* op = "gemb_fp8_gemv_bf16in";
  GEMB_TRY(validate_fp8_gemv(op, act_bf16, w, w_scales, out, rows, k));
  GEMB_REQUIRE(out_dtype == GEMB_F32 || out_dtype == GEMB_BF16, "%s: output dtype must be GEMB_F32 or GEMB_BF16", op);
  GEMB_ENTER(op);
  Fp8Group grp{};
  grp.n = 1;
  grp.p[0] = {w, w_scales, out, rows};
  if (out_dtype == GEMB_BF16) return launch_fp8_gemv<true, true>(op, act_bf16, nullptr, grp, k, stream);
  return launch_fp8_gemv<true, false>(op, act_bf16, nullptr, grp, k, stream);
}

int32_t gemb_nvfp4_gemv(const uint8_t* act, const uint8_t* act_scales, const uint8_t* w,
                        const uint8_t* w_scales, float* out, uint64_t rows, uint64_t k, float ga,
                        float gw, gemb_stream_t stream) {
  const char* op = "gemb_nvfp4_gemv";
  GEMB_REQUIRE(act && act_scales && w && w_scales && out, "%s: pointers must be nonnull", op);
  GEMB_TRY(validate_nvfp4_gemv(op, rows, k, ga, gw));
  GEMB_REQUIRE(reinterpret_cast<uintptr_t>(act) % 16 == 0 && reinterpret_cast<uintptr_t>(w) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(w_scales) % 2 == 0,
               "%s: activation and weight must be 16-byte aligned, weight scales 2-byte aligned", op);
  GEMB_ENTER(op);
  return launch_nvfp4_gemv<false>(op, act, act_scales, w, w_scales, nullptr, nullptr, out, nullptr,
                                  nullptr, rows, k, ga * gw, 1.0f, stream);
}

int32_t gemb_nvfp4_gemv_batch(const uint8_t* act, const uint8_t* act_scales, const uint8_t* w, const uint8_t* w_scales,
                              float* out, uint64_t tokens, uint64_t rows, uint64_t k, float ga, float gw,
                              gemb_stream_t stream) {
  const char* op = "gemb_nvfp4_gemv_batch";
  GEMB_REQUIRE(act && act_scales && w && w_scales && out, "%s: pointers must be nonnull", op);
  GEMB_TRY(validate_nvfp4_gemv(op, rows, k, ga, gw));
  GEMB_REQUIRE(tokens >= 1 && tokens <= 8, "%s: between 1 and 8 tokens (larger batches go through gemb_nvfp4_gemm_bf16)", op);
  GEMB_REQUIRE(tokens * ((k + 1023) / 1024 * 1024 * 2 + (k / 16) * 4) <= 200 * 1024,
               "%s: tokens * K exceeds the shared-memory staging limit", op);
  GEMB_REQUIRE(reinterpret_cast<uintptr_t>(act) % 16 == 0 && reinterpret_cast<uintptr_t>(w) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(w_scales) % 2 == 0,
               "%s: activation and weight must be 16-byte aligned, weight scales 2-byte aligned", op);
  GEMB_ENTER(op);
  const float div = ga * gw;
  switch (tokens) {
    case 1: return launch_nvfp4_gemv<false>(op, act, act_scales, w, w_scales, nullptr, nullptr, out, nullptr, nullptr, rows,
                                            k, div, 1.0f, stream);
    case 2: return launch_nvfp4_gemv_batch_variant<2>(op, act, act_scales, w, w_scales, out, rows, k, div, stream);
    case 3: return launch_nvfp4_gemv_batch_variant<3>(op, act, act_scales, w, w_scales, out, rows, k, div, stream);
    case 4: return launch_nvfp4_gemv_batch_variant<4>(op, act, act_scales, w, w_scales, out, rows, k, div, stream);
    case 5: return launch_nvfp4_gemv_batch_variant<5>(op, act, act_scales, w, w_scales, out, rows, k, div, stream);
    case 6: return launch_nvfp4_gemv_batch_variant<6>(op, act, act_scales, w, w_scales, out, rows, k, div, stream);
    case 7: return launch_nvfp4_gemv_batch_variant<7>(op, act, act_scales, w, w_scales, out, rows, k, div, stream);
    default: return launch_nvfp4_gemv_batch_variant<8>(op, act, act_scales, w, w_scales, out, rows, k, div, stream);
  }
}

int32_t gemb_nvfp4_gemv_gate_up(const uint8_t* act, const uint8_t* act_scales, const uint8_t* gate_w,
                                const uint8_t* gate_s, const uint8_t* up_w, const uint8_t* up_s,
                                float* gate_out, float* up_out, float* product, uint64_t rows,
                                uint64_t k, float gate_ga, float gate_gw, float up_ga, float up_gw,
                                gemb_stream_t stream) {
  const char* op = "gemb_nvfp4_gemv_gate_up";
  GEMB_REQUIRE(act && act_scales && gate_w && gate_s && up_w && up_s && product,
               "%s: required pointers must be nonnull", op);
  GEMB_REQUIRE((gate_out == nullptr) == (up_out == nullptr),
               "%s: gate and up outputs must both be present or both null", op);
  GEMB_TRY(validate_nvfp4_gemv(op, rows, k, gate_ga, gate_gw));
  GEMB_TRY(validate_nvfp4_gemv(op, rows, k, up_ga, up_gw));
  GEMB_REQUIRE(reinterpret_cast<uintptr_t>(act) % 16 == 0 && reinterpret_cast<uintptr_t>(gate_w) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(up_w) % 16 == 0 && reinterpret_cast<uintptr_t>(gate_s) % 2 == 0 &&
                   reinterpret_cast<uintptr_t>(up_s) % 2 == 0,
               "%s: activation and weights must be 16-byte aligned, weight scales 2-byte aligned", op);
  GEMB_ENTER(op);
  return launch_nvfp4_gemv<true>(op, act, act_scales, gate_w, gate_s, up_w, up_s, gate_out, up_out,
                                 product, rows, k, gate_ga * gate_gw, up_ga * up_gw, stream);
}

int32_t gemb_nvfp4_gemv_gate_up_batch(const uint8_t* act, const uint8_t* act_scales, const uint8_t* gate_w,
                                      const uint8_t* gate_s, const uint8_t* up_w, const uint8_t* up_s, float* gate_out,
                                      float* up_out, float* product, uint64_t tokens, uint64_t rows, uint64_t k,
                                      float gate_ga, float gate_gw, float up_ga, float up_gw, gemb_stream_t stream) {
  const char* op = "gemb_nvfp4_gemv_gate_up_batch";
  GEMB_REQUIRE(tokens >= 1 && tokens <= 65535, "%s: between 1 and 65,535 tokens", op);
  // One fused gate/up launch per token (the verifier's batches are a handful of tokens): every
  // token's result is bit-identical to the single-token operator.
  for (uint64_t t = 0; t < tokens; ++t)
    GEMB_TRY(gemb_nvfp4_gemv_gate_up(act + t * (k / 2), act_scales + t * (k / 16), gate_w, gate_s, up_w, up_s,
                                     gate_out ? gate_out + t * rows : nullptr, up_out ? up_out + t * rows : nullptr,
                                     product + t * rows, rows, k, gate_ga, gate_gw, up_ga, up_gw, stream));
  return GEMB_OK;
}

}  // extern "C"
