// Prefill projections: tcgen05 GEMMs with TMEM accumulators and TMA-staged operand tiles.
//
//   NVFP4  D[M,N] = alpha * sum_k (A e2m1 * SFA ue4m3)(B e2m1 * SFB ue4m3)   kind::mxf4nvf4.block16
//   FP8    D[M,N] = (sum_k A e4m3 * B e4m3) * a_scale[m] * w_scale[n]          kind::f8f6f4
//
// A is the activation [M, K] (tokens), B the weight [N, K] (output rows), both K-major, so
// D = A * B^T lands with one token per TMEM lane and one output feature per TMEM column.
//
// One persistent CTA per SM, six warps:
//   warp 0   producer: one elected lane issues TMA tile loads (128-byte swizzle, no multicast)
//            for A and B and 1-D bulk copies for the interleaved block scales into a ring of
//            kStages shared-memory stages, each guarded by a full/empty mbarrier pair;
//   warp 1   MMA issuer: owns the 512 TMEM columns; per stage issues one tcgen05.mma per 32
//            bytes of K and commits the stage's empty barrier; after the last K step commits
//            the accumulator barrier;
//   warps 2-5 and the last four warps: epilogue, two sets of four; each warp drains its 32 TMEM
//            lanes 64 columns at a time, the sets taking alternate 64-column sub-tiles (two
//            tcgen05.ld in flight), scales, rounds to bf16, writes a 32 x 128-byte block into
//            its own swizzled staging buffer and issues a TMA store (which also clips the
//            token / row tails).  With kAccStages = 2 the
//            accumulators are double buffered in TMEM so the epilogue of tile i overlaps the
//            main loop of tile i+1.
//   warps 6-9 (NVFP4 only) scale movers: each copies the stage's block scales from shared
//            memory into its quarter of TMEM with tcgen05.st (one 128-bit shared load feeds four
//            TMEM columns) and arrives on the stage's scales-ready barrier.  Doing this with
//            tcgen05.cp from the MMA thread costs a third of the tensor-pipe time, because those
//            copies queue in front of the MMAs.
// Tiles are walked with the token-tile index fastest so CTAs running at the same time share the
// same weight tile through L2.
//
// Per stage a tile needs 128 B of K per row: 256 E2M1 or 128 E4M3 elements.  K only has to be
// a multiple of 64 (NVFP4) / 32 (FP8): the last stage issues fewer MMAs, TMA zero-fills the
// rest of its box.
//
// Every mbarrier wait is bounded; on expiry the kernel records a code in g_gemm_error, stops
// issuing work, and still releases its TMEM before returning.
#include <cuda.h>

#include <algorithm>
#include <mutex>

#include "common.cuh"
#include "ptx.cuh"

namespace gemb {

__device__ int g_gemm_error = 0;

namespace {

constexpr int kGemmThreadsFp8 = 320;   // producer, MMA, 2 x 4 epilogue warps
constexpr int kGemmThreadsFp4 = 448;   // producer, MMA, 4 epilogue, 4 scale movers, 4 more epilogue warps
constexpr int BM = 128;

struct GemmParams {
  const uint8_t* sfa;            // NVFP4: interleaved activation scales
  const uint8_t* sfb;            // NVFP4: interleaved weight scales
  const float* a_scales;         // FP8: per-token scales
  const uint16_t* w_scales;      // FP8: per-row bf16 scales
  uint16_t* out;                 // bf16 [M, N]
  uint32_t m, n, k;              // k in elements
  float alpha;                   // NVFP4: 1 / (ga * gw)
  // Grouped (mixture-of-experts) mode when plan != null: token tiles come from the device-side
  // plan (plan[0] tiles, tile_expert at plan + 3 + experts), the weight is [experts, n, K].
  const int32_t* plan;
  const float* w_divisors;       // per-expert weight global divisors (null: alpha is used)
  float ga;                      // activation global divisor (with w_divisors)
  uint32_t experts;
  // Gated epilogue (gated != 0): the weight rows interleave gate and up features in runs of 32
  // (gemb_nvfp4_pack_gate_up), so every 64 accumulator columns hold 32 gate + 32 up values of
  // the same features; the epilogue writes the NVFP4-quantised GELU product instead of bf16.
  uint32_t gated;
  uint32_t out_f32;              // NVFP4 only: store fp32 (acc * alpha) instead of bf16 (row-split partial sums)
  float alpha_up;                // 1 / (ga * gw_up); `alpha` is the gate's
  float g_product;               // input divisor of the down projection
  uint8_t* out_packed;           // [M, n/4] payload of the product (n/2 features)
  uint8_t* out_scales;           // interleaved scales of the product
};

template <bool kFp4, int BN, int kStages, int kAccStages>
struct Cfg {
  static constexpr int kKPerStage = kFp4 ? 256 : 128;      // elements covered by 128 bytes
  static constexpr int kKPerMma = kFp4 ? 64 : 32;          // elements per tcgen05.mma
  static constexpr int kABytes = BM * 128;
  static constexpr int kBBytes = BN * 128;
  // Weight scales are stored in 128-row groups.  A 192-wide tile starts on a group boundary
  // (even tiles) or 64 rows into a group (odd tiles): it always stages two whole groups in shared
  // memory and the scale movers write just the six 32-row columns the tile covers into TMEM.
  static constexpr int kSfbGroups = BN <= 128 ? 1 : 2;
  static constexpr int kSfaBytes = kFp4 ? 2048 : 0;        // 4 chunks of 512 B
  static constexpr int kSfbBytes = kFp4 ? kSfbGroups * 2048 : 0;
  static constexpr int kStageBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;
  static constexpr int kEpiBytes = 4 * 2 * 4096;          // 4 warps x 2 buffers x (32 rows x 128 B)
  static constexpr int kBarrierBytes = 1024;
  static constexpr int kSmemBytes = kStages * kStageBytes + kEpiBytes + kBarrierBytes + 1024;  // + alignment slack
  // TMEM columns: accumulators first, then a ring of scale regions (one per step in flight).
  static constexpr int kAccCols = kAccStages * BN;
  static constexpr int kSfaCols = 16;                      // 4 MMAs x 4 columns
  static constexpr int kSfbColsPerMma = BN / 32;
  static constexpr int kSfbCols = 4 * kSfbColsPerMma;
  static constexpr int kSfColsPerStage = kFp4 ? kSfaCols + kSfbCols : 0;
  static constexpr int kSfStages = !kFp4 ? 1 : ((512 - kAccCols) / kSfColsPerStage < kStages ? (512 - kAccCols) / kSfColsPerStage : kStages);
  static_assert(!kFp4 || kSfStages >= 2, "TMEM budget exceeded");
  static_assert(kAccCols + (kFp4 ? kSfStages * kSfColsPerStage : 0) <= 512, "TMEM budget exceeded");
  static_assert(BN % 64 == 0 && BN <= 256, "BN must be 128, 192 or 256");
  static_assert(kSmemBytes <= 227 * 1024, "shared memory budget exceeded");
};

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

template <bool kFp4, int BN, int kStages, int kAccStages>
__global__ void __launch_bounds__(kFp4 ? kGemmThreadsFp4 : kGemmThreadsFp8, 1)
gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
            const __grid_constant__ CUtensorMap map_out, const GemmParams p) {
  using C = Cfg<kFp4, BN, kStages, kAccStages>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stage_a = smem;
  uint8_t* stage_b = stage_a + kStages * C::kABytes;
  uint8_t* epi_stage = stage_b + kStages * C::kBBytes;
  uint8_t* stage_sfa = epi_stage + C::kEpiBytes;
  uint8_t* stage_sfb = stage_sfa + kStages * C::kSfaBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(stage_sfb + kStages * C::kSfbBytes);
  uint64_t* full = bars;
  uint64_t* empty = full + kStages;
  uint64_t* acc_full = empty + kStages;
  uint64_t* acc_empty = acc_full + kAccStages;
  uint64_t* sf_ready = acc_empty + kAccStages;   // per smem stage: scales are in TMEM
  uint64_t* sf_free = sf_ready + kStages;        // per TMEM scale region: its MMAs have completed
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(sf_free + kStages);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(&full[s], 1);
      ptx::mbar_init(&empty[s], 1);
      ptx::mbar_init(&sf_ready[s], 4);
      ptx::mbar_init(&sf_free[s], 1);
    }
    for (int s = 0; s < kAccStages; ++s) {
      ptx::mbar_init(&acc_full[s], 1);
      ptx::mbar_init(&acc_empty[s], 8);
    }
    *abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::prefetch_tensormap(&map_a);
    ptx::prefetch_tensormap(&map_b);
    ptx::prefetch_tensormap(&map_out);
  }
  if (warp == 1) ptx::tmem_alloc(tmem_holder, 512);
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  const uint32_t m_tiles = p.plan ? static_cast<uint32_t>(__ldg(p.plan)) : (p.m + BM - 1) / BM;
  const uint32_t n_tiles = (p.n + BN - 1) / BN;
  const int32_t* tile_expert = p.plan ? p.plan + 3 + p.experts : nullptr;
  const uint32_t num_tiles = m_tiles * n_tiles;
  const uint32_t k_stages = (p.k + C::kKPerStage - 1) / C::kKPerStage;
  const uint32_t k_groups_pad = (p.k / 16 + 3) / 4;  // 512-byte scale chunks per 128-row group

  // Tile order: groups of 16 token tiles; inside a group the token tile runs fastest, so the
  // CTAs of a wave share a few weight tiles and the group's activations stay in L2 while every
  // weight tile passes over them.
  auto tile_coords = [&](uint32_t tile, uint32_t& mt, uint32_t& nt) {
    constexpr uint32_t kGroupM = 16;
    const uint32_t per_group = kGroupM * n_tiles;
    const uint32_t first_m = (tile / per_group) * kGroupM;
    const uint32_t gm = min(kGroupM, m_tiles - first_m);
    const uint32_t within = tile % per_group;
    mt = first_m + within % gm;
    nt = within / gm;
  };

  auto fail_wait = [&](int code) {
    atomicCAS(&g_gemm_error, 0, code);
    *abort_flag = 1;
  };

  if (warp == 0) {
    // ------------------------------- producer -------------------------------------------------
    if (ptx::elect_one()) {
      uint32_t stage = 0, phase = 0;
      for (uint32_t tile = blockIdx.x; tile < num_tiles && !*abort_flag; tile += gridDim.x) {
        uint32_t mt, nt;
        tile_coords(tile, mt, nt);
        const uint32_t expert = tile_expert ? static_cast<uint32_t>(__ldg(tile_expert + mt)) : 0u;
        for (uint32_t ks = 0; ks < k_stages; ++ks) {
          if (!ptx::mbar_wait(&empty[stage], phase ^ 1)) { fail_wait(1); break; }
          const uint32_t k0 = ks * C::kKPerStage;
          const uint32_t n_mma = min(4u, (p.k - k0) / C::kKPerMma);
          uint32_t bytes = C::kABytes + C::kBBytes;
          if constexpr (kFp4) {
            const uint32_t groups_per_matrix = (p.n + 127) / 128;
            const uint32_t g0 = expert * groups_per_matrix + (nt * BN) / 128;
            const uint32_t total_groups = groups_per_matrix * (tile_expert ? p.experts : 1u);
            const uint32_t n_groups = min(static_cast<uint32_t>(C::kSfbGroups), total_groups - g0);
            bytes += n_mma * 512 * (1 + n_groups);
            ptx::mbar_expect_tx(&full[stage], bytes);
            ptx::bulk_load_1d(stage_sfa + stage * C::kSfaBytes,
                              p.sfa + (static_cast<uint64_t>(mt) * k_groups_pad + ks * 4) * 512, n_mma * 512,
                              &full[stage]);
            for (uint32_t g = 0; g < n_groups; ++g)
              ptx::bulk_load_1d(stage_sfb + stage * C::kSfbBytes + g * 2048,
                                p.sfb + (static_cast<uint64_t>(g0 + g) * k_groups_pad + ks * 4) * 512,
                                n_mma * 512, &full[stage]);
          } else {
            ptx::mbar_expect_tx(&full[stage], bytes);
          }
          ptx::tma_load_2d(stage_a + stage * C::kABytes, &map_a, &full[stage], static_cast<int32_t>(ks * 128),
                           static_cast<int32_t>(mt * BM));
          ptx::tma_load_2d(stage_b + stage * C::kBBytes, &map_b, &full[stage], static_cast<int32_t>(ks * 128),
                           static_cast<int32_t>(expert * p.n + nt * BN));
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -----------------------------------------------
    // The CTA's work is a flat sequence of steps (tile, k stage).
    if (ptx::elect_one()) {
      constexpr uint32_t idesc = kFp4 ? ptx::idesc_nvfp4(BM, BN) : ptx::idesc_e4m3(BM, BN);
      const uint32_t my_tiles = blockIdx.x < num_tiles ? (num_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
      const uint32_t total_steps = my_tiles * k_stages;
      uint32_t as = 0, aphase = 0;
      uint32_t stage = 0, phase = 0;
      for (uint32_t step = 0; step < total_steps && !*abort_flag; ++step) {
        const uint32_t ks = step % k_stages;
        if (ks == 0) {
          if (!ptx::mbar_wait(&acc_empty[as], aphase ^ 1)) { fail_wait(2); break; }
          ptx::tc_fence_after();
        }
        // NVFP4 waits for the scale movers (who waited for the operands); FP8 for the operands.
        if (!ptx::mbar_wait(kFp4 ? &sf_ready[stage] : &full[stage], phase)) { fail_wait(3); break; }
        ptx::tc_fence_after();
        const uint32_t tmem_acc = tmem_base + as * BN;
        const uint32_t n_mma = min(4u, (p.k - ks * C::kKPerStage) / C::kKPerMma);
        const uint64_t a_desc = ptx::smem_desc_k128_swizzled(ptx::smem_addr(stage_a + stage * C::kABytes));
        const uint64_t b_desc = ptx::smem_desc_k128_swizzled(ptx::smem_addr(stage_b + stage * C::kBBytes));
        if constexpr (kFp4) {
          const uint32_t region = step % C::kSfStages;
          const uint32_t tsfa = tmem_base + C::kAccCols + region * C::kSfColsPerStage;
          const uint32_t tsfb = tsfa + C::kSfaCols;
          for (uint32_t j = 0; j < n_mma; ++j)
            ptx::tc_mma_nvfp4(tmem_acc, a_desc + j * 2, b_desc + j * 2, idesc, tsfa + j * 4,
                              tsfb + j * C::kSfbColsPerMma, (ks | j) != 0 ? 1u : 0u);
        } else {
          for (uint32_t j = 0; j < n_mma; ++j)
            ptx::tc_mma_f8(tmem_acc, a_desc + j * 2, b_desc + j * 2, idesc, (ks | j) != 0 ? 1u : 0u);
        }
        ptx::tc_commit(&empty[stage]);
        if constexpr (kFp4) ptx::tc_commit(&sf_free[step % C::kSfStages]);
        if (++stage == kStages) { stage = 0; phase ^= 1; }
        if (ks + 1 == k_stages) {
          ptx::tc_commit(&acc_full[as]);
          if (++as == kAccStages) { as = 0; aphase ^= 1; }
        }
      }
    }
  } else if (kFp4 && warp >= 6 && warp < 10) {
    // ------------------------------- scale movers (NVFP4) ------------------------------------
    if constexpr (kFp4) {
      const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
      const uint32_t my_tiles = blockIdx.x < num_tiles ? (num_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
      const uint32_t total_steps = my_tiles * k_stages;
      uint32_t stage = 0, phase = 0;
      for (uint32_t step = 0; step < total_steps && !*abort_flag; ++step) {
        if (!ptx::mbar_wait(&full[stage], phase)) { fail_wait(5); break; }
        // The TMEM region is reused every kSfStages steps: wait until the MMAs that read its
        // previous contents have completed.
        const uint32_t region = step % C::kSfStages;
        if (!ptx::mbar_wait(&sf_free[region], ((step / C::kSfStages) & 1) ^ 1)) { fail_wait(6); break; }
        ptx::tc_fence_after();
        const uint32_t ks = step % k_stages;
        const uint32_t n_mma = min(4u, (p.k - ks * C::kKPerStage) / C::kKPerMma);
        const uint32_t tsfa = tmem_base + C::kAccCols + region * C::kSfColsPerStage + lane_base;
        const uint32_t tsfb = tsfa + C::kSfaCols;
        const uint8_t* sfa_s = stage_sfa + stage * C::kSfaBytes + lane * 16;
        const uint8_t* sfb_s = stage_sfb + stage * C::kSfbBytes + lane * 16;
        // A 512-byte chunk holds, for row r of 32, sixteen bytes: four 32-row groups x four K
        // blocks.  Lane r's 16 bytes are exactly its four TMEM columns for one MMA.
        uint32_t mt, nt;
        tile_coords(blockIdx.x + (step / k_stages) * gridDim.x, mt, nt);
        const bool mid_group = ((nt * BN) % 128) != 0;  // only possible for 192-wide tiles
        for (uint32_t j = 0; j < n_mma; ++j) {
          ptx::tc_st_32x32b_x4(tsfa + j * 4, *reinterpret_cast<const uint4*>(sfa_s + j * 512));
          const uint4 g0 = *reinterpret_cast<const uint4*>(sfb_s + j * 512);
          if constexpr (BN == 128) {
            ptx::tc_st_32x32b_x4(tsfb + j * 4, g0);
          } else {
            const uint4 g1 = *reinterpret_cast<const uint4*>(sfb_s + 2048 + j * 512);
            if constexpr (BN == 256) {
              ptx::tc_st_32x32b_x4(tsfb + j * 8, g0);
              ptx::tc_st_32x32b_x4(tsfb + j * 8 + 4, g1);
            } else if (mid_group) {   // rows 64..127 of the first group, then the whole second
              ptx::tc_st_32x32b_x2(tsfb + j * 6, g0.z, g0.w);
              ptx::tc_st_32x32b_x4(tsfb + j * 6 + 2, g1);
            } else {                  // the whole first group, then rows 0..63 of the second
              ptx::tc_st_32x32b_x4(tsfb + j * 6, g0);
              ptx::tc_st_32x32b_x2(tsfb + j * 6 + 4, g1.x, g1.y);
            }
          }
        }
        ptx::tc_wait_st();
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&sf_ready[stage]);
        if (++stage == kStages) { stage = 0; phase ^= 1; }
      }
    }
  } else {
    // ------------------------------- epilogue -------------------------------------------------
    // Two sets of four warps; set s drains the 64-column sub-tiles s, s+2, ... of every tile.
    const uint32_t quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter+32) belong to this warp
    const uint32_t set = warp >= 6 ? 1u : 0u;
    uint8_t* my_stage = epi_stage + (set * 4 + quarter) * 4096;
    uint32_t as = 0, aphase = 0;
    for (uint32_t tile = blockIdx.x; tile < num_tiles && !*abort_flag; tile += gridDim.x) {
      uint32_t mt, nt;
      tile_coords(tile, mt, nt);
      if (!ptx::mbar_wait(&acc_full[as], aphase)) { fail_wait(4); break; }
      ptx::tc_fence_after();
      const uint32_t row0 = mt * BM + quarter * 32;
      float row_scale = p.alpha;
      if constexpr (!kFp4) row_scale = row0 + lane < p.m ? __ldg(p.a_scales + row0 + lane) : 0.0f;
      if (kFp4 && p.w_divisors != nullptr)
        row_scale = __fdiv_rn(1.0f, __fmul_rn(p.ga, __ldg(p.w_divisors + (tile_expert ? __ldg(tile_expert + mt) : 0))));
      const uint32_t tmem_acc = tmem_base + as * BN + ((quarter * 32) << 16);
      bool released = false;
#pragma unroll 1
      for (uint32_t c = set; c < BN / 64; c += 2) {
        const uint32_t col0 = nt * BN + c * 64;
        if (col0 >= p.n || row0 >= p.m) break;  // warp-uniform
        uint32_t v0[32], v1[32];
        ptx::tc_ld_32x32b_x32(tmem_acc + c * 64, v0);
        ptx::tc_ld_32x32b_x32(tmem_acc + c * 64 + 32, v1);
        uint32_t ws_pair = 0;  // FP8: lane l holds the bf16 scales of columns col0 + 2l, col0 + 2l + 1
        if constexpr (!kFp4) {
          const uint32_t c0 = min(col0 + 2 * lane, p.n - 2);
          ws_pair = __ldg(reinterpret_cast<const uint32_t*>(p.w_scales + c0));
        }
        if (kFp4 && p.gated) {
          // v0 = 32 gate values, v1 = 32 up values of features f0 .. f0+31 for this thread's token.
          ptx::tc_wait_ld();
          const uint32_t f0 = col0 / 2, inter = p.n / 2;
          float alpha_g = row_scale, alpha_u = p.w_divisors != nullptr ? row_scale : p.alpha_up;
          uint32_t words[4];
          uint8_t sb[2];
#pragma unroll
          for (int b = 0; b < 2; ++b) {
            float prod[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              // bf16 projection boundaries, bf16 GELU, bf16 product: src/cuda/nvfp4/reference.cu:177-190
              const float gv = bf16_round(__fmul_rn(__uint_as_float(v0[b * 16 + i]), alpha_g));
              const float uv = bf16_round(__fmul_rn(__uint_as_float(v1[b * 16 + i]), alpha_u));
              const float inner = 0.7978845608028654f * (gv + 0.044715f * gv * gv * gv);
              const float gelu = bf16_round(0.5f * gv * (1.0f + tanhf(inner)));
              prod[i] = bf16_round(gelu * uv);
            }
            quantize_block16<false>(prod, p.g_product, words[2 * b], words[2 * b + 1], sb[b]);
          }
          const uint32_t row = row0 + lane;
          if (row < p.m) {
            *reinterpret_cast<uint4*>(p.out_packed + static_cast<uint64_t>(row) * (inter / 2) + f0 / 2) =
                make_uint4(words[0], words[1], words[2], words[3]);
            const uint32_t c_pad = (inter / 16 + 3) / 4 * 4;
            *reinterpret_cast<uint16_t*>(p.out_scales + interleaved_scale_offset(row, f0 / 16, c_pad)) =
                static_cast<uint16_t>(sb[0]) | (static_cast<uint16_t>(sb[1]) << 8);
          }
          continue;
        }
        if (kFp4 && p.out_f32) {
          // fp32 output: two 32-column boxes (128 bytes per row each) through the same staging buffer.
          ptx::tc_wait_ld();
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            if (col0 + half * 32 >= p.n) break;
            if (lane == 0) ptx::bulk_wait_group_read<0>();
            __syncwarp();
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              const uint32_t* v = half == 0 ? v0 : v1;
              *reinterpret_cast<uint4*>(my_stage + lane * 128 + ((q ^ (lane & 7)) << 4)) = make_uint4(
                  __float_as_uint(__fmul_rn(__uint_as_float(v[4 * q]), row_scale)),
                  __float_as_uint(__fmul_rn(__uint_as_float(v[4 * q + 1]), row_scale)),
                  __float_as_uint(__fmul_rn(__uint_as_float(v[4 * q + 2]), row_scale)),
                  __float_as_uint(__fmul_rn(__uint_as_float(v[4 * q + 3]), row_scale)));
            }
            ptx::fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              ptx::tma_store_2d(&map_out, my_stage, static_cast<int32_t>(col0 + half * 32), static_cast<int32_t>(row0));
              ptx::bulk_commit_group();
            }
          }
          continue;
        }
        // The staging buffer about to be overwritten was handed to a TMA store one sub-tile ago.
        if (lane == 0) ptx::bulk_wait_group_read<0>();
        __syncwarp();
        ptx::tc_wait_ld();
        if (c + 2 >= BN / 64) {
          // This warp's last sub-tile is in registers: the accumulator can be overwritten while
          // the conversion and the store below are still running.
          ptx::tc_fence_before();
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(&acc_empty[as]);
          released = true;
        }
        uint8_t* sbuf = my_stage;
        auto convert = [&](const uint32_t (&v)[32], int half) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint32_t packed[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int e = q * 8 + i * 2;  // column within this 32-column half
              float lo = __uint_as_float(v[e]), hi = __uint_as_float(v[e + 1]);
              if constexpr (kFp4) {
                lo = __fmul_rn(lo, row_scale);
                hi = __fmul_rn(hi, row_scale);
              } else {
                // (acc * a_scale) * w_scale, in that order: src/cuda/fp8/cutlass_sm120.cu:49-63.
                const uint32_t wp = __shfl_sync(0xFFFFFFFFu, ws_pair, half * 16 + e / 2);
                lo = __fmul_rn(__fmul_rn(lo, row_scale), __uint_as_float(wp << 16));
                hi = __fmul_rn(__fmul_rn(hi, row_scale), __uint_as_float(wp & 0xFFFF0000u));
              }
              packed[i] = pack_bf16x2(lo, hi);
            }
            // 16-byte chunk j of row `lane`, stored at chunk j ^ (lane % 8): the 128-byte swizzle
            // the output tensor map expects, and conflict free for the warp.
            const int j = half * 4 + q;
            *reinterpret_cast<uint4*>(sbuf + lane * 128 + ((j ^ (lane & 7)) << 4)) =
                make_uint4(packed[0], packed[1], packed[2], packed[3]);
          }
        };
        convert(v0, 0);
        convert(v1, 1);
        ptx::fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          ptx::tma_store_2d(&map_out, sbuf, static_cast<int32_t>(col0), static_cast<int32_t>(row0));
          ptx::bulk_commit_group();
        }
      }
      if (!released) {
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&acc_empty[as]);
      }
      if (++as == kAccStages) { as = 0; aphase ^= 1; }
    }
    if (lane == 0) ptx::bulk_wait_group_all();
  }

  // ------------------------------- teardown ---------------------------------------------------
  ptx::tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // Give copies that are still in flight a bounded time to land before the CTA exits.
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, 512);
  }
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                   CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                   CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
    else
      cudaGetLastError();
  });
  return fn;
}

// Byte matrix [rows, row_bytes] row-major -> tiles of 128 bytes x box_rows rows, 128-byte swizzle.
int32_t make_byte_map(const char* op, CUtensorMap* map, const void* base, uint64_t rows, uint64_t row_bytes,
                      uint32_t box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return fail(GEMB_UNSUPPORTED, "%s: cuTensorMapEncodeTiled is not available from the driver", op);
  const cuuint64_t dims[2] = {row_bytes, rows};
  const cuuint64_t strides[1] = {row_bytes};
  const cuuint32_t box[2] = {128, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(GEMB_INTERNAL, "%s: cuTensorMapEncodeTiled failed with CUresult %d", op, int(r));
  return GEMB_OK;
}

// bf16 matrix [rows, cols] row-major -> boxes of 64 columns (128 bytes) x 32 rows, 128-byte swizzle.
int32_t make_out_map(const char* op, CUtensorMap* map, void* base, uint64_t rows, uint64_t cols) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return fail(GEMB_UNSUPPORTED, "%s: cuTensorMapEncodeTiled is not available from the driver", op);
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {cols * 2};
  const cuuint32_t box[2] = {64, 32};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(GEMB_INTERNAL, "%s: cuTensorMapEncodeTiled failed with CUresult %d", op, int(r));
  return GEMB_OK;
}

// fp32 matrix [rows, cols] row-major -> boxes of 32 columns (128 bytes) x 32 rows, 128-byte swizzle.
int32_t make_out_map_f32(const char* op, CUtensorMap* map, void* base, uint64_t rows, uint64_t cols) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return fail(GEMB_UNSUPPORTED, "%s: cuTensorMapEncodeTiled is not available from the driver", op);
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {cols * 4};
  const cuuint32_t box[2] = {32, 32};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, base, dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(GEMB_INTERNAL, "%s: cuTensorMapEncodeTiled failed with CUresult %d", op, int(r));
  return GEMB_OK;
}

int g_gemm_bn = 0;  // 0 = automatic; gemb_set_tuning(GEMB_TUNE_GEMM_BN, 128 | 256)

template <bool kFp4, int BN, int kStages, int kAccStages>
int32_t launch_gemm(const char* op, const void* a, const void* b, const GemmParams& p, cudaStream_t stream) {
  using C = Cfg<kFp4, BN, kStages, kAccStages>;
  auto kern = gemm_kernel<kFp4, BN, kStages, kAccStages>;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  dev &= 63;
  if (!configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
    if (e != cudaSuccess) return fail(GEMB_INTERNAL, "%s: %s: %s", op, cudaGetErrorName(e), cudaGetErrorString(e));
    configured[dev] = true;
  }
  const uint64_t row_bytes = kFp4 ? p.k / 2 : p.k;
  CUtensorMap map_a, map_b, map_out;
  GEMB_TRY(make_byte_map(op, &map_a, a, p.m, row_bytes, BM));
  GEMB_TRY(make_byte_map(op, &map_b, b, static_cast<uint64_t>(p.n) * (p.plan ? p.experts : 1u), row_bytes, BN));
  if (p.out_f32)
    GEMB_TRY(make_out_map_f32(op, &map_out, p.out, p.m, p.n));
  else if (p.gated)  // the tensor-map store path is unused; describe the payload buffer so the map is valid
    GEMB_TRY(make_out_map(op, &map_out, p.out_packed, p.m, p.n / 8));
  else
    GEMB_TRY(make_out_map(op, &map_out, p.out, p.m, p.n));
  const uint32_t tiles = ((p.m + BM - 1) / BM) * ((p.n + BN - 1) / BN);
  const unsigned grid = std::min<uint32_t>(tiles, static_cast<uint32_t>(sm_count()));
  kern<<<grid, kFp4 ? kGemmThreadsFp4 : kGemmThreadsFp8, C::kSmemBytes, stream>>>(map_a, map_b, map_out, p);
  return check_launch(op);
}

int32_t validate_gemm(const char* op, uint64_t tokens, uint64_t rows, uint64_t k, uint64_t k_multiple) {
  GEMB_REQUIRE(tokens > 0 && rows > 0 && k > 0, "%s: geometry must be nonzero", op);
  GEMB_REQUIRE(k % k_multiple == 0, "%s: contracting extent must be a multiple of %llu", op,
               static_cast<unsigned long long>(k_multiple));
  GEMB_REQUIRE(rows % 8 == 0, "%s: rows must be a multiple of 8", op);
  GEMB_REQUIRE(tokens < (1ull << 31) && rows < (1ull << 31) && k < (1ull << 31), "%s: extent too large", op);
  return GEMB_OK;
}

}  // namespace

int32_t gemm_set_tuning(int32_t knob, int32_t value) {
  if (knob == GEMB_TUNE_GEMM_BN) {
    GEMB_REQUIRE(value == 0 || value == 128 || value == 192 || value == 256,
                 "gemb_set_tuning: GEMM tile width must be 0 (auto), 128, 192 or 256");
    g_gemm_bn = value;
    return GEMB_OK;
  }
  return fail(GEMB_INVALID_ARGUMENT, "gemb_set_tuning: unknown knob %d", knob);
}

}  // namespace gemb

using namespace gemb;

extern "C" {

int32_t gemb_nvfp4_gemm_bf16(const uint8_t* act, const uint8_t* act_scales_interleaved, const uint8_t* w,
                             const uint8_t* w_scales_interleaved, uint16_t* out, uint64_t tokens,
                             uint64_t rows, uint64_t k, float ga, float gw, gemb_stream_t stream) {
  const char* op = "gemb_nvfp4_gemm_bf16";
  GEMB_REQUIRE(act && act_scales_interleaved && w && w_scales_interleaved && out, "%s: pointers must be nonnull", op);
  GEMB_TRY(validate_gemm(op, tokens, rows, k, 64));
  GEMB_REQUIRE(positive_finite(ga) && positive_finite(gw) && std::isfinite(ga * gw) && ga * gw > 0.0f,
               "%s: global divisors must be positive and finite", op);
  GEMB_REQUIRE(reinterpret_cast<uintptr_t>(act) % 16 == 0 && reinterpret_cast<uintptr_t>(w) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(act_scales_interleaved) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(w_scales_interleaved) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(out) % 16 == 0,
               "%s: all buffers must be 16-byte aligned", op);
  GEMB_TRY(require_sm100(op));
  GemmParams p{};
  p.sfa = act_scales_interleaved;
  p.sfb = w_scales_interleaved;
  p.out = out;
  p.m = static_cast<uint32_t>(tokens);
  p.n = static_cast<uint32_t>(rows);
  p.k = static_cast<uint32_t>(k);
  p.alpha = 1.0f / (ga * gw);  // one multiply in the epilogue, as src/cuda/nvfp4/cutlass_sm120.cu:551-552
  const int bn = g_gemm_bn ? g_gemm_bn : 256;  // 256 measured fastest; 192 and 128 stay selectable
  if (bn == 128) return launch_gemm<true, 128, 5, 2>(op, act, w, p, stream);
  if (bn == 192) return launch_gemm<true, 192, 4, 2>(op, act, w, p, stream);
  return launch_gemm<true, 256, 3, 1>(op, act, w, p, stream);
}

int32_t gemb_nvfp4_gemm_f32(const uint8_t* act, const uint8_t* act_scales_interleaved, const uint8_t* w,
                            const uint8_t* w_scales_interleaved, float* out, uint64_t tokens, uint64_t rows,
                            uint64_t k, float ga, float gw, gemb_stream_t stream) {
  const char* op = "gemb_nvfp4_gemm_f32";
  GEMB_REQUIRE(act && act_scales_interleaved && w && w_scales_interleaved && out, "%s: pointers must be nonnull", op);
  GEMB_TRY(validate_gemm(op, tokens, rows, k, 64));
  GEMB_REQUIRE(positive_finite(ga) && positive_finite(gw) && std::isfinite(ga * gw) && ga * gw > 0.0f,
               "%s: global divisors must be positive and finite", op);
  GEMB_REQUIRE(reinterpret_cast<uintptr_t>(act) % 16 == 0 && reinterpret_cast<uintptr_t>(w) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(act_scales_interleaved) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(w_scales_interleaved) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(out) % 16 == 0,
               "%s: all buffers must be 16-byte aligned", op);
  GEMB_TRY(require_sm100(op));
  GemmParams p{};
  p.sfa = act_scales_interleaved;
  p.sfb = w_scales_interleaved;
  p.out = reinterpret_cast<uint16_t*>(out);
  p.out_f32 = 1;
  p.m = static_cast<uint32_t>(tokens);
  p.n = static_cast<uint32_t>(rows);
  p.k = static_cast<uint32_t>(k);
  p.alpha = 1.0f / (ga * gw);
  const int bn = g_gemm_bn ? g_gemm_bn : 256;
  if (bn == 128) return launch_gemm<true, 128, 5, 2>(op, act, w, p, stream);
  if (bn == 192) return launch_gemm<true, 192, 4, 2>(op, act, w, p, stream);
  return launch_gemm<true, 256, 3, 1>(op, act, w, p, stream);
}

int32_t gemb_moe_grouped_gemm_bf16(const uint8_t* act, const uint8_t* act_scales_interleaved, const uint8_t* w,
                                   const uint8_t* w_scales_interleaved, uint16_t* out, const int32_t* plan,
                                   uint64_t padded_rows_max, uint64_t experts, uint64_t rows_per_expert,
                                   uint64_t k, float ga, const float* w_divisors, gemb_stream_t stream) {
  const char* op = "gemb_moe_grouped_gemm_bf16";
  GEMB_REQUIRE(act && act_scales_interleaved && w && w_scales_interleaved && out && plan && w_divisors,
               "%s: pointers must be nonnull", op);
  GEMB_TRY(validate_gemm(op, padded_rows_max, rows_per_expert, k, 64));
  GEMB_REQUIRE(padded_rows_max % 128 == 0, "%s: padded row capacity must be a multiple of 128", op);
  GEMB_REQUIRE(rows_per_expert % 128 == 0, "%s: rows per expert must be a multiple of 128", op);
  GEMB_REQUIRE(experts > 0 && experts <= 4096 && experts * rows_per_expert < (1ull << 31), "%s: bad expert count", op);
  GEMB_REQUIRE(positive_finite(ga), "%s: activation global divisor must be positive and finite", op);
  GEMB_REQUIRE(reinterpret_cast<uintptr_t>(act) % 16 == 0 && reinterpret_cast<uintptr_t>(w) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(act_scales_interleaved) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(w_scales_interleaved) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(out) % 16 == 0,
               "%s: all buffers must be 16-byte aligned", op);
  GEMB_TRY(require_sm100(op));
  GemmParams p{};
  p.sfa = act_scales_interleaved;
  p.sfb = w_scales_interleaved;
  p.out = out;
  p.m = static_cast<uint32_t>(padded_rows_max);
  p.n = static_cast<uint32_t>(rows_per_expert);
  p.k = static_cast<uint32_t>(k);
  p.plan = plan;
  p.w_divisors = w_divisors;
  p.ga = ga;
  p.experts = static_cast<uint32_t>(experts);
  p.alpha = 1.0f;
  const int bn = g_gemm_bn ? g_gemm_bn : 256;
  if (bn == 128) return launch_gemm<true, 128, 5, 2>(op, act, w, p, stream);
  if (bn == 192) return launch_gemm<true, 192, 4, 2>(op, act, w, p, stream);
  return launch_gemm<true, 256, 3, 1>(op, act, w, p, stream);
}

// ---------------------------------------------------------------------------------------------
// Gate/up weight packing for the gated epilogue: output row (f / 32) * 64 + which * 32 + f % 32
// holds feature f of the gate (which = 0) or up (which = 1) matrix; scales follow their rows and
// are written in the interleaved layout.
// ---------------------------------------------------------------------------------------------
namespace gemb {
namespace {
__global__ void __launch_bounds__(256)
pack_gate_up_kernel(const uint8_t* __restrict__ gate, const uint8_t* __restrict__ gate_s,
                    const uint8_t* __restrict__ up, const uint8_t* __restrict__ up_s,
                    uint8_t* __restrict__ out, uint8_t* __restrict__ out_s, uint32_t inter, uint32_t k) {
  const uint32_t chunks = k / 32;                 // 16-byte payload chunks per row
  const uint64_t idx = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<uint64_t>(2) * inter * chunks) return;
  const uint32_t orow = static_cast<uint32_t>(idx / chunks), c = static_cast<uint32_t>(idx % chunks);
  const uint32_t which = (orow / 32) & 1, f = (orow / 64) * 32 + orow % 32;
  const uint8_t* src = (which ? up : gate) + static_cast<uint64_t>(f) * (k / 2) + c * 16;
  const uint8_t* ssrc = (which ? up_s : gate_s) + static_cast<uint64_t>(f) * (k / 16) + c * 2;
  *reinterpret_cast<uint4*>(out + static_cast<uint64_t>(orow) * (k / 2) + c * 16) = __ldg(reinterpret_cast<const uint4*>(src));
  const uint32_t c_pad = (k / 16 + 3) / 4 * 4;
  *reinterpret_cast<uint16_t*>(out_s + interleaved_scale_offset(orow, c * 2, c_pad)) =
      __ldg(reinterpret_cast<const uint16_t*>(ssrc));
}
}  // namespace
}  // namespace gemb

extern "C" int32_t gemb_nvfp4_pack_gate_up(const uint8_t* gate_packed, const uint8_t* gate_scales,
                                           const uint8_t* up_packed, const uint8_t* up_scales,
                                           uint8_t* fused_packed, uint8_t* fused_interleaved_scales,
                                           uint64_t intermediate, uint64_t k, gemb_stream_t stream) {
  const char* op = "gemb_nvfp4_pack_gate_up";
  GEMB_REQUIRE(gate_packed && gate_scales && up_packed && up_scales && fused_packed && fused_interleaved_scales,
               "%s: pointers must be nonnull", op);
  GEMB_REQUIRE(intermediate > 0 && intermediate % 32 == 0 && intermediate < (1ull << 30),
               "%s: intermediate size must be a nonzero multiple of 32", op);
  GEMB_REQUIRE(k > 0 && k % 64 == 0 && k < (1ull << 31), "%s: contracting extent must be a nonzero multiple of 64", op);
  GEMB_REQUIRE(reinterpret_cast<uintptr_t>(gate_packed) % 16 == 0 && reinterpret_cast<uintptr_t>(up_packed) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(fused_packed) % 16 == 0 && reinterpret_cast<uintptr_t>(gate_scales) % 2 == 0 &&
                   reinterpret_cast<uintptr_t>(up_scales) % 2 == 0 && reinterpret_cast<uintptr_t>(fused_interleaved_scales) % 4 == 0,
               "%s: payloads must be 16-byte, scales 2-byte aligned", op);
  GEMB_TRY(require_sm100(op));
  cudaError_t e = cudaMemsetAsync(fused_interleaved_scales, 0, gemb_interleaved_scale_bytes(2 * intermediate, k), stream);
  if (e != cudaSuccess) return fail(GEMB_INTERNAL, "%s: %s: %s", op, cudaGetErrorName(e), cudaGetErrorString(e));
  const uint64_t work = 2 * intermediate * (k / 32);
  pack_gate_up_kernel<<<static_cast<unsigned>((work + 255) / 256), 256, 0, stream>>>(
      gate_packed, gate_scales, up_packed, up_scales, fused_packed, fused_interleaved_scales,
      static_cast<uint32_t>(intermediate), static_cast<uint32_t>(k));
  return check_launch(op);
}

static int32_t launch_gated(const char* op, const uint8_t* act, const uint8_t* w, GemmParams& p, cudaStream_t stream) {
  const int bn = g_gemm_bn ? g_gemm_bn : 256;
  if (bn == 128) return launch_gemm<true, 128, 5, 2>(op, act, w, p, stream);
  return launch_gemm<true, 256, 3, 1>(op, act, w, p, stream);   // 192 is not a multiple of 64 gate/up runs per tile pair
}

int32_t gemb_nvfp4_gemm_gated_quant(const uint8_t* act, const uint8_t* act_scales_interleaved, const uint8_t* w_fused,
                                    const uint8_t* w_scales_interleaved, uint8_t* product_packed,
                                    uint8_t* product_interleaved_scales, uint64_t tokens, uint64_t intermediate,
                                    uint64_t k, float ga, float gw_gate, float gw_up, float product_divisor,
                                    gemb_stream_t stream) {
  const char* op = "gemb_nvfp4_gemm_gated_quant";
  GEMB_REQUIRE(act && act_scales_interleaved && w_fused && w_scales_interleaved && product_packed && product_interleaved_scales,
               "%s: pointers must be nonnull", op);
  GEMB_TRY(validate_gemm(op, tokens, 2 * intermediate, k, 64));
  GEMB_REQUIRE(intermediate % 32 == 0, "%s: intermediate size must be a multiple of 32", op);
  GEMB_REQUIRE(positive_finite(ga) && positive_finite(gw_gate) && positive_finite(gw_up) && positive_finite(product_divisor) &&
                   std::isfinite(ga * gw_gate) && std::isfinite(ga * gw_up),
               "%s: global divisors must be positive and finite", op);
  GEMB_REQUIRE(reinterpret_cast<uintptr_t>(act) % 16 == 0 && reinterpret_cast<uintptr_t>(w_fused) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(act_scales_interleaved) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(w_scales_interleaved) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(product_packed) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(product_interleaved_scales) % 4 == 0,
               "%s: all buffers must be 16-byte aligned", op);
  GEMB_TRY(require_sm100(op));
  GemmParams p{};
  p.sfa = act_scales_interleaved;
  p.sfb = w_scales_interleaved;
  p.m = static_cast<uint32_t>(tokens);
  p.n = static_cast<uint32_t>(2 * intermediate);
  p.k = static_cast<uint32_t>(k);
  p.alpha = 1.0f / (ga * gw_gate);
  p.alpha_up = 1.0f / (ga * gw_up);
  p.gated = 1;
  p.g_product = product_divisor;
  p.out_packed = product_packed;
  p.out_scales = product_interleaved_scales;
  return launch_gated(op, act, w_fused, p, stream);
}

int32_t gemb_moe_grouped_gemm_gated_quant(const uint8_t* act, const uint8_t* act_scales_interleaved, const uint8_t* w_fused,
                                          const uint8_t* w_scales_interleaved, uint8_t* product_packed,
                                          uint8_t* product_interleaved_scales, const int32_t* plan,
                                          uint64_t padded_rows_max, uint64_t experts, uint64_t intermediate, uint64_t k,
                                          float ga, const float* w_divisors, float product_divisor, gemb_stream_t stream) {
  const char* op = "gemb_moe_grouped_gemm_gated_quant";
  GEMB_REQUIRE(act && act_scales_interleaved && w_fused && w_scales_interleaved && product_packed &&
                   product_interleaved_scales && plan && w_divisors,
               "%s: pointers must be nonnull", op);
  GEMB_TRY(validate_gemm(op, padded_rows_max, 2 * intermediate, k, 64));
  GEMB_REQUIRE(padded_rows_max % 128 == 0, "%s: padded row capacity must be a multiple of 128", op);
  GEMB_REQUIRE((2 * intermediate) % 128 == 0, "%s: intermediate size must be a multiple of 64", op);
  GEMB_REQUIRE(experts > 0 && experts <= 4096 && experts * 2 * intermediate < (1ull << 31), "%s: bad expert count", op);
  GEMB_REQUIRE(positive_finite(ga) && positive_finite(product_divisor), "%s: global divisors must be positive and finite", op);
  GEMB_REQUIRE(reinterpret_cast<uintptr_t>(act) % 16 == 0 && reinterpret_cast<uintptr_t>(w_fused) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(act_scales_interleaved) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(w_scales_interleaved) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(product_packed) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(product_interleaved_scales) % 4 == 0,
               "%s: all buffers must be 16-byte aligned", op);
  GEMB_TRY(require_sm100(op));
  GemmParams p{};
  p.sfa = act_scales_interleaved;
  p.sfb = w_scales_interleaved;
  p.m = static_cast<uint32_t>(padded_rows_max);
  p.n = static_cast<uint32_t>(2 * intermediate);
  p.k = static_cast<uint32_t>(k);
  p.plan = plan;
  p.w_divisors = w_divisors;
  p.ga = ga;
  p.experts = static_cast<uint32_t>(experts);
  p.alpha = 1.0f;
  p.gated = 1;
  p.g_product = product_divisor;
  p.out_packed = product_packed;
  p.out_scales = product_interleaved_scales;
  return launch_gated(op, act, w_fused, p, stream);
}

int32_t gemb_fp8_gemm_bf16(const uint8_t* act, const float* act_scales, const uint8_t* w,
                           const uint16_t* w_scales_bf16, uint16_t* out, uint64_t tokens, uint64_t rows,
                           uint64_t k, gemb_stream_t stream) {
  const char* op = "gemb_fp8_gemm_bf16";
  GEMB_REQUIRE(act && act_scales && w && w_scales_bf16 && out, "%s: pointers must be nonnull", op);
  GEMB_TRY(validate_gemm(op, tokens, rows, k, 32));
  GEMB_REQUIRE(reinterpret_cast<uintptr_t>(act) % 16 == 0 && reinterpret_cast<uintptr_t>(w) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(out) % 16 == 0,
               "%s: activation, weight and output must be 16-byte aligned", op);
  GEMB_TRY(require_sm100(op));
  GemmParams p{};
  p.a_scales = act_scales;
  p.w_scales = w_scales_bf16;
  p.out = out;
  p.m = static_cast<uint32_t>(tokens);
  p.n = static_cast<uint32_t>(rows);
  p.k = static_cast<uint32_t>(k);
  p.alpha = 1.0f;
  const int bn = g_gemm_bn == 128 ? 128 : 256;
  if (bn == 128) return launch_gemm<false, 128, 6, 2>(op, act, w, p, stream);
  return launch_gemm<false, 256, 4, 2>(op, act, w, p, stream);
}

int32_t gemb_check_device_status(void) {
  const char* op = "gemb_check_device_status";
  int code = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&code, g_gemm_error, sizeof code);
  if (e != cudaSuccess) return fail(GEMB_INTERNAL, "%s: %s: %s", op, cudaGetErrorName(e), cudaGetErrorString(e));
  if (code != 0) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_gemm_error, &zero, sizeof zero);
    return fail(GEMB_INTERNAL, "%s: a GEMM kernel gave up waiting on a pipeline barrier (role %d)", op, code);
  }
  const int gemv_code = gemv_take_device_error();
  if (gemv_code != 0)
    return fail(GEMB_INTERNAL, "%s: a GEMV kernel gave up waiting on a pipeline barrier (role %d)", op, gemv_code);
  return GEMB_OK;
}

}  // extern "C"
