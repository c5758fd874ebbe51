// Prefill projections: tcgen05 GEMMs with TMEM accumulators and TMA-staged operand tiles.
//
//   NVFP4  D[M,N] = alpha * sum_k (A e2m1 * SFA ue4m3)(B e2m1 * SFB ue4m3)   kind::mxf4nvf4.block16
//   FP8    D[M,N] = (sum_k A e4m3 * B e4m3) * a_scale[m] * w_scale[n]          kind::f8f6f4
//
// A is the activation [M, K] (tokens), B the weight [N, K] (output rows), both K-major, so
// D = A * B^T lands with one token per TMEM lane and one output feature per TMEM column.
//
// One persistent CTA per SM.  Dense calls pair the CTAs (clusters of two, tcgen05 cta_group::2):
// the pair owns a 256 x 256 tile, each CTA stages its own 128 activation rows and 128 of the 256
// weight rows, the even CTA issues every MMA, each CTA accumulates and stores its own 128 rows.
// Grouped (mixture-of-experts) calls keep one CTA per 128 x 256 tile.  Warp roles:
//   producer (warp 0): one elected lane issues TMA tile loads (128-byte swizzle, no multicast)
//            for A and B and 1-D bulk copies for the interleaved block scales into a ring of
//            kStages shared-memory stages, each guarded by a full/empty mbarrier pair;
//   MMA issuer (warp 1): per stage one tcgen05.mma per 32 bytes of K, then a commit of the stage's
//            empty barrier; after the last K step a commit of the accumulator barrier.  In the odd
//            CTA of a pair this warp only relays "operands landed" to the issuer (FP8);
//   epilogue, two sets of four warps: each warp drains its 32 TMEM lanes 64 columns at a time,
//            the sets taking alternate 64-column sub-tiles; scales, rounds to bf16, stages a
//            32 x 128-byte block in its own swizzled buffer and issues a TMA store (which also
//            clips the token / row tails).  FP8 double-buffers the accumulator; NVFP4 has room
//            for one (256 columns + the scale regions), so its epilogue releases the accumulator
//            as early as it can: first sub-tile converted in registers, second loaded, release,
//            and only then the staging and the stores;
//   scale movers (NVFP4), two sets of four warps: copy a stage's block scales from shared memory
//            into the stage's TMEM region with tcgen05.st and arrive on its scales-ready barrier.
//            Doing this with tcgen05.cp from the MMA thread costs a third of the tensor-pipe
//            time, because those copies queue in front of the MMAs.
// NVFP4 lays the roles out on warpgroup boundaries (warps 0-3 producer / issuer / two idle, 4-7
// and 12-15 epilogue, 8-11 and 16-19 movers) so that setmaxnreg can move registers from the
// producer, issuer and movers to the epilogue, which holds 96 accumulator values per thread
// between the accumulator becoming full and its release.
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
constexpr int kGemmThreadsFp4 = 640;   // warpgroups: control (producer, MMA, 2 idle), epilogue, movers, epilogue, movers
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
  // Pushing epilogue (push_meta != null; grouped bf16 output only): row r of the padded row space
  // is not stored at out[r] but at row push_meta[r].y of the bf16 [push_rows, n] buffer
  // push_dst[push_meta[r].x] -- for expert parallelism the buffer of the GPU that owns the token,
  // written with plain 16-byte stores over NVLink while the next tile's MMAs run.  Only the first
  // push_tile_rows[tile] rows of a tile are real assignments; the rest is padding and is dropped.
  const int2* push_meta;
  const int32_t* push_tile_rows;
  uint8_t* push_dst[16];
  uint32_t push_ranks;
  uint32_t push_rows;
  uint32_t m_out;                // rows of the buffer the output tensor map describes (0: m)
  // Up projection with a materialised gate (gate_in != null): the accumulator holds Up [M, n], the
  // bf16 Gate [M, n] is read in the epilogue, which writes the quantised GELU product like `gated`.
  const uint16_t* gate_in;
  // Grouped calls on CTA pairs: only the tiles of experts [expert_lo, expert_hi) (expert_hi = 0: all of them).
  uint32_t expert_lo, expert_hi;
};

template <bool kFp4, int BN, int kStages, int kAccStages, bool kPair = false>
struct Cfg {
  static constexpr int kKPerStage = kFp4 ? 256 : 128;      // elements covered by 128 bytes
  static constexpr int kKPerMma = kFp4 ? 64 : 32;          // elements per tcgen05.mma
  static constexpr int kABytes = BM * 128;
  static constexpr int kBRows = kPair ? BN / 2 : BN;       // weight rows this CTA stages
  static constexpr int kBBytes = kBRows * 128;
  // Weight scales are stored in 128-row groups: a 256-wide tile stages two of them.
  static constexpr int kSfbGroups = BN / 128;
  static constexpr int kSfaBytes = kFp4 ? 2048 : 0;        // 4 chunks of 512 B
  static constexpr int kSfbBytes = kFp4 ? kSfbGroups * 2048 : 0;
  static constexpr int kStageBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;
  static constexpr int kEpiBytes = 8 * 4096;               // eight epilogue warps x one staging buffer (32 rows x 128 B)
  static constexpr int kBarrierBytes = 1024;
  static constexpr int kSmemBytes = kStages * kStageBytes + kEpiBytes + kBarrierBytes + 1024;  // + alignment slack
  // TMEM columns: accumulators first, then one scale region per shared-memory stage.  A stage's
  // "empty" barrier (its MMAs have completed) therefore also frees its scale region, and a stage
  // that is full again proves it: the scale movers need no barrier of their own for the region.
  static constexpr int kAccCols = kAccStages * BN;
  static constexpr int kSfaCols = 16;                      // 4 MMAs x 4 columns
  static constexpr int kSfbColsPerMma = BN / 32;
  static constexpr int kSfbCols = 4 * kSfbColsPerMma;
  static constexpr int kSfColsPerStage = kFp4 ? kSfaCols + kSfbCols : 0;
  static_assert(kAccCols + kStages * kSfColsPerStage <= 512, "TMEM budget exceeded");
  static_assert(BN == 128 || BN == 256, "BN must be 128 or 256");
    static_assert(kSmemBytes <= 227 * 1024, "shared memory budget exceeded");
};

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

template <bool kFp4, int BN, int kStages, int kAccStages, bool kPair>
__global__ void __launch_bounds__(kFp4 ? kGemmThreadsFp4 : kGemmThreadsFp8, 1)
gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
            const __grid_constant__ CUtensorMap map_out, const GemmParams p) {
  using C = Cfg<kFp4, BN, kStages, kAccStages, kPair>;
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
  uint64_t* sf_ready = acc_empty + kAccStages;   // per stage: its scales are in TMEM
  uint64_t* peer_full = sf_ready + kStages;      // pairs, FP8: the odd CTA's operands have landed
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(peer_full + kStages);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // CTA pairs: the even CTA (rank 0) issues every MMA; the barriers that gate it (scales ready,
  // accumulator drained, peer operands landed) live in its shared memory and collect arrivals
  // from both CTAs.  The MMA's completion is committed to the same barrier in both CTAs.
  const uint32_t rank = kPair ? ptx::cluster_ctarank() : 0u;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(&full[s], 1);
      ptx::mbar_init(&empty[s], 1);
      ptx::mbar_init(&sf_ready[s], kPair ? 8 : 4);
      ptx::mbar_init(&peer_full[s], 1);
    }
    for (int s = 0; s < kAccStages; ++s) {
      ptx::mbar_init(&acc_full[s], 1);
      ptx::mbar_init(&acc_empty[s], kPair ? 16 : 8);
    }
    *abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::prefetch_tensormap(&map_a);
    ptx::prefetch_tensormap(&map_b);
    ptx::prefetch_tensormap(&map_out);
  }
  if (warp == 1) {
    if constexpr (kPair) ptx::tmem_alloc_pair(tmem_holder, 512);
    else ptx::tmem_alloc(tmem_holder, 512);
  }
  ptx::tc_fence_before();
  if constexpr (kPair) ptx::cluster_sync();
  else __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  // A device-side plan is clamped to the buffers' capacity (p.m rows): whatever it holds, no tile
  // beyond the activation, scale and output buffers is touched.
  // Grouped mode: experts are padded to 256 rows, so a 128-row tile may hold padding only.  A single
  // CTA walks the plan's list of tiles that hold real rows; a pair walks all 256-row units (the even
  // tile of a unit is always real) and takes the expert from the even tile.
  // plan entries behind the expert offsets: {expert of tile i (-1: padding only), i-th tile that holds real rows},
  // then, behind the last tile's pair, the number of tiles that hold real rows.
  const int32_t* tile_info = p.plan ? p.plan + 3 + p.experts : nullptr;
  const uint32_t plan_tiles = p.plan ? min(static_cast<uint32_t>(__ldg(p.plan)), p.m / BM) : 0u;
  const uint32_t m_tiles = p.plan ? (kPair ? plan_tiles : min(static_cast<uint32_t>(__ldg(tile_info + 2 * plan_tiles)), plan_tiles))
                                  : (p.m + BM - 1) / BM;
  const uint32_t n_tiles = (p.n + BN - 1) / BN;
  const int32_t* tile_expert = tile_info;   // stride 2
  // A work unit is one 128-row token tile, or for pairs two consecutive ones (rank picks which).
  uint32_t m_units = kPair ? (m_tiles + 1) / 2 : m_tiles;
  uint32_t unit0 = 0;   // first 256-row unit of the call's expert range
  if constexpr (kPair) {
    if (p.plan != nullptr && p.expert_hi != 0) {   // padded offsets are multiples of 256 rows: whole units
      const uint32_t lo_t = min(static_cast<uint32_t>(__ldg(p.plan + 2 + min(p.expert_lo, p.experts))) / BM, plan_tiles);
      const uint32_t hi_t = min(static_cast<uint32_t>(__ldg(p.plan + 2 + min(p.expert_hi, p.experts))) / BM, plan_tiles);
      unit0 = lo_t / 2;
      m_units = hi_t > lo_t ? (hi_t - lo_t + 1) / 2 : 0u;
    }
  }
  const uint32_t num_tiles = m_units * n_tiles;
  const uint32_t first_tile = kPair ? blockIdx.x >> 1 : blockIdx.x;
  const uint32_t tile_stride = kPair ? gridDim.x >> 1 : gridDim.x;
  const uint32_t my_tiles = first_tile < num_tiles ? (num_tiles - first_tile + tile_stride - 1) / tile_stride : 0;
  const uint32_t k_stages = (p.k + C::kKPerStage - 1) / C::kKPerStage;
  const uint32_t k_groups_pad = (p.k / 16 + 3) / 4;  // 512-byte scale chunks per 128-row group
  auto tile_expert_of = [&](uint32_t mt) -> int32_t {
    return __ldg(tile_expert + 2 * (kPair ? (mt & ~1u) : mt));
  };

  // Tile order: groups of 16 token tiles; inside a group the token tile runs fastest, so the
  // CTAs of a wave share a few weight tiles and the group's activations stay in L2 while every
  // weight tile passes over them.
  auto tile_coords = [&](uint32_t tile, uint32_t& mt, uint32_t& nt) {
    constexpr uint32_t kGroupM = kPair ? 8 : 16;
    const uint32_t per_group = kGroupM * n_tiles;
    const uint32_t first_m = (tile / per_group) * kGroupM;
    const uint32_t gm = min(kGroupM, m_units - first_m);
    const uint32_t within = tile % per_group;
    mt = first_m + within % gm;
    if constexpr (kPair) mt = (mt + unit0) * 2 + rank;
    else if (tile_info != nullptr) mt = min(static_cast<uint32_t>(__ldg(tile_info + 2 * mt + 1)), p.m / BM - 1);
    nt = within / gm;
  };
  // Completion of the MMAs issued so far, signalled to the same barrier of both CTAs of a pair.
  const uint32_t bars_rank0 = kPair ? ptx::cluster_map(bars, 0) : 0u;
  const uint32_t bars_rank1 = kPair ? ptx::cluster_map(bars, 1) : 0u;
  auto commit = [&](uint64_t* bar) {
    if constexpr (kPair) {
      const uint32_t off = static_cast<uint32_t>(reinterpret_cast<uint8_t*>(bar) - reinterpret_cast<uint8_t*>(bars));
      ptx::tc_commit_pair(bars_rank0 + off);
      ptx::tc_commit_pair(bars_rank1 + off);
    } else {
      ptx::tc_commit(bar);
    }
  };
  // Arrival on a barrier that gates the MMA issuer.
  auto arrive_issuer = [&](uint64_t* bar) {
    if constexpr (kPair) ptx::mbar_arrive_cluster(ptx::cluster_map(bar, 0));
    else ptx::mbar_arrive(bar);
  };
  auto wait_issuer = [&](uint64_t* bar, uint32_t parity) {
    if constexpr (kPair) return ptx::mbar_wait_cluster(bar, parity);
    else return ptx::mbar_wait(bar, parity);
  };

  auto fail_wait = [&](int code) {
    atomicCAS(&g_gemm_error, 0, code);
    *abort_flag = 1;
  };

  // NVFP4: 640 threads start with 96 registers each.  The control warpgroup (to 40) and the two
  // mover warpgroups (to 72) hand back 128 * (56 + 2 * 24) = 13,312 registers; the two epilogue
  // warpgroups (to 144) take 128 * 2 * 48 = 12,288 of them.  An inc can only be served from what
  // the same CTA has released, so the decs must cover the incs (the inc waits for them).  Each
  // setmaxnreg is the first thing its whole warpgroup executes inside the branch it governs.
  const bool is_ctrl = kFp4 ? warp < 4 : warp < 2;
  const bool is_mover = kFp4 && ((warp >= 8 && warp < 12) || warp >= 16);
  if (is_ctrl) {
  if constexpr (kFp4) ptx::reg_dec<40>();
  if (warp == 0) {
    // ------------------------------- producer -------------------------------------------------
    if (ptx::elect_one()) {
      uint32_t stage = 0, phase = 0;
      for (uint32_t tile = first_tile; tile < num_tiles && !*abort_flag; tile += tile_stride) {
        uint32_t mt, nt;
        tile_coords(tile, mt, nt);
        const uint32_t expert = tile_expert ? min(static_cast<uint32_t>(tile_expert_of(mt)), p.experts - 1) : 0u;
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
            // The odd CTA of a pair may sit past the last token tile: its rows are never stored,
            // it just reads the last tile's scales again.
            ptx::bulk_load_1d(stage_sfa + stage * C::kSfaBytes,
                              p.sfa + (static_cast<uint64_t>(min(mt, (p.plan ? p.m / BM : m_tiles) - 1)) * k_groups_pad + ks * 4) * 512,
                              n_mma * 512, &full[stage]);
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
                           static_cast<int32_t>(expert * p.n + nt * BN + rank * C::kBRows));
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1 && rank != 0) {
    // ------------------------------- odd CTA of a pair: relay (FP8) ---------------------------
    // Tells the issuer in the even CTA that this CTA's operands have landed.  NVFP4 needs no
    // relay: the scale movers, who wait for the operands, arrive on the issuer's barrier.
    if (!kFp4 && ptx::elect_one()) {
      const uint32_t total_steps = my_tiles * k_stages;
      uint32_t stage = 0, phase = 0;
      for (uint32_t step = 0; step < total_steps && !*abort_flag; ++step) {
        if (!ptx::mbar_wait(&full[stage], phase)) { fail_wait(7); break; }
        arrive_issuer(&peer_full[stage]);
        if (++stage == kStages) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -----------------------------------------------
    // One thread issues everything.  Its instruction stream is on the critical path (an MMA
    // takes about 50 clocks to issue and 128 to execute, a barrier poll about 160 to return),
    // so the barrier of the NEXT step is polled before this step's MMAs are issued and the
    // answer is only looked at one iteration later.
    if (ptx::elect_one()) {
      constexpr uint32_t kM = kPair ? 2 * BM : BM;
      constexpr uint32_t idesc = kFp4 ? ptx::idesc_nvfp4(kM, BN) : ptx::idesc_e4m3(kM, BN);
      uint32_t as = 0, aphase = 0;
      uint32_t stage = 0, phase = 0;
      bool ready = false;
      for (uint32_t t = 0; t < my_tiles && !*abort_flag; ++t) {
        if (!wait_issuer(&acc_empty[as], aphase ^ 1)) { fail_wait(2); break; }
        const uint32_t tmem_acc = tmem_base + as * BN;
        uint32_t k_left = p.k;
        bool ok = true;
        for (uint32_t ks = 0; ks < k_stages; ++ks, k_left -= C::kKPerStage) {
          // NVFP4 waits for the scale movers (who waited for the operands); FP8 for the operands.
          if (!ready) {
            if constexpr (kFp4) {
              ok = wait_issuer(&sf_ready[stage], phase);
            } else {
              ok = ptx::mbar_wait(&full[stage], phase);
              if constexpr (kPair) ok = ok && wait_issuer(&peer_full[stage], phase);
            }
            if (!ok) { fail_wait(3); break; }
          }
          ptx::tc_fence_after();
          const uint32_t next_stage = stage + 1 == kStages ? 0 : stage + 1;
          const uint32_t next_phase = stage + 1 == kStages ? phase ^ 1 : phase;
          const uint32_t n_mma = min(4u, k_left / C::kKPerMma);
          const uint64_t a_desc = ptx::smem_desc_k128_swizzled(ptx::smem_addr(stage_a + stage * C::kABytes));
          const uint64_t b_desc = ptx::smem_desc_k128_swizzled(ptx::smem_addr(stage_b + stage * C::kBBytes));
          // What the next step will wait for: NVFP4 the scale movers (who waited for the operands),
          // FP8 the operands of this CTA and, in a pair, of the odd CTA.
          uint64_t* poll0 = kFp4 ? &sf_ready[next_stage] : &full[next_stage];
          uint64_t* poll1 = (!kFp4 && kPair) ? &peer_full[next_stage] : poll0;
          if constexpr (kFp4) {
            const uint32_t tsfa = tmem_base + C::kAccCols + stage * C::kSfColsPerStage;
            const uint32_t tsfb = tsfa + C::kSfaCols;
            if (n_mma == 4) {
              if constexpr (kPair)
                ready = ptx::tc_mma4_nvfp4_pair_poll(tmem_acc, a_desc, b_desc, idesc, ks, tsfa, tsfb,
                                                     C::kSfbColsPerMma, poll0, poll1, next_phase);
              else
                ready = ptx::tc_mma4_nvfp4_poll(tmem_acc, a_desc, b_desc, idesc, ks, tsfa, tsfb,
                                                C::kSfbColsPerMma, poll0, poll1, next_phase);
            } else {
              ready = false;
              for (uint32_t j = 0; j < n_mma; ++j) {
                if constexpr (kPair)
                  ptx::tc_mma_nvfp4_pair(tmem_acc, a_desc + j * 2, b_desc + j * 2, idesc, tsfa + j * 4,
                                         tsfb + j * C::kSfbColsPerMma, (ks | j) != 0 ? 1u : 0u);
                else
                  ptx::tc_mma_nvfp4(tmem_acc, a_desc + j * 2, b_desc + j * 2, idesc, tsfa + j * 4,
                                    tsfb + j * C::kSfbColsPerMma, (ks | j) != 0 ? 1u : 0u);
              }
            }
          } else {
            if (n_mma == 4) {
              if constexpr (kPair)
                ready = ptx::tc_mma4_f8_pair_poll(tmem_acc, a_desc, b_desc, idesc, ks, poll0, poll1, next_phase);
              else
                ready = ptx::tc_mma4_f8_poll(tmem_acc, a_desc, b_desc, idesc, ks, poll0, poll1, next_phase);
            } else {
              ready = false;
              for (uint32_t j = 0; j < n_mma; ++j) {
                if constexpr (kPair)
                  ptx::tc_mma_f8_pair(tmem_acc, a_desc + j * 2, b_desc + j * 2, idesc, (ks | j) != 0 ? 1u : 0u);
                else
                  ptx::tc_mma_f8(tmem_acc, a_desc + j * 2, b_desc + j * 2, idesc, (ks | j) != 0 ? 1u : 0u);
              }
            }
          }
          commit(&empty[stage]);   // frees the operand stage and, NVFP4, its scale region
          stage = next_stage;
          phase = next_phase;
        }
        if (!ok) break;
        commit(&acc_full[as]);
        if (++as == kAccStages) { as = 0; aphase ^= 1; }
      }
    }
  }  // warps 2 and 3 of the NVFP4 control warpgroup are idle
  } else if (is_mover) {
    // ------------------------------- scale movers (NVFP4) ------------------------------------
    // Two sets of four warps (one warp per TMEM lane quarter), since one trip of this loop
    // (barrier poll, shared loads, tcgen05.st, wait, arrive) takes longer than a step's four
    // MMAs.  Set 0 owns the even stages and set 1 the odd ones: every use of a stage's barrier is
    // then seen by the same warps in order, which the parity waits rely on (a waiter that skipped
    // a phase would take the older phase's completion for the one it wants).  Per stage each
    // lane reads its 16-byte rows of the staged scale chunks (one row = the four TMEM columns of
    // one MMA) and writes them to the stage's TMEM region with two wide tcgen05.st.  The set's
    // next barrier is polled while the loads are in flight.
    if constexpr (kFp4) {
      ptx::reg_dec<72>();
      const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
      const uint32_t total_steps = my_tiles * k_stages;
      static_assert(kStages % 2 == 1 && kStages >= 3, "the mover sets split an odd number of stages");
      const uint32_t mset = warp >= 16 ? 1u : 0u;
      uint32_t stage = mset, phase = 0, step = mset, ks = mset % k_stages;
      bool ready = false;
      while (step < total_steps && !*abort_flag) {
        if (!ready && !ptx::mbar_wait(&full[stage], phase)) { fail_wait(5); break; }
        // A full stage means its previous MMAs completed (the producer waited for that), so the
        // stage's TMEM scale region is free as well.
        ptx::tc_fence_after();
        const uint32_t n_mma = min(4u, (p.k - ks * C::kKPerStage) / C::kKPerMma);
        const uint32_t tsfa = tmem_base + C::kAccCols + stage * C::kSfColsPerStage + lane_base;
        const uint32_t tsfb = tsfa + C::kSfaCols;
        const uint8_t* sfa_s = stage_sfa + stage * C::kSfaBytes + lane * 16;
        const uint8_t* sfb_s = stage_sfb + stage * C::kSfbBytes + lane * 16;
        // This set's next stage: two further, or back to its first one (set 0 wraps from the last
        // stage to stage 0, one step later; set 1 from the last but one to stage 1, three later).
        uint32_t next_stage = stage + 2, next_phase = phase, delta = 2;
        if (next_stage >= kStages) {
          next_stage = mset;
          next_phase ^= 1;
          delta = mset ? 3 : 1;
        }
        if (n_mma == 4) {
          uint4 a4[4], b4[4 * C::kSfbGroups];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            a4[j] = *reinterpret_cast<const uint4*>(sfa_s + j * 512);
#pragma unroll
            for (int g = 0; g < C::kSfbGroups; ++g)
              b4[j * C::kSfbGroups + g] = *reinterpret_cast<const uint4*>(sfb_s + g * 2048 + j * 512);
          }
          ready = ptx::mbar_test_wait(&full[next_stage], next_phase);
          ptx::tc_st_32x32b_x16(tsfa, a4);
          if constexpr (C::kSfbGroups == 2) ptx::tc_st_32x32b_x32(tsfb, b4);
          else ptx::tc_st_32x32b_x16(tsfb, b4);
        } else {
          // Last stage of a K that is not a multiple of 256: fewer MMAs, fewer scale rows staged.
          ready = false;
          for (uint32_t j = 0; j < n_mma; ++j) {
            ptx::tc_st_32x32b_x4(tsfa + j * 4, *reinterpret_cast<const uint4*>(sfa_s + j * 512));
            for (int g = 0; g < C::kSfbGroups; ++g)
              ptx::tc_st_32x32b_x4(tsfb + j * C::kSfbColsPerMma + g * 4,
                                   *reinterpret_cast<const uint4*>(sfb_s + g * 2048 + j * 512));
          }
        }
        ptx::tc_wait_st();
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) arrive_issuer(&sf_ready[stage]);
        stage = next_stage;
        phase = next_phase;
        step += delta;
        ks += delta;
        while (ks >= k_stages) ks -= k_stages;
      }
    }
  } else {
    // ------------------------------- epilogue -------------------------------------------------
    // Two sets of four warps; set s drains the 64-column sub-tiles s, s+2, ... of every tile.
    if constexpr (kFp4) ptx::reg_inc<144>();
    const uint32_t quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter+32) belong to this warp
    const uint32_t set = warp >= (kFp4 ? 12 : 6) ? 1u : 0u;
    uint8_t* my_stage = epi_stage + (set * 4 + quarter) * 4096;
    uint32_t as = 0, aphase = 0;
    for (uint32_t tile = first_tile; tile < num_tiles && !*abort_flag; tile += tile_stride) {
      uint32_t mt, nt;
      tile_coords(tile, mt, nt);
      // In a pair the odd CTA may own a padding-only tile: it takes part in the barriers, nothing else.
      const bool dead = kPair && tile_expert != nullptr && (mt >= p.m / BM || __ldg(tile_expert + 2 * mt) < 0);
      // The staging buffer must be free again (the previous tile's last store has read it); checked
      // here, while the tile is still being computed, rather than after the accumulator is full.
      if (lane == 0) ptx::bulk_wait_group_read<0>();
      __syncwarp();
      if (!ptx::mbar_wait(&acc_full[as], aphase)) { fail_wait(4); break; }
      ptx::tc_fence_after();
      const uint32_t row0 = mt * BM + quarter * 32;
      float row_scale = p.alpha;
      if constexpr (!kFp4) row_scale = row0 + lane < p.m ? __ldg(p.a_scales + row0 + lane) : 0.0f;
      if (kFp4 && p.w_divisors != nullptr)
        row_scale = __fdiv_rn(1.0f, __fmul_rn(p.ga, __ldg(p.w_divisors + (tile_expert ? min(static_cast<uint32_t>(tile_expert_of(mt)), p.experts - 1) : 0u))));
      const uint32_t tmem_acc = tmem_base + as * BN + ((quarter * 32) << 16);
      bool released = false, pending = false;
      uint32_t pending_col = 0;
      uint32_t packed[32];  // one converted sub-tile: 16-byte chunk j of this lane's row = packed[4j .. 4j+3]
      // Stages `packed` in this warp's swizzled buffer and hands it to a TMA store.
      // Pushing epilogue: where this lane's row goes, and how many of the warp's 32 rows are real.
      int2 push_to = make_int2(-1, 0);
      uint32_t push_valid = 0;
      if (kFp4 && p.push_meta != nullptr && !dead) {
        const uint32_t tile_rows = min(static_cast<uint32_t>(__ldg(p.push_tile_rows + mt)), static_cast<uint32_t>(BM));
        push_valid = tile_rows > quarter * 32 ? min(32u, tile_rows - quarter * 32) : 0u;
        if (static_cast<uint32_t>(lane) < push_valid) {
          push_to = __ldg(p.push_meta + row0 + lane);
          if (static_cast<uint32_t>(push_to.x) >= p.push_ranks || static_cast<uint32_t>(push_to.y) >= p.push_rows) {
            atomicCAS(&g_gemm_error, 0, 8);   // a destination outside the buffers: recorded, the row is dropped
            push_to.x = -1;
          }
        }
      }
      auto stage_and_store = [&](uint32_t col) {
        if (kFp4 && p.push_meta != nullptr) {
          __syncwarp();   // the previous sub-tile's pushes have read the buffer
#pragma unroll
          for (int j = 0; j < 8; ++j)
            *reinterpret_cast<uint4*>(my_stage + lane * 128 + ((j ^ (lane & 7)) << 4)) =
                make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
          __syncwarp();
          // Eight lanes take one row: 8 x 16 bytes = one full 128-byte line of the destination row.
          const uint32_t chunk = lane & 7;
#pragma unroll
          for (int it = 0; it < 8; ++it) {
            const uint32_t r = it * 4 + (lane >> 3);
            const int dst_rank = __shfl_sync(0xFFFFFFFFu, push_to.x, r);
            const int dst_row = __shfl_sync(0xFFFFFFFFu, push_to.y, r);
            if (dst_rank < 0 || col + chunk * 8 >= p.n) continue;
            const uint4 v = *reinterpret_cast<const uint4*>(my_stage + r * 128 + ((chunk ^ (r & 7)) << 4));
            uint8_t* dst = p.push_dst[dst_rank] + (static_cast<uint64_t>(dst_row) * p.n + col + chunk * 8) * 2;
            asm volatile("st.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
          }
          pending = false;
          return;
        }
        if (lane == 0) ptx::bulk_wait_group_read<0>();  // the previous store has read the buffer
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 8; ++j)
          // chunk j of row `lane` goes to chunk j ^ (lane % 8): the 128-byte swizzle the output
          // tensor map expects, and conflict free for the warp.
          *reinterpret_cast<uint4*>(my_stage + lane * 128 + ((j ^ (lane & 7)) << 4)) =
              make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
        ptx::fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          ptx::tma_store_2d(&map_out, my_stage, static_cast<int32_t>(col), static_cast<int32_t>(row0));
          ptx::bulk_commit_group();
        }
        pending = false;
      };
      // Gated epilogue, second half: packed[i] = {bf16 gate, bf16 up} of feature f0 + i -> GELU, product,
      // NVFP4 quantisation (two 16-blocks), 16 payload bytes and two scale bytes per row.
      auto emit_gated = [&](uint32_t col) {
        const uint32_t f0 = col / 2, inter = p.n / 2;
        uint32_t words[4];
        uint8_t sb[2];
#pragma unroll
        for (int b = 0; b < 2; ++b) {
          float prod[16];
#pragma unroll
          for (int i = 0; i < 16; ++i)   // bf16 boundaries of src/cuda/nvfp4/reference.cu:177-190
            prod[i] = gelu_tanh_product(__uint_as_float(packed[b * 16 + i] << 16), __uint_as_float(packed[b * 16 + i] & 0xFFFF0000u));
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
        pending = false;
      };
#pragma unroll 1
      for (uint32_t c = set; c < BN / 64; c += 2) {
        const uint32_t col0 = nt * BN + c * 64;
        if (col0 >= p.n || row0 >= p.m || dead) break;  // warp-uniform
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
          // Like the plain path, nothing slow sits between "accumulator full" and its release: a
          // sub-tile is only scaled and rounded to bf16 pairs (the first step of the boundary
          // arithmetic anyway) and kept in `packed`; the GELU, the product and the quantiser run
          // after the warp's last sub-tile is in registers and the accumulator has been released.
          ptx::tc_wait_ld();
          if (c + 2 >= BN / 64 || col0 + 128 >= p.n) {
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) arrive_issuer(&acc_empty[as]);
            released = true;
          }
          if (pending) emit_gated(pending_col);
          const float alpha_g = row_scale, alpha_u = p.w_divisors != nullptr ? row_scale : p.alpha_up;
#pragma unroll
          for (int i = 0; i < 32; ++i)
            packed[i] = pack_bf16x2(__fmul_rn(__uint_as_float(v0[i]), alpha_g), __fmul_rn(__uint_as_float(v1[i]), alpha_u));
          pending = true;
          pending_col = col0;
          continue;
        }
        if (kFp4 && p.gate_in != nullptr) {
          // 64 up values of features col0 .. col0+63 for this thread's token; the gate of the same
          // features comes from memory (bf16, 128 bytes of the token's row).
          ptx::tc_wait_ld();
          if (c + 2 >= BN / 64 || col0 + 128 >= p.n) {
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) arrive_issuer(&acc_empty[as]);
            released = true;
          }
          const uint32_t row = row0 + lane;
          if (row < p.m) {
            const uint4* gp = reinterpret_cast<const uint4*>(p.gate_in + static_cast<uint64_t>(row) * p.n + col0);
            const uint32_t c_pad = (p.n / 16 + 3) / 4 * 4;
#pragma unroll
            for (int b = 0; b < 4; ++b) {
              if (col0 + b * 16 >= p.n) break;
              const uint4 ga4 = __ldg(gp + 2 * b), gb4 = __ldg(gp + 2 * b + 1);
              const uint32_t gw[8] = {ga4.x, ga4.y, ga4.z, ga4.w, gb4.x, gb4.y, gb4.z, gb4.w};
              float prod[16];
#pragma unroll
              for (int i = 0; i < 16; ++i) {
                const uint32_t acc = b < 2 ? v0[b * 16 + i] : v1[(b - 2) * 16 + i];
                const float uv = bf16_round(__fmul_rn(__uint_as_float(acc), row_scale));
                const float gv = __uint_as_float((i & 1) ? (gw[i >> 1] & 0xFFFF0000u) : (gw[i >> 1] << 16));
                prod[i] = gelu_tanh_product(gv, uv);
              }
              uint32_t lo, hi;
              uint8_t sb;
              quantize_block16<false>(prod, p.g_product, lo, hi, sb);
              *reinterpret_cast<uint2*>(p.out_packed + static_cast<uint64_t>(row) * (p.n / 2) + (col0 + b * 16) / 2) = make_uint2(lo, hi);
              p.out_scales[interleaved_scale_offset(row, (col0 + b * 16) / 16, c_pad)] = sb;
            }
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
        // Plain bf16 output.  Nothing slow may sit between the accumulator becoming full and its
        // release (the MMA issuer is idle meanwhile): a warp's first sub-tile is only converted,
        // registers to registers; once its last one is in registers too the accumulator is
        // released, and the staging and the TMA stores of both follow.
        ptx::tc_wait_ld();
        if (c + 2 >= BN / 64) {
          ptx::tc_fence_before();
          __syncwarp();
          if (lane == 0) arrive_issuer(&acc_empty[as]);
          released = true;
        }
        if (pending) stage_and_store(pending_col);
#pragma unroll
        for (int half = 0; half < 2; ++half) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int e = q * 8 + i * 2;  // column within this 32-column half
              float lo = __uint_as_float(half == 0 ? v0[e] : v1[e]);
              float hi = __uint_as_float(half == 0 ? v0[e + 1] : v1[e + 1]);
              if constexpr (kFp4) {
                lo = __fmul_rn(lo, row_scale);
                hi = __fmul_rn(hi, row_scale);
              } else {
                // (acc * a_scale) * w_scale, in that order: src/cuda/fp8/cutlass_sm120.cu:49-63.
                const uint32_t wp = __shfl_sync(0xFFFFFFFFu, ws_pair, half * 16 + e / 2);
                lo = __fmul_rn(__fmul_rn(lo, row_scale), __uint_as_float(wp << 16));
                hi = __fmul_rn(__fmul_rn(hi, row_scale), __uint_as_float(wp & 0xFFFF0000u));
              }
              packed[(half * 4 + q) * 4 + i] = pack_bf16x2(lo, hi);
            }
          }
        }
        pending = true;
        pending_col = col0;
      }
      if (pending) {
        if (kFp4 && p.gated) emit_gated(pending_col);
        else stage_and_store(pending_col);
      }
      if (!released) {
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) arrive_issuer(&acc_empty[as]);
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
  // Neither CTA of a pair may leave while the other can still reach its shared memory or barriers.
  if constexpr (kPair) ptx::cluster_sync();
  if (warp == 1) {
    ptx::tc_fence_after();
    if constexpr (kPair) ptx::tmem_dealloc_pair(tmem_base, 512);
    else ptx::tmem_dealloc(tmem_base, 512);
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

int g_gemm_bn = 0;    // 0 = automatic; gemb_set_tuning(GEMB_TUNE_GEMM_BN, 128 | 256)
int g_gemm_pair = 0;  // 0 = automatic (pairs for the dense 256-wide tile), 1 = never, 2 = always

bool use_pairs() { return g_gemm_pair != 1 && (g_gemm_bn == 0 || g_gemm_bn == 256 || g_gemm_pair == 2); }

// Grouped calls run on CTA pairs when the experts are expected to hold many 128-row tiles each.  A pair
// works in units of 256 rows, so it also multiplies the padding rows behind every expert (on average
// 128 per expert against 64 for single CTAs that walk the list of real tiles): measured on 128 experts,
// pairs win from about 768 rows per expert (16,384 tokens top-8: gate/up 328 against 350 us) and lose
// below (4,096 tokens: 132 against 123 us, down 103 against 90 us).  The expectation is the rows the caller announced (the layer calls know how
// many assignments they route) or else what the capacity of the padded row space implies.
thread_local uint64_t g_grouped_rows_hint = 0;
// Upper bound on the persistent grid of the GEMMs this thread launches (0 = none): lets a caller run two
// GEMMs side by side on disjoint sets of SMs instead of having their CTAs take turns.
thread_local uint32_t g_gemm_cta_cap = 0;
// Expert range of the grouped GEMMs this thread launches next on CTA pairs ({0, 0}: all experts).
thread_local uint32_t g_expert_lo = 0, g_expert_hi = 0;
bool grouped_pairs(uint64_t padded_rows_max, uint64_t experts) {
  if (!use_pairs()) return false;
  uint64_t rows = g_grouped_rows_hint;
  if (rows == 0) rows = padded_rows_max / 128 > 2 * experts ? (padded_rows_max / 128 - 2 * experts) * 128 : 0;
  return g_gemm_pair == 2 || rows >= 768 * experts;
}

template <bool kFp4, int BN, int kStages, int kAccStages, bool kPair = false>
int32_t launch_gemm(const char* op, const void* a, const void* b, const GemmParams& p, cudaStream_t stream) {
  using C = Cfg<kFp4, BN, kStages, kAccStages, kPair>;
  auto kern = gemm_kernel<kFp4, BN, kStages, kAccStages, kPair>;
  constexpr unsigned kThreads = kFp4 ? kGemmThreadsFp4 : kGemmThreadsFp8;
  // First call per device and kernel variant: shared-memory opt-in and the pair occupancy,
  // serialised so that two host threads cannot race on it.
  static bool configured[64] = {false};
  static int max_pairs[64] = {0};
  static std::mutex configure_mutex;
  int dev = 0;
  cudaGetDevice(&dev);
  dev &= 63;
  std::lock_guard<std::mutex> configure_lock(configure_mutex);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cudaLaunchConfig_t cfg{};
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = C::kSmemBytes;
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = kPair ? 1 : 0;
  if (!configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
    if (e != cudaSuccess) return fail(GEMB_INTERNAL, "%s: %s: %s", op, cudaGetErrorName(e), cudaGetErrorString(e));
    if constexpr (kPair) {
      // How many CTA pairs the device can hold at once: the persistent grid is sized to it.
      cfg.gridDim = dim3(static_cast<unsigned>(sm_count()) & ~1u);
      int clusters = 0;
      e = cudaOccupancyMaxActiveClusters(&clusters, kern, &cfg);
      if (e != cudaSuccess || clusters <= 0) {
        cudaGetLastError();
        return fail(GEMB_INTERNAL, "%s: CTA pairs cannot be scheduled on this device (%s)", op, cudaGetErrorName(e));
      }
      max_pairs[dev] = clusters;
    }
    configured[dev] = true;
  }
  const uint64_t row_bytes = kFp4 ? p.k / 2 : p.k;
  CUtensorMap map_a, map_b, map_out;
  GEMB_TRY(make_byte_map(op, &map_a, a, p.m, row_bytes, BM));
  GEMB_TRY(make_byte_map(op, &map_b, b, static_cast<uint64_t>(p.n) * (p.plan ? p.experts : 1u), row_bytes, C::kBRows));
  if (p.out_f32)
    GEMB_TRY(make_out_map_f32(op, &map_out, p.out, p.m, p.n));
  else if (p.gated)  // the tensor-map store path is unused; describe the payload buffer so the map is valid
    GEMB_TRY(make_out_map(op, &map_out, p.out_packed, p.m, p.n / 8));
  else if (p.gate_in != nullptr)
    GEMB_TRY(make_out_map(op, &map_out, p.out_packed, p.m, p.n / 4));
  else
    GEMB_TRY(make_out_map(op, &map_out, p.out, p.m_out ? p.m_out : p.m, p.n));
  const uint32_t m_tiles = (p.m + BM - 1) / BM, n_tiles = (p.n + BN - 1) / BN;
  if constexpr (kPair) {
    const uint32_t units = ((m_tiles + 1) / 2) * n_tiles;
    uint32_t pairs_max = static_cast<uint32_t>(max_pairs[dev]);
    if (g_gemm_cta_cap != 0) pairs_max = std::max(1u, std::min(pairs_max, g_gemm_cta_cap / 2));
    cfg.gridDim = dim3(2 * std::min<uint32_t>(units, pairs_max));
  } else {
    uint32_t ctas_max = static_cast<uint32_t>(sm_count());
    if (g_gemm_cta_cap != 0) ctas_max = std::max(1u, std::min(ctas_max, g_gemm_cta_cap));
    cfg.gridDim = dim3(std::min<uint32_t>(m_tiles * n_tiles, ctas_max));
  }
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, map_a, map_b, map_out, p);
  if (e != cudaSuccess) return fail(GEMB_INTERNAL, "%s: %s: %s", op, cudaGetErrorName(e), cudaGetErrorString(e));
  return check_launch(op);
}

// NVFP4 tile variants.  256 x 256 pair tiles hold one accumulator (256 TMEM columns plus the scale regions
// fill the 512); 256 x 128 pair tiles hold two, so a tile's epilogue runs under the next tile's MMAs, at
// the operand traffic per flop of the single-CTA 128 x 256 tile.
//
// Automatic choice: 256 wide, except where that leaves SMs without a tile or the tiles are too coarse to
// balance -- a dense call with fewer 256-wide tiles than SMs (decode-size batches of the shared branch: 23 us
// instead of 29), and the grouped gate/up GEMM with the GELU epilogue up to 128 announced assignments per
// expert (its 1,408 interleaved columns are 5.5 tiles of 256 but 11 of 128; on 128 experts 37 us instead
// of 41 at 64 tokens, 89 instead of 92 at 2,048; from 4,096 tokens, 256 rows per expert, the wide tile wins).
int32_t launch_fp4(const char* op, const void* act, const void* w, const GemmParams& params, bool pairs, cudaStream_t stream) {
  GemmParams p = params;
  if (p.plan != nullptr) {
    p.expert_lo = g_expert_lo;
    p.expert_hi = g_expert_hi;
  }
  int bn = g_gemm_bn;
  if (bn == 0) {
    bool narrow;
    if (p.plan != nullptr)
      narrow = p.gated && g_grouped_rows_hint != 0 && g_grouped_rows_hint <= 128ull * p.experts;
    else
      narrow = static_cast<uint64_t>((p.m + BM - 1) / BM) * ((p.n + 255) / 256) < static_cast<uint64_t>(sm_count());
    bn = narrow ? 128 : 256;
    if (narrow) pairs = false;
  }
  if (bn == 128) {
    if (pairs) return launch_gemm<true, 128, 5, 2, true>(op, act, w, p, stream);
    return launch_gemm<true, 128, 5, 2>(op, act, w, p, stream);
  }
  if (pairs) return launch_gemm<true, 256, 5, 1, true>(op, act, w, p, stream);
  return launch_gemm<true, 256, 3, 1>(op, act, w, p, stream);
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

void set_grouped_rows_hint(uint64_t rows) { g_grouped_rows_hint = rows; }
void set_gemm_cta_cap(uint32_t ctas) { g_gemm_cta_cap = ctas; }
void set_grouped_expert_range(uint32_t lo, uint32_t hi) {
  g_expert_lo = lo;
  g_expert_hi = hi;
}
bool grouped_uses_pairs(uint64_t padded_rows_max, uint64_t experts) {
  return g_gemm_bn != 128 && grouped_pairs(padded_rows_max, experts);
}

int32_t gemm_set_tuning(int32_t knob, int32_t value) {
  if (knob == GEMB_TUNE_GEMM_BN) {
    GEMB_REQUIRE(value == 0 || value == 128 || value == 256,
                 "gemb_set_tuning: GEMM tile width must be 0 (auto), 128 or 256");
    g_gemm_bn = value;
    return GEMB_OK;
  }
  if (knob == GEMB_TUNE_GEMM_PAIR) {
    GEMB_REQUIRE(value >= 0 && value <= 2, "gemb_set_tuning: GEMM pairing must be 0 (auto), 1 (off) or 2 (on)");
    g_gemm_pair = value;
    return GEMB_OK;
  }
  return ep_set_tuning(knob, value);
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
  GEMB_ENTER(op);
  GemmParams p{};
  p.sfa = act_scales_interleaved;
  p.sfb = w_scales_interleaved;
  p.out = out;
  p.m = static_cast<uint32_t>(tokens);
  p.n = static_cast<uint32_t>(rows);
  p.k = static_cast<uint32_t>(k);
  p.alpha = 1.0f / (ga * gw);  // one multiply in the epilogue, as src/cuda/nvfp4/cutlass_sm120.cu:551-552
  return launch_fp4(op, act, w, p, use_pairs(), stream);
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
  GEMB_ENTER(op);
  GemmParams p{};
  p.sfa = act_scales_interleaved;
  p.sfb = w_scales_interleaved;
  p.out = reinterpret_cast<uint16_t*>(out);
  p.out_f32 = 1;
  p.m = static_cast<uint32_t>(tokens);
  p.n = static_cast<uint32_t>(rows);
  p.k = static_cast<uint32_t>(k);
  p.alpha = 1.0f / (ga * gw);
  return launch_fp4(op, act, w, p, use_pairs(), stream);
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
  GEMB_ENTER(op);
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
  return launch_fp4(op, act, w, p, grouped_pairs(padded_rows_max, experts), stream);
}

// Grouped down projection whose epilogue stores every real row at its destination in one of
// `ranks` bf16 [dst_rows, rows_per_expert] buffers (dst_host: their device addresses, a host array;
// buffers of other GPUs are peer-mapped) instead of the padded row space: meta[r] = {destination
// buffer, destination row} per padded row, tile_rows[t] = real rows of 128-row tile t.
}  // extern "C"
namespace gemb {
int32_t grouped_gemm_push(const char* op, const uint8_t* act, const uint8_t* act_scales_interleaved, const uint8_t* w,
                          const uint8_t* w_scales_interleaved, const int32_t* plan, uint64_t padded_rows_max,
                          uint64_t experts, uint64_t rows_per_expert, uint64_t k, float ga, const float* w_divisors,
                          const int32_t* meta, const int32_t* tile_rows, const uint64_t* dst_host, uint64_t ranks,
                          uint64_t rank, uint64_t dst_rows, gemb_stream_t stream) {
  GEMB_REQUIRE(act && act_scales_interleaved && w && w_scales_interleaved && plan && w_divisors && meta && tile_rows && dst_host,
               "%s: pointers must be nonnull", op);
  GEMB_TRY(validate_gemm(op, padded_rows_max, rows_per_expert, k, 64));
  GEMB_REQUIRE(padded_rows_max % 128 == 0 && rows_per_expert % 128 == 0, "%s: rows must come in multiples of 128", op);
  GEMB_REQUIRE(experts > 0 && experts <= 4096 && experts * rows_per_expert < (1ull << 31), "%s: bad expert count", op);
  GEMB_REQUIRE(ranks >= 1 && ranks <= 16 && rank < ranks && dst_rows > 0 && dst_rows < (1ull << 31), "%s: bad destination geometry", op);
  GEMB_REQUIRE(positive_finite(ga), "%s: activation global divisor must be positive and finite", op);
  GemmParams p{};
  p.sfa = act_scales_interleaved;
  p.sfb = w_scales_interleaved;
  p.m = static_cast<uint32_t>(padded_rows_max);
  p.n = static_cast<uint32_t>(rows_per_expert);
  p.k = static_cast<uint32_t>(k);
  p.plan = plan;
  p.w_divisors = w_divisors;
  p.ga = ga;
  p.experts = static_cast<uint32_t>(experts);
  p.alpha = 1.0f;
  p.push_meta = reinterpret_cast<const int2*>(meta);
  p.push_tile_rows = tile_rows;
  p.push_ranks = static_cast<uint32_t>(ranks);
  p.push_rows = static_cast<uint32_t>(dst_rows);
  for (uint64_t r = 0; r < ranks; ++r) {
    GEMB_REQUIRE(dst_host[r] != 0 && dst_host[r] % 16 == 0, "%s: every destination buffer must be mapped and 16-byte aligned", op);
    p.push_dst[r] = reinterpret_cast<uint8_t*>(dst_host[r]);
  }
  p.out = reinterpret_cast<uint16_t*>(dst_host[rank]);   // describes the (unused) tensor-map store target
  p.m_out = static_cast<uint32_t>(dst_rows);
  return launch_fp4(op, act, w, p, grouped_pairs(padded_rows_max, experts), stream);
}
}  // namespace gemb
extern "C" {

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
  GEMB_ENTER(op);
  cudaError_t e = cudaMemsetAsync(fused_interleaved_scales, 0, gemb_interleaved_scale_bytes(2 * intermediate, k), stream);
  if (e != cudaSuccess) return fail(GEMB_INTERNAL, "%s: %s: %s", op, cudaGetErrorName(e), cudaGetErrorString(e));
  const uint64_t work = 2 * intermediate * (k / 32);
  pack_gate_up_kernel<<<static_cast<unsigned>((work + 255) / 256), 256, 0, stream>>>(
      gate_packed, gate_scales, up_packed, up_scales, fused_packed, fused_interleaved_scales,
      static_cast<uint32_t>(intermediate), static_cast<uint32_t>(k));
  return check_launch(op);
}

static int32_t launch_gated(const char* op, const uint8_t* act, const uint8_t* w, GemmParams& p, cudaStream_t stream) {
  return launch_fp4(op, act, w, p, p.plan ? grouped_pairs(p.m, p.experts) : use_pairs(), stream);
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
  GEMB_ENTER(op);
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

int32_t gemb_nvfp4_gemm_up_gated_quant(const uint8_t* act, const uint8_t* act_scales_interleaved, const uint8_t* up_w,
                                       const uint8_t* up_scales_interleaved, const uint16_t* gate_bf16,
                                       uint8_t* product_packed, uint8_t* product_interleaved_scales, uint64_t tokens,
                                       uint64_t rows, uint64_t k, float ga, float gw_up, float product_divisor,
                                       gemb_stream_t stream) {
  const char* op = "gemb_nvfp4_gemm_up_gated_quant";
  GEMB_REQUIRE(act && act_scales_interleaved && up_w && up_scales_interleaved && gate_bf16 && product_packed &&
                   product_interleaved_scales,
               "%s: pointers must be nonnull", op);
  GEMB_TRY(validate_gemm(op, tokens, rows, k, 64));
  GEMB_REQUIRE(rows % 64 == 0, "%s: rows must be a multiple of 64", op);
  GEMB_REQUIRE(positive_finite(ga) && positive_finite(gw_up) && positive_finite(product_divisor) && std::isfinite(ga * gw_up),
               "%s: global divisors must be positive and finite", op);
  GEMB_REQUIRE(reinterpret_cast<uintptr_t>(act) % 16 == 0 && reinterpret_cast<uintptr_t>(up_w) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(act_scales_interleaved) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(up_scales_interleaved) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(gate_bf16) % 16 == 0 && reinterpret_cast<uintptr_t>(product_packed) % 16 == 0,
               "%s: all buffers must be 16-byte aligned", op);
  GEMB_ENTER(op);
  GemmParams p{};
  p.sfa = act_scales_interleaved;
  p.sfb = up_scales_interleaved;
  p.m = static_cast<uint32_t>(tokens);
  p.n = static_cast<uint32_t>(rows);
  p.k = static_cast<uint32_t>(k);
  p.alpha = 1.0f / (ga * gw_up);
  p.gate_in = gate_bf16;
  p.g_product = product_divisor;
  p.out_packed = product_packed;
  p.out_scales = product_interleaved_scales;
  return launch_gated(op, act, up_w, p, stream);
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
  GEMB_ENTER(op);
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
  GEMB_ENTER(op);
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
  if (use_pairs()) return launch_gemm<false, 256, 6, 2, true>(op, act, w, p, stream);
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
    if (code == 8)
      return fail(GEMB_INTERNAL, "%s: a pushing GEMM epilogue met a destination outside the receive buffers and dropped the row", op);
    return fail(GEMB_INTERNAL, "%s: a GEMM kernel gave up waiting on a pipeline barrier (role %d)", op, code);
  }
  const int gemv_code = gemv_take_device_error();
  if (gemv_code != 0)
    return fail(GEMB_INTERNAL, "%s: a GEMV kernel gave up waiting on a pipeline barrier (role %d)", op, gemv_code);
  const int ep_code = ep_take_device_error();
  if (ep_code == 5)
    return fail(GEMB_INTERNAL, "%s: an expert-parallel flag barrier gave up waiting for a peer (check 5)", op);
  if (ep_code != 0)
    return fail(GEMB_INTERNAL, "%s: an expert-parallel kernel met positions outside its buffers and skipped or clamped them (check %d)", op, ep_code);
  const int moe_code = moe_take_device_error();
  if (moe_code == 1)
    return fail(GEMB_DATA_LOSS, "%s: the router met a non-finite logit; the token got zero routing weights", op);
  if (moe_code != 0)
    return fail(GEMB_DATA_LOSS, "%s: an expert id outside [0, experts) reached the permutation and was clamped", op);
  return GEMB_OK;
}

}  // extern "C"
