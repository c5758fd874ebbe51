// Thin inline-PTX wrappers for the sm_100a features the GEMM kernels use: mbarriers, TMA tile
// loads (no multicast anywhere), 1-D bulk copies, tensor memory (TMEM) management and the
// tcgen05 MMA / copy / load instructions.  Every wait is bounded.
#pragma once

#include <cstdint>

namespace gemb {
namespace ptx {

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "elect.sync _|p, 0xFFFFFFFF;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

// ---- mbarrier -------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count));
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_addr(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Non-blocking poll (try_wait may suspend the thread for a while when the phase is still open).
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_addr(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: returns false when the barrier did not flip within `limit` polls.  Each poll
// may itself block for a hardware-defined short time, so the limit is of the order of a second.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, uint32_t limit = 1u << 22) {
  for (uint32_t i = 0; i < limit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if (i > 4096) __nanosleep(64);
  }
  return false;
}

// ---- CTA pairs (clusters of two) --------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// Every thread of every CTA in the cluster must call this (it is a full cluster barrier).
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n"
               "barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address, in the cluster's shared window, of the same shared variable in CTA `rank`.
__device__ __forceinline__ uint32_t cluster_map(const void* p, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr(p)), "r"(rank));
  return r;
}
// Arrive on a barrier of any CTA in the cluster (address from cluster_map), release at cluster scope.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// Bounded wait on a barrier of this CTA that threads of the peer CTA arrive on.
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity, uint32_t limit = 1u << 22) {
  for (uint32_t i = 0; i < limit; ++i) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(smem_addr(bar)), "r"(parity)
        : "memory");
    if (ok) return true;
    if (i > 4096) __nanosleep(64);
  }
  return false;
}

// ---- register re-allocation between warpgroups -------------------------------------------------
// All four warps of a warpgroup (warps 4i .. 4i+3) must execute the same one.  `inc` blocks until
// other warpgroups have released enough registers with `dec`.
template <int kRegs>
__device__ __forceinline__ void reg_dec() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegs));
}
template <int kRegs>
__device__ __forceinline__ void reg_inc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegs));
}

// ---- TMA -------------------------------------------------------------------------------------
__device__ __forceinline__ void prefetch_tensormap(const void* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}
// 2-D tiled load global -> shared of this CTA, completion on `bar` (transaction bytes).
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const void* map, uint64_t* bar, int32_t x,
                                            int32_t y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_addr(smem_dst)), "l"(map), "r"(smem_addr(bar)), "r"(x), "r"(y)
      : "memory");
}
// 1-D bulk copy global -> shared; both addresses 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_load_1d(void* smem_dst, const void* gmem_src, uint32_t bytes,
                                             uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(smem_addr(smem_dst)), "l"(gmem_src), "r"(bytes), "r"(smem_addr(bar))
      : "memory");
}

// 2-D tiled store shared -> global (bulk async-group completion).  Out-of-range parts of the box
// are clipped by the hardware.
__device__ __forceinline__ void tma_store_2d(const void* map, const void* smem_src, int32_t x, int32_t y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map),
               "r"(smem_addr(smem_src)), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Waits until at most `kPending` of this thread's bulk groups still read their shared source.
template <int kPending>
__device__ __forceinline__ void bulk_wait_group_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(kPending) : "memory");
}
__device__ __forceinline__ void bulk_wait_group_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// ---- tensor memory ---------------------------------------------------------------------------
// Whole-warp: allocates `cols` (power of two >= 32) TMEM columns, base address written to smem.
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_addr(smem_result)),
               "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
// CTA-pair forms: one warp of EACH CTA of the pair executes them; both CTAs get the same columns.
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_result, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_addr(smem_result)),
               "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// Arrives on `bar` once every tcgen05 operation this thread issued before has completed.
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_addr(bar))
               : "memory");
}
// Pair form: tracks the pair MMAs this thread issued; `cluster_addr` may name a barrier of either CTA.
__device__ __forceinline__ void tc_commit_pair(uint32_t cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_addr)
               : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]^T with E2M1 operands and one UE4M3 scale per 16 K elements.
__device__ __forceinline__ void tc_mma_nvfp4(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc,
                                             uint32_t idesc, uint32_t tmem_sfa, uint32_t tmem_sfb,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n"
      "}\n"
      ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb)
      : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]^T with 8-bit float operands (E4M3 here), fp32 accumulate.
__device__ __forceinline__ void tc_mma_f8(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n"
      "}\n"
      ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// CTA-pair forms, issued by one thread of the even CTA: a 256 x N tile, rows 0..127 accumulate in
// the even CTA's TMEM and rows 128..255 in the odd CTA's; each CTA supplies its own 128 rows of A
// and N/2 rows of B from the same shared-memory offsets, and its own scale columns in TMEM.
__device__ __forceinline__ void tc_mma_nvfp4_pair(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc,
                                                  uint32_t idesc, uint32_t tmem_sfa, uint32_t tmem_sfb,
                                                  uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n"
      "}\n"
      ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb)
      : "memory");
}
__device__ __forceinline__ void tc_mma_f8_pair(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc,
                                               uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n"
      "}\n"
      ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// One pipeline step of the MMA issuer in a single asm block: a non-blocking poll of the NEXT
// step's barrier(s) (pass the same barrier twice when there is only one) whose result is read
// only after the step's four MMAs have been issued, so the poll's latency hides behind them.
// The four MMAs cover consecutive 32-byte K slices (descriptor + 2 each); the first one
// overwrites the accumulator when `accumulate` is 0.
__device__ __forceinline__ bool tc_mma4_nvfp4_poll(
    uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate,
    uint32_t tmem_sfa, uint32_t tmem_sfb, uint32_t sfb_stride, uint64_t* poll0, uint64_t* poll1, uint32_t parity) {
  uint32_t ready;
  asm volatile(
      "{\n"
      ".reg .pred p, t, q0, q1;\n"
      ".reg .b64 a1, a2, a3, b1, b2, b3;\n"
      ".reg .b32 sa1, sa2, sa3, sb1, sb2, sb3;\n"
      "mbarrier.test_wait.parity.shared::cta.b64 q0, [%9], %11;\n"
      "mbarrier.test_wait.parity.shared::cta.b64 q1, [%10], %11;\n"
      "setp.ne.b32 p, %5, 0;\n"
      "setp.eq.u32 t, 0, 0;\n"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%1], %2, %3, %4, [%6], [%7], p;\n"
      "add.u64 a1, %2, 2;\n"
      "add.u64 b1, %3, 2;\n"
      "add.u32 sa1, %6, 4;\n"
      "mad.lo.u32 sb1, %8, 1, %7;\n"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%1], a1, b1, %4, [sa1], [sb1], t;\n"
      "add.u64 a2, %2, 4;\n"
      "add.u64 b2, %3, 4;\n"
      "add.u32 sa2, %6, 8;\n"
      "mad.lo.u32 sb2, %8, 2, %7;\n"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%1], a2, b2, %4, [sa2], [sb2], t;\n"
      "add.u64 a3, %2, 6;\n"
      "add.u64 b3, %3, 6;\n"
      "add.u32 sa3, %6, 12;\n"
      "mad.lo.u32 sb3, %8, 3, %7;\n"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%1], a3, b3, %4, [sa3], [sb3], t;\n"
      "and.pred q0, q0, q1;\n"
      "selp.u32 %0, 1, 0, q0;\n"
      "}\n"
      : "=r"(ready)
      : "r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb),
        "r"(sfb_stride), "r"(smem_addr(poll0)), "r"(smem_addr(poll1)), "r"(parity)
      : "memory");
  return ready != 0;
}
__device__ __forceinline__ bool tc_mma4_nvfp4_pair_poll(
    uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate,
    uint32_t tmem_sfa, uint32_t tmem_sfb, uint32_t sfb_stride, uint64_t* poll0, uint64_t* poll1, uint32_t parity) {
  uint32_t ready;
  asm volatile(
      "{\n"
      ".reg .pred p, t, q0, q1;\n"
      ".reg .b64 a1, a2, a3, b1, b2, b3;\n"
      ".reg .b32 sa1, sa2, sa3, sb1, sb2, sb3;\n"
      "mbarrier.test_wait.parity.shared::cta.b64 q0, [%9], %11;\n"
      "mbarrier.test_wait.parity.shared::cta.b64 q1, [%10], %11;\n"
      "setp.ne.b32 p, %5, 0;\n"
      "setp.eq.u32 t, 0, 0;\n"
      "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.block16 [%1], %2, %3, %4, [%6], [%7], p;\n"
      "add.u64 a1, %2, 2;\n"
      "add.u64 b1, %3, 2;\n"
      "add.u32 sa1, %6, 4;\n"
      "mad.lo.u32 sb1, %8, 1, %7;\n"
      "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.block16 [%1], a1, b1, %4, [sa1], [sb1], t;\n"
      "add.u64 a2, %2, 4;\n"
      "add.u64 b2, %3, 4;\n"
      "add.u32 sa2, %6, 8;\n"
      "mad.lo.u32 sb2, %8, 2, %7;\n"
      "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.block16 [%1], a2, b2, %4, [sa2], [sb2], t;\n"
      "add.u64 a3, %2, 6;\n"
      "add.u64 b3, %3, 6;\n"
      "add.u32 sa3, %6, 12;\n"
      "mad.lo.u32 sb3, %8, 3, %7;\n"
      "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.block16 [%1], a3, b3, %4, [sa3], [sb3], t;\n"
      "and.pred q0, q0, q1;\n"
      "selp.u32 %0, 1, 0, q0;\n"
      "}\n"
      : "=r"(ready)
      : "r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb),
        "r"(sfb_stride), "r"(smem_addr(poll0)), "r"(smem_addr(poll1)), "r"(parity)
      : "memory");
  return ready != 0;
}
__device__ __forceinline__ bool tc_mma4_f8_poll(
    uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate,
    uint64_t* poll0, uint64_t* poll1, uint32_t parity) {
  uint32_t ready;
  asm volatile(
      "{\n"
      ".reg .pred p, t, q0, q1;\n"
      ".reg .b64 a1, a2, a3, b1, b2, b3;\n"
      "mbarrier.test_wait.parity.shared::cta.b64 q0, [%6], %8;\n"
      "mbarrier.test_wait.parity.shared::cta.b64 q1, [%7], %8;\n"
      "setp.ne.b32 p, %5, 0;\n"
      "setp.eq.u32 t, 0, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%1], %2, %3, %4, p;\n"
      "add.u64 a1, %2, 2;\n"
      "add.u64 b1, %3, 2;\n"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%1], a1, b1, %4, t;\n"
      "add.u64 a2, %2, 4;\n"
      "add.u64 b2, %3, 4;\n"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%1], a2, b2, %4, t;\n"
      "add.u64 a3, %2, 6;\n"
      "add.u64 b3, %3, 6;\n"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%1], a3, b3, %4, t;\n"
      "and.pred q0, q0, q1;\n"
      "selp.u32 %0, 1, 0, q0;\n"
      "}\n"
      : "=r"(ready)
      : "r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(smem_addr(poll0)),
        "r"(smem_addr(poll1)), "r"(parity)
      : "memory");
  return ready != 0;
}
__device__ __forceinline__ bool tc_mma4_f8_pair_poll(
    uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate,
    uint64_t* poll0, uint64_t* poll1, uint32_t parity) {
  uint32_t ready;
  asm volatile(
      "{\n"
      ".reg .pred p, t, q0, q1;\n"
      ".reg .b64 a1, a2, a3, b1, b2, b3;\n"
      "mbarrier.test_wait.parity.shared::cta.b64 q0, [%6], %8;\n"
      "mbarrier.test_wait.parity.shared::cta.b64 q1, [%7], %8;\n"
      "setp.ne.b32 p, %5, 0;\n"
      "setp.eq.u32 t, 0, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%1], %2, %3, %4, p;\n"
      "add.u64 a1, %2, 2;\n"
      "add.u64 b1, %3, 2;\n"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%1], a1, b1, %4, t;\n"
      "add.u64 a2, %2, 4;\n"
      "add.u64 b2, %3, 4;\n"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%1], a2, b2, %4, t;\n"
      "add.u64 a3, %2, 6;\n"
      "add.u64 b3, %3, 6;\n"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%1], a3, b3, %4, t;\n"
      "and.pred q0, q0, q1;\n"
      "selp.u32 %0, 1, 0, q0;\n"
      "}\n"
      : "=r"(ready)
      : "r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(smem_addr(poll0)),
        "r"(smem_addr(poll1)), "r"(parity)
      : "memory");
  return ready != 0;
}
// TMEM -> registers: this warp's 32 lanes x 32 consecutive 32-bit columns.
__device__ __forceinline__ void tc_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
        "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]),
        "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]),
        "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
// Registers -> TMEM: this warp's 32 lanes x 4 consecutive 32-bit columns.
__device__ __forceinline__ void tc_st_32x32b_x4(uint32_t taddr, const uint4& v) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};" ::"r"(taddr), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}
// Wide forms: 16 / 32 consecutive columns from an array of uint4 (element j = columns 4j .. 4j+3).
__device__ __forceinline__ void tc_st_32x32b_x16(uint32_t taddr, const uint4 (&v)[4]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr), "r"(v[0].x), "r"(v[0].y), "r"(v[0].z), "r"(v[0].w), "r"(v[1].x), "r"(v[1].y), "r"(v[1].z), "r"(v[1].w), "r"(v[2].x), "r"(v[2].y), "r"(v[2].z), "r"(v[2].w), "r"(v[3].x), "r"(v[3].y), "r"(v[3].z), "r"(v[3].w)
               : "memory");
}
__device__ __forceinline__ void tc_st_32x32b_x32(uint32_t taddr, const uint4 (&v)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr), "r"(v[0].x), "r"(v[0].y), "r"(v[0].z), "r"(v[0].w), "r"(v[1].x), "r"(v[1].y), "r"(v[1].z), "r"(v[1].w), "r"(v[2].x), "r"(v[2].y), "r"(v[2].z), "r"(v[2].w), "r"(v[3].x), "r"(v[3].y), "r"(v[3].z), "r"(v[3].w), "r"(v[4].x), "r"(v[4].y), "r"(v[4].z), "r"(v[4].w), "r"(v[5].x), "r"(v[5].y), "r"(v[5].z), "r"(v[5].w), "r"(v[6].x), "r"(v[6].y), "r"(v[6].z), "r"(v[6].w), "r"(v[7].x), "r"(v[7].y), "r"(v[7].z), "r"(v[7].w)
               : "memory");
}
__device__ __forceinline__ void tc_st_32x32b_x2(uint32_t taddr, uint32_t v0, uint32_t v1) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x2.b32 [%0], {%1, %2};" ::"r"(taddr), "r"(v0), "r"(v1) : "memory");
}
__device__ __forceinline__ void tc_wait_st() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tc_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ---- descriptors -----------------------------------------------------------------------------
// Shared-memory matrix descriptor, K-major operand tile whose rows are 128 bytes wide and
// stored with the 128-byte swizzle (what a TMA box of 128 x rows bytes with SWIZZLE_128B
// writes): 8-row groups are 1024 bytes apart (stride byte offset), the leading offset is unused.
__device__ __forceinline__ uint64_t smem_desc_k128_swizzled(uint32_t saddr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3FFFF) >> 4);        // start address, bits [0,14)
  d |= static_cast<uint64_t>(1024 >> 4) << 32;               // stride byte offset, bits [32,46)
  d |= 1ull << 46;                                           // descriptor version (sm_100)
  d |= 2ull << 61;                                           // layout: SWIZZLE_128B
  return d;
}
// Descriptor of a 32-row x 16-byte scale block stored densely (no swizzle): 8-row x 16-byte
// core matrices, 128 bytes apart.
__device__ __forceinline__ uint64_t smem_desc_scale_block(uint32_t saddr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>(128 >> 4) << 32;
  d |= 1ull << 46;
  return d;
}
// Instruction descriptor, block-scaled E2M1 x E2M1 (kind::mxf4nvf4), UE4M3 scales, both K-major.
__host__ __device__ constexpr uint32_t idesc_nvfp4(int m, int n) {
  return (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) | (0u << 23) |
         (static_cast<uint32_t>(m >> 4) << 24);
}
// Instruction descriptor, E4M3 x E4M3 (kind::f8f6f4), fp32 accumulator, both K-major.
__host__ __device__ constexpr uint32_t idesc_e4m3(int m, int n) {
  return (1u << 4) | (0u << 7) | (0u << 10) | (static_cast<uint32_t>(n >> 3) << 17) |
         (static_cast<uint32_t>(m >> 4) << 24);
}

}  // namespace ptx
}  // namespace gemb
