// Expert parallelism over peer memory (NVLink / NVSwitch): the dispatch and the combine of the
// mixture-of-experts layer as kernels that PULL rows straight out of the other GPUs' buffers with
// plain global loads, instead of an all-to-all followed by local gather / scatter passes.
//
// Setting: R ranks (one process per GPU), E experts, rank r owns experts [r*E/R, (r+1)*E/R).
// Every rank routes its own tokens over all E experts and leaves, in a buffer its peers can map,
// one quantised message row per assignment in (expert, token, slot) order -- i.e. already grouped
// by owner.  The per-expert counts of all ranks, C[s][e], are all-gathered (R*E integers; the
// collective doubles as the "send buffers are complete" barrier).  Everything else follows from
// C by arithmetic, identically on every rank, so no indices travel and nothing is read back to
// the host:
//
//   rows of expert e held by source s start at      src(s, e) = sum_{e' < e} C[s][e']
//   on e's owner they land, source after source, at dst(s, e) = pad(e) + sum_{s' < s} C[s'][e]
//   pad(e) = start of e in the owner's padded row space (every expert starts on a multiple of
//            128 rows, as the grouped GEMM wants)
//
// which is the (expert, global token, slot) order of the single-GPU layer.  After the grouped
// GEMMs a second tiny collective says "expert outputs are complete", and each token's owner
// combines its top-k contributions in slot order by reading the rows at dst(me, e) + j from the
// owners' output buffers.
//
// gem16 has no multi-GPU code; this protocol is the library's own.
#include <algorithm>

#include "common.cuh"
#include "moe_layer.h"

namespace gemb {

// Set when a position computed from the counts falls outside a buffer (the counts were not what
// the protocol promises, e.g. read before the peers had written them): the access is skipped.
__device__ int g_ep_error = 0;

int ep_take_device_error() {
  int code = 0;
  if (cudaMemcpyFromSymbol(&code, g_ep_error, sizeof code) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  if (code != 0) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_ep_error, &zero, sizeof zero);
  }
  return code;
}

// Polls a flag barrier makes before it gives up (about 500 ns each once past the first 64):
// gemb_set_tuning(GEMB_TUNE_EP_BARRIER_SPINS, n); the default is about three seconds.
int g_ep_barrier_spins = 1 << 22;
int g_ep_split_sms = 0;    // large batches: experts in two halves, the first half's push on this many SMs (0: one pass)
int g_ep_shared_sms = 40;  // large batches: SMs given to the shared branch beside the pushing down GEMM (0: in line)

int32_t ep_set_tuning(int32_t knob, int32_t value) {
  if (knob == GEMB_TUNE_EP_BARRIER_SPINS) {
    GEMB_REQUIRE(value >= 0 && value <= (1 << 24), "gemb_set_tuning: barrier polls must be in [0, 2^24] (0 = default)");
    g_ep_barrier_spins = value == 0 ? 1 << 22 : value;
    return GEMB_OK;
  }
  if (knob == GEMB_TUNE_EP_SPLIT_SMS) {
    GEMB_REQUIRE(value >= 0 && value <= 128 && value % 2 == 0, "gemb_set_tuning: SMs for the first half's push must be even, in [0, 128]");
    g_ep_split_sms = value;
    return GEMB_OK;
  }
  if (knob == GEMB_TUNE_EP_SHARED_SMS) {
    GEMB_REQUIRE(value >= 0 && value <= 128 && value % 2 == 0, "gemb_set_tuning: SMs for the shared branch must be even, in [0, 128]");
    g_ep_shared_sms = value;
    return GEMB_OK;
  }
  return moe_set_tuning(knob, value);
}

namespace {

constexpr uint32_t kMaxRanks = 16;
constexpr uint32_t kMaxExperts = 1024;

struct PeerPtrs {
  const uint8_t* p[kMaxRanks];
};

// One CTA.  counts_all: [ranks][experts].  tile_rows (optional): real rows of every 128-row tile.
constexpr uint32_t kPlanSmemCounts = 4096;
__device__ __forceinline__ void
ep_plan_body(const int32_t* counts_all_global, uint32_t ranks, uint32_t experts, uint32_t me,
             int32_t* __restrict__ plan, int32_t* __restrict__ recv_prefix, int32_t* __restrict__ recv_src,
             int32_t* __restrict__ recv_dst, int32_t* __restrict__ out_base, uint32_t capacity_rows,
             uint32_t send_rows, int32_t* __restrict__ tile_rows) {
  const int32_t* counts_all = counts_all_global;
  extern __shared__ int sm[];
  const uint32_t el = experts / ranks;
  // A single thread walking global memory waits for every load in turn (about a quarter of a
  // microsecond each); the serial prefix sums below therefore work on a shared-memory copy of the
  // counts whenever it fits (ranks * experts <= 4,096, which covers 16 ranks x 256 experts).
  if (ranks * experts <= kPlanSmemCounts) {
    int* copy = sm + 5 * experts;
    for (uint32_t i = threadIdx.x; i < ranks * experts; i += blockDim.x) copy[i] = counts_all_global[i];
    __syncthreads();
    counts_all = copy;
  }
  // Counts that cannot be (negative, more than a rank can send, or more padded rows than the
  // buffers hold -- e.g. read after a barrier gave up, while a peer was still writing them) give
  // an empty plan: no tile, no segment, every combine base out of range (the combine skips those).
  __shared__ int bad;
  if (threadIdx.x == 0) bad = 0;
  __syncthreads();
  for (uint32_t s = threadIdx.x; s < ranks; s += blockDim.x) {
    int64_t sent = 0;
    bool neg = false;
    for (uint32_t e0 = 0; e0 < experts; e0 += 8) {
      int c[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) c[j] = e0 + j < experts ? counts_all[s * experts + e0 + j] : 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        neg |= c[j] < 0;
        sent += c[j];
      }
    }
    if (neg || sent > static_cast<int64_t>(send_rows)) bad = 1;
  }
  // padded rows of my experts: one thread per expert, combined with a shared-memory atomic
  __shared__ unsigned long long padded_total;
  if (threadIdx.x == 0) padded_total = 0ull;
  __syncthreads();
  for (uint32_t e = me * el + threadIdx.x; e < (me + 1) * el; e += blockDim.x) {
    int64_t t = 0;
    for (uint32_t s = 0; s < ranks; ++s) t += max(counts_all[s * experts + e], 0);
    atomicAdd(&padded_total, static_cast<unsigned long long>((t + 255) / 256 * 256));
  }
  __syncthreads();
  if (threadIdx.x == 0 && padded_total > static_cast<unsigned long long>(capacity_rows)) bad = 1;
  __syncthreads();
  if (bad) {
    if (threadIdx.x == 0) {
      atomicCAS(&g_ep_error, 0, 6);
      plan[0] = 0;
      plan[1] = 0;
      plan[3 + el] = 0;
    }
    for (uint32_t e = threadIdx.x; e <= el; e += blockDim.x) plan[2 + e] = 0;
    for (uint32_t g = threadIdx.x; g <= ranks * el; g += blockDim.x) recv_prefix[g] = 0;
    for (uint32_t g = threadIdx.x; g < ranks * el; g += blockDim.x) recv_src[g] = recv_dst[g] = 0;
    for (uint32_t e = threadIdx.x; e < experts; e += blockDim.x) out_base[e] = -(1 << 30);
    return;
  }
  int* tot = sm;                    // [experts] rows of expert e over all sources
  int* pad = tot + experts;         // [experts] start of e in its owner's padded row space
  int* before_me = pad + experts;   // [experts] sum_{s' < me} C[s'][e]
  int* my_pad = before_me + experts;  // [experts] start of e in MY local padded space (single-GPU plan of my tokens)
  int* live_off = my_pad + experts;   // [local experts] first entry of the expert in the list of real tiles
  for (uint32_t e = threadIdx.x; e < experts; e += blockDim.x) {
    int t = 0, b = 0;
    for (uint32_t s = 0; s < ranks; ++s) {
      const int c = counts_all[s * experts + e];
      if (s < me) b += c;
      t += c;
    }
    tot[e] = t;
    before_me[e] = b;
  }
  __syncthreads();
  // Padded offsets restart at every owner's first expert; one thread per owner, plus one for mine.
  if (threadIdx.x < ranks) {
    const uint32_t d = threadIdx.x;
    // A serial prefix sum in one thread: the loads of eight values are issued together, so an iteration
    // costs one add instead of one shared-memory round trip.  live_off (the first entry of every local
    // expert in the list of tiles that hold real rows) rides along for this rank's own experts.
    int po = 0, lo = 0;
    for (uint32_t e0 = d * el; e0 < (d + 1) * el; e0 += 8) {
      int t[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) t[j] = e0 + j < (d + 1) * el ? tot[e0 + j] : 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (e0 + j >= (d + 1) * el) break;
        pad[e0 + j] = po;
        po += (t[j] + 255) / 256 * 256;
        if (d == me) {
          live_off[e0 + j - d * el] = lo;
          lo += (t[j] + 127) / 128;
        }
      }
    }
    if (d == me) {
      plan[0] = po / 128;
      plan[1] = po;
      plan[2 + el] = po;
      plan[3 + el + 2 * (po / 128)] = lo;
    }
  } else if (threadIdx.x == 32) {   // another warp, so that it runs beside the owners' threads
    int po = 0;
    for (uint32_t e0 = 0; e0 < experts; e0 += 8) {
      int t[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) t[j] = e0 + j < experts ? counts_all[me * experts + e0 + j] : 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (e0 + j >= experts) break;
        my_pad[e0 + j] = po;
        po += (t[j] + 255) / 256 * 256;
      }
    }
  }
  __syncthreads();
  for (uint32_t e = threadIdx.x; e < experts; e += blockDim.x)
    out_base[e] = pad[e] + before_me[e] - my_pad[e];
  int32_t* info = plan + 3 + el;   // pairs {expert of tile i, i-th tile with real rows}, then the number of those
  for (uint32_t e = threadIdx.x; e < el; e += blockDim.x) {
    const uint32_t ge = me * el + e;
    plan[2 + e] = pad[ge];
    const int end = pad[ge] + (tot[ge] + 255) / 256 * 256;
    for (int tile = pad[ge] / 128, j = 0; tile < end / 128; ++tile, ++j) {
      const int real = max(0, min(128, tot[ge] - (tile * 128 - pad[ge])));
      info[2 * tile] = real > 0 ? static_cast<int32_t>(e) : -1;   // -1: padding only
      if (real > 0) info[2 * (live_off[e] + j) + 1] = tile;
      if (tile_rows != nullptr) tile_rows[tile] = real;
    }
  }
  // Segments (source s, local expert e) in source-major order: one thread per source.
  __shared__ int rows_from[kMaxRanks];
  if (threadIdx.x < ranks) {
    int n = 0;
    for (uint32_t e0 = 0; e0 < el; e0 += 8) {
      int c[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) c[j] = e0 + j < el ? counts_all[threadIdx.x * experts + me * el + e0 + j] : 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) n += c[j];
    }
    rows_from[threadIdx.x] = n;
  }
  __syncthreads();
  for (uint32_t g = threadIdx.x; g < ranks * el; g += blockDim.x) {   // destination: rows of the sources before s
    const uint32_t s = g / el, ge = me * el + g % el;
    int b = 0;
    for (uint32_t s2 = 0; s2 < s; ++s2) b += counts_all[s2 * experts + ge];
    recv_dst[g] = pad[ge] + b;
  }
  if (threadIdx.x < ranks) {
    const uint32_t s = threadIdx.x;
    int run = 0, src = 0;
    for (uint32_t s2 = 0; s2 < s; ++s2) run += rows_from[s2];
    for (uint32_t e0 = 0; e0 < me * el; e0 += 8) {
      int c[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) c[j] = e0 + j < me * el ? counts_all[s * experts + e0 + j] : 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) src += c[j];
    }
    for (uint32_t e0 = 0; e0 < el; e0 += 8) {
      int c[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) c[j] = e0 + j < el ? counts_all[s * experts + me * el + e0 + j] : 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (e0 + j >= el) break;
        const uint32_t g = s * el + e0 + j;
        recv_prefix[g] = run;
        recv_src[g] = src;
        run += c[j];
        src += c[j];
      }
    }
    if (s == ranks - 1) recv_prefix[ranks * el] = run;
  }
}

__global__ void __launch_bounds__(256)
ep_plan_kernel(const int32_t* __restrict__ counts_all, uint32_t ranks, uint32_t experts, uint32_t me,
               int32_t* __restrict__ plan, int32_t* __restrict__ recv_prefix, int32_t* __restrict__ recv_src,
               int32_t* __restrict__ recv_dst, int32_t* __restrict__ out_base, uint32_t capacity_rows,
               uint32_t send_rows, int32_t* __restrict__ tile_rows) {
  ep_plan_body(counts_all, ranks, experts, me, plan, recv_prefix, recv_src, recv_dst, out_base, capacity_rows, send_rows,
               tile_rows);
}

// Cross-GPU barrier on flags in peer-mapped memory: every rank bumps its own epoch for barrier
// `which`, publishes it to slot [which][rank] of every rank's flag array (release, system scope)
// and waits until all slots of its own array have reached that epoch (acquire).  The kernels
// before it in the stream have completed, so their writes are in this GPU's memory before the flag
// leaves; a peer that has seen the flag may read them over NVLink.  The epoch lives on the device,
// so a captured launch stays valid when replayed.  The wait is bounded: on expiry the kernel
// records the fact and returns (the launches that follow then work on stale data and the caller
// sees the error at its next gemb_check_device_status()).
// One warp; the ranks run on different GPUs (never several ranks of one barrier on the same GPU).
__device__ __forceinline__ void
ep_barrier_warp(const PeerPtrs& flag_arrays, uint32_t ranks, uint32_t me, uint32_t which, uint32_t* __restrict__ epochs,
                uint32_t spin_limit) {
  const uint32_t lane = threadIdx.x & 31;
  uint32_t e = 0;
  if (lane == 0) {
    e = epochs[which] + 1;
    epochs[which] = e;
  }
  e = __shfl_sync(0xFFFFFFFFu, e, 0);
  if (lane < ranks) {
    uint32_t* theirs = reinterpret_cast<uint32_t*>(const_cast<uint8_t*>(flag_arrays.p[lane])) + which * kMaxRanks + me;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(theirs), "r"(e) : "memory");
    const uint32_t* mine = reinterpret_cast<const uint32_t*>(flag_arrays.p[me]) + which * kMaxRanks + lane;
    bool ok = false;
    for (uint32_t i = 0; i < spin_limit && !ok; ++i) {
      uint32_t v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
      ok = static_cast<int32_t>(v - e) >= 0;   // epochs only grow; a peer may already be one barrier ahead
      if (!ok && i > 64) __nanosleep(500);   // about three seconds in all at the default limit
    }
    if (!ok) atomicCAS(&g_ep_error, 0, 5);
  }
}

__global__ void __launch_bounds__(32)
ep_barrier_kernel(PeerPtrs flag_arrays, uint32_t ranks, uint32_t me, uint32_t which, uint32_t* __restrict__ epochs,
                  uint32_t spin_limit) {
  ep_barrier_warp(flag_arrays, ranks, me, which, epochs, spin_limit);
}

// Barrier 0, the read of every rank's per-expert counts and the position arithmetic in ONE launch
// of one CTA: warp 0 runs the flag barrier (when `barrier` is set; its acquire loads order the
// reads below after the peers' writes), then all threads copy the peers' counts into counts_all
// (when `gather` is set; otherwise counts_all is the caller's) and the CTA derives the plan.
__global__ void __launch_bounds__(256)
ep_sync_plan_kernel(PeerPtrs flag_arrays, PeerPtrs count_buffers, uint32_t ranks, uint32_t experts, uint32_t me,
                    uint32_t* __restrict__ epochs, uint32_t spin_limit, int barrier, int gather,
                    int32_t* __restrict__ counts_all, int32_t* __restrict__ plan, int32_t* __restrict__ recv_prefix,
                    int32_t* __restrict__ recv_src, int32_t* __restrict__ recv_dst, int32_t* __restrict__ out_base,
                    uint32_t capacity_rows, uint32_t send_rows, int32_t* __restrict__ tile_rows) {
  if (barrier && threadIdx.x < 32) ep_barrier_warp(flag_arrays, ranks, me, 0, epochs, spin_limit);
  __syncthreads();
  if (gather) {
    for (uint32_t i = threadIdx.x; i < ranks * experts; i += blockDim.x) {
      const uint32_t s = i / experts, e = i % experts;
      int32_t v;
      asm volatile("ld.relaxed.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(reinterpret_cast<const int32_t*>(count_buffers.p[s]) + e) : "memory");
      counts_all[i] = v;
    }
    __syncthreads();
  }
  ep_plan_body(counts_all, ranks, experts, me, plan, recv_prefix, recv_src, recv_dst, out_base, capacity_rows, send_rows,
               tile_rows);
}

// Quantises each local token once (EXACT NVFP4 contract, src/numeric/nvfp4.cpp:139-150) and PUSHES one
// message row per assignment -- payload | compact block scales | assignment index (token * topk +
// slot) -- into the message buffer of the rank that owns the expert (plain stores, peer memory for
// another rank).  A rank's message buffer holds one region of send_rows rows per source rank; inside its
// region a row sits at the assignment's position in the source's (expert, token, slot) order, which
// follows from the permutation's outputs alone: offsets[e] + (slot_rows[i] - padded_offset[e]).  So the
// source needs nobody else's counts to place a row, and the owner finds it where the position
// arithmetic over all counts says (recv_src).  One CTA per token, one thread per 16-element block.
__global__ void __launch_bounds__(256)
ep_pack_kernel(const uint16_t* __restrict__ x, const int32_t* __restrict__ ids, const int32_t* __restrict__ slot_rows,
               const int32_t* __restrict__ offsets, const int32_t* __restrict__ plan, PeerPtrs msg, uint32_t me, uint32_t el,
               uint32_t hidden, uint32_t topk, uint32_t experts, uint32_t msg_bytes, uint32_t send_rows, float g) {
  const uint32_t t = blockIdx.x;
  __shared__ uint8_t* dst[32];
  extern __shared__ __align__(16) uint8_t pack_sc[];   // the token's hidden/16 scale bytes
  if (threadIdx.x < topk) {
    const uint64_t i = static_cast<uint64_t>(t) * topk + threadIdx.x;
    const uint32_t e = static_cast<uint32_t>(__ldg(ids + i));
    uint8_t* d = nullptr;
    if (e < experts) {
      const int64_t q = static_cast<int64_t>(__ldg(offsets + e)) + __ldg(slot_rows + i) - __ldg(plan + 2 + e);
      if (q >= 0 && q < static_cast<int64_t>(send_rows))
        d = const_cast<uint8_t*>(msg.p[e / el]) + (static_cast<uint64_t>(me) * send_rows + static_cast<uint64_t>(q)) * msg_bytes;
    }
    if (d == nullptr) atomicCAS(&g_ep_error, 0, 7);   // cannot be; the row is not written
    dst[threadIdx.x] = d;
  }
  __syncthreads();
  const uint32_t blocks = hidden / 16;
  for (uint32_t c = threadIdx.x; c < blocks; c += blockDim.x) {
    const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<uint64_t>(t) * hidden + c * 16);
    const uint4 a = __ldg(src), b = __ldg(src + 1);
    const uint32_t ww[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    float v[16];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      v[2 * i] = __uint_as_float(ww[i] << 16);
      v[2 * i + 1] = __uint_as_float(ww[i] & 0xFFFF0000u);
    }
    uint32_t lo, hi;
    uint8_t sb;
    quantize_block16<false>(v, g, lo, hi, sb);
    pack_sc[c] = sb;
    for (uint32_t s = 0; s < topk; ++s)
      if (dst[s] != nullptr) *reinterpret_cast<uint2*>(dst[s] + c * 8) = make_uint2(lo, hi);
  }
  __syncthreads();
  // the scales as 16-byte pieces (hidden is a multiple of 256, so hidden / 16 bytes are whole pieces), then the index
  const uint32_t pieces = blocks / 16;
  for (uint32_t idx = threadIdx.x; idx < pieces * topk; idx += blockDim.x) {
    const uint32_t s = idx / pieces, q = idx % pieces;
    if (dst[s] != nullptr)
      *reinterpret_cast<uint4*>(dst[s] + hidden / 2 + q * 16) = *reinterpret_cast<const uint4*>(pack_sc + q * 16);
  }
  if (threadIdx.x < topk && dst[threadIdx.x] != nullptr)
    *reinterpret_cast<int32_t*>(dst[threadIdx.x] + hidden / 2 + hidden / 16) = static_cast<int32_t>(t * topk + threadIdx.x);
}

// counts_all[s][e] = the per-expert counts rank s left in its peer-mapped buffer.
__global__ void __launch_bounds__(256)
ep_gather_counts_kernel(PeerPtrs count_buffers, uint32_t ranks, uint32_t experts, int32_t* __restrict__ counts_all) {
  for (uint32_t i = threadIdx.x; i < ranks * experts; i += blockDim.x) {
    const uint32_t s = i / experts, e = i % experts;
    counts_all[i] = *(reinterpret_cast<const volatile int32_t*>(count_buffers.p[s]) + e);
  }
}

// kPullPayloadVecs: 16-byte payload vectors per lane and row (4: hidden <= 4,096; 8: hidden <= 8,192).
// Persistent grid, one warp per received row: copies the E2M1 payload into the padded row space and
// the compact block scales into the interleaved layout.
template <int kPullPayloadVecs>
__global__ void __launch_bounds__(256)
ep_pull_dispatch_kernel(PeerPtrs peers, const int32_t* __restrict__ recv_prefix, const int32_t* __restrict__ recv_src,
                        const int32_t* __restrict__ recv_dst, uint32_t segments, uint32_t el, uint32_t hidden,
                        uint32_t msg_bytes, uint32_t c_pad, uint8_t* __restrict__ packed,
                        uint8_t* __restrict__ scales, uint32_t send_rows, uint32_t rows_max, int2* __restrict__ row_meta) {
  constexpr int kPullScaleWords = kPullPayloadVecs / 2;   // 4-byte scale words per lane and row
  extern __shared__ int sm[];
  int* prefix = sm;  // [segments + 1]
  for (uint32_t i = threadIdx.x; i <= segments; i += blockDim.x) prefix[i] = recv_prefix[i];
  __syncthreads();
  uint32_t total = static_cast<uint32_t>(prefix[segments]);
  if (total > rows_max) {  // cannot be: every received row has a place in the padded row space
    if (threadIdx.x == 0) atomicCAS(&g_ep_error, 0, 1);
    total = 0;
  }
  const uint32_t lane = threadIdx.x & 31;
  const uint32_t warps = gridDim.x * (blockDim.x >> 5);
  const uint32_t payload_vecs = hidden / 32;   // 16-byte vectors of payload per row
  const uint32_t scale_words = hidden / 64;    // 4-byte words of scales per row (four K blocks each)
  for (uint32_t r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); r < total; r += warps) {
    uint32_t lo = 0, hi = segments;            // last segment whose prefix is <= r
    while (hi - lo > 1) {
      const uint32_t mid = (lo + hi) >> 1;
      if (static_cast<uint32_t>(prefix[mid]) <= r) lo = mid; else hi = mid;
    }
    const uint32_t j = r - static_cast<uint32_t>(prefix[lo]);
    const uint64_t srow = static_cast<uint64_t>(static_cast<uint32_t>(__ldg(recv_src + lo))) + j;
    const uint64_t d = static_cast<uint64_t>(static_cast<uint32_t>(__ldg(recv_dst + lo))) + j;
    if (srow >= send_rows || d >= rows_max) {
      if (lane == 0) atomicCAS(&g_ep_error, 0, 2);
      continue;
    }
    const uint8_t* src = peers.p[lo / el] + srow * msg_bytes;
    // Every load of the row (over NVLink for a remote source) is issued before the first store: a row is
    // small, so what hides the latency is the loads in flight per warp, and a store that waited for its
    // own load in program order would hold back the loads behind it.
    uint4 pv[kPullPayloadVecs];
#pragma unroll
    for (int i = 0; i < kPullPayloadVecs; ++i) {
      const uint32_t v = i * 32 + lane;
      pv[i] = v < payload_vecs ? *reinterpret_cast<const uint4*>(src + v * 16) : make_uint4(0u, 0u, 0u, 0u);
    }
    uint32_t sv[kPullScaleWords];
#pragma unroll
    for (int i = 0; i < kPullScaleWords; ++i) {
      const uint32_t w = i * 32 + lane;
      sv[i] = w < scale_words ? *reinterpret_cast<const uint32_t*>(src + hidden / 2 + w * 4) : 0u;
    }
    // Where the row's result has to go: {source rank, the assignment index the source wrote behind the scales}.
    int assignment = 0;
    if (row_meta != nullptr && lane == 0) assignment = *reinterpret_cast<const int32_t*>(src + hidden / 2 + hidden / 16);
#pragma unroll
    for (int i = 0; i < kPullPayloadVecs; ++i) {
      const uint32_t v = i * 32 + lane;
      if (v < payload_vecs) *reinterpret_cast<uint4*>(packed + d * (hidden / 2) + v * 16) = pv[i];
    }
#pragma unroll
    for (int i = 0; i < kPullScaleWords; ++i) {
      const uint32_t w = i * 32 + lane;
      if (w < scale_words) *reinterpret_cast<uint32_t*>(scales + interleaved_scale_offset(d, w * 4, c_pad)) = sv[i];
    }
    if (row_meta != nullptr && lane == 0) row_meta[d] = make_int2(static_cast<int>(lo / el), assignment);
  }
}

// Deterministic combine (slot order, one fma per slot) with the expert outputs read from their owners.
__global__ void __launch_bounds__(256)
ep_pull_combine_kernel(PeerPtrs peers, const int32_t* __restrict__ ids, const int32_t* __restrict__ slot_rows,
                       const int32_t* __restrict__ out_base, const float* __restrict__ weights,
                       const uint16_t* __restrict__ shared_out, uint16_t* __restrict__ out, uint32_t tokens,
                       uint32_t hidden, uint32_t topk, uint32_t el, uint32_t experts, uint32_t rows_max) {
  const uint32_t chunks = hidden / 8;
  const uint64_t idx = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<uint64_t>(tokens) * chunks) return;
  const uint32_t t = static_cast<uint32_t>(idx / chunks), c = static_cast<uint32_t>(idx % chunks);
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
  for (uint32_t s = 0; s < topk; ++s) {
    const uint64_t a = static_cast<uint64_t>(t) * topk + s;
    const float wv = __ldg(weights + a);
    const uint32_t e = static_cast<uint32_t>(__ldg(ids + a));
    if (e >= experts) {
      atomicCAS(&g_ep_error, 0, 3);
      continue;
    }
    const int64_t r = static_cast<int64_t>(__ldg(out_base + e)) + __ldg(slot_rows + a);
    if (r < 0 || r >= static_cast<int64_t>(rows_max)) {
      atomicCAS(&g_ep_error, 0, 4);
      continue;
    }
    const uint4 v = *(reinterpret_cast<const uint4*>(peers.p[e / el] + r * hidden * 2) + c);
    const uint32_t ww[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      acc[2 * i] = fmaf(wv, __uint_as_float(ww[i] << 16), acc[2 * i]);
      acc[2 * i + 1] = fmaf(wv, __uint_as_float(ww[i] & 0xFFFF0000u), acc[2 * i + 1]);
    }
  }
  if (shared_out != nullptr) {
    const uint4 v = __ldg(reinterpret_cast<const uint4*>(shared_out + static_cast<uint64_t>(t) * hidden) + c);
    const uint32_t ww[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      acc[2 * i] = __fadd_rn(acc[2 * i], __uint_as_float(ww[i] << 16));
      acc[2 * i + 1] = __fadd_rn(acc[2 * i + 1], __uint_as_float(ww[i] & 0xFFFF0000u));
    }
  }
  uint32_t packed[4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
    packed[i] = static_cast<uint32_t>(float_to_bf16_bits(acc[2 * i])) |
                (static_cast<uint32_t>(float_to_bf16_bits(acc[2 * i + 1])) << 16);
  *(reinterpret_cast<uint4*>(out + static_cast<uint64_t>(t) * hidden) + c) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
}

// ---------------------------------------------------------------------------------------------
// Tensor-parallel reduction over peer memory: the all-reduce behind a K-split projection as a
// reduce-scatter and an all-gather made of plain peer loads.  Rank r owns token rows
// [r*T/R, (r+1)*T/R): it sums every rank's fp32 partial of those rows in rank order (so all ranks
// agree bit for bit and the result does not depend on timing), rounds once to bf16 and writes its
// slice of its own peer-mapped output; after a barrier every rank copies the other slices from
// their owners.  Per rank (R-1)/R of the fp32 matrix and (R-1)/R of the bf16 matrix cross NVLink,
// against 2(R-1)/R of the fp32 matrix for a ring all-reduce.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
tp_reduce_rows_kernel(PeerPtrs partials, uint32_t ranks, uint64_t row_begin, uint64_t row_end, uint32_t hidden,
                      uint16_t* __restrict__ out) {
  const uint32_t vecs = hidden / 4;
  const uint64_t work = (row_end - row_begin) * vecs;
  for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < work;
       i += static_cast<uint64_t>(gridDim.x) * blockDim.x) {
    const uint64_t off = (row_begin + i / vecs) * hidden + (i % vecs) * 4;   // element offset
    float4 acc = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(partials.p[0]) + off);
    for (uint32_t s = 1; s < ranks; ++s) {
      const float4 v = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(partials.p[s]) + off);
      acc.x = __fadd_rn(acc.x, v.x);
      acc.y = __fadd_rn(acc.y, v.y);
      acc.z = __fadd_rn(acc.z, v.z);
      acc.w = __fadd_rn(acc.w, v.w);
    }
    const uint32_t lo = static_cast<uint32_t>(float_to_bf16_bits(acc.x)) | (static_cast<uint32_t>(float_to_bf16_bits(acc.y)) << 16);
    const uint32_t hi = static_cast<uint32_t>(float_to_bf16_bits(acc.z)) | (static_cast<uint32_t>(float_to_bf16_bits(acc.w)) << 16);
    *reinterpret_cast<uint2*>(out + off) = make_uint2(lo, hi);
  }
}

__global__ void __launch_bounds__(256)
tp_gather_rows_kernel(PeerPtrs slices, uint32_t ranks, uint32_t me, uint64_t tokens, uint32_t hidden,
                      uint16_t* __restrict__ out) {
  const uint32_t vecs = hidden / 8;   // 16-byte pieces per row
  const uint64_t work = tokens * vecs;
  for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < work;
       i += static_cast<uint64_t>(gridDim.x) * blockDim.x) {
    const uint64_t row = i / vecs;
    // owner of the row: the rank whose slice [s*T/R, (s+1)*T/R) holds it
    uint32_t owner = static_cast<uint32_t>((row * ranks + ranks - 1) / tokens);
    while (owner > 0 && row < owner * tokens / ranks) --owner;
    while (owner + 1 < ranks && row >= (owner + 1) * tokens / ranks) ++owner;
    if (owner == me) continue;
    const uint64_t off = row * hidden + (i % vecs) * 8;
    *reinterpret_cast<uint4*>(out + off) = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(slices.p[owner]) + off);
  }
}

int32_t load_peers(const char* op, const uint64_t* peer_ptrs, uint64_t ranks, PeerPtrs* out) {
  GEMB_REQUIRE(peer_ptrs != nullptr, "%s: peer pointer table must be nonnull", op);
  GEMB_REQUIRE(ranks >= 1 && ranks <= kMaxRanks, "%s: between 1 and %u ranks are supported", op, kMaxRanks);
  for (uint64_t r = 0; r < kMaxRanks; ++r) {
    out->p[r] = r < ranks ? reinterpret_cast<const uint8_t*>(peer_ptrs[r]) : nullptr;
    GEMB_REQUIRE(r >= ranks || (out->p[r] != nullptr && peer_ptrs[r] % 16 == 0),
                 "%s: every rank's buffer must be mapped and 16-byte aligned", op);
  }
  return GEMB_OK;
}

}  // namespace
}  // namespace gemb

using namespace gemb;

extern "C" {

uint64_t gemb_moe_ep_plan_ints(uint64_t capacity_rows, uint64_t local_experts) {
  // tiles, padded rows, local_experts + 1 padded offsets, one expert id per possible tile (every
  // expert's rows are padded to a multiple of 256: at most capacity / 128 + 2 per expert tiles)
  // the same again for the list of tiles that hold real rows, plus its length
  return 3 + local_experts + 2 * ((capacity_rows + 127) / 128 + 2 * local_experts) + 1;
}

int32_t gemb_moe_ep_plan(const int32_t* counts_all, uint64_t ranks, uint64_t experts, uint64_t rank,
                         int32_t* plan, int32_t* recv_prefix, int32_t* recv_src_rows, int32_t* recv_dst_rows,
                         int32_t* combine_row_base, uint64_t capacity_rows, uint64_t send_rows_per_rank,
                         gemb_stream_t stream) {
  const char* op = "gemb_moe_ep_plan";
  GEMB_REQUIRE(counts_all && plan && recv_prefix && recv_src_rows && recv_dst_rows && combine_row_base,
               "%s: pointers must be nonnull", op);
  GEMB_REQUIRE(ranks >= 1 && ranks <= kMaxRanks && rank < ranks, "%s: bad rank geometry", op);
  GEMB_REQUIRE(experts >= ranks && experts <= kMaxExperts && experts % ranks == 0,
               "%s: experts must be a multiple of ranks, at most %u", op, kMaxExperts);
  GEMB_REQUIRE(capacity_rows > 0 && capacity_rows < (1ull << 31) && capacity_rows % 128 == 0 &&
                   send_rows_per_rank > 0 && send_rows_per_rank < (1ull << 31),
               "%s: buffer capacities must be nonzero (padded rows a multiple of 128)", op);
  GEMB_ENTER(op);
  ep_plan_kernel<<<1, 256, (5 * experts + (ranks * experts <= kPlanSmemCounts ? ranks * experts : 0)) * sizeof(int), stream>>>(
      counts_all, static_cast<uint32_t>(ranks), static_cast<uint32_t>(experts), static_cast<uint32_t>(rank), plan,
      recv_prefix, recv_src_rows, recv_dst_rows, combine_row_base, static_cast<uint32_t>(capacity_rows),
      static_cast<uint32_t>(send_rows_per_rank), nullptr);
  return check_launch(op);
}

int32_t gemb_moe_ep_barrier(const uint64_t* peer_flag_arrays_host, uint64_t ranks, uint64_t rank, uint64_t which,
                            uint32_t* local_epochs, gemb_stream_t stream) {
  const char* op = "gemb_moe_ep_barrier";
  PeerPtrs peers;
  GEMB_TRY(load_peers(op, peer_flag_arrays_host, ranks, &peers));
  GEMB_REQUIRE(rank < ranks && which < 2 && local_epochs != nullptr, "%s: bad rank, barrier index or epoch pointer", op);
  GEMB_ENTER(op);
  ep_barrier_kernel<<<1, 32, 0, stream>>>(peers, static_cast<uint32_t>(ranks), static_cast<uint32_t>(rank),
                                          static_cast<uint32_t>(which), local_epochs,
                                          static_cast<uint32_t>(g_ep_barrier_spins));
  return check_launch(op);
}

int32_t gemb_moe_ep_gather_counts(const uint64_t* peer_count_buffers_host, uint64_t ranks, uint64_t experts,
                                  int32_t* counts_all, gemb_stream_t stream) {
  const char* op = "gemb_moe_ep_gather_counts";
  PeerPtrs peers;
  GEMB_TRY(load_peers(op, peer_count_buffers_host, ranks, &peers));
  GEMB_REQUIRE(counts_all != nullptr && experts >= 1 && experts <= kMaxExperts, "%s: bad arguments", op);
  GEMB_ENTER(op);
  ep_gather_counts_kernel<<<1, 256, 0, stream>>>(peers, static_cast<uint32_t>(ranks), static_cast<uint32_t>(experts), counts_all);
  return check_launch(op);
}

int32_t gemb_tp_reduce_rows(const uint64_t* peer_partials_host, uint64_t ranks, uint64_t rank, uint64_t tokens,
                            uint64_t hidden, uint16_t* out_bf16, gemb_stream_t stream) {
  const char* op = "gemb_tp_reduce_rows";
  PeerPtrs peers;
  GEMB_TRY(load_peers(op, peer_partials_host, ranks, &peers));
  GEMB_REQUIRE(out_bf16 != nullptr && rank < ranks, "%s: bad output pointer or rank", op);
  GEMB_REQUIRE(tokens > 0 && tokens < (1ull << 31) && hidden > 0 && hidden % 8 == 0 && hidden < (1ull << 24),
               "%s: hidden must be a nonzero multiple of 8", op);
  GEMB_REQUIRE(reinterpret_cast<uintptr_t>(out_bf16) % 16 == 0, "%s: output must be 16-byte aligned", op);
  GEMB_ENTER(op);
  const uint64_t begin = rank * tokens / ranks, end = (rank + 1) * tokens / ranks;
  if (end == begin) return GEMB_OK;
  const uint64_t work = (end - begin) * (hidden / 4);
  const uint64_t ctas = std::min<uint64_t>((work + 255) / 256, static_cast<uint64_t>(sm_count()) * 16);
  tp_reduce_rows_kernel<<<static_cast<unsigned>(ctas), 256, 0, stream>>>(peers, static_cast<uint32_t>(ranks), begin, end,
                                                                        static_cast<uint32_t>(hidden), out_bf16);
  return check_launch(op);
}

int32_t gemb_tp_gather_rows(const uint64_t* peer_outputs_host, uint64_t ranks, uint64_t rank, uint64_t tokens,
                            uint64_t hidden, uint16_t* out_bf16, gemb_stream_t stream) {
  const char* op = "gemb_tp_gather_rows";
  PeerPtrs peers;
  GEMB_TRY(load_peers(op, peer_outputs_host, ranks, &peers));
  GEMB_REQUIRE(out_bf16 != nullptr && rank < ranks, "%s: bad output pointer or rank", op);
  GEMB_REQUIRE(tokens > 0 && tokens < (1ull << 31) && hidden > 0 && hidden % 8 == 0 && hidden < (1ull << 24),
               "%s: hidden must be a nonzero multiple of 8", op);
  GEMB_REQUIRE(reinterpret_cast<uintptr_t>(out_bf16) % 16 == 0, "%s: output must be 16-byte aligned", op);
  GEMB_ENTER(op);
  if (ranks == 1) return GEMB_OK;
  const uint64_t work = tokens * (hidden / 8);
  const uint64_t ctas = std::min<uint64_t>((work + 255) / 256, static_cast<uint64_t>(sm_count()) * 16);
  tp_gather_rows_kernel<<<static_cast<unsigned>(ctas), 256, 0, stream>>>(peers, static_cast<uint32_t>(ranks),
                                                                        static_cast<uint32_t>(rank), tokens,
                                                                        static_cast<uint32_t>(hidden), out_bf16);
  return check_launch(op);
}

int32_t gemb_moe_ep_pull_dispatch(const uint64_t* peer_send_buffers_host, uint64_t ranks, uint64_t local_experts,
                                  const int32_t* recv_prefix, const int32_t* recv_src_rows,
                                  const int32_t* recv_dst_rows, uint8_t* packed_e2m1, uint8_t* interleaved_scales,
                                  uint64_t hidden, uint64_t message_row_bytes, uint64_t send_rows_per_rank,
                                  uint64_t padded_rows_max, gemb_stream_t stream) {
  const char* op = "gemb_moe_ep_pull_dispatch";
  PeerPtrs peers;
  GEMB_TRY(load_peers(op, peer_send_buffers_host, ranks, &peers));
  GEMB_REQUIRE(recv_prefix && recv_src_rows && recv_dst_rows && packed_e2m1 && interleaved_scales,
               "%s: pointers must be nonnull", op);
  GEMB_REQUIRE(local_experts >= 1 && ranks * local_experts <= kMaxExperts, "%s: bad expert geometry", op);
  GEMB_REQUIRE(hidden > 0 && hidden % 64 == 0 && hidden <= 8192, "%s: hidden must be a nonzero multiple of 64, at most 8,192", op);
  GEMB_REQUIRE(message_row_bytes % 16 == 0 && message_row_bytes >= hidden / 2 + hidden / 16,
               "%s: a message row holds the payload and the block scales, padded to 16 bytes", op);
  GEMB_REQUIRE(reinterpret_cast<uintptr_t>(packed_e2m1) % 16 == 0 && reinterpret_cast<uintptr_t>(interleaved_scales) % 4 == 0,
               "%s: outputs must be 16-byte (payload) and 4-byte (scales) aligned", op);
  GEMB_REQUIRE(send_rows_per_rank > 0 && send_rows_per_rank < (1ull << 31) && padded_rows_max > 0 &&
                   padded_rows_max < (1ull << 31) && padded_rows_max % 128 == 0,
               "%s: buffer capacities must be nonzero (padded rows a multiple of 128)", op);
  GEMB_ENTER(op);
  const uint32_t segments = static_cast<uint32_t>(ranks * local_experts);
  const uint32_t c_pad = static_cast<uint32_t>((hidden / 16 + 3) / 4 * 4);
  if (hidden <= 4096)
    ep_pull_dispatch_kernel<4><<<static_cast<unsigned>(sm_count()) * 8, 256, (segments + 1) * sizeof(int), stream>>>(
      peers, recv_prefix, recv_src_rows, recv_dst_rows, segments, static_cast<uint32_t>(local_experts),
      static_cast<uint32_t>(hidden), static_cast<uint32_t>(message_row_bytes), c_pad, packed_e2m1, interleaved_scales,
      static_cast<uint32_t>(send_rows_per_rank), static_cast<uint32_t>(padded_rows_max), nullptr);
  else
    ep_pull_dispatch_kernel<8><<<static_cast<unsigned>(sm_count()) * 8, 256, (segments + 1) * sizeof(int), stream>>>(
      peers, recv_prefix, recv_src_rows, recv_dst_rows, segments, static_cast<uint32_t>(local_experts),
      static_cast<uint32_t>(hidden), static_cast<uint32_t>(message_row_bytes), c_pad, packed_e2m1, interleaved_scales,
      static_cast<uint32_t>(send_rows_per_rank), static_cast<uint32_t>(padded_rows_max), nullptr);
  return check_launch(op);
}

int32_t gemb_moe_ep_pull_combine(const uint64_t* peer_expert_outputs_host, uint64_t ranks, uint64_t local_experts,
                                 const int32_t* top_ids, const int32_t* slot_rows, const int32_t* combine_row_base,
                                 const float* top_weights, const uint16_t* shared_bf16, uint16_t* out_bf16,
                                 uint64_t tokens, uint64_t hidden, uint64_t topk, uint64_t padded_rows_max,
                                 gemb_stream_t stream) {
  const char* op = "gemb_moe_ep_pull_combine";
  PeerPtrs peers;
  GEMB_TRY(load_peers(op, peer_expert_outputs_host, ranks, &peers));
  GEMB_REQUIRE(top_ids && slot_rows && combine_row_base && top_weights && out_bf16, "%s: pointers must be nonnull", op);
  GEMB_REQUIRE(tokens > 0 && tokens < (1ull << 31) && topk >= 1 && topk <= 32, "%s: bad geometry", op);
  GEMB_REQUIRE(local_experts >= 1 && ranks * local_experts <= kMaxExperts, "%s: bad expert geometry", op);
  GEMB_REQUIRE(hidden > 0 && hidden % 8 == 0 && hidden < (1ull << 31), "%s: hidden must be a nonzero multiple of 8", op);
  GEMB_REQUIRE(padded_rows_max > 0 && padded_rows_max < (1ull << 31), "%s: output capacity must be nonzero", op);
  GEMB_REQUIRE(reinterpret_cast<uintptr_t>(out_bf16) % 16 == 0 && reinterpret_cast<uintptr_t>(shared_bf16) % 16 == 0,
               "%s: buffers must be 16-byte aligned", op);
  GEMB_ENTER(op);
  const uint64_t work = tokens * (hidden / 8);
  ep_pull_combine_kernel<<<static_cast<unsigned>((work + 255) / 256), 256, 0, stream>>>(
      peers, top_ids, slot_rows, combine_row_base, top_weights, shared_bf16, out_bf16, static_cast<uint32_t>(tokens),
      static_cast<uint32_t>(hidden), static_cast<uint32_t>(topk), static_cast<uint32_t>(local_experts),
      static_cast<uint32_t>(ranks * local_experts), static_cast<uint32_t>(padded_rows_max));
  return check_launch(op);
}

// ---------------------------------------------------------------------------------------------
// One expert-parallel layer: workspace planning and the launch sequence.
// ---------------------------------------------------------------------------------------------
}  // extern "C"

namespace gemb {
namespace {

struct EpBuffers {
  MoeCommonBuffers c;
  uint64_t cap;         // assignments this rank can receive: tokens * topk * ranks
  uint64_t rows_max;    // padded rows of its local experts for that many
  uint64_t el;
  int32_t* counts_all;
  int32_t* plan;
  int32_t* recv_prefix;
  int32_t* recv_src;
  int32_t* recv_dst;
  int32_t* row_base;
  int32_t* tile_rows;
  int32_t* row_meta;
  uint8_t* a_packed;
  uint8_t* a_scales;
  uint16_t* gate_up;
  uint8_t* p_packed;
  uint8_t* p_scales;
};

uint64_t carve_ep(const gemb_moe_layer_weights* w, uint64_t tokens, uint64_t ranks, uint8_t* base, EpBuffers* b) {
  uint64_t cursor = 0;
  carve_common(w, tokens, base, &cursor, &b->c);
  auto take = [&](uint64_t bytes) {
    uint8_t* p = base ? base + cursor : nullptr;
    cursor += (bytes + 255) / 256 * 256;
    return p;
  };
  const uint64_t h = w->hidden, i = w->intermediate, e = w->experts;
  b->el = e / ranks;
  b->cap = tokens * w->topk * ranks;
  b->rows_max = gemb_moe_padded_rows_max(b->cap, b->el, 1);
  b->counts_all = reinterpret_cast<int32_t*>(take(ranks * e * 4));
  b->plan = reinterpret_cast<int32_t*>(take(gemb_moe_ep_plan_ints(b->cap, b->el) * 4));
  b->recv_prefix = reinterpret_cast<int32_t*>(take((ranks * b->el + 1) * 4));
  b->recv_src = reinterpret_cast<int32_t*>(take(ranks * b->el * 4));
  b->recv_dst = reinterpret_cast<int32_t*>(take(ranks * b->el * 4));
  b->row_base = reinterpret_cast<int32_t*>(take(e * 4));
  b->tile_rows = reinterpret_cast<int32_t*>(take(b->rows_max / 128 * 4));
  b->row_meta = reinterpret_cast<int32_t*>(take(b->rows_max * 8));
  b->a_packed = take(b->rows_max * h / 2);
  b->a_scales = take(gemb_interleaved_scale_bytes(b->rows_max, h));
  b->gate_up = w->gate_up_fused ? nullptr : reinterpret_cast<uint16_t*>(take(b->rows_max * 2 * i * 2));
  b->p_packed = take(b->rows_max * i / 2);
  b->p_scales = take(gemb_interleaved_scale_bytes(b->rows_max, i));
  return cursor;
}

int32_t validate_ep(const char* op, const gemb_moe_layer_weights* w, uint64_t tokens, uint64_t ranks) {
  GEMB_REQUIRE(w != nullptr, "%s: weights must be nonnull", op);
  GEMB_REQUIRE(ranks >= 1 && ranks <= kMaxRanks && w->experts % ranks == 0, "%s: experts must be a multiple of the rank count (at most %u ranks)",
               op, kMaxRanks);
  GEMB_TRY(validate_moe_weights(op, w, tokens, w->experts / ranks));
  GEMB_REQUIRE(w->hidden % 256 == 0 && w->hidden <= 8192, "%s: hidden must be a multiple of 256, at most 8,192", op);
  GEMB_REQUIRE(tokens * w->topk * ranks < (1ull << 31), "%s: tokens * topk * ranks must fit 31 bits", op);
  return GEMB_OK;
}

struct EpCall {
  EpBuffers b;
  PeerPtrs send, recv, counts, flags;
  uint64_t msg_bytes;
};

int32_t prepare_ep(const char* op, const gemb_moe_layer_weights* w, const gemb_moe_ep_comm* comm, uint64_t tokens,
                   void* workspace, uint64_t workspace_bytes, EpCall* call) {
  GEMB_REQUIRE(comm != nullptr, "%s: comm must be nonnull", op);
  GEMB_TRY(validate_ep(op, w, tokens, comm->ranks));
  GEMB_REQUIRE(comm->rank < comm->ranks && comm->local_epochs != nullptr, "%s: bad rank or epoch pointer", op);
  GEMB_REQUIRE(workspace != nullptr && reinterpret_cast<uintptr_t>(workspace) % 256 == 0, "%s: workspace must be 256-byte aligned", op);
  const uint64_t need = carve_ep(w, tokens, comm->ranks, static_cast<uint8_t*>(workspace), &call->b);
  GEMB_REQUIRE(workspace_bytes >= need, "%s: workspace too small (%llu bytes needed)", op, static_cast<unsigned long long>(need));
  GEMB_TRY(load_peers(op, comm->send_buffers_host, comm->ranks, &call->send));
  GEMB_TRY(load_peers(op, comm->recv_buffers_host, comm->ranks, &call->recv));
  GEMB_TRY(load_peers(op, comm->count_buffers_host, comm->ranks, &call->counts));
  GEMB_TRY(load_peers(op, comm->flag_arrays_host, comm->ranks, &call->flags));
  call->msg_bytes = gemb_moe_ep_message_row_bytes(w->hidden);
  return require_sm100(op);
}

int32_t ep_stage_send(const char* op, const gemb_moe_layer_weights* w, const gemb_moe_ep_comm* comm, const EpCall& call,
                      const uint16_t* x, uint64_t tokens, gemb_stream_t stream) {
  const EpBuffers& b = call.b;
  int32_t* my_counts = reinterpret_cast<int32_t*>(const_cast<uint8_t*>(call.counts.p[comm->rank]));
  if (moe_stage_on(kStageRoute)) GEMB_TRY(moe_route_stage(w, x, tokens, b.c, my_counts, stream));
  if (!moe_stage_on(kStagePack)) return GEMB_OK;
  const uint32_t h = static_cast<uint32_t>(w->hidden);
  const unsigned threads = static_cast<unsigned>(std::min<uint64_t>(256, (h / 16 + 31) / 32 * 32));
  ep_pack_kernel<<<static_cast<unsigned>(tokens), threads, h / 16, stream>>>(
      x, b.c.ids, b.c.slot_rows, b.c.offsets, b.c.plan, call.send, static_cast<uint32_t>(comm->rank),
      static_cast<uint32_t>(b.el), h, static_cast<uint32_t>(w->topk), static_cast<uint32_t>(w->experts), static_cast<uint32_t>(call.msg_bytes),
      static_cast<uint32_t>(tokens * w->topk), w->gate_up.input_divisor);
  return check_launch(op);
}

// Flag barrier 0 + counts + position arithmetic, then the gather of the pushed rows into the padded row space.
int32_t ep_stage_exchange(const char* op, const gemb_moe_layer_weights* w, const gemb_moe_ep_comm* comm, const EpCall& call,
                          uint64_t tokens, bool barriers, gemb_stream_t stream) {
  const EpBuffers& b = call.b;
  const uint32_t ranks = static_cast<uint32_t>(comm->ranks), me = static_cast<uint32_t>(comm->rank);
  const uint32_t e = static_cast<uint32_t>(w->experts), el = static_cast<uint32_t>(b.el);
  const uint64_t h = w->hidden, n = tokens * w->topk;
  if (!moe_stage_on(kStageExchange)) return GEMB_OK;
  ep_sync_plan_kernel<<<1, 256, (5 * e + (ranks * e <= kPlanSmemCounts ? ranks * e : 0)) * sizeof(int), stream>>>(
      call.flags, call.counts, ranks, e, me, comm->local_epochs, static_cast<uint32_t>(g_ep_barrier_spins), barriers ? 1 : 0,
      barriers ? 1 : 0, b.counts_all, b.plan, b.recv_prefix, b.recv_src, b.recv_dst, b.row_base,
      static_cast<uint32_t>(b.rows_max), static_cast<uint32_t>(n), b.tile_rows);
  GEMB_TRY(check_launch(op));
  const uint32_t segments = ranks * el;
  const uint32_t c_pad = static_cast<uint32_t>((h / 16 + 3) / 4 * 4);
  // The rows were pushed: source s's rows lie in region s of this rank's own message buffer.
  PeerPtrs regions{};
  for (uint32_t s = 0; s < ranks; ++s) regions.p[s] = call.send.p[me] + static_cast<uint64_t>(s) * n * call.msg_bytes;
  if (h <= 4096)
    ep_pull_dispatch_kernel<4><<<static_cast<unsigned>(sm_count()) * 8, 256, (segments + 1) * sizeof(int), stream>>>(
      regions, b.recv_prefix, b.recv_src, b.recv_dst, segments, el, static_cast<uint32_t>(h),
      static_cast<uint32_t>(call.msg_bytes), c_pad, b.a_packed, b.a_scales, static_cast<uint32_t>(n),
      static_cast<uint32_t>(b.rows_max), reinterpret_cast<int2*>(b.row_meta));
  else
    ep_pull_dispatch_kernel<8><<<static_cast<unsigned>(sm_count()) * 8, 256, (segments + 1) * sizeof(int), stream>>>(
      regions, b.recv_prefix, b.recv_src, b.recv_dst, segments, el, static_cast<uint32_t>(h),
      static_cast<uint32_t>(call.msg_bytes), c_pad, b.a_packed, b.a_scales, static_cast<uint32_t>(n),
      static_cast<uint32_t>(b.rows_max), reinterpret_cast<int2*>(b.row_meta));
  return check_launch(op);
}

// Grouped gate/up GEMM (+ GELU + requantisation) of the local experts, or of the range the caller set.
int32_t ep_stage_gate_up(const char* op, const gemb_moe_layer_weights* w, const EpCall& call, uint64_t tokens,
                         gemb_stream_t stream) {
  (void)op;
  const EpBuffers& b = call.b;
  const uint32_t el = static_cast<uint32_t>(b.el);
  const uint64_t h = w->hidden, i = w->intermediate, n = tokens * w->topk;
  const gemb_nvfp4_binding& gu = w->gate_up;
  const gemb_nvfp4_binding& dn = w->down;
  // with balanced routing this rank's experts receive about as many rows as the rank routes itself
  struct Hint {
    explicit Hint(uint64_t rows) { set_grouped_rows_hint(rows); }
    ~Hint() { set_grouped_rows_hint(0); }
  } hint(n);
  if (w->gate_up_fused != nullptr) {
    if (moe_stage_on(kStageGateUp))
    GEMB_TRY(gemb_moe_grouped_gemm_gated_quant(b.a_packed, b.a_scales, w->gate_up_fused, w->gate_up_fused_scales, b.p_packed,
                                               b.p_scales, b.plan, b.rows_max, el, i, h, gu.input_divisor,
                                               gu.weight_divisors_device, dn.input_divisor, stream));
  } else {
    if (moe_stage_on(kStageGateUp))
    GEMB_TRY(gemb_moe_grouped_gemm_bf16(b.a_packed, b.a_scales, gu.packed_weight, gu.scales_interleaved, b.gate_up, b.plan,
                                        b.rows_max, el, 2 * i, h, gu.input_divisor, gu.weight_divisors_device, stream));
    if (moe_stage_on(kStageGelu))
    GEMB_TRY(gemb_moe_expert_gelu_quantize(b.gate_up, b.plan, b.p_packed, b.p_scales, b.rows_max, i, dn.input_divisor, stream));
  }
  return GEMB_OK;
}

int32_t ep_stage_experts(const char* op, const gemb_moe_layer_weights* w, const gemb_moe_ep_comm* comm, const EpCall& call,
                         uint64_t tokens, bool barriers, gemb_stream_t stream) {
  GEMB_TRY(ep_stage_exchange(op, w, comm, call, tokens, barriers, stream));
  return ep_stage_gate_up(op, w, call, tokens, stream);
}

int32_t ep_stage_down(const char* op, const gemb_moe_layer_weights* w, const gemb_moe_ep_comm* comm, const EpCall& call,
                      uint64_t tokens, gemb_stream_t stream) {
  const EpBuffers& b = call.b;
  const gemb_nvfp4_binding& dn = w->down;
  const uint32_t el = static_cast<uint32_t>(b.el);
  const uint64_t h = w->hidden, i = w->intermediate, n = tokens * w->topk;
  if (!moe_stage_on(kStageDown)) return GEMB_OK;
  struct Hint {
    explicit Hint(uint64_t rows) { set_grouped_rows_hint(rows); }
    ~Hint() { set_grouped_rows_hint(0); }
  } hint(n);
  return grouped_gemm_push(op, b.p_packed, b.p_scales, dn.packed_weight, dn.scales_interleaved, b.plan, b.rows_max, el, h, i,
                           dn.input_divisor, dn.weight_divisors_device, b.row_meta, b.tile_rows, comm->recv_buffers_host,
                           comm->ranks, comm->rank, n, stream);
}

int32_t ep_stage_combine(const char* op, const gemb_moe_layer_weights* w, const gemb_moe_ep_comm* comm, const EpCall& call,
                         uint16_t* out, uint64_t tokens, bool barriers, gemb_stream_t stream) {
  if (barriers && moe_stage_on(kStageExchange)) {
    ep_barrier_kernel<<<1, 32, 0, stream>>>(call.flags, static_cast<uint32_t>(comm->ranks), static_cast<uint32_t>(comm->rank), 1,
                                            comm->local_epochs, static_cast<uint32_t>(g_ep_barrier_spins));
    GEMB_TRY(check_launch(op));
  }
  if (!moe_stage_on(kStageCombine)) return GEMB_OK;
  const uint16_t* rows = reinterpret_cast<const uint16_t*>(call.recv.p[comm->rank]);
  return gemb_moe_combine(rows, nullptr, call.b.c.weights, w->shared_intermediate ? call.b.c.s_out : nullptr, out, tokens,
                          w->hidden, w->topk, stream);
}

// Grid caps and expert ranges of the GEMM launches of the calling thread, for the duration of a scope.
struct Cap {
  explicit Cap(uint32_t ctas) { set_gemm_cta_cap(ctas); }
  ~Cap() { set_gemm_cta_cap(0); }
};
struct Range {
  Range(uint32_t lo, uint32_t hi) { set_grouped_expert_range(lo, hi); }
  ~Range() { set_grouped_expert_range(0, 0); }
};

// The layer behind the pack kernel with the local experts in two halves: exchange; gate/up of the first half;
// then the first half's pushing down GEMM on C SMs of the side stream beside the second half's gate/up GEMM
// on the others; then the second half's push beside the shared branch; join; barrier 1 and combine.
int32_t ep_forward_two_halves(const char* op, const gemb_moe_layer_weights* w, const gemb_moe_ep_comm* comm, const EpCall& call,
                              const uint16_t* x, uint16_t* out, uint64_t tokens, gemb_stream_t stream, gemb_stream_t side_stream,
                              void* fork_event, void* join_event) {
  const bool shared = w->shared_intermediate != 0;
  const uint32_t el = static_cast<uint32_t>(call.b.el);
  const uint32_t sms = static_cast<uint32_t>(sm_count()), c1 = std::min(static_cast<uint32_t>(g_ep_split_sms), sms - 2) & ~1u;
  const uint32_t s_sms = shared ? std::min(static_cast<uint32_t>(std::max(g_ep_shared_sms, 2)), sms - 2) & ~1u : 0u;
  GEMB_TRY(ep_stage_exchange(op, w, comm, call, tokens, true, stream));
  {
    Range first(0, el / 2);
    GEMB_TRY(ep_stage_gate_up(op, w, call, tokens, stream));
    GEMB_TRY(stream_fork(op, stream, side_stream, fork_event));
    Cap cap(c1);
    GEMB_TRY(ep_stage_down(op, w, comm, call, tokens, side_stream));
  }
  // "first half pushed", recorded on the side stream here and waited for by the main stream only before its own push
  cudaError_t ce = cudaEventRecord(static_cast<cudaEvent_t>(join_event), side_stream);
  if (ce != cudaSuccess) return fail(GEMB_INTERNAL, "%s: %s: %s", op, cudaGetErrorName(ce), cudaGetErrorString(ce));
  {
    Range second(el / 2, el);
    {
      Cap cap((sms - c1) & ~1u);
      GEMB_TRY(ep_stage_gate_up(op, w, call, tokens, stream));
    }
    ce = cudaStreamWaitEvent(stream, static_cast<cudaEvent_t>(join_event), 0);
    if (ce != cudaSuccess) return fail(GEMB_INTERNAL, "%s: %s: %s", op, cudaGetErrorName(ce), cudaGetErrorString(ce));
    if (shared) {
      Cap cap(s_sms);
      GEMB_TRY(moe_shared_stage(w, x, tokens, call.b.c, side_stream));
    }
    Cap cap(shared ? (sms - s_sms) & ~1u : 0u);
    GEMB_TRY(ep_stage_down(op, w, comm, call, tokens, stream));
  }
  GEMB_TRY(stream_join(op, stream, side_stream, fork_event));
  return ep_stage_combine(op, w, comm, call, out, tokens, true, stream);
}

}  // namespace
}  // namespace gemb

extern "C" {

uint64_t gemb_moe_ep_message_row_bytes(uint64_t hidden) { return (hidden / 2 + hidden / 16 + 4 + 15) / 16 * 16; }

uint64_t gemb_moe_ep_layer_workspace_bytes(const gemb_moe_layer_weights* weights, uint64_t tokens, uint64_t ranks) {
  if (validate_ep("gemb_moe_ep_layer_workspace_bytes", weights, tokens, ranks) != GEMB_OK) return 0;
  EpBuffers b;
  return carve_ep(weights, tokens, ranks, nullptr, &b);
}

int32_t gemb_moe_ep_layer_records(const gemb_moe_layer_weights* weights, uint64_t tokens, uint64_t ranks, void* workspace,
                                  gemb_moe_records* records) {
  const char* op = "gemb_moe_ep_layer_records";
  GEMB_TRY(validate_ep(op, weights, tokens, ranks));
  GEMB_REQUIRE(workspace != nullptr && records != nullptr && reinterpret_cast<uintptr_t>(workspace) % 256 == 0,
               "%s: workspace (256-byte aligned) and records must be nonnull", op);
  EpBuffers b;
  carve_ep(weights, tokens, ranks, static_cast<uint8_t*>(workspace), &b);
  *records = gemb_moe_records{b.c.logits, b.c.ids, b.c.weights, b.c.counts, b.c.offsets, b.c.perm,
                              b.c.slot_rows, b.plan, nullptr, b.rows_max, b.counts_all};
  return GEMB_OK;
}

int32_t gemb_moe_ep_layer_stage(const gemb_moe_layer_weights* w, const gemb_moe_ep_comm* comm, const uint16_t* x, uint16_t* out,
                                uint64_t tokens, void* workspace, uint64_t workspace_bytes, int32_t stage, int32_t barriers,
                                gemb_stream_t stream) {
  const char* op = "gemb_moe_ep_layer_stage";
  EpCall call;
  GEMB_TRY(prepare_ep(op, w, comm, tokens, workspace, workspace_bytes, &call));
  GEMB_REQUIRE(stage >= 0 && stage <= 2, "%s: stage must be 0, 1 or 2", op);
  if (stage == 0) {
    GEMB_REQUIRE(x != nullptr, "%s: input must be nonnull", op);
    if (w->shared_intermediate != 0) GEMB_TRY(moe_shared_stage(w, x, tokens, call.b.c, stream));
    return ep_stage_send(op, w, comm, call, x, tokens, stream);
  }
  if (stage == 1) {
    GEMB_TRY(ep_stage_experts(op, w, comm, call, tokens, barriers != 0, stream));
    return ep_stage_down(op, w, comm, call, tokens, stream);
  }
  GEMB_REQUIRE(out != nullptr, "%s: output must be nonnull", op);
  return ep_stage_combine(op, w, comm, call, out, tokens, barriers != 0, stream);
}

int32_t gemb_moe_ep_layer_forward(const gemb_moe_layer_weights* w, const gemb_moe_ep_comm* comm, const uint16_t* x, uint16_t* out,
                                  uint64_t tokens, void* workspace, uint64_t workspace_bytes, gemb_stream_t stream,
                                  gemb_stream_t side_stream, void* fork_event, void* join_event) {
  const char* op = "gemb_moe_ep_layer_forward";
  EpCall call;
  GEMB_TRY(prepare_ep(op, w, comm, tokens, workspace, workspace_bytes, &call));
  GEMB_REQUIRE(x != nullptr && out != nullptr, "%s: input and output must be nonnull", op);
  const bool shared = w->shared_intermediate != 0;
  // Small batches: the shared branch on the side stream from the start.  Large ones: in line, behind the
  // pushing down GEMM, so that it runs while the slower ranks' rows are still arriving and only then
  // does this rank wait at the second barrier.
  const bool forked = shared && side_stream != nullptr && fork_event != nullptr && join_event != nullptr && fork_pays(tokens);
  if (forked) {
    GEMB_TRY(stream_fork(op, stream, side_stream, fork_event));
    if (moe_stage_on(kStageShared)) GEMB_TRY(moe_shared_stage(w, x, tokens, call.b.c, side_stream));
  }
  GEMB_TRY(ep_stage_send(op, w, comm, call, x, tokens, stream));
  // Large batches, GEMB_TUNE_EP_SPLIT_SMS = C > 0: the local experts in two halves, so that the NVLink-bound
  // pushing down GEMM of the first half (side stream, C SMs) runs beside the gate/up GEMM of the second (the
  // other SMs), and the second half's pushing down GEMM beside the shared branch.  Needs the grouped GEMMs on
  // CTA pairs (an expert range is a range of 256-row units) and the fused gate/up epilogue.
  const uint32_t el = static_cast<uint32_t>(call.b.el);
  bool split = !forked && g_ep_split_sms > 0 && comm->ranks > 1 && el >= 2 && side_stream != nullptr && fork_event != nullptr &&
               join_event != nullptr && w->gate_up_fused != nullptr && moe_stage_on(kStageGateUp) && moe_stage_on(kStageDown) &&
               moe_stage_on(kStageShared) && moe_stage_on(kStageExchange);
  if (split) {
    set_grouped_rows_hint(tokens * w->topk);
    split = grouped_uses_pairs(call.b.rows_max, el);
    set_grouped_rows_hint(0);
  }
  if (split) return ep_forward_two_halves(op, w, comm, call, x, out, tokens, stream, side_stream, fork_event, join_event);
  GEMB_TRY(ep_stage_experts(op, w, comm, call, tokens, true, stream));
  // The pushing down GEMM is bound by NVLink, not by the SMs: with GEMB_TUNE_EP_SHARED_SMS = S the shared
  // branch's GEMMs run beside it on S SMs of their own (both grids capped, so all CTAs are resident at
  // once and none waits for another kernel's CTA to leave an SM).
  const bool beside = shared && !forked && g_ep_shared_sms > 0 && comm->ranks > 1 && side_stream != nullptr &&
                      fork_event != nullptr && join_event != nullptr && moe_stage_on(kStageShared) && moe_stage_on(kStageDown);
  if (beside) {
    GEMB_TRY(stream_fork(op, stream, side_stream, fork_event));
    {
      Cap cap(static_cast<uint32_t>(g_ep_shared_sms));
      GEMB_TRY(moe_shared_stage(w, x, tokens, call.b.c, side_stream));
    }
    {
      Cap cap(static_cast<uint32_t>(sm_count() - g_ep_shared_sms) & ~1u);
      GEMB_TRY(ep_stage_down(op, w, comm, call, tokens, stream));
    }
    GEMB_TRY(stream_join(op, stream, side_stream, join_event));
  } else {
    GEMB_TRY(ep_stage_down(op, w, comm, call, tokens, stream));
    if (shared && !forked && moe_stage_on(kStageShared)) GEMB_TRY(moe_shared_stage(w, x, tokens, call.b.c, stream));
  }
  if (forked) GEMB_TRY(stream_join(op, stream, side_stream, join_event));
  return ep_stage_combine(op, w, comm, call, out, tokens, true, stream);
}

}  // extern "C"
