// Internal: pieces of the mixture-of-experts layer shared by the single-GPU and the
// expert-parallel entry points (workspace carving, routing stage, shared dense branch).
#pragma once

#include "common.cuh"

namespace gemb {

struct MoeCommonBuffers {
  float* logits;
  int32_t* ids;
  float* weights;
  int32_t* counts;
  int32_t* offsets;
  int32_t* perm;
  int32_t* slot_rows;
  int32_t* plan;
  void* permute_ws;
  uint64_t permute_ws_bytes;
  uint16_t* router_x;      // router input transform output (specification mode), else null
  uint8_t* s_packed;       // shared branch: quantised tokens
  uint8_t* s_scales;
  uint16_t* s_gate_up;     // three-launch form only
  uint8_t* s_p_packed;
  uint8_t* s_p_scales;
  uint16_t* s_out;
};

// Geometry, pointer and divisor checks of a layer descriptor whose expert stacks hold
// `local_experts` matrices.
int32_t validate_moe_weights(const char* op, const gemb_moe_layer_weights* w, uint64_t tokens, uint64_t local_experts);
// Advances *cursor over the common buffers; fills `b` with pointers when base is nonnull.
void carve_common(const gemb_moe_layer_weights* w, uint64_t tokens, uint8_t* base, uint64_t* cursor, MoeCommonBuffers* b);
// Router (input transform when configured, logits, softmax / top-k) and the stable permutation.
// counts_out overrides where the per-expert counts go (the expert-parallel layer keeps them in
// peer-visible memory); null = b.counts.
int32_t moe_route_stage(const gemb_moe_layer_weights* w, const uint16_t* x, uint64_t tokens, const MoeCommonBuffers& b,
                        int32_t* counts_out, gemb_stream_t stream);
// Shared dense FFN of every token into b.s_out.
int32_t moe_shared_stage(const gemb_moe_layer_weights* w, const uint16_t* x, uint64_t tokens, const MoeCommonBuffers& b,
                         gemb_stream_t stream);
// Grouped projection with the pushing epilogue (csrc/gemm.cu).
int32_t grouped_gemm_push(const char* op, const uint8_t* act, const uint8_t* act_scales_interleaved, const uint8_t* w,
                          const uint8_t* w_scales_interleaved, const int32_t* plan, uint64_t padded_rows_max,
                          uint64_t experts, uint64_t rows_per_expert, uint64_t k, float ga, const float* w_divisors,
                          const int32_t* meta, const int32_t* tile_rows, const uint64_t* dst_host, uint64_t ranks,
                          uint64_t rank, uint64_t dst_rows, gemb_stream_t stream);
// Announces how many rows the calling thread's next grouped GEMMs will really hold (0: unknown),
// for their choice between single CTAs and CTA pairs (csrc/gemm.cu).
void set_grouped_rows_hint(uint64_t rows);
// Upper bound on the persistent grid of the GEMMs the calling thread launches next (0: none), so that two
// GEMMs on two streams can each keep a set of SMs to themselves.
void set_gemm_cta_cap(uint32_t ctas);
// Restricts the calling thread's next grouped GEMMs to the experts [lo, hi) ({0, 0}: all).  Takes effect on
// CTA pairs only, which grouped_uses_pairs predicts for the rows announced with set_grouped_rows_hint.
void set_grouped_expert_range(uint32_t lo, uint32_t hi);
bool grouped_uses_pairs(uint64_t padded_rows_max, uint64_t experts);
// Stage selection of the layer calls (gemb_set_tuning(GEMB_TUNE_MOE_STAGE_MASK, ...)).
enum : int { kStageRoute = 1, kStagePack = 2, kStageGateUp = 4, kStageGelu = 8, kStageDown = 16, kStageCombine = 32,
             kStageShared = 64, kStageExchange = 128 };
bool moe_stage_on(int bit);
// Whether a batch of this many tokens is small enough for the shared branch to gain from a second stream.
bool fork_pays(uint64_t tokens);
// Fork: side_stream waits for what `stream` holds so far.  Join: `stream` waits for side_stream.
int32_t stream_fork(const char* op, gemb_stream_t stream, gemb_stream_t side_stream, void* event);
int32_t stream_join(const char* op, gemb_stream_t stream, gemb_stream_t side_stream, void* event);

}  // namespace gemb
