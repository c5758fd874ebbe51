// Whole-layer entry points of the mixture-of-experts path: workspace planning, the launch
// sequence of one layer on one GPU, and the router's input transform.  Host code only sequences
// the operator entry points of this library; every one of them is stream-ordered and allocates
// nothing, so a layer call is capturable as it stands.
//
// gem16 reserves these entry points (gem16::internal::LaunchMoe*, src/cuda/moe/) in
// docs/plans/gemma4-26b/milestones/M11_CUDA_MOE_REFERENCE.md:26-45 and
// M15_GROUPED_MOE_PREFILL.md:27-33 but holds no code for them; the stage order is that of
// docs/plans/gemma4-26b/specs/MOE_PREFILL_KERNEL_SPEC.md:34-47.
#include <cmath>

#include "common.cuh"
#include "moe_layer.h"

namespace gemb {

namespace {

// r = bf16(((x * inv) * scale) * root): one thread per token walks the row (the sum of squares is a
// single fma chain in ascending k, which is the contract), then the CTA's threads rescale the
// rows together.  A mode of the router, not a hot kernel.
__global__ void __launch_bounds__(128)
router_input_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ scale, uint16_t* __restrict__ out,
                    uint32_t tokens, uint32_t hidden, float eps, float root) {
  __shared__ float inv_s[128];
  const uint32_t t0 = blockIdx.x * 128;
  const uint32_t t = t0 + threadIdx.x;
  if (t < tokens) {
    const uint16_t* row = x + static_cast<uint64_t>(t) * hidden;
    float ss = 0.0f;
    for (uint32_t i = 0; i < hidden; i += 8) {
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(row + i));
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float lo = __uint_as_float(w[j] << 16), hi = __uint_as_float(w[j] & 0xFFFF0000u);
        ss = fmaf(lo, lo, ss);
        ss = fmaf(hi, hi, ss);
      }
    }
    const float mean = __fadd_rn(__fdiv_rn(ss, static_cast<float>(hidden)), eps);
    inv_s[threadIdx.x] = __fdiv_rn(1.0f, __fsqrt_rn(mean));
  }
  __syncthreads();
  const uint32_t rows = min(128u, tokens - t0);
  for (uint64_t idx = threadIdx.x; idx < static_cast<uint64_t>(rows) * hidden; idx += 128) {
    const uint32_t r = static_cast<uint32_t>(idx / hidden), c = static_cast<uint32_t>(idx % hidden);
    const uint64_t off = static_cast<uint64_t>(t0 + r) * hidden + c;
    float v = __fmul_rn(bf16_bits_to_float(__ldg(x + off)), inv_s[r]);
    v = __fmul_rn(v, bf16_bits_to_float(__ldg(scale + c)));
    out[off] = float_to_bf16_bits(__fmul_rn(v, root));
  }
}

uint64_t align256(uint64_t v) { return (v + 255) / 256 * 256; }

}  // namespace

extern int g_router_tile;
int g_moe_stage_mask = 0;   // 0 = every stage
bool moe_stage_on(int bit) { return g_moe_stage_mask == 0 || (g_moe_stage_mask & bit) != 0; }

int32_t moe_set_tuning(int32_t knob, int32_t value) {
  if (knob == GEMB_TUNE_MOE_STAGE_MASK) {
    GEMB_REQUIRE(value >= 0 && value < 256, "gemb_set_tuning: the stage mask has eight bits");
    g_moe_stage_mask = value;
    return GEMB_OK;
  }
  if (knob == GEMB_TUNE_ROUTER_TILE) {
    GEMB_REQUIRE(value == 0 || value == 1 || value == 8 || value == 16 || value == 32 || value == 56 || value == 64,
                 "gemb_set_tuning: router tile must be 0 (auto), 1 (expert-per-thread kernels), 8, 16, 32, 56 or 64");
    g_router_tile = value;
    return GEMB_OK;
  }
  return fail(GEMB_INVALID_ARGUMENT, "gemb_set_tuning: unknown knob %d", knob);
}

int32_t validate_moe_weights(const char* op, const gemb_moe_layer_weights* w, uint64_t tokens, uint64_t local_experts) {
  GEMB_REQUIRE(w != nullptr, "%s: weights must be nonnull", op);
  GEMB_REQUIRE(tokens > 0 && tokens * w->topk < (1ull << 31), "%s: token count must be nonzero and fit 31 bits", op);
  GEMB_REQUIRE(w->experts >= 32 && w->experts % 32 == 0 && w->experts <= 256, "%s: experts must be a multiple of 32 in [32, 256]", op);
  GEMB_REQUIRE(w->topk >= 1 && w->topk <= 32 && w->topk <= w->experts, "%s: top-k must be in [1, 32] and at most the expert count", op);
  GEMB_REQUIRE(w->hidden >= 128 && w->hidden % 128 == 0 && w->hidden < (1ull << 24), "%s: hidden must be a multiple of 128", op);
  GEMB_REQUIRE(w->intermediate >= 64 && w->intermediate % 64 == 0 && w->intermediate < (1ull << 24),
               "%s: expert intermediate size must be a multiple of 64", op);
  GEMB_REQUIRE(w->shared_intermediate % 64 == 0 && w->shared_intermediate < (1ull << 24),
               "%s: shared intermediate size must be a multiple of 64", op);
  GEMB_REQUIRE(w->router_weight != nullptr, "%s: router weight must be nonnull", op);
  GEMB_REQUIRE(w->router_input_scale == nullptr || positive_finite(w->router_epsilon),
               "%s: the router's RMSNorm epsilon must be positive and finite", op);
  const gemb_nvfp4_binding& gu = w->gate_up;
  const gemb_nvfp4_binding& dn = w->down;
  GEMB_REQUIRE(gu.experts == local_experts && dn.experts == local_experts,
               "%s: the expert stacks must hold %llu matrices", op, static_cast<unsigned long long>(local_experts));
  GEMB_REQUIRE(gu.rows == 2 * w->intermediate && gu.contracting == w->hidden && dn.rows == w->hidden &&
                   dn.contracting == w->intermediate,
               "%s: expert stack geometry must be gate_up [2*intermediate, hidden], down [hidden, intermediate]", op);
  GEMB_REQUIRE((w->gate_up_fused != nullptr) == (w->gate_up_fused_scales != nullptr),
               "%s: fused gate/up weight and scales go together", op);
  GEMB_REQUIRE(w->gate_up_fused != nullptr || (gu.packed_weight != nullptr && gu.scales_interleaved != nullptr),
               "%s: gate/up weights are missing", op);
  GEMB_REQUIRE(dn.packed_weight && dn.scales_interleaved && gu.weight_divisors_device && dn.weight_divisors_device,
               "%s: down weights and the per-expert divisors must be nonnull", op);
  GEMB_REQUIRE(positive_finite(gu.input_divisor) && positive_finite(dn.input_divisor),
               "%s: input divisors must be positive and finite", op);
  if (w->shared_intermediate != 0) {
    const gemb_nvfp4_binding& sg = w->shared_gate_up;
    const gemb_nvfp4_binding& sd = w->shared_down;
    GEMB_REQUIRE(sg.rows == 2 * w->shared_intermediate && sg.contracting == w->hidden && sd.rows == w->hidden &&
                     sd.contracting == w->shared_intermediate && sg.experts == 0 && sd.experts == 0,
                 "%s: shared branch geometry must be gate_up [2*shared_intermediate, hidden], down [hidden, shared_intermediate]", op);
    GEMB_REQUIRE((w->shared_gate_up_fused != nullptr) == (w->shared_gate_up_fused_scales != nullptr),
                 "%s: fused shared gate/up weight and scales go together", op);
    GEMB_REQUIRE(w->shared_gate_up_fused != nullptr || (sg.packed_weight != nullptr && sg.scales_interleaved != nullptr),
                 "%s: shared gate/up weights are missing", op);
    GEMB_REQUIRE(sd.packed_weight && sd.scales_interleaved, "%s: shared down weights must be nonnull", op);
    GEMB_REQUIRE(positive_finite(sg.input_divisor) && positive_finite(sd.input_divisor) && positive_finite(sg.weight_divisor) &&
                     positive_finite(sd.weight_divisor),
                 "%s: shared branch divisors must be positive and finite", op);
  }
  return GEMB_OK;
}

// Carves the routing half of a layer's workspace (shared by the single-GPU and the expert-parallel
// layer): records, permutation scratch, the router's transformed input and the shared branch.
void carve_common(const gemb_moe_layer_weights* w, uint64_t tokens, uint8_t* base, uint64_t* cursor, MoeCommonBuffers* b) {
  auto take = [&](uint64_t bytes) {
    uint8_t* p = base ? base + *cursor : nullptr;
    *cursor += align256(bytes);
    return p;
  };
  const uint64_t e = w->experts, k = w->topk, h = w->hidden, n = tokens * k;
  b->logits = reinterpret_cast<float*>(take(tokens * e * 4));
  b->ids = reinterpret_cast<int32_t*>(take(n * 4));
  b->weights = reinterpret_cast<float*>(take(n * 4));
  b->counts = reinterpret_cast<int32_t*>(take(e * 4));
  b->offsets = reinterpret_cast<int32_t*>(take((e + 1) * 4));
  b->perm = reinterpret_cast<int32_t*>(take(n * 4));
  b->slot_rows = reinterpret_cast<int32_t*>(take(n * 4));
  b->plan = reinterpret_cast<int32_t*>(take(gemb_moe_plan_ints(tokens, e, k) * 4));
  b->permute_ws_bytes = gemb_moe_permute_workspace_bytes(tokens, e, k);
  b->permute_ws = take(b->permute_ws_bytes);
  b->router_x = w->router_input_scale ? reinterpret_cast<uint16_t*>(take(tokens * h * 2)) : nullptr;
  const uint64_t si = w->shared_intermediate;
  if (si != 0) {
    b->s_packed = take(tokens * h / 2);
    b->s_scales = take(gemb_interleaved_scale_bytes(tokens, h));
    b->s_gate_up = w->shared_gate_up_fused ? nullptr : reinterpret_cast<uint16_t*>(take(tokens * 2 * si * 2));
    b->s_p_packed = take(tokens * si / 2);
    b->s_p_scales = take(gemb_interleaved_scale_bytes(tokens, si));
    b->s_out = reinterpret_cast<uint16_t*>(take(tokens * h * 2));
  } else {
    b->s_packed = b->s_scales = b->s_p_packed = b->s_p_scales = nullptr;
    b->s_gate_up = b->s_out = nullptr;
  }
}

int32_t moe_route_stage(const gemb_moe_layer_weights* w, const uint16_t* x, uint64_t tokens, const MoeCommonBuffers& b,
                        int32_t* counts_out, gemb_stream_t stream) {
  const uint16_t* rx = x;
  if (w->router_input_scale != nullptr) {
    GEMB_TRY(gemb_moe_router_input(x, w->router_input_scale, b.router_x, tokens, w->hidden, w->router_epsilon, stream));
    rx = b.router_x;
  }
  GEMB_TRY(gemb_moe_router_logits(rx, w->router_weight, w->router_bias, b.logits, tokens, w->hidden, w->experts, stream));
  GEMB_TRY(gemb_moe_route(b.logits, w->per_expert_scale, b.ids, b.weights, nullptr, tokens, w->experts, w->topk, stream));
  return gemb_moe_permute(b.ids, counts_out ? counts_out : b.counts, b.offsets, b.perm, b.slot_rows, b.plan, b.permute_ws,
                          b.permute_ws_bytes, tokens, w->experts, w->topk, stream);
}

int32_t moe_shared_stage(const gemb_moe_layer_weights* w, const uint16_t* x, uint64_t tokens, const MoeCommonBuffers& b,
                         gemb_stream_t stream) {
  const gemb_nvfp4_binding& sg = w->shared_gate_up;
  const gemb_nvfp4_binding& sd = w->shared_down;
  const uint64_t h = w->hidden, si = w->shared_intermediate;
  GEMB_TRY(gemb_nvfp4_quantize(x, GEMB_BF16, b.s_packed, b.s_scales, tokens, h, sg.input_divisor, GEMB_SCALES_INTERLEAVED,
                               GEMB_QUANT_EXACT, stream));
  if (w->shared_gate_up_fused != nullptr) {
    GEMB_TRY(gemb_nvfp4_gemm_gated_quant(b.s_packed, b.s_scales, w->shared_gate_up_fused, w->shared_gate_up_fused_scales,
                                         b.s_p_packed, b.s_p_scales, tokens, si, h, sg.input_divisor, sg.weight_divisor,
                                         sg.weight_divisor, sd.input_divisor, stream));
  } else {
    GEMB_TRY(gemb_nvfp4_gemm_bf16(b.s_packed, b.s_scales, sg.packed_weight, sg.scales_interleaved, b.s_gate_up, tokens,
                                  2 * si, h, sg.input_divisor, sg.weight_divisor, stream));
    GEMB_TRY(gemb_moe_expert_gelu_quantize(b.s_gate_up, nullptr, b.s_p_packed, b.s_p_scales, tokens, si, sd.input_divisor,
                                           stream));
  }
  return gemb_nvfp4_gemm_bf16(b.s_p_packed, b.s_p_scales, sd.packed_weight, sd.scales_interleaved, b.s_out, tokens, h, si,
                              sd.input_divisor, sd.weight_divisor, stream);
}

// Whether the shared branch goes to the side stream.  Up to about a thousand tokens the layer's kernels
// leave SMs idle and a second stream fills them (15 % at 64 tokens).  Beyond that every kernel fills the
// GPU, so two streams cannot beat the sum of the kernels -- and the persistent GEMMs of the two streams,
// one CTA per SM with a fixed share of tiles each, can only take turns on an SM: whichever CTAs start
// late finish late, and the same captured graph was measured at either 477 or 637 us (4,096 tokens)
// depending on how the CTAs happened to interleave.  In line the layer is the sum of its kernels, every time.
bool fork_pays(uint64_t tokens) { return tokens <= 1024; }

int32_t stream_fork(const char* op, gemb_stream_t stream, gemb_stream_t side_stream, void* event) {
  cudaError_t e = cudaEventRecord(static_cast<cudaEvent_t>(event), stream);
  if (e == cudaSuccess) e = cudaStreamWaitEvent(side_stream, static_cast<cudaEvent_t>(event), 0);
  if (e != cudaSuccess) return fail(GEMB_INTERNAL, "%s: %s: %s", op, cudaGetErrorName(e), cudaGetErrorString(e));
  return GEMB_OK;
}
int32_t stream_join(const char* op, gemb_stream_t stream, gemb_stream_t side_stream, void* event) {
  return stream_fork(op, side_stream, stream, event);
}

namespace {

struct LayerBuffers {
  MoeCommonBuffers c;
  uint64_t rows_max;
  uint8_t* a_packed;
  uint8_t* a_scales;
  uint16_t* gate_up;   // three-launch form only
  uint8_t* p_packed;
  uint8_t* p_scales;
  uint16_t* y;
};

uint64_t carve_layer(const gemb_moe_layer_weights* w, uint64_t tokens, uint8_t* base, LayerBuffers* b) {
  uint64_t cursor = 0;
  carve_common(w, tokens, base, &cursor, &b->c);
  auto take = [&](uint64_t bytes) {
    uint8_t* p = base ? base + cursor : nullptr;
    cursor += align256(bytes);
    return p;
  };
  const uint64_t h = w->hidden, i = w->intermediate;
  b->rows_max = gemb_moe_padded_rows_max(tokens, w->experts, w->topk);
  b->a_packed = take(b->rows_max * h / 2);
  b->a_scales = take(gemb_interleaved_scale_bytes(b->rows_max, h));
  b->gate_up = w->gate_up_fused ? nullptr : reinterpret_cast<uint16_t*>(take(b->rows_max * 2 * i * 2));
  b->p_packed = take(b->rows_max * i / 2);
  b->p_scales = take(gemb_interleaved_scale_bytes(b->rows_max, i));
  b->y = reinterpret_cast<uint16_t*>(take(b->rows_max * h * 2));
  return cursor;
}

}  // namespace
}  // namespace gemb

using namespace gemb;

extern "C" {

uint64_t gemb_struct_bytes(int32_t which) {
  switch (which) {
    case 0: return sizeof(gemb_fp8_binding);
    case 1: return sizeof(gemb_nvfp4_binding);
    case 2: return sizeof(gemb_moe_layer_weights);
    case 3: return sizeof(gemb_moe_records);
    case 4: return sizeof(gemb_moe_ep_comm);
    default: return 0;
  }
}

int32_t gemb_moe_router_input(const uint16_t* x_bf16, const uint16_t* scale_bf16, uint16_t* out_bf16, uint64_t tokens,
                              uint64_t hidden, float epsilon, gemb_stream_t stream) {
  const char* op = "gemb_moe_router_input";
  GEMB_REQUIRE(x_bf16 && scale_bf16 && out_bf16, "%s: pointers must be nonnull", op);
  GEMB_REQUIRE(tokens > 0 && tokens < (1ull << 31) && hidden > 0 && hidden % 8 == 0 && hidden < (1ull << 24),
               "%s: hidden must be a nonzero multiple of 8", op);
  GEMB_REQUIRE(positive_finite(epsilon), "%s: epsilon must be positive and finite", op);
  GEMB_REQUIRE(reinterpret_cast<uintptr_t>(x_bf16) % 16 == 0, "%s: input must be 16-byte aligned", op);
  GEMB_ENTER(op);
  const float root = 1.0f / std::sqrt(static_cast<float>(hidden));
  router_input_kernel<<<static_cast<unsigned>((tokens + 127) / 128), 128, 0, stream>>>(
      x_bf16, scale_bf16, out_bf16, static_cast<uint32_t>(tokens), static_cast<uint32_t>(hidden), epsilon, root);
  return check_launch(op);
}

uint64_t gemb_moe_layer_workspace_bytes(const gemb_moe_layer_weights* weights, uint64_t tokens) {
  if (validate_moe_weights("gemb_moe_layer_workspace_bytes", weights, tokens, weights ? weights->experts : 0) != GEMB_OK)
    return 0;
  LayerBuffers b;
  return carve_layer(weights, tokens, nullptr, &b);
}

int32_t gemb_moe_layer_records(const gemb_moe_layer_weights* weights, uint64_t tokens, void* workspace,
                               gemb_moe_records* records) {
  const char* op = "gemb_moe_layer_records";
  GEMB_TRY(validate_moe_weights(op, weights, tokens, weights ? weights->experts : 0));
  GEMB_REQUIRE(workspace != nullptr && records != nullptr && reinterpret_cast<uintptr_t>(workspace) % 256 == 0,
               "%s: workspace (256-byte aligned) and records must be nonnull", op);
  LayerBuffers b;
  carve_layer(weights, tokens, static_cast<uint8_t*>(workspace), &b);
  *records = gemb_moe_records{b.c.logits, b.c.ids, b.c.weights, b.c.counts, b.c.offsets, b.c.perm,
                              b.c.slot_rows, b.c.plan, b.y, b.rows_max, nullptr};
  return GEMB_OK;
}

int32_t gemb_moe_layer_forward(const gemb_moe_layer_weights* w, const uint16_t* x, uint16_t* out, uint64_t tokens,
                               void* workspace, uint64_t workspace_bytes, gemb_stream_t stream, gemb_stream_t side_stream,
                               void* fork_event, void* join_event) {
  const char* op = "gemb_moe_layer_forward";
  GEMB_TRY(validate_moe_weights(op, w, tokens, w ? w->experts : 0));
  GEMB_REQUIRE(x && out && workspace && reinterpret_cast<uintptr_t>(workspace) % 256 == 0,
               "%s: input, output and workspace (256-byte aligned) must be nonnull", op);
  LayerBuffers b;
  const uint64_t need = carve_layer(w, tokens, static_cast<uint8_t*>(workspace), &b);
  GEMB_REQUIRE(workspace_bytes >= need, "%s: workspace too small (%llu bytes needed)", op, static_cast<unsigned long long>(need));
  GEMB_ENTER(op);
  const bool shared = w->shared_intermediate != 0;
  const bool forked = shared && side_stream != nullptr && fork_event != nullptr && join_event != nullptr && fork_pays(tokens);
  struct Hint {
    explicit Hint(uint64_t rows) { set_grouped_rows_hint(rows); }
    ~Hint() { set_grouped_rows_hint(0); }
  } hint(tokens * w->topk);
  // The shared dense branch depends only on x: beside routing and the expert GEMMs when the caller
  // gave a second stream and the batch is small enough for that to pay, first otherwise.
  if (forked) GEMB_TRY(stream_fork(op, stream, side_stream, fork_event));
  if (shared && moe_stage_on(kStageShared)) GEMB_TRY(moe_shared_stage(w, x, tokens, b.c, forked ? side_stream : stream));
  if (moe_stage_on(kStageRoute)) GEMB_TRY(moe_route_stage(w, x, tokens, b.c, nullptr, stream));
  const gemb_nvfp4_binding& gu = w->gate_up;
  const gemb_nvfp4_binding& dn = w->down;
  const uint64_t h = w->hidden, i = w->intermediate, e = w->experts;
  if (moe_stage_on(kStagePack))
    GEMB_TRY(gemb_moe_dispatch_quantize(x, b.c.slot_rows, b.a_packed, b.a_scales, tokens, h, w->topk, gu.input_divisor, stream));
  if (w->gate_up_fused != nullptr) {
    if (moe_stage_on(kStageGateUp))
    GEMB_TRY(gemb_moe_grouped_gemm_gated_quant(b.a_packed, b.a_scales, w->gate_up_fused, w->gate_up_fused_scales, b.p_packed,
                                               b.p_scales, b.c.plan, b.rows_max, e, i, h, gu.input_divisor,
                                               gu.weight_divisors_device, dn.input_divisor, stream));
  } else {
    if (moe_stage_on(kStageGateUp))
    GEMB_TRY(gemb_moe_grouped_gemm_bf16(b.a_packed, b.a_scales, gu.packed_weight, gu.scales_interleaved, b.gate_up, b.c.plan,
                                        b.rows_max, e, 2 * i, h, gu.input_divisor, gu.weight_divisors_device, stream));
    if (moe_stage_on(kStageGelu))
    GEMB_TRY(gemb_moe_expert_gelu_quantize(b.gate_up, b.c.plan, b.p_packed, b.p_scales, b.rows_max, i, dn.input_divisor, stream));
  }
  if (moe_stage_on(kStageDown))
  GEMB_TRY(gemb_moe_grouped_gemm_bf16(b.p_packed, b.p_scales, dn.packed_weight, dn.scales_interleaved, b.y, b.c.plan,
                                      b.rows_max, e, h, i, dn.input_divisor, dn.weight_divisors_device, stream));
  if (forked) GEMB_TRY(stream_join(op, stream, side_stream, join_event));
  if (!moe_stage_on(kStageCombine)) return GEMB_OK;
  return gemb_moe_combine(b.y, b.c.slot_rows, b.c.weights, shared ? b.c.s_out : nullptr, out, tokens, h, w->topk, stream);
}

}  // extern "C"
