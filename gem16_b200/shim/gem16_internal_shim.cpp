// Drop-in shim: defines gem16's operator launchers (namespace gem16::internal, declared in the
// gem16 tree under src/cuda/nvfp4/*.h and src/cuda/fp8/*.h) on top of the gemb200 C ABI.
//
// Compile this file inside the gem16 tree (-I <gem16>/include -I <gem16>/src -I <gemb200>/include,
// link libgemb200.so) in place of the SM120 operator sources.  Each function keeps the
// reference's signature and error convention (gem16::Status, include/gem16/status.h) and
// forwards; status codes map one to one.
//
// Layout contract that changes with the operator library (see the header of include/gemb200.h):
// NVFP4 weights are the checkpoint's row-major payload; "tiled" weight-scale arguments are
// compact [rows, K/16] for the T=1 launchers and 128x4-interleaved for the batch launchers;
// scratch and workspace arguments are accepted and ignored.
#include "cuda/fp8/cutlass_sm120.h"
#include "cuda/fp8/reference.h"
#include "cuda/fp8/sm120.h"
#include "cuda/nvfp4/cutlass_sm120.h"
#include "cuda/nvfp4/gemv.h"
#include "cuda/nvfp4/mlp.h"
#include "cuda/nvfp4/reference.h"
#include "cuda/nvfp4/sm120.h"
#include "cuda/output_head.h"
#include "gemb200.h"

namespace gem16::internal {
namespace {

Status ToStatus(std::int32_t rc) {
  if (rc == GEMB_OK) return Status::Ok();
  return Status(static_cast<StatusCode>(rc), gemb_last_error());
}
gemb_stream_t S(cudaStream_t stream) { return reinterpret_cast<gemb_stream_t>(stream); }

}  // namespace

// ---- src/cuda/nvfp4/reference.h -----------------------------------------------------------
Status LaunchNvfp4ReferenceActivationQuantization(const float* input, std::uint8_t* packed,
                                                  std::uint8_t* scales, std::uint64_t elements,
                                                  float divisor, cudaStream_t stream) {
  return ToStatus(gemb_nvfp4_quantize(input, GEMB_F32, packed, scales, 1, elements, divisor,
                                      GEMB_SCALES_COMPACT, GEMB_QUANT_RCP_APPROX, S(stream)));
}
Status LaunchRmsNormNvfp4ActivationQuantizationBatch(const float* input, const std::uint16_t* weight,
                                                     std::uint8_t* packed, std::uint8_t* scales,
                                                     std::uint64_t tokens, std::uint64_t k, float eps,
                                                     float divisor, cudaStream_t stream) {
  return ToStatus(gemb_nvfp4_rmsnorm_quantize(input, GEMB_F32, weight, packed, scales, tokens, k, eps,
                                              divisor, GEMB_SCALES_COMPACT, GEMB_QUANT_RCP_APPROX, S(stream)));
}
Status LaunchRmsNormNvfp4ActivationQuantizationBf16Batch(const std::uint16_t* input,
                                                         const std::uint16_t* weight, std::uint8_t* packed,
                                                         std::uint8_t* scales, std::uint64_t tokens,
                                                         std::uint64_t k, float eps, float divisor,
                                                         cudaStream_t stream) {
  return ToStatus(gemb_nvfp4_rmsnorm_quantize(input, GEMB_BF16, weight, packed, scales, tokens, k, eps,
                                              divisor, GEMB_SCALES_COMPACT, GEMB_QUANT_RCP_APPROX, S(stream)));
}
Status LaunchGatedGeluNvfp4ActivationQuantization(const float* gate, const float* up, std::uint8_t* packed,
                                                  std::uint8_t* scales, std::uint64_t elements, float divisor,
                                                  cudaStream_t stream) {
  return ToStatus(gemb_nvfp4_gated_gelu_quantize(gate, up, GEMB_F32, packed, scales, 1, elements, divisor,
                                                 GEMB_SCALES_COMPACT, GEMB_QUANT_RCP_APPROX, S(stream)));
}
Status LaunchGatedGeluNvfp4ActivationQuantizationBf16(const std::uint16_t* gate, const std::uint16_t* up,
                                                      std::uint8_t* packed, std::uint8_t* scales,
                                                      std::uint64_t elements, float divisor,
                                                      cudaStream_t stream) {
  return ToStatus(gemb_nvfp4_gated_gelu_quantize(gate, up, GEMB_BF16, packed, scales, 1, elements, divisor,
                                                 GEMB_SCALES_COMPACT, GEMB_QUANT_RCP_APPROX, S(stream)));
}
Status LaunchNvfp4ReferenceProjection(const std::uint8_t* act, const std::uint8_t* act_scales,
                                      const std::uint8_t* weight, const std::uint8_t* weight_scales,
                                      float* output, std::uint64_t rows, std::uint64_t k, float ga, float gw,
                                      cudaStream_t stream) {
  return ToStatus(gemb_nvfp4_reference_projection(act, act_scales, weight, weight_scales, output, 1, rows, k,
                                                  ga, gw, S(stream)));
}
Status LaunchNvfp4ReferenceProjectionBatch(const std::uint8_t* act, const std::uint8_t* act_scales,
                                           const std::uint8_t* weight, const std::uint8_t* weight_scales,
                                           float* output, std::uint64_t tokens, std::uint64_t rows,
                                           std::uint64_t k, float ga, float gw, cudaStream_t stream) {
  return ToStatus(gemb_nvfp4_reference_projection(act, act_scales, weight, weight_scales, output, tokens, rows,
                                                  k, ga, gw, S(stream)));
}

// ---- src/cuda/nvfp4/sm120.h, gemv.h ----------------------------------------------------------
Status LaunchNvfp4Sm120DirectProjection(const std::uint8_t* act, const std::uint8_t* act_scales,
                                        const std::uint8_t* weight, const std::uint8_t* weight_scales,
                                        float* output, std::uint64_t rows, std::uint64_t k, float ga, float gw,
                                        cudaStream_t stream) {
  return ToStatus(gemb_nvfp4_gemv(act, act_scales, weight, weight_scales, output, rows, k, ga, gw, S(stream)));
}
Status LaunchNvfp4SimtGemvProjection(const std::uint8_t* act, const std::uint8_t* act_scales,
                                     const std::uint8_t* weight, const std::uint8_t* weight_scales,
                                     float* output, std::uint64_t rows, std::uint64_t k, float ga, float gw,
                                     cudaStream_t stream) {
  return ToStatus(gemb_nvfp4_gemv(act, act_scales, weight, weight_scales, output, rows, k, ga, gw, S(stream)));
}
Status LaunchNvfp4Sm120FusedGateUp(const std::uint8_t* act, const std::uint8_t* act_scales,
                                   const std::uint8_t* gate_weight, const std::uint8_t* gate_scales,
                                   const std::uint8_t* up_weight, const std::uint8_t* up_scales,
                                   float* gate_output, float* up_output, float* product_output,
                                   std::uint64_t rows, std::uint64_t k, float gate_ga, float gate_gw,
                                   float up_ga, float up_gw, cudaStream_t stream) {
  return ToStatus(gemb_nvfp4_gemv_gate_up(act, act_scales, gate_weight, gate_scales, up_weight, up_scales,
                                          gate_output, up_output, product_output, rows, k, gate_ga, gate_gw,
                                          up_ga, up_gw, S(stream)));
}
// fp32-output batch form: the verifier's 3 or 5 tokens stream the weights once like the T=1 kernel.
Status LaunchNvfp4Sm120DirectProjectionBatch(const std::uint8_t* act, const std::uint8_t* act_scales,
                                             const std::uint8_t* weight, const std::uint8_t* weight_scales, float* output,
                                             std::uint64_t tokens, std::uint64_t rows, std::uint64_t k, float ga, float gw,
                                             cudaStream_t stream) {
  if (tokens > 8U) return Status(StatusCode::kUnsupported, "more than 8 tokens: use the prefill GEMM (bf16 output)");
  return ToStatus(gemb_nvfp4_gemv_batch(act, act_scales, weight, weight_scales, output, tokens, rows, k, ga, gw, S(stream)));
}
Status LaunchNvfp4Sm120DirectProjectionBf16Batch(const std::uint8_t* act, const std::uint8_t* act_scales_interleaved,
                                                 const std::uint8_t* weight,
                                                 const std::uint8_t* weight_scales_interleaved,
                                                 std::uint16_t* output, std::uint64_t tokens, std::uint64_t rows,
                                                 std::uint64_t k, float ga, float gw, cudaStream_t stream) {
  return ToStatus(gemb_nvfp4_gemm_bf16(act, act_scales_interleaved, weight, weight_scales_interleaved, output,
                                       tokens, rows, k, ga, gw, S(stream)));
}

// ---- src/cuda/nvfp4/cutlass_sm120.h -------------------------------------------------------------
Status LaunchNvfp4CutlassInterleaveActivationScales(const std::uint8_t* compact, std::uint8_t* interleaved,
                                                    std::uint64_t tokens, std::uint64_t k,
                                                    cudaStream_t stream) {
  return ToStatus(gemb_nvfp4_interleave_scales(compact, interleaved, tokens, k, S(stream)));
}
Status LaunchNvfp4CutlassProjectionBf16Batch(const std::uint8_t* act, const std::uint8_t* act_scales_interleaved,
                                             const std::uint8_t* weight,
                                             const std::uint8_t* weight_scales_interleaved, std::uint8_t*,
                                             std::uint8_t*, void*, std::size_t, std::uint16_t* output,
                                             std::uint64_t tokens, std::uint64_t rows, std::uint64_t k, float ga,
                                             float gw, cudaStream_t stream) {
  return ToStatus(gemb_nvfp4_gemm_bf16(act, act_scales_interleaved, weight, weight_scales_interleaved, output,
                                       tokens, rows, k, ga, gw, S(stream)));
}

// ---- src/cuda/fp8/reference.h -----------------------------------------------------------------
Status LaunchFp8ReferenceTokenQuantization(const float* input, std::uint8_t* output, float* scale,
                                           std::uint64_t elements, cudaStream_t stream) {
  return ToStatus(gemb_fp8_quantize(input, GEMB_F32, output, scale, 1, elements, S(stream)));
}
Status LaunchFp8ReferenceTokenQuantizationBatch(const float* input, std::uint8_t* output, float* scales,
                                                std::uint64_t tokens, std::uint64_t k, cudaStream_t stream) {
  return ToStatus(gemb_fp8_quantize(input, GEMB_F32, output, scales, tokens, k, S(stream)));
}
Status LaunchFp8ReferenceTokenQuantizationBf16Batch(const std::uint16_t* input, std::uint8_t* output,
                                                    float* scales, std::uint64_t tokens, std::uint64_t k,
                                                    cudaStream_t stream) {
  return ToStatus(gemb_fp8_quantize(input, GEMB_BF16, output, scales, tokens, k, S(stream)));
}
Status LaunchRmsNormFp8TokenQuantizationBatch(const float* input, const std::uint16_t* weight,
                                              std::uint8_t* output, float* scales, std::uint64_t tokens,
                                              std::uint64_t k, float eps, cudaStream_t stream) {
  return ToStatus(gemb_fp8_rmsnorm_quantize(input, GEMB_F32, weight, output, scales, tokens, k, eps, S(stream)));
}
Status LaunchRmsNormFp8TokenQuantizationBf16Batch(const std::uint16_t* input, const std::uint16_t* weight,
                                                  std::uint8_t* output, float* scales, std::uint64_t tokens,
                                                  std::uint64_t k, float eps, cudaStream_t stream) {
  return ToStatus(gemb_fp8_rmsnorm_quantize(input, GEMB_BF16, weight, output, scales, tokens, k, eps, S(stream)));
}
Status LaunchFp8ReferenceProjection(const std::uint8_t* act, const float* act_scale, const std::uint8_t* weight,
                                    const std::uint16_t* weight_scales, float* output, std::uint64_t rows,
                                    std::uint64_t k, cudaStream_t stream) {
  return ToStatus(gemb_fp8_reference_projection(act, act_scale, weight, weight_scales, output, 1, rows, k, S(stream)));
}
Status LaunchFp8ReferenceProjectionBatch(const std::uint8_t* act, const float* act_scales,
                                         const std::uint8_t* weight, const std::uint16_t* weight_scales,
                                         float* output, std::uint64_t tokens, std::uint64_t rows, std::uint64_t k,
                                         cudaStream_t stream) {
  return ToStatus(gemb_fp8_reference_projection(act, act_scales, weight, weight_scales, output, tokens, rows, k,
                                                S(stream)));
}

// ---- src/cuda/fp8/sm120.h, cutlass_sm120.h -------------------------------------------------------
Status LaunchFp8Sm120DirectProjection(const std::uint8_t* act, const float* act_scale, const std::uint8_t* weight,
                                      const std::uint16_t* weight_scales, float* output, std::uint64_t rows,
                                      std::uint64_t k, cudaStream_t stream) {
  return ToStatus(gemb_fp8_gemv(act, act_scale, weight, weight_scales, output, rows, k, S(stream)));
}
Status LaunchFp8Sm120GroupedQkvProjection(const std::uint8_t* act, const float* act_scale,
                                          const std::uint8_t* q_weight, const std::uint16_t* q_scales,
                                          float* q_output, std::uint64_t q_rows, const std::uint8_t* k_weight,
                                          const std::uint16_t* k_scales, float* k_output, std::uint64_t k_rows,
                                          const std::uint8_t* v_weight, const std::uint16_t* v_scales,
                                          float* v_output, std::uint64_t v_rows, std::uint64_t k,
                                          cudaStream_t stream) {
  return ToStatus(gemb_fp8_gemv_qkv(act, act_scale, q_weight, q_scales, q_output, q_rows, k_weight, k_scales,
                                    k_output, k_rows, v_weight, v_scales, v_output, v_rows, k, S(stream)));
}
// Small batches (the speculative-decoding verifier) stream the weights once like the T=1 kernel; the
// reference's function also accepts prefill-sized batches, which belong to the GEMM (bf16 output).
Status LaunchFp8Sm120DirectProjectionBatch(const std::uint8_t* act, const float* act_scales, const std::uint8_t* weight,
                                           const std::uint16_t* weight_scales, float* output, std::uint64_t tokens,
                                           std::uint64_t rows, std::uint64_t k, cudaStream_t stream) {
  if (tokens > 8U) return Status(StatusCode::kUnsupported, "more than 8 tokens: use the prefill GEMM (bf16 output)");
  return ToStatus(gemb_fp8_gemv_batch(act, act_scales, weight, weight_scales, output, tokens, rows, k, S(stream)));
}
Status LaunchFp8Sm120GroupedQkvProjectionBatch(const std::uint8_t* act, const float* act_scales,
                                               const std::uint8_t* q_weight, const std::uint16_t* q_scales,
                                               float* q_output, std::uint64_t q_rows, const std::uint8_t* k_weight,
                                               const std::uint16_t* k_scales, float* k_output, std::uint64_t k_rows,
                                               const std::uint8_t* v_weight, const std::uint16_t* v_scales,
                                               float* v_output, std::uint64_t v_rows, std::uint64_t tokens,
                                               std::uint64_t k, cudaStream_t stream) {
  if (tokens > 8U) return Status(StatusCode::kUnsupported, "more than 8 tokens: use the prefill GEMM (bf16 output)");
  return ToStatus(gemb_fp8_gemv_qkv_batch(act, act_scales, q_weight, q_scales, q_output, q_rows, k_weight, k_scales,
                                          k_output, k_rows, v_weight, v_scales, v_output, v_rows, tokens, k, S(stream)));
}
Status LaunchFp8CutlassProjectionBatch(const std::uint8_t* act, const float* act_scales,
                                       const std::uint8_t* weight, const std::uint16_t* weight_scales,
                                       std::uint16_t* output, std::uint64_t tokens, std::uint64_t rows,
                                       std::uint64_t k, void*, std::size_t, cudaStream_t stream) {
  return ToStatus(gemb_fp8_gemm_bf16(act, act_scales, weight, weight_scales, output, tokens, rows, k, S(stream)));
}

// ---- src/cuda/output_head.h ------------------------------------------------------------------------
// The reference's kernels are specialised to its vocabulary and width; the same constants go in here.
// OutputHeadCandidate is {float value; uint32 token}, the record gemb_output_head_candidates writes,
// 4,096 per hidden row (kOutputHeadCandidateBlocks == gemb_output_head_candidate_blocks()).
namespace {
constexpr std::uint64_t kShimVocabulary = 262144U, kShimHidden = 3840U;
}  // namespace
Status LaunchFusedOutputHeadCandidates(const std::uint16_t* weights, const float* hidden,
                                       const std::uint32_t* suppressed, std::uint32_t suppressed_count,
                                       const DecodeControl* control, OutputHeadCandidate* candidates,
                                       float* diagnostic_logits, cudaStream_t stream) {
  // the reference reads control->suppressed_token_count on the device when control is non-null
  const std::uint32_t* dynamic_count = control == nullptr ? nullptr : &control->suppressed_token_count;
  return ToStatus(gemb_output_head_candidates(weights, hidden, 1, suppressed, suppressed_count, dynamic_count, candidates,
                                              diagnostic_logits, kShimVocabulary, kShimHidden, S(stream)));
}
Status LaunchFusedOutputHeadBatchCandidates(const std::uint16_t* weights, const float* hidden,
                                            const std::uint32_t* suppressed, std::uint32_t suppressed_count,
                                            std::uint64_t rows, OutputHeadCandidate* candidates,
                                            float* diagnostic_logits, cudaStream_t stream) {
  if (rows == 0U || rows > 5U) return Status(StatusCode::kInvalidArgument, "batched output-head row count is invalid");
  return ToStatus(gemb_output_head_candidates(weights, hidden, rows, suppressed, suppressed_count, nullptr, candidates,
                                              diagnostic_logits, kShimVocabulary, kShimHidden, S(stream)));
}
Status LaunchOutputHeadCandidateArgmax(const OutputHeadCandidate* candidates, std::uint32_t* selected,
                                       cudaStream_t stream) {
  return ToStatus(gemb_output_head_argmax(candidates, 1, selected, S(stream)));
}
Status LaunchOutputHeadBatchArgmax(const OutputHeadCandidate* candidates, std::uint64_t rows, std::uint32_t* selected,
                                   cudaStream_t stream) {
  return ToStatus(gemb_output_head_argmax(candidates, rows, selected, S(stream)));
}

// ---- launchers beside the projections that the engine calls on the same path ------------------
Status LaunchNvfp4CutlassUpGatedGeluQuantizedBatch(
    const std::uint8_t* act, const std::uint8_t* act_scales_interleaved, const std::uint8_t* up_weight,
    const std::uint8_t* up_weight_scales, std::uint8_t*, std::uint8_t*, void*, std::size_t,
    const std::uint16_t* gate_bf16, std::uint8_t* product_packed, std::uint8_t* product_scales,
    std::uint64_t tokens, std::uint64_t rows, std::uint64_t k, float ga, float gw, float product_divisor,
    const float*, cudaStream_t stream) {
  return ToStatus(gemb_nvfp4_gemm_up_gated_quant(act, act_scales_interleaved, up_weight, up_weight_scales, gate_bf16,
                                                 product_packed, product_scales, tokens, rows, k, ga, gw,
                                                 product_divisor, S(stream)));
}
Status LaunchNvfp4Sm120FusedGateUpBatch(const std::uint8_t* act, const std::uint8_t* act_scales,
                                        const std::uint8_t* gate_weight, const std::uint8_t* gate_scales,
                                        const std::uint8_t* up_weight, const std::uint8_t* up_scales,
                                        float* gate_output, float* up_output, float* product_output,
                                        std::uint64_t tokens, std::uint64_t rows, std::uint64_t k, float gate_ga,
                                        float gate_gw, float up_ga, float up_gw, cudaStream_t stream) {
  return ToStatus(gemb_nvfp4_gemv_gate_up_batch(act, act_scales, gate_weight, gate_scales, up_weight, up_scales,
                                                gate_output, up_output, product_output, tokens, rows, k, gate_ga,
                                                gate_gw, up_ga, up_gw, S(stream)));
}
Status LaunchGeluTanhProduct(const float* gate, const float* up, float* output, std::uint64_t elements,
                             cudaStream_t stream) {
  return ToStatus(gemb_gelu_tanh_product_f32(gate, up, output, elements, S(stream)));
}
Status LaunchAddResidual(const float* mlp_output, const float* residual, float* output, std::uint64_t elements,
                         cudaStream_t stream) {
  return ToStatus(gemb_add_residual_f32(mlp_output, residual, output, elements, S(stream)));
}
Status LaunchOutputHeadLogits(const std::uint16_t* weights, const float* hidden, float* logits, cudaStream_t stream) {
  return ToStatus(gemb_output_head_candidates(weights, hidden, 1, nullptr, 0, nullptr, nullptr, logits, 262144, 3840,
                                              S(stream)));
}
Status LaunchLogitArgmax(const float* logits, const std::uint32_t* suppressed, std::uint32_t suppressed_count,
                         std::uint32_t* selected, cudaStream_t stream) {
  return ToStatus(gemb_logit_argmax(logits, suppressed, suppressed_count, selected, 262144, S(stream)));
}

// ---- src/cuda/layer/reference.h: the RMSNorm + residual forms on both sides of every linear ------
Status LaunchRmsNormResidualBf16(const float* input, const std::uint16_t* weight_bf16, const float* residual,
                                 float* normalized_output, float* output, std::uint64_t vectors, std::uint64_t width,
                                 float epsilon, const std::uint16_t* scalar_bf16, cudaStream_t stream) {
  return ToStatus(gemb_rmsnorm_residual(input, GEMB_F32, weight_bf16, residual, normalized_output, output, GEMB_F32,
                                        vectors, width, epsilon, scalar_bf16, S(stream)));
}
Status LaunchRmsNormResidualBf16Input(const std::uint16_t* input_bf16, const std::uint16_t* weight_bf16,
                                      const float* residual, float* normalized_output, float* output,
                                      std::uint64_t vectors, std::uint64_t width, float epsilon,
                                      const std::uint16_t* scalar_bf16, cudaStream_t stream) {
  return ToStatus(gemb_rmsnorm_residual(input_bf16, GEMB_BF16, weight_bf16, residual, normalized_output, output, GEMB_F32,
                                        vectors, width, epsilon, scalar_bf16, S(stream)));
}
Status LaunchRmsNormResidualPhysicalBf16(const std::uint16_t* input_bf16, const std::uint16_t* weight_bf16,
                                         const std::uint16_t* residual_bf16, std::uint16_t* output_bf16,
                                         std::uint64_t vectors, std::uint64_t width, float epsilon,
                                         const std::uint16_t* scalar_bf16, cudaStream_t stream) {
  return ToStatus(gemb_rmsnorm_residual(input_bf16, GEMB_BF16, weight_bf16, residual_bf16, nullptr, output_bf16, GEMB_BF16,
                                        vectors, width, epsilon, scalar_bf16, S(stream)));
}

}  // namespace gem16::internal
