/* gemb200 -- B200 (sm_100a) implementation of gem16's quantized-weight contraction path.
 *
 * C ABI.  Every entry point mirrors one operator launcher of `namespace gem16::internal`
 * (cited per function as file:line inside the gem16 tree) or, for the MoE path where gem16
 * holds only specifications, the record layouts those specifications define.
 *
 * Conventions (same as the reference launchers):
 *   - every pointer is a DEVICE pointer owned by the caller unless its name ends in `_host`;
 *   - operators allocate nothing, never synchronise, and are ordered on `stream`;
 *   - the return value is a gemb_status; on failure gemb_last_error() holds the message
 *     (thread local), formatted like the reference's "op: cudaErrorName: string";
 *   - null pointers, bad geometry and non-finite / non-positive divisors are rejected with
 *     GEMB_INVALID_ARGUMENT before anything is launched (src/cuda/nvfp4/reference.cu:270-284).
 *   - there is no CPU fallback: without an sm_100 device every launch fails with
 *     GEMB_UNSUPPORTED.
 *
 * Data formats (src/numeric/nvfp4.cpp:13-15,58-70; docs/CHECKPOINT_FORMAT.md:62-95):
 *   NVFP4  packed E2M1, element 2i in the low nibble of byte i; one E4M3FN scale byte per 16
 *          contiguous K elements; one fp32 "global divisor" per tensor.
 *   FP8    E4M3FN bytes; activations carry one fp32 scale per token, weights one bf16 scale per
 *          output row.
 *   bf16   raw uint16 bit patterns.
 */
#ifndef GEMB200_H_
#define GEMB200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* gemb_stream_t; /* identical to cudaStream_t */

/* Mirrors gem16::StatusCode, include/gem16/status.h:9-19, value for value. */
typedef enum gemb_status {
  GEMB_OK = 0,
  GEMB_INVALID_ARGUMENT = 1,
  GEMB_NOT_FOUND = 2,
  GEMB_IO_ERROR = 3,
  GEMB_DATA_LOSS = 4,
  GEMB_UNSUPPORTED = 5,
  GEMB_RESOURCE_EXHAUSTED = 6,
  GEMB_CANCELLED = 7,
  GEMB_INTERNAL = 8
} gemb_status;

/* Element type of an activation input. */
enum { GEMB_F32 = 0, GEMB_BF16 = 1 };
/* Where an NVFP4 quantizer writes its block scales.
 *   COMPACT      row-major [tokens, K/16]                     (src/cuda/nvfp4/reference.cu:99-101)
 *   INTERLEAVED  rows padded to 128, K/16 padded to 4, byte offset
 *                ((r/128)*(C/4)+c/4)*512 + (r%32)*16 + ((r%128)/32)*4 + c%4, padding zero
 *                                                             (src/cuda/nvfp4/cutlass_sm120.cu:160-194)
 */
enum { GEMB_SCALES_COMPACT = 0, GEMB_SCALES_INTERLEAVED = 1 };
/* Which of the reference's two quantizer contracts to follow.
 *   EXACT       q = E2M1((x*g) / decode(scale)), scale = E4M3((amax*(1/6))*g)   -- the host
 *               oracle, src/numeric/nvfp4.cpp:134-150.  Default; what parity is checked against.
 *   RCP_APPROX  q = E2M1(x * rcp(decode(scale) * rcp(g))), scale = E4M3((amax*rcp(6))*g) with
 *               rcp.approx.ftz.f32 -- the reference's device kernels,
 *               src/cuda/nvfp4/reference.cu:39-43,60-78.
 */
enum { GEMB_QUANT_EXACT = 0, GEMB_QUANT_RCP_APPROX = 1 };

const char* gemb_last_error(void);
const char* gemb_status_name(int32_t status);
/* ABI version of this header; bumped on any signature change. */
int32_t gemb_abi_version(void);
/* GEMB_OK when the current CUDA device is compute capability 10.x, else GEMB_UNSUPPORTED.
 * Counterpart of the device gate at src/cuda/engine/inference_engine_initialize.cuh:14-19. */
int32_t gemb_device_check(void);
/* Benchmark hook: overrides an automatic launch heuristic process-wide (not thread safe; meant
 * for sweeps).  No counterpart in the reference, which has no runtime kernel selectors
 * (docs/ARCHITECTURE.md:289).  Knobs: GEMB_TUNE_GEMV_ROWS = weight rows per warp in the decode
 * GEMVs, value 0 (automatic), 1, 2 or 4; GEMB_TUNE_GEMV_PDL = launch the decode GEMVs with
 * programmatic stream serialization so a GEMV's weight prefetch overlaps the tail of the kernel
 * before it (1, default) or not (0); GEMB_TUNE_GEMM_BN = output-feature width of a prefill GEMM
 * tile, 0 (automatic), 128 or 256; GEMB_TUNE_GEMV_IMPL = FP8 decode GEMV data path, 0 (automatic),
 * 1 (direct global loads; also selects the SIMT form of the FP8 small-batch GEMVs, whose per-token
 * results are bit-identical to gemb_fp8_gemv) or 2 (bulk-copy ring through shared memory wherever it fits);
 * GEMB_TUNE_GEMM_PAIR = dense prefill GEMMs on CTA pairs (two SMs share one 256 x 256 tile and
 * each stages half of the weight tile), 0 (automatic), 1 (never) or 2 (always, when the tile is 256 wide);
 * GEMB_TUNE_EP_BARRIER_SPINS = how many times gemb_moe_ep_barrier polls its flags before it gives
 * up and records the fact (about 500 ns per poll; 0 = the default of 2^22, about three seconds) --
 * a deployment's failure-detection latency, and what lets a test see the give-up path quickly;
 * GEMB_TUNE_MOE_STAGE_MASK = which stages the two layer calls launch (bit 0 router + permutation, 1
 * dispatch / pack, 2 grouped gate/up GEMM, 3 separate GELU requantisation, 4 grouped down GEMM, 5
 * combine, 6 shared branch, 7 flag barriers + position arithmetic + pull; 0 = all): with a subset
 * the call re-runs just those launches on what the previous full call left in the workspace, so a
 * benchmark can time one kernel of the sequence in place.  Results of a partial call are not a layer;
 * GEMB_TUNE_EP_SHARED_SMS = for batches above 1,024 tokens per rank, how many SMs (even) the shared branch's
 * GEMMs get beside the NVLink-bound pushing down GEMM of gemb_moe_ep_layer_forward when a side stream is
 * given (default 40, measured best of 0 / 40 / 56 / 72 on two GPUs; 0: the shared branch runs in line behind it);
 * GEMB_TUNE_EP_SPLIT_SMS = for the same batches, C > 0 runs the local experts in two halves: the pushing down
 * GEMM of the first half on C SMs beside the gate/up GEMM of the second half, the second half's pushing down GEMM
 * beside the shared branch (0, the default: one pass over all local experts; at two GPUs the two-half schedule
 * measured 1.23-1.35 ms per layer against 1.00 ms, because neither push is light enough on the SMs);
 * GEMB_TUNE_ROUTER_TILE = which router-logits kernel runs: 0 automatic, 1 the expert-per-thread kernels
 * wherever they apply, 8 / 16 / 32 / 56 / 64 the tiled kernel with that many tokens per CTA (same bits from all). */
enum {
  GEMB_TUNE_GEMV_ROWS = 1,
  GEMB_TUNE_GEMV_PDL = 2,
  GEMB_TUNE_GEMM_BN = 3,
  GEMB_TUNE_GEMV_IMPL = 4,
  GEMB_TUNE_GEMM_PAIR = 5,
  GEMB_TUNE_EP_BARRIER_SPINS = 6,
  GEMB_TUNE_MOE_STAGE_MASK = 7,
  GEMB_TUNE_ROUTER_TILE = 8,
  GEMB_TUNE_EP_SHARED_SMS = 9,
  GEMB_TUNE_EP_SPLIT_SMS = 10
};
int32_t gemb_set_tuning(int32_t knob, int32_t value);
/* Bytes of an INTERLEAVED scale buffer for `rows` rows of K elements. */
uint64_t gemb_interleaved_scale_bytes(uint64_t rows, uint64_t contracting_elements);

/* ------------------------------------------------------------------------------------------
 * Activation quantizers
 * ---------------------------------------------------------------------------------------- */

/* NVFP4 block quantizer over [tokens, K], K % 16 == 0.
 * Replaces LaunchNvfp4ReferenceActivationQuantization, src/cuda/nvfp4/reference.h:13-19
 * (call with tokens = 1, K = elements for the flattened form). */
int32_t gemb_nvfp4_quantize(const void* input, int32_t input_dtype, uint8_t* packed_e2m1,
                            uint8_t* block_scales_e4m3fn, uint64_t tokens,
                            uint64_t elements_per_token, float global_divisor,
                            int32_t scale_layout, int32_t quant_mode, gemb_stream_t stream);

/* RMSNorm -> bf16 state rounding -> NVFP4 quantizer, one pass per token.
 * Replaces LaunchRmsNormNvfp4ActivationQuantizationBatch / ...Bf16Batch,
 * src/cuda/nvfp4/reference.h:23-47.  weight_bf16 may be null (no learned weight). */
int32_t gemb_nvfp4_rmsnorm_quantize(const void* input, int32_t input_dtype,
                                    const uint16_t* weight_bf16, uint8_t* packed_e2m1,
                                    uint8_t* block_scales_e4m3fn, uint64_t tokens,
                                    uint64_t elements_per_token, float epsilon,
                                    float global_divisor, int32_t scale_layout,
                                    int32_t quant_mode, gemb_stream_t stream);

/* bf16(gate), bf16(up) -> bf16 gelu_tanh(gate) -> bf16 product -> NVFP4 quantizer.
 * Replaces LaunchGatedGeluNvfp4ActivationQuantization / ...Bf16,
 * src/cuda/nvfp4/reference.h:52-70. */
int32_t gemb_nvfp4_gated_gelu_quantize(const void* gate, const void* up, int32_t input_dtype,
                                       uint8_t* packed_e2m1, uint8_t* block_scales_e4m3fn,
                                       uint64_t tokens, uint64_t elements_per_token,
                                       float global_divisor, int32_t scale_layout,
                                       int32_t quant_mode, gemb_stream_t stream);

/* Compact -> interleaved block scales (padding written as zero).
 * Replaces LaunchNvfp4CutlassInterleaveActivationScales, src/cuda/nvfp4/cutlass_sm120.h:11-16. */
int32_t gemb_nvfp4_interleave_scales(const uint8_t* compact_scales, uint8_t* interleaved_scales,
                                     uint64_t rows, uint64_t contracting_elements,
                                     gemb_stream_t stream);

/* FP8 dynamic per-token quantizer: scale = amax/448 (1 for an all-zero token), q = E4M3(x/scale).
 * Replaces LaunchFp8ReferenceTokenQuantization{,Batch,Bf16Batch},
 * src/cuda/fp8/reference.h:11-33. */
int32_t gemb_fp8_quantize(const void* input, int32_t input_dtype, uint8_t* output_e4m3fn,
                          float* output_scales, uint64_t tokens, uint64_t elements_per_token,
                          gemb_stream_t stream);

/* RMSNorm -> bf16 -> FP8 per-token quantizer.
 * Replaces LaunchRmsNormFp8TokenQuantizationBatch / ...Bf16Batch,
 * src/cuda/fp8/reference.h:37-58. */
int32_t gemb_fp8_rmsnorm_quantize(const void* input, int32_t input_dtype,
                                  const uint16_t* weight_bf16, uint8_t* output_e4m3fn,
                                  float* output_scales, uint64_t tokens,
                                  uint64_t elements_per_token, float epsilon,
                                  gemb_stream_t stream);

/* RMSNorm + residual (+ layer scalar) with bf16 boundaries: n = bf16(x * inv * w), v = bf16(n +
 * residual), v = bf16(v * scalar) when scalar_bf16 is non-null; weight_bf16 may be null.  input is fp32
 * or bf16 (input_dtype); residual and output are both fp32 or both bf16 (residual_output_dtype; bf16
 * needs a bf16 input); normalized_output (fp32, optional) receives n.
 * Replaces LaunchRmsNormResidualBf16, ...Bf16Input and ...PhysicalBf16, src/cuda/layer/reference.h:45-71
 * (kernels src/cuda/norm/reference.cu:66-160). */
int32_t gemb_rmsnorm_residual(const void* input, int32_t input_dtype, const uint16_t* weight_bf16,
                              const void* residual, float* normalized_output, void* output,
                              int32_t residual_output_dtype, uint64_t vectors, uint64_t width, float epsilon,
                              const uint16_t* scalar_bf16, gemb_stream_t stream);

/* out = bf16(gelu_tanh(gate)) * up in fp32, and out = a + b: the MLP's elementwise bridges.
 * Replace LaunchGeluTanhProduct and LaunchAddResidual, src/cuda/nvfp4/mlp.h:13-23. */
int32_t gemb_gelu_tanh_product_f32(const float* gate, const float* up, float* output, uint64_t elements,
                                   gemb_stream_t stream);
int32_t gemb_add_residual_f32(const float* values, const float* residual, float* output, uint64_t elements,
                              gemb_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * Batch-1 decode projections (HBM-streaming GEMV).  Weights are row-major [rows, K] in the
 * checkpoint's source layout; NVFP4 block scales are COMPACT [rows, K/16].
 * ---------------------------------------------------------------------------------------- */

/* y[row] = (sum_k qa qw) * a_scale * bf16(w_scale[row]), fp32 out.  K % 16 == 0.
 * Replaces LaunchFp8Sm120DirectProjection, src/cuda/fp8/sm120.h:14-22. */
int32_t gemb_fp8_gemv(const uint8_t* activation_e4m3fn, const float* activation_scale,
                      const uint8_t* weight_e4m3fn, const uint16_t* weight_scales_bf16,
                      float* output, uint64_t rows, uint64_t contracting_elements,
                      gemb_stream_t stream);

/* One launch for Q, K and V (V may be null with v_rows = 0).
 * Replaces LaunchFp8Sm120GroupedQkvProjection, src/cuda/fp8/sm120.h:27-43. */
int32_t gemb_fp8_gemv_qkv(const uint8_t* activation_e4m3fn, const float* activation_scale,
                          const uint8_t* q_weight, const uint16_t* q_scales_bf16, float* q_output,
                          uint64_t q_rows, const uint8_t* k_weight, const uint16_t* k_scales_bf16,
                          float* k_output, uint64_t k_rows, const uint8_t* v_weight,
                          const uint16_t* v_scales_bf16, float* v_output, uint64_t v_rows,
                          uint64_t contracting_elements, gemb_stream_t stream);

/* Small-batch forms for the speculative-decoding verifier (second row of the path's "next" list):
 * 1..8 tokens share one pass over the weights.  activation [tokens, K] E4M3, activation_scales
 * [tokens], output fp32 [tokens, rows] (per projection for the grouped form).  With two or more
 * tokens the dot products run on the warp-level tensor-core path (mma.sync m16n8k32, E4M3 x E4M3 ->
 * fp32, the instruction the reference's batch kernel issues, src/cuda/fp8/sm120.cu:101): exact where
 * every partial sum is representable (the reference's fixture, tests/cuda/nvfp4_reference_test.cu:1131),
 * else within the single-token budget of the binary64 value but not bit-identical to gemb_fp8_gemv,
 * since the order of the fp32 additions differs.  tokens * K (K padded to 512) <= 102,400.
 * Replace LaunchFp8Sm120DirectProjectionBatch and LaunchFp8Sm120GroupedQkvProjectionBatch
 * (src/cuda/fp8/sm120.h:45-79) for tokens <= 8; larger batches are prefill and belong to
 * gemb_fp8_gemm_bf16. */
int32_t gemb_fp8_gemv_batch(const uint8_t* activation_e4m3fn, const float* activation_scales,
                            const uint8_t* weight_e4m3fn, const uint16_t* weight_scales_bf16,
                            float* output, uint64_t tokens, uint64_t rows,
                            uint64_t contracting_elements, gemb_stream_t stream);
int32_t gemb_fp8_gemv_qkv_batch(const uint8_t* activation_e4m3fn, const float* activation_scales,
                                const uint8_t* q_weight, const uint16_t* q_scales_bf16, float* q_output,
                                uint64_t q_rows, const uint8_t* k_weight, const uint16_t* k_scales_bf16,
                                float* k_output, uint64_t k_rows, const uint8_t* v_weight,
                                const uint16_t* v_scales_bf16, float* v_output, uint64_t v_rows,
                                uint64_t tokens, uint64_t contracting_elements, gemb_stream_t stream);

/* Per-token FP8 quantization of a bf16 vector fused into the GEMV (each CTA re-derives the
 * token scale and bytes; results are bit-identical to gemb_fp8_quantize + gemb_fp8_gemv).
 * Fuses the decode pair at src/cuda/engine/inference_engine_decode_graphs.cuh:287-290.
 * output_dtype: GEMB_F32 or GEMB_BF16 (round-to-nearest-even). */
int32_t gemb_fp8_gemv_bf16in(const uint16_t* activation_bf16, const uint8_t* weight_e4m3fn,
                             const uint16_t* weight_scales_bf16, void* output,
                             int32_t output_dtype, uint64_t rows, uint64_t contracting_elements,
                             gemb_stream_t stream);

/* y[row] = (sum_k qa sa qw sw) / (ga * gw), fp32 out.  K % 64 == 0, rows % 8 == 0
 * (the reference's native geometry rule, src/cuda/nvfp4/sm120.cu:708-711).
 * Replaces LaunchNvfp4Sm120DirectProjection, src/cuda/nvfp4/sm120.h:14-24. */
int32_t gemb_nvfp4_gemv(const uint8_t* packed_activation_e2m1, const uint8_t* activation_scales,
                        const uint8_t* packed_weight_e2m1, const uint8_t* weight_scales,
                        float* output, uint64_t rows, uint64_t contracting_elements,
                        float activation_global_divisor, float weight_global_divisor,
                        gemb_stream_t stream);

/* Small-batch form (1..8 tokens, the verifier's MLP projections): activation [tokens, K/2] with
 * COMPACT scales [tokens, K/16], output fp32 [tokens, rows]; per token bit-identical to
 * gemb_nvfp4_gemv.  Replaces LaunchNvfp4Sm120DirectProjectionBatch (src/cuda/nvfp4/sm120.h:26-37)
 * for tokens <= 8; larger batches are prefill and belong to gemb_nvfp4_gemm_bf16. */
int32_t gemb_nvfp4_gemv_batch(const uint8_t* packed_activation_e2m1, const uint8_t* activation_scales,
                              const uint8_t* packed_weight_e2m1, const uint8_t* weight_scales,
                              float* output, uint64_t tokens, uint64_t rows,
                              uint64_t contracting_elements, float activation_global_divisor,
                              float weight_global_divisor, gemb_stream_t stream);

/* Gate and Up in one launch with the bf16 boundaries and the GELU-tanh product in the epilogue;
 * gate_output / up_output may be null.
 * Replaces LaunchNvfp4Sm120FusedGateUp, src/cuda/nvfp4/sm120.h:58-74. */
int32_t gemb_nvfp4_gemv_gate_up(const uint8_t* packed_activation_e2m1,
                                const uint8_t* activation_scales,
                                const uint8_t* packed_gate_weight, const uint8_t* gate_weight_scales,
                                const uint8_t* packed_up_weight, const uint8_t* up_weight_scales,
                                float* gate_output, float* up_output, float* product_output,
                                uint64_t rows, uint64_t contracting_elements,
                                float gate_activation_global_divisor,
                                float gate_weight_global_divisor,
                                float up_activation_global_divisor,
                                float up_weight_global_divisor, gemb_stream_t stream);

/* The same for 1..65,535 tokens (the verifier's batches are a handful): activation [tokens, K/2]
 * with COMPACT scales [tokens, K/16], outputs [tokens, rows]; per token bit-identical to
 * gemb_nvfp4_gemv_gate_up, which it launches once per token.
 * Replaces LaunchNvfp4Sm120FusedGateUpBatch, src/cuda/nvfp4/sm120.h:75-92. */
int32_t gemb_nvfp4_gemv_gate_up_batch(const uint8_t* packed_activation_e2m1, const uint8_t* activation_scales,
                                      const uint8_t* packed_gate_weight, const uint8_t* gate_weight_scales,
                                      const uint8_t* packed_up_weight, const uint8_t* up_weight_scales,
                                      float* gate_output, float* up_output, float* product_output,
                                      uint64_t tokens, uint64_t rows, uint64_t contracting_elements,
                                      float gate_activation_global_divisor, float gate_weight_global_divisor,
                                      float up_activation_global_divisor, float up_weight_global_divisor,
                                      gemb_stream_t stream);

/* y[row] = bf16( sum_k x[k] * W[row][k] ) kept as fp32: fp32 activation, bf16 weights [rows, K],
 * fp32 accumulation, one bf16 rounding of the result.  K % 8 == 0, K <= 12,288.  The assistant
 * model's projections; replaces the Bf16GemvKernel launches of src/cuda/mtp/assistant.cu:99-122. */
int32_t gemb_bf16_gemv(const float* input, const uint16_t* weight_bf16, float* output, uint64_t rows,
                       uint64_t contracting_elements, gemb_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * Prefill projections (tcgen05 GEMM, TMEM accumulators, TMA-staged tiles), bf16 output [tokens,
 * rows].  Operands are row-major and K-major: activation [tokens, K], weight [rows, K].
 * ---------------------------------------------------------------------------------------- */

/* NVFP4 W4A4: out = bf16( (sum_k qa sa qw sw) * (1 / (ga * gw)) ).  Both scale buffers use the
 * INTERLEAVED layout (rows padded to 128); K % 64 == 0, rows % 8 == 0; any token count.
 * Replaces LaunchNvfp4CutlassProjectionBf16Batch, src/cuda/nvfp4/cutlass_sm120.h:24-39.  The
 * reference re-tiles its Row8/K64 weights into scratch on every call (PrepareWeightKernel,
 * src/cuda/nvfp4/cutlass_sm120.cu:196-252); here weights are stored once, row-major with
 * interleaved scales, so the scratch and workspace arguments disappear. */
int32_t gemb_nvfp4_gemm_bf16(const uint8_t* packed_activation_e2m1,
                             const uint8_t* interleaved_activation_scales,
                             const uint8_t* packed_weight_e2m1,
                             const uint8_t* interleaved_weight_scales, uint16_t* output_bf16,
                             uint64_t tokens, uint64_t rows, uint64_t contracting_elements,
                             float activation_global_divisor, float weight_global_divisor,
                             gemb_stream_t stream);

/* Same contraction with fp32 output [tokens, rows] = acc * (1 / (ga * gw)), no bf16 rounding: the
 * partial sums of a row-split (K-sharded) projection, to be all-reduced and rounded once.  The
 * reference has no multi-GPU path; its nearest relative is the fp32-output batch projection
 * LaunchNvfp4Sm120DirectProjectionBatch, src/cuda/nvfp4/sm120.h:26-37. */
int32_t gemb_nvfp4_gemm_f32(const uint8_t* packed_activation_e2m1,
                            const uint8_t* interleaved_activation_scales,
                            const uint8_t* packed_weight_e2m1, const uint8_t* interleaved_weight_scales,
                            float* output_f32, uint64_t tokens, uint64_t rows,
                            uint64_t contracting_elements, float activation_global_divisor,
                            float weight_global_divisor, gemb_stream_t stream);

/* Gate and Up projections, GELU and requantisation in ONE kernel.  The fused weight holds the
 * gate and up rows interleaved in runs of 32 features (gemb_nvfp4_pack_gate_up), so each token's
 * accumulator row carries gate and up of the same features side by side and the epilogue emits
 * product = bf16(bf16(gelu_tanh(bf16(gate))) * bf16(up)) already NVFP4-quantised (EXACT contract)
 * with the down projection's input divisor: payload [tokens, intermediate/2] + INTERLEAVED
 * scales, byte-identical to gemb_nvfp4_gemm_bf16 (gate), (up) + gemb_nvfp4_gated_gelu_quantize.
 * intermediate % 32 == 0, K % 64 == 0.
 * Replaces LaunchNvfp4CutlassProjectionBf16Batch (gate) + LaunchNvfp4CutlassUpGatedGeluQuantizedBatch,
 * src/cuda/nvfp4/cutlass_sm120.h:24-66 (the reference fuses only the Up GEMM with the epilogue and
 * reads a materialised bf16 Gate; here neither projection is written to memory). */
int32_t gemb_nvfp4_gemm_gated_quant(const uint8_t* packed_activation_e2m1,
                                    const uint8_t* interleaved_activation_scales,
                                    const uint8_t* fused_gate_up_weight,
                                    const uint8_t* fused_interleaved_weight_scales,
                                    uint8_t* product_packed_e2m1, uint8_t* product_interleaved_scales,
                                    uint64_t tokens, uint64_t intermediate,
                                    uint64_t contracting_elements, float activation_global_divisor,
                                    float gate_weight_global_divisor, float up_weight_global_divisor,
                                    float product_global_divisor, gemb_stream_t stream);

/* The reference's own split of the same step: the Gate projection is already materialised as bf16
 * [tokens, rows]; this call runs the Up projection and its epilogue reads the gate, applies the
 * bf16 boundaries, the GELU-tanh product and the NVFP4 quantiser (EXACT contract) with the down
 * projection's input divisor.  Output as gemb_nvfp4_gemm_gated_quant; byte-identical to
 * gemb_nvfp4_gemm_bf16 (up) + gemb_nvfp4_gated_gelu_quantize.  rows % 64 == 0, K % 64 == 0.
 * Replaces LaunchNvfp4CutlassUpGatedGeluQuantizedBatch, src/cuda/nvfp4/cutlass_sm120.h:47-67. */
int32_t gemb_nvfp4_gemm_up_gated_quant(const uint8_t* packed_activation_e2m1,
                                       const uint8_t* interleaved_activation_scales,
                                       const uint8_t* packed_up_weight_e2m1,
                                       const uint8_t* interleaved_up_weight_scales, const uint16_t* gate_bf16,
                                       uint8_t* product_packed_e2m1, uint8_t* product_interleaved_scales,
                                       uint64_t tokens, uint64_t rows, uint64_t contracting_elements,
                                       float activation_global_divisor, float up_weight_global_divisor,
                                       float product_global_divisor, gemb_stream_t stream);

/* Builds the fused gate/up weight of gemb_nvfp4_gemm_gated_quant from the two row-major NVFP4
 * matrices [intermediate, K/2] with COMPACT scales: output row (f/32)*64 + which*32 + f%32 holds
 * feature f of gate (which = 0) or up (which = 1); output scales are INTERLEAVED.  A load-time
 * step, the counterpart of the reference's host tiler (src/cuda/nvfp4/sm120_layout.cpp:58-145). */
int32_t gemb_nvfp4_pack_gate_up(const uint8_t* gate_packed, const uint8_t* gate_scales,
                                const uint8_t* up_packed, const uint8_t* up_scales,
                                uint8_t* fused_packed, uint8_t* fused_interleaved_scales,
                                uint64_t intermediate, uint64_t contracting_elements,
                                gemb_stream_t stream);

/* FP8 W8A8: out = bf16( ((sum_k qa qw) * a_scale[token]) * bf16(w_scale[row]) ).  K % 32 == 0,
 * rows % 8 == 0.  Replaces LaunchFp8CutlassProjectionBatch, src/cuda/fp8/cutlass_sm120.h:17-28
 * (no workspace needed). */
int32_t gemb_fp8_gemm_bf16(const uint8_t* activation_e4m3fn, const float* activation_scales,
                           const uint8_t* weight_e4m3fn, const uint16_t* weight_scales_bf16,
                           uint16_t* output_bf16, uint64_t tokens, uint64_t rows,
                           uint64_t contracting_elements, gemb_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * Mixture-of-experts path.  gem16 holds no MoE code yet: the entry points implement the records
 * and ordering rules its specifications define, at the places its plan reserves for them
 * (src/cuda/moe/router_reference.cu, prefill_{router,permute,reduce}.cu,
 * docs/plans/gemma4-26b/milestones/M11_CUDA_MOE_REFERENCE.md:26-45, M15_GROUPED_MOE_PREFILL.md:27-33).
 * Stages are separate observable launches; nothing is read back to the host between them.
 * ---------------------------------------------------------------------------------------- */

/* logits[t][e] = bias[e] + sum_k x[t][k] * w[e][k], fp32, exactly one fused multiply-add per k
 * in ascending k (bias may be null = 0).  x is bf16 [tokens, hidden], w fp32 [experts, hidden].
 * docs/plans/gemma4-26b/specs/MOE_ROUTER_SPEC.md:3-13 (projection), :27-38 (fp32, deterministic). */
int32_t gemb_moe_router_logits(const uint16_t* x_bf16, const float* router_weight, const float* bias,
                               float* logits, uint64_t tokens, uint64_t hidden, uint64_t experts,
                               gemb_stream_t stream);

/* fp32 softmax over all experts, the topk largest probabilities (the lower expert id wins a
 * tie), renormalised to sum one, then multiplied by per_expert_scale[id] when it is non-null.
 * Outputs RoutedExperts records as two arrays: top_ids[tokens, topk] int32 and
 * top_weights[tokens, topk] fp32; probabilities[tokens, experts] is optional (null to skip).
 * experts % 32 == 0, experts <= 256, topk <= 32.
 * docs/plans/gemma4-26b/specs/MOE_ROUTER_SPEC.md:27-73. */
int32_t gemb_moe_route(const float* logits, const float* per_expert_scale, int32_t* top_ids,
                       float* top_weights, float* probabilities, uint64_t tokens, uint64_t experts,
                       uint64_t topk, gemb_stream_t stream);

/* Sizes for gemb_moe_permute: scratch bytes, int32 entries of `plan`, and the upper bound of
 * padded rows (every expert's rows start on a multiple of 256) that dispatch / grouped GEMM /
 * combine buffers must hold. */
uint64_t gemb_moe_permute_workspace_bytes(uint64_t tokens, uint64_t experts, uint64_t topk);
uint64_t gemb_moe_plan_ints(uint64_t tokens, uint64_t experts, uint64_t topk);
uint64_t gemb_moe_padded_rows_max(uint64_t tokens, uint64_t experts, uint64_t topk);

/* Histogram(experts) -> exclusive prefix(experts + 1) -> stable permutation of the tokens*topk
 * assignments (assignment i = token * topk + slot; inside an expert i ascends).
 *   counts[experts], offsets[experts + 1], perm[tokens * topk] (perm[pos] = i)   -- the spec's
 *   records;  slot_rows[i] = row of assignment i in the padded per-expert row space;
 *   plan = {tiles, padded rows, padded_offsets[experts + 1], tiles x {expert of the tile or -1 for a
 *   tile of padding only, i-th tile that holds real rows}, number of tiles that hold real rows},
 *   consumed on the device by the grouped GEMM (no host readback).  Every expert's rows start on a
 *   multiple of 256, so a 128-row tile and the 256-row tile of a CTA pair never mix experts.
 *   1 <= experts <= 1024, topk <= 32.
 * docs/plans/gemma4-26b/specs/MOE_PREFILL_KERNEL_SPEC.md:19-58. */
int32_t gemb_moe_permute(const int32_t* top_ids, int32_t* counts, int32_t* offsets, int32_t* perm,
                         int32_t* slot_rows, int32_t* plan, void* workspace, uint64_t workspace_bytes,
                         uint64_t tokens, uint64_t experts, uint64_t topk, gemb_stream_t stream);

/* The same operation as gemb_moe_permute for hosts that can neither hand over a workspace nor
 * allocate one: an engine whose single load-time arena has no region to spare, or code inside a
 * section where cudaMalloc is off limits because it would synchronise the device or break a
 * stream capture.  The per-segment counts go to a 128 KiB array that lives inside the library
 * (every GPU that loads the library keeps it until exit).  Limits: tokens * topk <= 131,072
 * and experts <= 256; larger problems are rejected with GEMB_INVALID_ARGUMENT and must use
 * gemb_moe_permute.  The first call on each device looks up the array's device address
 * (cudaGetSymbolAddress, that device current): make that first call outside any stream
 * capture.  No cudaMalloc / cudaFree or allocating library call is made, ever.  All calls
 * share the one array: two calls whose kernels can overlap on the GPU (different streams,
 * no dependency) race on it and corrupt each other's result; calls ordered on one stream are
 * safe, and nothing has to be cleared between them.
 * This entry point has no counterpart in the reference. */
int32_t gemb_moe_permute_static(const int32_t* top_ids, int32_t* counts, int32_t* offsets,
                                int32_t* perm, int32_t* slot_rows, int32_t* plan, uint64_t tokens,
                                uint64_t experts, uint64_t topk, gemb_stream_t stream);

/* NVFP4-quantises each token's expert input once (EXACT contract) and writes payload and
 * INTERLEAVED block scales to the padded row of each of its topk assignments.
 * "activation + W2 input quantization" boundary of MOE_PREFILL_KERNEL_SPEC.md:34-47. */
int32_t gemb_moe_dispatch_quantize(const uint16_t* x_bf16, const int32_t* slot_rows,
                                   uint8_t* packed_e2m1, uint8_t* interleaved_scales,
                                   uint64_t tokens, uint64_t hidden, uint64_t topk,
                                   float global_divisor, gemb_stream_t stream);

/* Expert-parallel plumbing (gem16 has no multi-GPU code; docs/GEMMA4_26B.md:114-117 excludes it,
 * so these have no counterpart there).
 * gather_rows: dst row i = src row index[i] / index_divisor; row_bytes (multiple of 16) are copied,
 * rows are src_row_stride / dst_row_stride bytes apart -- packs quantised tokens in permutation
 * order into the dispatch message (index = perm, divisor = topk; payload and scales of one
 * assignment share a message row) and expert outputs back into arrival order for the combine
 * all-to-all (index = slot rows).
 * scatter_quantized: places already quantised rows (payload and COMPACT scales, both with
 * src_row_stride bytes between rows, as received) at slot_rows[i] of the padded row space and
 * converts their scales to the INTERLEAVED layout. */
int32_t gemb_moe_gather_rows(const void* src, void* dst, const int32_t* index, uint64_t index_divisor,
                             uint64_t rows, uint64_t row_bytes, uint64_t src_row_stride,
                             uint64_t dst_row_stride, gemb_stream_t stream);
int32_t gemb_moe_scatter_quantized(const uint8_t* packed_rows, const uint8_t* compact_scales,
                                   const int32_t* slot_rows, uint8_t* packed_e2m1,
                                   uint8_t* interleaved_scales, uint64_t rows, uint64_t hidden,
                                   uint64_t src_row_stride, gemb_stream_t stream);

/* Grouped expert projection over the padded row space: for every 128-row tile t of the plan,
 * out[rows of t] = bf16( A[rows of t] . W[tile_expert[t]]^T / (ga * w_divisors[expert]) ).
 * A: NVFP4 payload [padded_rows_max, K/2] + INTERLEAVED scales; W: [experts, rows_per_expert, K/2]
 * with each expert's scales INTERLEAVED back to back; w_divisors: fp32 [experts] on the device.
 * Experts with no assignment own no tile and cost nothing; nothing is read back to the host.
 * rows_per_expert % 128 == 0, K % 64 == 0.  "grouped W13 / grouped W2" of
 * docs/plans/gemma4-26b/specs/MOE_PREFILL_KERNEL_SPEC.md:34-66. */
int32_t gemb_moe_grouped_gemm_bf16(const uint8_t* packed_activation_e2m1,
                                   const uint8_t* interleaved_activation_scales,
                                   const uint8_t* packed_weight_e2m1,
                                   const uint8_t* interleaved_weight_scales, uint16_t* output_bf16,
                                   const int32_t* plan, uint64_t padded_rows_max, uint64_t experts,
                                   uint64_t rows_per_expert, uint64_t contracting_elements,
                                   float activation_global_divisor, const float* weight_global_divisors,
                                   gemb_stream_t stream);

/* Grouped form of gemb_nvfp4_gemm_gated_quant: per-expert fused gate/up weights
 * [experts, 2*intermediate, K/2] (each packed with gemb_nvfp4_pack_gate_up), one weight divisor per
 * expert; output = quantised product rows [padded_rows_max, intermediate/2] + INTERLEAVED scales,
 * ready for the grouped down projection.  Fuses "grouped W13 -> activation + W2 input
 * quantization" of docs/plans/gemma4-26b/specs/MOE_PREFILL_KERNEL_SPEC.md:34-47. */
int32_t gemb_moe_grouped_gemm_gated_quant(const uint8_t* packed_activation_e2m1,
                                          const uint8_t* interleaved_activation_scales,
                                          const uint8_t* fused_gate_up_weights,
                                          const uint8_t* fused_interleaved_weight_scales,
                                          uint8_t* product_packed_e2m1,
                                          uint8_t* product_interleaved_scales, const int32_t* plan,
                                          uint64_t padded_rows_max, uint64_t experts,
                                          uint64_t intermediate, uint64_t contracting_elements,
                                          float activation_global_divisor,
                                          const float* weight_global_divisors,
                                          float product_global_divisor, gemb_stream_t stream);

/* Expert activation boundary on the padded rows: gate_up bf16 [rows, 2*intermediate] (gate first),
 * product = bf16(bf16(gelu_tanh(gate)) * up), NVFP4-quantised (EXACT contract) with the down
 * projection's input divisor into payload [rows, intermediate/2] + INTERLEAVED scales.  Only
 * the plan's padded rows are processed (plan may be null: all rows_max rows).
 * Boundaries of src/cuda/nvfp4/reference.cu:177-217; fused gate_up order of
 * tools/capture_gemma4_26b_goldens.py:232-240. */
int32_t gemb_moe_expert_gelu_quantize(const uint16_t* gate_up_bf16, const int32_t* plan,
                                      uint8_t* packed_e2m1, uint8_t* interleaved_scales,
                                      uint64_t rows_max, uint64_t intermediate,
                                      float global_divisor, gemb_stream_t stream);

/* ---- output head (the first row of the path's "next" list: the tied bf16 head of the decode step) ----
 * For each of `rows` (1..8) fp32 hidden vectors [rows, hidden] and every vocabulary row v:
 *   logit[r][v] = tanhf(dot(bf16 W[v, :], hidden[r, :]) / 30) * 30        (fp32 accumulation)
 * Tokens on the suppression list never win; ties go to the lower token id.  The launch writes, per
 * hidden row, gemb_output_head_candidate_blocks() = 4,096 candidates {float value; uint32 token}
 * (candidates[r * 4096 + block]) and, when diagnostic_logits is non-null, every capped logit
 * [rows, vocabulary].  dynamic_suppressed_count, when non-null, is a device word that overrides
 * suppressed_count at run time (the reference reads it from DecodeControl).
 * Replaces LaunchFusedOutputHeadCandidates / LaunchFusedOutputHeadBatchCandidates
 * (src/cuda/output_head.h:19-30, kernels src/cuda/output_head.cu:55-110,113-186) and, with
 * diagnostic_logits, LaunchOutputHeadLogits (output_head.h:40-43).
 * gemb_output_head_argmax reduces the candidates of each row to selected[r]
 * (LaunchOutputHeadCandidateArgmax / LaunchOutputHeadBatchArgmax, output_head.h:32-38). */
/* candidates may be null when only the diagnostic logits are wanted (LaunchOutputHeadLogits).
 * gemb_logit_argmax picks the largest of `vocabulary` materialised logits that is not on the
 * suppression list, the lower token id on ties (LaunchLogitArgmax, output_head.h:44-48). */
uint64_t gemb_output_head_candidate_blocks(void);
int32_t gemb_logit_argmax(const float* logits, const uint32_t* suppressed, uint64_t suppressed_count,
                          uint32_t* selected, uint64_t vocabulary, gemb_stream_t stream);
int32_t gemb_output_head_candidates(const uint16_t* weights_bf16, const float* hidden_rows, uint64_t rows,
                                    const uint32_t* suppressed, uint64_t suppressed_count,
                                    const uint32_t* dynamic_suppressed_count, void* candidates,
                                    float* diagnostic_logits, uint64_t vocabulary, uint64_t hidden,
                                    gemb_stream_t stream);
int32_t gemb_output_head_argmax(const void* candidates, uint64_t rows, uint32_t* selected,
                                gemb_stream_t stream);

/* ---- expert parallelism over peer memory (no counterpart in the reference, which is single-GPU) ----
 * R ranks, E experts, rank r owns experts [r*E/R, (r+1)*E/R).  Every rank leaves its quantised
 * assignments, one message row each (payload | compact block scales, padded to 16 bytes) in
 * (expert, token, slot) order, in a buffer its peers have mapped; counts_all [R][E] holds every
 * rank's per-expert counts (all-gathered by the caller, which also orders the kernels below after
 * the peers' writes).  All row positions follow from counts_all; nothing is read back to the host.
 *
 * gemb_moe_ep_plan (one small launch) writes, for rank `rank`:
 *   plan              the grouped-GEMM plan of its local experts over the rows of ALL ranks
 *                     (layout of gemb_moe_permute's plan; gemb_moe_ep_plan_ints integers),
 *   recv_prefix       [R*E/R + 1] exclusive prefix of the segments (source, local expert) it receives,
 *   recv_src_rows     [R*E/R] first row of each segment in the source's send buffer,
 *   recv_dst_rows     [R*E/R] first row of each segment in its padded row space,
 *   combine_row_base  [E] for an assignment of ITS OWN tokens to expert e whose local slot row
 *                     (gemb_moe_permute's slot_rows) is p: the row of the result in the owner's
 *                     output buffer is combine_row_base[e] + p.
 * gemb_moe_ep_pull_dispatch reads the segments out of the peers' send buffers (peer_send_buffers_host:
 * R device addresses, host array) into payload [rows, hidden/2] + INTERLEAVED scales.
 * gemb_moe_ep_pull_combine is gemb_moe_combine with every expert row read from its owner's output
 * buffer (peer_expert_outputs_host: R device addresses of bf16 [rows, hidden]).
 * send_rows_per_rank / padded_rows_max (capacity_rows for the plan) are the capacities of the send
 * and of the padded buffers.  Counts that are not what the protocol promises (negative, more rows
 * than a rank can send, more padded rows than the capacity -- e.g. read after a barrier gave up)
 * make gemb_moe_ep_plan write an EMPTY plan and record the fact; a single position outside a
 * buffer is skipped and recorded by the pull kernels; gemb_check_device_status() then reports it,
 * instead of an access faulting. */
/* Ordering between the GPUs without a collective library.  gemb_moe_ep_barrier: rank `rank` bumps
 * its device-resident epoch for barrier `which` (0 or 1; local_epochs holds two words, zero at
 * start), stores it to slot [which][rank] of every rank's flag array (peer_flag_arrays_host: R device
 * addresses of 2 x 16 zero-initialised words) and waits, for a bounded time, until every slot of its
 * own array has reached the epoch.  Everything earlier in the stream is then visible to peers that
 * pass their own barrier.  Each rank must run on its own GPU.  gemb_moe_ep_gather_counts copies
 * every rank's per-expert counts (peer_count_buffers_host: R device addresses of E int32) into
 * counts_all [R][E] -- the input of gemb_moe_ep_plan -- after such a barrier. */
int32_t gemb_moe_ep_barrier(const uint64_t* peer_flag_arrays_host, uint64_t ranks, uint64_t rank, uint64_t which,
                            uint32_t* local_epochs, gemb_stream_t stream);
int32_t gemb_moe_ep_gather_counts(const uint64_t* peer_count_buffers_host, uint64_t ranks, uint64_t experts,
                                  int32_t* counts_all, gemb_stream_t stream);
uint64_t gemb_moe_ep_plan_ints(uint64_t capacity_rows, uint64_t local_experts);
int32_t gemb_moe_ep_plan(const int32_t* counts_all, uint64_t ranks, uint64_t experts, uint64_t rank,
                         int32_t* plan, int32_t* recv_prefix, int32_t* recv_src_rows,
                         int32_t* recv_dst_rows, int32_t* combine_row_base, uint64_t capacity_rows,
                         uint64_t send_rows_per_rank, gemb_stream_t stream);
int32_t gemb_moe_ep_pull_dispatch(const uint64_t* peer_send_buffers_host, uint64_t ranks,
                                  uint64_t local_experts, const int32_t* recv_prefix,
                                  const int32_t* recv_src_rows, const int32_t* recv_dst_rows,
                                  uint8_t* packed_e2m1, uint8_t* interleaved_scales, uint64_t hidden,
                                  uint64_t message_row_bytes, uint64_t send_rows_per_rank,
                                  uint64_t padded_rows_max, gemb_stream_t stream);
int32_t gemb_moe_ep_pull_combine(const uint64_t* peer_expert_outputs_host, uint64_t ranks,
                                 uint64_t local_experts, const int32_t* top_ids,
                                 const int32_t* slot_rows, const int32_t* combine_row_base,
                                 const float* top_weights, const uint16_t* shared_bf16,
                                 uint16_t* out_bf16, uint64_t tokens, uint64_t hidden, uint64_t topk,
                                 uint64_t padded_rows_max, gemb_stream_t stream);

/* Tensor-parallel reduction of a K-split projection over peer memory (no counterpart in the
 * reference).  peer_partials_host: R device addresses of fp32 partial results [tokens, hidden]
 * (gemb_nvfp4_gemm_f32 on each rank's K slice).  gemb_tp_reduce_rows sums, for the token rows rank
 * `rank` owns ([rank*T/R, (rank+1)*T/R)), the partials of all ranks in rank order, rounds once to
 * bf16 and writes those rows of out_bf16 [tokens, hidden]; gemb_tp_gather_rows then copies every
 * other rank's rows from its out buffer (peer_outputs_host).  The caller separates the GEMM, the
 * reduce and the gather with gemb_moe_ep_barrier (or any other barrier between the GPUs). */
int32_t gemb_tp_reduce_rows(const uint64_t* peer_partials_host, uint64_t ranks, uint64_t rank, uint64_t tokens,
                            uint64_t hidden, uint16_t* out_bf16, gemb_stream_t stream);
int32_t gemb_tp_gather_rows(const uint64_t* peer_outputs_host, uint64_t ranks, uint64_t rank, uint64_t tokens,
                            uint64_t hidden, uint16_t* out_bf16, gemb_stream_t stream);

/* out[t] = bf16( sum over slots in slot order of fma(weight[t][slot], y[slot_rows[t*topk+slot]])
 *                + shared[t] ), fp32 accumulation, no atomics; shared may be null; slot_rows may be
 * null when y already holds the rows in assignment order (row t*topk+slot).
 * docs/plans/gemma4-26b/specs/MOE_SEMANTICS_SPEC.md:74-83. */
int32_t gemb_moe_combine(const uint16_t* y_bf16, const int32_t* slot_rows, const float* top_weights,
                         const uint16_t* shared_bf16, uint16_t* out_bf16, uint64_t tokens,
                         uint64_t hidden, uint64_t topk, gemb_stream_t stream);

/* ------------------------------------------------------------------------------------------
 * Weight descriptors and whole-layer entry points.  The launch sequence, the buffer planning, the
 * fork / join of the shared branch and the expert-parallel protocol live here, in the library, so
 * that a C++ host only fills descriptors, hands over one workspace and makes one call per layer.
 * ---------------------------------------------------------------------------------------- */

/* Mirror gem16::internal::Fp8Binding and Nvfp4Binding (src/cuda/engine/target_model.h:15-30):
 * device pointers into the caller's weight arena plus geometry and divisors.  The NVFP4
 * descriptor keeps the reference's fields and adds what this library's layouts need. */
typedef struct gemb_fp8_binding {
  const uint8_t* weight;                /* [rows, contracting] E4M3FN */
  const uint16_t* scales;               /* [rows] bf16 bits */
  uint64_t rows;
  uint64_t contracting;
} gemb_fp8_binding;

typedef struct gemb_nvfp4_binding {
  const uint8_t* packed_weight;         /* [rows, K/2]; expert stack: [experts, rows, K/2] */
  const uint8_t* scales;                /* COMPACT [rows, K/16] (decode GEMV); may be null where only GEMMs run */
  const float* input_divisor_device;    /* optional device copy of input_divisor, as in the reference */
  float input_divisor;
  float weight_divisor;                 /* plain module; unused for a stack */
  uint64_t rows;
  uint64_t contracting;
  /* beyond the reference's fields */
  const uint8_t* scales_interleaved;    /* 128x4 interleave for the tcgen05 GEMMs; stack: experts back to back */
  const float* weight_divisors_device;  /* expert stack: fp32 [experts] */
  uint64_t experts;                     /* 0 = plain module, else the number of matrices in the stack */
} gemb_nvfp4_binding;

/* Checkpoint loader (load time, host side): opens a safetensors file, validates a module the way
 * gem16's loader does and binds it into the caller's device arena in this library's layouts.
 *   NVFP4 module `m`:  m.weight_packed U8 [rows, K/2] (or [experts, rows, K/2]), m.weight_scale F8_E4M3
 *     [.., rows, K/16], m.weight_global_scale and m.input_global_scale F32 [1] (or [experts]): all four
 *     required, exact dtypes and shapes, no NaN scale byte, positive finite divisors, K % 64 == 0,
 *     rows % 8 == 0  (src/model/manifest.cpp:344-365, src/cuda/engine/target_model.cu:361-388).
 *   FP8 module `m`:  m.weight F8_E4M3 [rows, K], m.weight_scale BF16 [rows, 1]  (manifest.cpp:366-372,
 *     target_model.cu:345-358).
 * rows / contracting_elements, when nonzero, must match the stored geometry (the reference binds with
 * the geometry the model expects).  Failures: GEMB_NOT_FOUND (no such weight tensor), GEMB_DATA_LOSS
 * (schema violations, as the reference reports them), GEMB_IO_ERROR, GEMB_UNSUPPORTED (unknown dtype).
 * The arena piece (gemb_checkpoint_*_bytes, 256-byte aligned) receives, for NVFP4: payload, COMPACT
 * scales, INTERLEAVED scales (per expert, back to back), the weight divisors and the input divisor as
 * device floats; binding->weight_divisor / input_divisor hold the first (or only) values. */
typedef struct gemb_checkpoint gemb_checkpoint;
int32_t gemb_checkpoint_open(const char* path, gemb_checkpoint** checkpoint);
void gemb_checkpoint_close(gemb_checkpoint* checkpoint);
uint64_t gemb_checkpoint_nvfp4_bytes(const gemb_checkpoint* checkpoint, const char* module);
int32_t gemb_checkpoint_bind_nvfp4(const gemb_checkpoint* checkpoint, const char* module, uint64_t rows,
                                   uint64_t contracting_elements, void* device_arena, uint64_t arena_bytes,
                                   gemb_nvfp4_binding* binding, gemb_stream_t stream);
uint64_t gemb_checkpoint_fp8_bytes(const gemb_checkpoint* checkpoint, const char* module);
int32_t gemb_checkpoint_bind_fp8(const gemb_checkpoint* checkpoint, const char* module, uint64_t rows,
                                 uint64_t contracting_elements, void* device_arena, uint64_t arena_bytes,
                                 gemb_fp8_binding* binding, gemb_stream_t stream);

/* One mixture-of-experts layer (26B-A4B shape: router, `experts` gated FFNs of which each token
 * uses `topk`, one shared dense FFN).  gate_up / shared_gate_up hold the fused projection of
 * tools/capture_gemma4_26b_goldens.py:232-240: rows = 2 * intermediate, gate rows first.  When the
 * *_fused pointers are set (weights re-ordered once by gemb_nvfp4_pack_gate_up) the gate/up GEMM,
 * the GELU and the requantisation run as ONE kernel and gate_up.packed_weight / scales_interleaved
 * may be null; otherwise they run as GEMM + gemb_moe_expert_gelu_quantize (byte-identical results).
 * Under expert parallelism the stacks hold this rank's experts only (gate_up.experts = experts / ranks).
 * Router: logits = x . router_weight^T + router_bias, or, when router_input_scale is set, the
 * specification's form  r = bf16(rmsnorm_noweight(x) * router_input_scale * hidden^-1/2),
 * logits = r . router_weight^T  (docs/plans/gemma4-26b/specs/MOE_ROUTER_SPEC.md:3-13); weights are
 * multiplied by per_expert_scale[id] when it is set (:41-63). */
typedef struct gemb_moe_layer_weights {
  uint64_t hidden;
  uint64_t experts;                     /* experts the router scores */
  uint64_t topk;
  uint64_t intermediate;
  uint64_t shared_intermediate;         /* 0 = no shared branch */
  const float* router_weight;           /* fp32 [experts, hidden] */
  const float* router_bias;             /* fp32 [experts] or null */
  const float* per_expert_scale;        /* fp32 [experts] or null */
  const uint16_t* router_input_scale;   /* bf16 [hidden] or null */
  float router_epsilon;                 /* of the router's RMSNorm (with router_input_scale) */
  gemb_nvfp4_binding gate_up;
  gemb_nvfp4_binding down;
  gemb_nvfp4_binding shared_gate_up;
  gemb_nvfp4_binding shared_down;
  const uint8_t* gate_up_fused;
  const uint8_t* gate_up_fused_scales;
  const uint8_t* shared_gate_up_fused;
  const uint8_t* shared_gate_up_fused_scales;
} gemb_moe_layer_weights;

/* Where a layer call leaves its routing records inside the workspace (device pointers), for
 * callers that want to observe them: RoutedExperts and Assignment records of
 * MOE_ROUTER_SPEC.md:65-73 and MOE_PREFILL_KERNEL_SPEC.md:19-32 as arrays. */
typedef struct gemb_moe_records {
  float* logits;            /* [tokens, experts] */
  int32_t* top_ids;         /* [tokens, topk] */
  float* top_weights;       /* [tokens, topk] */
  int32_t* counts;          /* [experts] */
  int32_t* offsets;         /* [experts + 1] */
  int32_t* perm;            /* [tokens * topk] */
  int32_t* slot_rows;       /* [tokens * topk] */
  int32_t* plan;            /* gemb_moe_plan_ints entries */
  uint16_t* expert_rows;    /* bf16 [padded_rows_max, hidden]: the experts' outputs (single-GPU layer only) */
  uint64_t padded_rows_max;
  int32_t* counts_all;      /* expert-parallel layer only: every rank's counts, [ranks, experts] */
} gemb_moe_records;

/* sizeof of the structs above as this build of the library sees them (0 = gemb_fp8_binding,
 * 1 = gemb_nvfp4_binding, 2 = gemb_moe_layer_weights, 3 = gemb_moe_records, 4 = gemb_moe_ep_comm),
 * so a binding in another language can check its own layout. */
uint64_t gemb_struct_bytes(int32_t which);

/* r = bf16( ((x * inv) * scale) * hidden^-1/2 ), inv = 1 / sqrt(sum_k x_k^2 / hidden + epsilon): the
 * router's input transform (MOE_ROUTER_SPEC.md:3-13).  The sum is one fp32 fma per k in ascending
 * k and every other step one IEEE operation, so r is reproducible bit for bit. */
int32_t gemb_moe_router_input(const uint16_t* x_bf16, const uint16_t* scale_bf16, uint16_t* out_bf16,
                              uint64_t tokens, uint64_t hidden, float epsilon, gemb_stream_t stream);

/* One layer on one GPU: router -> top-k -> stable permutation -> quantise and dispatch -> grouped
 * gate/up -> GELU + requantisation -> grouped down -> slot-ordered weighted combine + shared branch
 * (stage order of docs/plans/gemma4-26b/specs/MOE_PREFILL_KERNEL_SPEC.md:34-47; the entry point the
 * plan reserves as gem16::internal::LaunchMoe* under src/cuda/moe/, milestones M11 and M15).
 * x and out are bf16 [tokens, hidden].  The workspace (gemb_moe_layer_workspace_bytes, 256-byte
 * aligned) needs no initialisation and keeps the records of the last call.  Stream-ordered, no
 * allocation, no host synchronisation, capturable.  When side_stream, fork_event and join_event
 * (cudaEvent_t created by the caller, timing disabled) are all set and the batch holds at most 1,024
 * tokens, the shared branch runs on side_stream beside routing and the expert GEMMs and joins before
 * the combine; otherwise everything runs on `stream` (from about a thousand tokens on every kernel of
 * the layer fills the GPU, and two streams of persistent GEMMs only take turns).  Same results either way. */
uint64_t gemb_moe_layer_workspace_bytes(const gemb_moe_layer_weights* weights, uint64_t tokens);
int32_t gemb_moe_layer_records(const gemb_moe_layer_weights* weights, uint64_t tokens, void* workspace,
                               gemb_moe_records* records);
int32_t gemb_moe_layer_forward(const gemb_moe_layer_weights* weights, const uint16_t* x_bf16,
                               uint16_t* out_bf16, uint64_t tokens, void* workspace,
                               uint64_t workspace_bytes, gemb_stream_t stream, gemb_stream_t side_stream,
                               void* fork_event, void* join_event);

/* ---- one expert-parallel layer (no counterpart in the reference, which is single-GPU) ----
 * R ranks, one per GPU; rank r holds experts [r*E/R, (r+1)*E/R) (weights->gate_up.experts = E/R) and
 * `tokens` tokens of its own; the router is replicated.  Four buffers per rank must be mapped by
 * every rank (peer memory); `comm` carries, per buffer kind, the R device addresses as seen from
 * THIS rank (host arrays), entry [rank] being the rank's own buffer:
 *   send_buffers   message rows IN: R regions (one per source rank) of tokens * topk rows of
 *                  gemb_moe_ep_message_row_bytes(hidden) bytes each
 *   recv_buffers   tokens * topk expert output rows, bf16 [tokens * topk, hidden]
 *   count_buffers  int32 [experts]
 *   flag_arrays    2 x 16 words, zero before the first call
 * plus local_epochs: two device words of this rank, zero before the first call.
 * Per layer and rank: route the local tokens; quantise each token once and push one message row
 * per assignment (payload | block scales | assignment index) into the owner's message buffer, at
 * the row's position in this rank's (expert, token, slot) order inside this rank's region there;
 * flag barrier 0; read all ranks' counts and derive every row position from them; gather the rows
 * of the local experts out of the regions of the own message buffer into the grouped GEMM's padded
 * row space; grouped gate/up (+ GELU + requantisation)
 * and grouped down GEMM, whose epilogue stores each finished bf16 row straight into the recv
 * buffer of the token's owner (plain 16-byte stores to peer memory, overlapped with the MMAs);
 * flag barrier 1; slot-ordered combine from the local recv buffer plus the shared branch.
 * Output, ids, weights and counts equal the single-GPU layer's bit for bit.  Nothing is read back
 * to the host; the call is capturable, replays included (barrier epochs live on the device).
 * A barrier that gives up (a peer that never arrives) is recorded for gemb_check_device_status and
 * the layer then runs on an empty plan: no access leaves the buffers.  Every rank must call with
 * the same geometry, each on its own GPU. */
typedef struct gemb_moe_ep_comm {
  uint64_t ranks;
  uint64_t rank;
  const uint64_t* send_buffers_host;
  const uint64_t* recv_buffers_host;
  const uint64_t* count_buffers_host;
  const uint64_t* flag_arrays_host;
  uint32_t* local_epochs;
} gemb_moe_ep_comm;
uint64_t gemb_moe_ep_message_row_bytes(uint64_t hidden);
uint64_t gemb_moe_ep_layer_workspace_bytes(const gemb_moe_layer_weights* weights, uint64_t tokens, uint64_t ranks);
int32_t gemb_moe_ep_layer_records(const gemb_moe_layer_weights* weights, uint64_t tokens, uint64_t ranks,
                                  void* workspace, gemb_moe_records* records);
int32_t gemb_moe_ep_layer_forward(const gemb_moe_layer_weights* weights, const gemb_moe_ep_comm* comm,
                                  const uint16_t* x_bf16, uint16_t* out_bf16, uint64_t tokens, void* workspace,
                                  uint64_t workspace_bytes, gemb_stream_t stream, gemb_stream_t side_stream,
                                  void* fork_event, void* join_event);
/* The stages of gemb_moe_ep_layer_forward, separately callable so that several ranks can be walked
 * through the protocol on ONE GPU (tests; a host-side copy of the counts stands in for barrier 0):
 * stage 0 = route + pack (+ shared branch), 1 = positions + pull + expert GEMMs with the pushing
 * epilogue, 2 = combine.  With barriers = 0 the stages skip the flag barriers and stage 1 reads the
 * counts from the records' counts_all (gemb_moe_ep_layer_records), which the caller fills. */
int32_t gemb_moe_ep_layer_stage(const gemb_moe_layer_weights* weights, const gemb_moe_ep_comm* comm,
                                const uint16_t* x_bf16, uint16_t* out_bf16, uint64_t tokens, void* workspace,
                                uint64_t workspace_bytes, int32_t stage, int32_t barriers, gemb_stream_t stream);

/* Synchronises the device and reports what the kernels recorded since the last call (the record is
 * cleared): a GEMM, GEMV or flag-barrier wait that ran out, an expert-parallel position outside its
 * buffers (GEMB_INTERNAL); a non-finite router logit or an out-of-range expert id, the states
 * MOE_ROUTER_SPEC.md:117-130 wants visible rather than repaired (GEMB_DATA_LOSS); else GEMB_OK.
 * The kernels themselves never fault on such input: they skip or clamp the access.  The reference
 * has no counterpart: its kernels have no device-side waits. */
int32_t gemb_check_device_status(void);

/* ------------------------------------------------------------------------------------------
 * Scalar cross-check projections (one thread per output, fp32 fma in k order).  Slow on
 * purpose; they exist so large shapes can be checked on the GPU.
 * Replace LaunchNvfp4ReferenceProjectionBatch (src/cuda/nvfp4/reference.h:83-94) and
 * LaunchFp8ReferenceProjectionBatch (src/cuda/fp8/reference.h:69-78).
 * ---------------------------------------------------------------------------------------- */
int32_t gemb_nvfp4_reference_projection(const uint8_t* packed_activation_e2m1,
                                        const uint8_t* activation_scales,
                                        const uint8_t* packed_weight_e2m1,
                                        const uint8_t* weight_scales, float* output,
                                        uint64_t tokens, uint64_t rows,
                                        uint64_t contracting_elements,
                                        float activation_global_divisor,
                                        float weight_global_divisor, gemb_stream_t stream);
int32_t gemb_fp8_reference_projection(const uint8_t* activation_e4m3fn,
                                      const float* activation_scales,
                                      const uint8_t* weight_e4m3fn,
                                      const uint16_t* weight_scales_bf16, float* output,
                                      uint64_t tokens, uint64_t rows,
                                      uint64_t contracting_elements, gemb_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* GEMB200_H_ */
