/*
 * lightop_b200 -- C ABI of the B200 (sm_100a) kernels behind the fused
 * block-INT8 (W8A8, 128x128 weight blocks, 128-wide activation groups) MoE path.
 *
 * Conventions
 *   - every pointer is a DEVICE pointer unless the comment says "host";
 *   - `stream` is a cudaStream_t passed as void* (NULL = legacy default stream);
 *   - every function only enqueues work on `stream`: no host synchronisation and
 *     no allocation (scratch memory is passed in by the caller);
 *   - the return value is a status code, 0 on success; lo_last_error() returns
 *     a thread-local, human readable description of the last failure;
 *   - "reference" citations name files of the HYGON-AI/lightop project by their
 *     path inside that project.
 */
#ifndef LIGHTOP_B200_H_
#define LIGHTOP_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LO_OK 0
#define LO_ERR_INVALID_ARGUMENT 1
#define LO_ERR_CUDA 2
#define LO_ERR_UNSUPPORTED 3
#define LO_ERR_DEVICE_TIMEOUT 4

/* element type codes used by the `*_dtype` arguments */
#define LO_F32 0
#define LO_F16 1
#define LO_BF16 2
#define LO_I32 3
#define LO_I64 4
#define LO_U32 5

/* how the routed weight is applied in a grouped-GEMM epilogue */
#define LO_WEIGHT_NONE 0
#define LO_WEIGHT_FP32 1      /* acc_fp32 * w, then one rounding (reference Triton kernel, int8.py:521-530) */
#define LO_WEIGHT_BF16_PRODUCT 2 /* round(acc) * round(w), rounded again (reference torch model, benchmark_moe_int8.py:199-201) */

int lo_version(void);
const char *lo_last_error(void);

/* Number of SMs of the current device (grid sizing is done inside the library;
 * exported for the benchmark's reporting). */
int lo_sm_count(void);
/* Kernels this library has launched since it was loaded (all threads, all devices). */
long long lo_launch_count(void);

/*
 * Softmax over experts + top-k selection (+ optional renormalisation).
 * Replaces: topk_softmax, csrc/kernels/softmax/topk_softmax_kernels.cu:1716
 *           (pybind export csrc/pybind/export.cpp:546,1437).
 * gating [M,E] (LO_F32 / LO_F16 / LO_BF16, row-major), topk_weights [M,k] f32,
 * topk_ids [M,k] (LO_I32 / LO_U32 / LO_I64), token_expert_indices [M,k] i32
 * (= slot*M + token; may be NULL).  Ids come out in descending score order,
 * ties go to the lower expert id.  E <= 1024, k <= 32.
 */
int lo_topk_softmax(const void *gating, int gating_dtype, int64_t M, int E, int k, int renormalize,
                    float *topk_weights, void *topk_ids, int ids_dtype,
                    int32_t *token_expert_indices, void *stream);

/*
 * Expert-major stable ordering of the flat (token, slot) indices, each expert's
 * segment padded to block_size with the sentinel `numel`.
 * Replaces: moe_align_block_size, csrc/kernels/moe_align_sum_kernels.cu:1210
 *           (wrapper python/lightop/_lmslim_native/vllm_compat/moe_align_block_size.py:17).
 * topk_ids: `numel` ids (LO_I32 / LO_I64).  expert_map (i32 [num_experts]) may be NULL.
 *   map_mode 0: ignore expert_map;
 *   map_mode 1: ids are mapped through expert_map before counting and ids mapping
 *               to -1 are dropped (the wrapper's ignore_invalid_experts=True);
 *   map_mode 2: counting uses the unmapped ids and expert_ids[] is written as
 *               expert_map[expert] (the wrapper's default with an expert_map).
 * sorted_ids capacity >= numel + num_experts*(block_size-1) (or numel*block_size when
 * numel < num_experts); every slot up to the capacity is written (sentinel fill).
 * expert_ids: one entry per block up to its capacity; blocks past the padded total get -1.
 * num_tokens_post_pad: i32[1], stays on the device.
 * Within an expert the flat indices are ascending (deterministic), which is the order of
 * the reference's Python model (test/test_moe_align_block_size.py:79-87).
 */
int lo_moe_align_block_size(const void *topk_ids, int ids_dtype, int64_t numel, int num_experts,
                            int block_size, const int32_t *expert_map, int map_mode,
                            int32_t *sorted_ids, int64_t sorted_capacity,
                            int32_t *expert_ids, int64_t expert_ids_capacity,
                            int32_t *num_tokens_post_pad, void *stream);

/*
 * Per-token-group symmetric INT8 quantisation: per `group_size` consecutive
 * elements amax -> scale = amax/127 -> q = trunc(clamp(x / scale, -128, 127)).
 * Replaces: per_token_group_quant_int8,
 *           python/lightop/_lmslim_native/layers/gemm/int8_utils.py:125 (Triton kernel :74-122).
 * x: num_groups*group_size contiguous elements (LO_BF16 / LO_F16 / LO_F32);
 * q: int8 same count; s: f32 [num_groups].  group_size in {64,128,256}.
 * eps is rounded to the input type before the clamp, as the reference's torch model does
 * (test/moe_w8a8/benchmark_moe_int8.py:76).
 */
int lo_group_quant_int8(const void *x, int x_dtype, int64_t num_groups, int group_size, float eps,
                        int8_t *q, float *s, void *stream);

/*
 * out[t,:] = factor * sum_j in[t,j,:] (+ bias[t,:]), fp32 accumulation, one rounding.
 * Replaces: moe_sum, csrc/kernels/moe_align_sum_kernels.cu:1315 (kernels :604-760),
 *           python/lightop/moe_align_sum.py:12-29.
 * in [M,topk,H], out [M,H], bias [M,H] or NULL, all of `dtype` (LO_BF16 / LO_F16 / LO_F32).
 * expert_mask: optional uint8/bool [M,topk]; slot j is skipped where it is 0.
 * num_local_tokens: optional i32[1]; tokens >= that count are left untouched.
 * H must be a multiple of 8.
 */
int lo_moe_sum(const void *in, void *out, const void *bias, int dtype, int64_t M, int topk, int64_t H,
               float factor, const uint8_t *expert_mask, const int32_t *num_local_tokens, void *stream);

/*
 * Grouped block-INT8 GEMM over expert-sorted row blocks (unfused form):
 *   C[id, n] = sum_kb (A_q[id / top_k, kb] . B_q[e, n, kb]) * a_s[id / top_k, kb] * b_s[e, n/128, kb]
 * for every id in sorted_ids below `numel_valid`, e = expert_ids[block of id].
 * Replaces: fused_moe_kernel / invoke_fused_moe_kernel_int8,
 *           python/lightop/_lmslim_native/layers/fused_moe/int8.py:320-626, and the
 *           block-scale form of moe_gemm_w8a8, python/lightop/gemmopt.py:437-457.
 * A [rows_a,K] int8, a_scale [rows_a,K/128] f32, B [E,N,K] int8 contiguous,
 * b_scale [E,N/128,K/128] f32, C [numel_valid, N] bf16, topk_weights flat f32 [numel_valid] or NULL.
 * N and K multiples of 128; block_size <= 128 or a multiple of 128.
 * Blocks whose expert id is negative produce zero rows (int8.py:441-449).
 * workspace: lo_grouped_gemm_workspace_bytes(sorted_capacity, block_size, K) bytes of scratch, 256-byte aligned
 * (the block table and a copy of the activation rows in sorted order, which the kernel reads by TMA).
 */
size_t lo_grouped_gemm_workspace_bytes(int64_t sorted_capacity, int block_size, int64_t K);
int lo_moe_grouped_gemm_i8_block(const int8_t *A, const float *a_scale, int64_t rows_a,
                                 const int8_t *B, const float *b_scale, int E, int64_t N, int64_t K,
                                 void *C, const float *topk_weights, int weight_mode,
                                 const int32_t *sorted_ids, int64_t sorted_capacity,
                                 const int32_t *expert_ids, const int32_t *num_tokens_post_pad,
                                 int64_t numel_valid, int top_k, int block_size,
                                 void *workspace, size_t workspace_bytes, void *stream);

/*
 * The whole fused layer for one chunk of tokens: group-quantise x, sort by expert,
 * gate_up grouped GEMM with SiLU*mul + re-quantisation in its epilogue, down grouped
 * GEMM with the routed weight in its epilogue, top-k reduction.
 * Replaces: fused_experts_impl_int8 with use_int8_w8a8=True, block_shape=[128,128],
 *           python/lightop/_lmslim_native/layers/fused_moe/int8.py:628-908 (one chunk).
 * x [M,H] bf16; w1 [E,2I,H] int8; w2 [E,H,I] int8; w1_scale [E,2I/128,H/128] f32;
 * w2_scale [E,H/128,I/128] f32; topk_weights [M,topk] f32; topk_ids [M,topk] (LO_I32/LO_I64);
 * expert_map i32 [global_num_experts] or NULL (ids mapping to -1 contribute nothing);
 * cache3 [M,topk,H] bf16 scratch (the caller's cache13); shared_output [M,H] bf16 or NULL;
 * out [M,H] bf16 = routed_scaling_factor * sum_j w_j * expert_j(x) (+ shared_output).
 * apply_router_weight_on_input != 0 multiplies the gate_up result instead (requires topk == 1).
 * workspace: lo_fused_moe_workspace_bytes(...) bytes, 256-byte aligned.
 * status: optional i32[1] device word, set non-zero by a kernel whose bounded wait ran out.
 */
size_t lo_fused_moe_workspace_bytes(int64_t M, int E_local, int global_num_experts, int topk,
                                    int64_t H, int64_t I);
/* Byte offsets of the intermediates inside that workspace, for inspection and tests (host array out8):
 * [0] header i32 {num_tokens_post_pad, num_chunks}, [1] x_q int8 [cap,H] and [2] x_s f32 [cap,H/128]
 * (stage-1 quantisation, one row per sorted position), [3] sorted_ids i32 [cap], [4] chunk table,
 * [5] act_q int8 [cap,I] and [6] act_s f32 [cap,I/128] (stage-2 quantisation, sorted order),
 * [7] = cap, the number of sorted positions (not a byte offset).
 * No counterpart in the reference, whose intermediates are torch tensors (int8.py:681-695). */
int lo_fused_moe_workspace_layout(int64_t M, int E_local, int global_num_experts, int topk,
                                  int64_t H, int64_t I, int64_t *out8);
int lo_fused_moe_block_int8(const void *x, const int8_t *w1, const int8_t *w2,
                            const float *w1_scale, const float *w2_scale,
                            const float *topk_weights, const void *topk_ids, int ids_dtype,
                            const int32_t *expert_map, int global_num_experts,
                            int64_t M, int E_local, int topk, int64_t H, int64_t I,
                            void *cache3, const void *shared_output, void *out,
                            int apply_router_weight_on_input, float routed_scaling_factor,
                            void *workspace, size_t workspace_bytes, int32_t *status, void *stream);

/*
 * lo_fused_moe_block_int8 for callers that can neither allocate device memory nor are given any:
 * for example a latency-critical serving thread (cudaMalloc synchronises the whole device), a plugin
 * that only receives raw pointers from a runtime owning the allocator, or a cgo / JNI / Rust FFI
 * binding without an allocator handle.  It has no counterpart in the reference, whose Python layer
 * always allocates its intermediates with torch (int8.py:681-695).
 * Same arguments and results as lo_fused_moe_block_int8, minus the workspace: the scratch is a fixed
 * array of LO_NOALLOC_SCRATCH_BYTES inside the library image, reserved on every GPU that loads the
 * library until the process exits.  Limit: lo_fused_moe_workspace_bytes(M, E_local, global_num_experts,
 * topk, H, I) must not exceed LO_NOALLOC_SCRATCH_BYTES (64 MiB: the DeepSeek-V3 shape with top_k 8 and
 * 256 experts fits up to 402 tokens per call; lo_fused_moe_workspace_bytes gives the need of any shape); larger
 * shapes are rejected with LO_ERR_INVALID_ARGUMENT.
 * The first call on a device looks up the array's device address (cudaGetSymbolAddress, with that device
 * current); make that first call outside any stream capture.  The function calls no cudaMalloc / cudaFree
 * and no allocating library.  All calls on a device share the one array and leave their intermediates
 * in it: nothing needs clearing between calls, but two calls whose kernels overlap on the GPU (different
 * streams, or a concurrent call from another host thread) race on it -- serialise them.
 */
#define LO_NOALLOC_SCRATCH_BYTES (64u << 20)
int lo_fused_moe_block_int8_noalloc(const void *x, const int8_t *w1, const int8_t *w2,
                                    const float *w1_scale, const float *w2_scale,
                                    const float *topk_weights, const void *topk_ids, int ids_dtype,
                                    const int32_t *expert_map, int global_num_experts,
                                    int64_t M, int E_local, int topk, int64_t H, int64_t I,
                                    void *cache3, const void *shared_output, void *out,
                                    int apply_router_weight_on_input, float routed_scaling_factor,
                                    int32_t *status, void *stream);

/*
 * Expert side of expert parallelism: run gate_up -> SiLU*mul -> re-quantise -> down on rows that arrive
 * already group-quantised from other ranks.  xq [T,H] int8, xs [T,H/128] f32, row_expert i32 [T] (local
 * expert of the row; rows with an id outside [0,E_local) are skipped and their output row is left
 * untouched), row_weight f32 [T] or NULL (routed weight, applied as bf16(acc)*bf16(w)), out [T,H] bf16.
 * workspace: lo_fused_moe_workspace_bytes(T, E_local, E_local, 1, H, I) bytes.
 * The reference has no such entry point: its EP support stops at the local permutation kernels
 * (csrc/kernels/deepgemm_moe_permute.cu) and leaves the exchange and the expert-side driver to the
 * serving framework (test/test_ep_gather_scatter_moe.py:205-296 shows the intended sequence).
 */
int lo_expert_rows_block_int8(const int8_t *xq, const float *xs, const int32_t *row_expert,
                              const float *row_weight, const int8_t *w1, const int8_t *w2,
                              const float *w1_scale, const float *w2_scale, int64_t T, int E_local,
                              int64_t H, int64_t I, void *out, void *workspace, size_t workspace_bytes,
                              int32_t *status, void *stream);

/*
 * The same on records as lo_ep_dispatch_pack writes them (packed [T, lo_ep_dispatch_row_bytes(H)] u8, as received
 * from the other ranks): expert id and routed weight are read from the records, rows and scales are gathered from
 * them into expert order.  workspace: lo_expert_rows_packed_workspace_bytes(T, E_local, H, I) bytes.  No counterpart
 * in the reference (see lo_expert_rows_block_int8).
 */
size_t lo_expert_rows_packed_workspace_bytes(int64_t T, int E_local, int64_t H, int64_t I);
int lo_expert_rows_block_int8_packed(const uint8_t *packed, int64_t T, const int8_t *w1, const int8_t *w2,
                                     const float *w1_scale, const float *w2_scale, int E_local, int64_t H, int64_t I,
                                     void *out, void *workspace, size_t workspace_bytes, int32_t *status, void *stream);

/*
 * The same, with every output row stored at an address of its own instead of into one matrix: the received records
 * form `world` runs (source rank s sent records seg_first[s] .. seg_first[s + 1] - 1; seg_first has world + 1
 * entries, device memory) and record r of run s is written, as H bf16, to seg_ret[s] + (r - seg_first[s]) * 2H
 * (seg_ret: world device-side addresses in this process's address space, local memory or a mapping of a peer's
 * buffer from lo_peer_open; 0 = drop the run).  The down GEMM's epilogue stores the rows with plain 16-byte
 * stores, so the combine step of expert parallelism needs no collective, only a barrier after the kernel.
 * workspace: lo_expert_rows_packed_workspace_bytes.  No counterpart in the reference.
 */
int lo_expert_rows_block_int8_packed_put(const uint8_t *packed, int64_t T, const int8_t *w1, const int8_t *w2,
                                         const float *w1_scale, const float *w2_scale, int E_local, int64_t H,
                                         int64_t I, const int32_t *seg_first, const int64_t *seg_ret, int world,
                                         void *workspace, size_t workspace_bytes, int32_t *status, void *stream);

/*
 * Dense block-INT8 linear: C[m, n] = sum_kb (A_q[m, kb] . B_q[n, kb]) * a_s[m, kb] * b_s[n/128, kb], bf16 out.
 * Replaces: the dense block-INT8 matmul of the reference -- matmul_block_int8 / apply_w8a8_block_int8_linear
 *           (python/lightop/_lmslim_native/layers/gemm/int8_utils.py:298-429) and gemm_w8a8_asm
 *           (python/lightop/gemmopt.py:633-639, csrc/asm/asm_gemm_w8a8.cu:136-147).
 * A [M,K] int8, a_scale [M,K/128] f32 (row-major), B [N,K] int8, b_scale [ceil(N/128), K/128] f32, C [M,N] bf16.
 * K a multiple of 128; N arbitrary (weight rows past N read as zero and are not stored).
 * Same kernel as the grouped GEMM with one expert.  workspace: lo_block_int8_linear_workspace_bytes(M).
 */
size_t lo_block_int8_linear_workspace_bytes(int64_t M);
int lo_block_int8_linear(const int8_t *A, const float *a_scale, const int8_t *B, const float *b_scale,
                         int64_t M, int64_t N, int64_t K, void *C, void *workspace, size_t workspace_bytes,
                         int32_t *status, void *stream);

/* ---------------------------------------------------------------------------
 * Routers upstream of the expert layer other than plain softmax top-k.
 * ------------------------------------------------------------------------- */

/*
 * Grouped, bias-corrected sigmoid gate (DeepSeek-V3 style).  Per token: p = sigmoid(x) in fp32, selection
 * score s = p + bias; the score of an expert group (E / num_expert_group consecutive experts) is the sum of its
 * two largest s; the topk_group best groups stay; among their experts the (topk - n_share_experts_fusion)
 * largest s are taken in descending order (ties: lower id); weight = p / sum(p of the taken) times
 * routed_scaling_factor when apply_routed_scaling_factor_on_output (and the factor is > 0).  The fused shared
 * experts fill the remaining slots with ids E, E+1, ... and weight (1 / routed_scaling_factor) times the same
 * output factor.  x [M,E] f32/f16/bf16, bias [E] f32/f16/bf16, topk_weights [M,topk] f32, topk_ids [M,topk]
 * LO_I32 or LO_I64.  E <= 1024, num_expert_group <= 32, topk <= 32; any configuration that satisfies the
 * reference's argument rules is accepted (its kernels cover a fixed table of layouts only).
 * Replaces: op.moe_fused_gate, csrc/kernels/moe_gate/moe_fused_gate.cu:1331-1420 (python/lightop/moe_fused_gate.py:10-31).
 */
int lo_moe_fused_gate(const void *x, int x_dtype, const void *bias, int bias_dtype, int64_t M, int E,
                      int num_expert_group, int topk_group, int topk, int n_share_experts_fusion,
                      float routed_scaling_factor, int apply_routed_scaling_factor_on_output,
                      float *topk_weights, void *topk_ids, int ids_dtype, void *stream);

/*
 * The general form of the gate above, which also covers the reference's ungrouped variants:
 *   score p = sigmoid(x) (LO_GATE_SIGMOID) or sqrt(log1p(exp(x))) (LO_GATE_SQRT_SOFTPLUS); selection on p + bias with
 *   the group limit (num_expert_group = topk_group = 1 for none); routed weight = p / (renormalize ? sum + norm_eps : 1)
 *   * out_scale; shared-expert slots (ids E + j) carry p = sum / shared_div through the same formula.
 *   bias_row_stride: 0 for one bias [E] shared by all tokens, else the element stride of a per-token bias [M, E].
 *   num_token_non_padded (device scalar, LO_I32 / LO_I64, or NULL): rows at or beyond it get weight 0 and id
 *   padding_id; the count is read on the device, so it may change between replays of a captured graph.
 * Replaces (with the parameters its Python layer derives, lightop_b200/moe/routing.py): op.kimi_k2_moe_fused_gate
 * (csrc/kernels/moe_gate/moe_fused_gate_kimi_k2.cu; model test/ci_tests/test_kimi_k2_moe_fused_gate.py:14-43) and
 * op.moe_fused_gate_sqrtsoftplus (csrc/kernels/moe_gate/moe_fused_gate_sqrtsoftplus.cu; model
 * test/ci_tests/test_moe_fused_gate_sqrtsoftplus.py:9-45), with its padded forms ..._v41_hcu_fused (padding id 0)
 * and ..._v41_hcu_deepep (padding id -1) (csrc/kernels/moe_gate/moe_fused_gate_sqrtsoftplus.cu:205-212, :378-421).
 */
#define LO_GATE_SIGMOID 0
#define LO_GATE_SQRT_SOFTPLUS 1
#define LO_GATE_SQRT_SOFTPLUS_SAFE 2 /* softplus(x) = x beyond 20: the reference's "v41" entry points */
int lo_moe_gate_topk(const void *x, int x_dtype, const void *bias, int bias_dtype, int64_t bias_row_stride,
                     int64_t M, int E,
                     int num_expert_group, int topk_group, int topk, int n_shared, int score_fn,
                     int renormalize, float norm_eps, float out_scale, float shared_div,
                     const void *num_token_non_padded, int num_token_dtype, int padding_id,
                     float *topk_weights, void *topk_ids, int ids_dtype, void *stream);

/*
 * In-place post-processing of top-k ids: ids of tokens at or beyond *num_token_non_padded become -1, the others
 * go through the logical -> physical expert map (ids outside [0, map_size) become -1).  Either pointer may be
 * NULL to skip that step.  topk_ids [M,topk] LO_I32 / LO_I64; the map and the count are LO_I32 / LO_I64 device data.
 * Replaces: op.topk_ids_postprocess, csrc/kernels/topk/topk_ids_postprocess.cu:30-66.
 */
int lo_topk_ids_postprocess(void *topk_ids, int ids_dtype, int64_t M, int64_t topk,
                            const void *logical_to_physical_map, int map_dtype, int64_t map_size,
                            const void *num_token_non_padded, int num_token_dtype, void *stream);

/* ---------------------------------------------------------------------------
 * Per-channel W8A8 mode of the same MoE layer (one scale per token, one per output channel).
 * ------------------------------------------------------------------------- */

/*
 * Per-token (whole-row) INT8 quantisation: absmax = max(max|x|, 1e-10); s[m] = absmax / 127;
 * q = rint(x * (127 / absmax)) (round half to even).  x [M, K] f32 / f16 / bf16, any K >= 1.
 * Replaces: per_token_quant_int8, python/lightop/_lmslim_native/layers/gemm/int8_utils.py:21-71
 * (exported as lightop.quant.per_token_quant_int8, python/lightop/quant/int8.py:35).
 */
int lo_per_token_quant_int8(const void *x, int x_dtype, int64_t M, int64_t K, int8_t *q, float *s, void *stream);

/*
 * SiLU(gate) * up and per-token INT8 quantisation of bf16 rows [rows, 2*d] (gate columns first):
 * act = bf16(bf16(silu(gate)) * up); s[row] = max|act| / 127; q = sat(rint(act * (127 / max))); a row of
 * zeros gets scale 0.  q int8 [rows, d], s f32 [rows].
 * Replaces: op.fuse_silu_mul_quant, csrc/kernels/gated_activation/fuse_silu_mul_quant.cu:90-131
 * (python/lightop/fuse_silu_mul_quant.py:44-62), whose reference model is silu_and_mul followed by
 * a dynamic per-token int8 quantisation (test/test_fuse_silu_mul_quant.py:11-14).
 */
int lo_silu_mul_quant_int8(const void *input, int64_t rows, int64_t d, int8_t *q, float *s, void *stream);

/*
 * Grouped per-channel INT8 GEMM over expert-sorted row blocks:
 *   C[id, n] = float(sum_k A_q[id / top_k, k] * B_q[e, n, k]) (* w[id] if LO_WEIGHT_FP32) * a_s[id / top_k] * b_s[e, n]
 * (LO_WEIGHT_BF16_PRODUCT: bf16 of the scaled sum times bf16(w[id])).  a_scale f32 [rows_a], b_scale f32 [E, N];
 * the other arguments and the workspace (lo_grouped_gemm_workspace_bytes) are those of
 * lo_moe_grouped_gemm_i8_block.
 * Replaces: op.moe_gemm_w8a8 (native per-channel MoE GEMM, csrc/moe_gemm/w8a8/moe_w8a8.cu:2389,
 * python/lightop/gemmopt.py:437-457) and the per_channel_quant branch of the Triton fused_moe_kernel
 * (python/lightop/_lmslim_native/layers/fused_moe/int8.py:466-474,509,519-532).
 */
int lo_moe_grouped_gemm_i8_channel(const int8_t *A, const float *a_scale, int64_t rows_a,
                                   const int8_t *B, const float *b_scale, int E, int64_t N, int64_t K,
                                   void *C, const float *topk_weights, int weight_mode,
                                   const int32_t *sorted_ids, int64_t sorted_capacity,
                                   const int32_t *expert_ids, const int32_t *num_tokens_post_pad,
                                   int64_t numel_valid, int top_k, int block_size,
                                   void *workspace, size_t workspace_bytes, void *stream);

/*
 * One chunk of the fused per-channel W8A8 MoE layer: align -> per-token quant -> gate_up GEMM ->
 * SiLU*mul + per-token quant -> down GEMM (routed weight in fp32 before the scales, as the reference's
 * kernel does) -> top-k sum.  w1 int8 [E, 2I, H], w2 int8 [E, H, I], w1_scale f32 [E, 2I], w2_scale f32 [E, H];
 * every other argument as in lo_fused_moe_block_int8 (x_dtype must be LO_BF16).
 * Replaces: fused_experts_impl_int8 with per_channel_quant=True and block_shape=None
 * (python/lightop/_lmslim_native/layers/fused_moe/int8.py:735-905) and fused_experts_impl_int8_marlin
 * (python/lightop/_lmslim_native/layers/fused_moe/int8_marlin.py:165-386; that variant takes weights
 * pre-shuffled for the reference's matrix cores, this one the plain [E, N, K] layout).
 */
size_t lo_fused_moe_channel_workspace_bytes(int64_t M, int E_local, int global_num_experts, int topk,
                                            int64_t H, int64_t I);
int lo_fused_moe_channel_int8(const void *x, int x_dtype, const int8_t *w1, const int8_t *w2,
                              const float *w1_scale, const float *w2_scale,
                              const float *topk_weights, const void *topk_ids, int ids_dtype,
                              const int32_t *expert_map, int global_num_experts,
                              int64_t M, int E_local, int topk, int64_t H, int64_t I,
                              void *cache3, const void *shared_output, void *out,
                              int apply_router_weight_on_input, float routed_scaling_factor,
                              void *workspace, size_t workspace_bytes, int32_t *status, void *stream);

/*
 * fuse_silu_mul_quant on the masked expert-parallel layout: input bf16 [groups, group_rows, 2*d]; only the first
 * tokens_per_group[g] (i32, device) rows of group g are processed, the others are left untouched.
 * q int8 [groups, group_rows, d], s f32 [groups, group_rows].
 * Replaces: op.fuse_silu_mul_quant_ep, csrc/kernels/gated_activation/fuse_silu_mul_quant_ep.cu
 * (python/lightop/fuse_silu_mul_quant.py:235-252).
 */
int lo_silu_mul_quant_int8_masked(const void *input, int64_t groups, int64_t group_rows, int64_t d,
                                  const int32_t *tokens_per_group, int8_t *q, float *s, void *stream);

/*
 * Per-channel grouped INT8 GEMMs on rows that are already grouped by expert (the layouts expert-parallel
 * dispatchers produce): C[m, n] = float(sum_k A_q[m, k] * B_q[e(m), n, k]) * a_s[m] * b_s[e(m), n], bf16 out.
 *   contiguous: A [M, K], m_indices i32 [M] = expert of each row, -1 for padding rows (their output rows are
 *               left untouched).  Layout contract: an expert's rows are consecutive, padding rows come at the end
 *               of its range, and every 128-row block holds rows of one expert (ranges padded to a multiple of
 *               128); a block that breaks the contract is skipped and code 20 is written to *status.
 *   masked:     A [E, max_m, K], masked_m i32 [E] = rows that exist per expert; C [E, max_m, N].
 * a_scale f32 [rows], B int8 [E, N, K] (plain layout), b_scale f32 [E, N].  N and K multiples of 128.
 * workspace: lo_m_grouped_gemm_workspace_bytes(total rows, E) bytes, 256-byte aligned.
 * Replaces: op.m_grouped_w8a8_gemm_nt_contig_asm (python/lightop/gemmopt.py:744-751) and
 * op.m_grouped_marlin_w8a8_gemm_nt_masked_asm (python/lightop/gemmopt.py:604-617), which take weights
 * pre-shuffled for the reference's matrix cores; reference models test/w8a8/test_w8a8_deepgemm_contig.py:106-147
 * and test/deepgemm/w8a8_moe_groupgemm_mask_marlin_correctness.py:40-57.
 */
size_t lo_m_grouped_gemm_workspace_bytes(int64_t total_rows, int num_groups);
int lo_m_grouped_w8a8_gemm_nt_contig(const int8_t *A, const float *a_scale, const int8_t *B, const float *b_scale,
                                     void *C, const int32_t *m_indices, int64_t M, int E, int64_t N, int64_t K,
                                     void *workspace, size_t workspace_bytes, int32_t *status, void *stream);
int lo_m_grouped_w8a8_gemm_nt_masked(const int8_t *A, const float *a_scale, const int8_t *B, const float *b_scale,
                                     void *C, const int32_t *masked_m, int E, int64_t max_m, int64_t N, int64_t K,
                                     void *workspace, size_t workspace_bytes, int32_t *status, void *stream);

/*
 * Per-stage timing of lo_fused_moe_block_int8 for benchmarks: while enabled (per host thread), the
 * call records CUDA events between its five kernels (align, group quant, gate_up GEMM, down GEMM,
 * top-k sum); lo_profile_read waits for the last one and returns the five durations in
 * milliseconds (host array).  No counterpart in the reference, which times with
 * triton.testing.do_bench around the whole call (test/moe_w8a8/moe_benchmark.py:918-932).
 */
int lo_profile_enable(int on);
int lo_profile_read(float *ms5);

/*
 * Expert-parallel local permutation: copy every (token, slot) whose expert is local into the
 * expert-contiguous, `alignment`-padded layout; record where it went.
 * Replaces: ep_scatter, csrc/kernels/deepgemm_moe_permute.cu:1080 (export.cpp:611,1765).
 * aq [T,H] int8; aq_scale [T,S] f32 (S = 1 as in the reference, or H/128 group scales);
 * topk_ids [T,k] (LO_I32/LO_I64); expert_map i32 or NULL; expert_num_tokens i32 [local_E] (in: counts);
 * aq_out [rows,H]; aq_scale_out [rows,S]; m_indices i32 [rows] (expert of the row, -1 padding);
 * inv_perm i32 [T,k] (destination row, -1 if not local).  Placement is stable (ascending flat index).
 */
int lo_ep_scatter(const int8_t *aq, const float *aq_scale, int scale_cols,
                  const void *topk_ids, int ids_dtype, const int32_t *expert_map,
                  const int32_t *expert_num_tokens, int8_t *aq_out, float *aq_scale_out,
                  int32_t *m_indices, int32_t *inv_perm, int64_t T, int k, int64_t H, int64_t rows,
                  int local_num_experts, int alignment, void *stream);

/*
 * Dispatch payload of expert parallelism across ranks: one record per routed (token, slot), records grouped by
 * destination rank in stable order, so that ONE all-to-all carries everything the expert side needs.
 * Record (lo_ep_dispatch_row_bytes(H) bytes, a multiple of 16): int8 row [H] | group scales f32 [H/128] |
 * i32 expert id on the destination rank | f32 routed weight | padding.
 * aq [T,H] int8, aq_scale [T,H/128] f32, topk_ids [T,k] (LO_I32/LO_I64), topk_weights f32 [T,k],
 * rank_of_expert i32 [global experts]; packed [T*k, record] u8, dest_rank i32 [T*k] (rank of every record),
 * inv_perm i32 [T,k] (record of every slot), counts i32 [world] (records per destination rank, on the device).
 * The reference has no counterpart: its expert-parallel kernels (csrc/kernels/deepgemm_moe_permute.cu:1080-1188)
 * permute rows on one device and leave the exchange to the serving framework.
 */
int64_t lo_ep_dispatch_row_bytes(int64_t H);
int lo_ep_dispatch_pack(const int8_t *aq, const float *aq_scale, const void *topk_ids, int ids_dtype,
                        const float *topk_weights, const int32_t *rank_of_expert, int64_t T, int k, int64_t H,
                        int experts_per_rank, int world, uint8_t *packed, int32_t *dest_rank, int32_t *inv_perm,
                        int32_t *counts, void *stream);

/*
 * The two halves of lo_ep_dispatch_pack for a dispatch without a collective.  lo_ep_dispatch_plan computes only the
 * bookkeeping (dest_rank, inv_perm, counts as above).  Once the ranks have exchanged their counts,
 * lo_ep_dispatch_put writes the record of every (token, slot) straight to its destination: seg_first[d] is the
 * packed position of this rank's first record for rank d and seg_dst[d] the address where that record belongs in
 * rank d's receive buffer (both device arrays of `world` entries; addresses in this process's address space, from
 * lo_peer_open for the other ranks; 0 = send nothing to d).  Plain stores only.  No counterpart in the reference.
 */
int lo_ep_dispatch_plan(const void *topk_ids, int ids_dtype, const int32_t *rank_of_expert, int64_t T, int k,
                        int world, int32_t *dest_rank, int32_t *inv_perm, int32_t *counts, void *stream);
int lo_ep_dispatch_put(const int8_t *aq, const float *aq_scale, const void *topk_ids, int ids_dtype,
                       const float *topk_weights, const int32_t *rank_of_expert, const int32_t *inv_perm,
                       int64_t T, int k, int64_t H, int experts_per_rank, int world, const int32_t *seg_first,
                       const int64_t *seg_dst, void *stream);

/*
 * Device buffers that other processes of the node may write (the landing zones of the two calls above).
 * lo_peer_alloc: a device allocation of its own on the current device.  lo_peer_export: its inter-process handle
 * (lo_peer_handle_bytes() bytes, to be sent to the other ranks by any means).  lo_peer_open: maps a handle received
 * from another process into this one and enables peer access; the returned address is valid on the current device.
 * lo_peer_close / lo_peer_free undo them (close every mapping before the owner frees).  A process must not open
 * its own handle: it uses the pointer.  No counterpart in the reference.
 */
int lo_peer_alloc(size_t bytes, void **ptr);
/* n 32-bit words from device memory into page-locked, device-addressable host memory, by a kernel rather than a copy
 * engine (a small read does not queue behind a large device-to-host copy of another stream).  Stream-ordered. */
int lo_words_to_host(const int32_t *src, int32_t *dst_host, int64_t n, void *stream);
int lo_peer_free(void *ptr);
int lo_peer_handle_bytes(void);
int lo_peer_export(const void *ptr, uint8_t *handle);
int lo_peer_open(const uint8_t *handle, void **ptr);
int lo_peer_close(void *ptr);

/*
 * Per-row expert id of the aligned contiguous layout.
 * Replaces: ep_build_m_indices, csrc/kernels/deepgemm_moe_permute.cu:833 (export.cpp:1137).
 */
int lo_ep_build_m_indices(const void *topk_ids, int ids_dtype, int64_t numel, int32_t *m_indices,
                          int64_t rows, int local_num_experts, int alignment, void *stream);

/*
 * out[t,:] = sum over local slots j of w[t,j] * a[inv_perm[t,j], :], fp32 accumulation.
 * Replaces: ep_gather, csrc/kernels/deepgemm_moe_permute.cu:1235 (kernel :947-1022).
 * a [rows,H] bf16; out [T,H] bf16.
 */
int lo_ep_gather(const void *a, const void *topk_ids, int ids_dtype, const float *topk_weights,
                 const int32_t *inv_perm, const int32_t *expert_map, void *out,
                 int64_t T, int k, int64_t H, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* LIGHTOP_B200_H_ */
