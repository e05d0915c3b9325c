/* b200q - C ABI of the sm_100a packed-GGUF quantized-inference kernels.
 *
 * Every entry point
 *   - takes plain device pointers and sizes (no framework types),
 *   - takes the CUDA stream as a `void*` (a `cudaStream_t`; NULL = legacy default stream),
 *   - only enqueues work: no allocation, no synchronisation, no host read-back, so calls
 *     can be captured into a CUDA graph (exceptions are stated on the function),
 *   - validates its arguments on the host BEFORE any launch and returns
 *       0 = ok, 1 = invalid argument, 2 = CUDA launch/runtime error, 3 = unsupported shape;
 *     `b200q_last_error()` gives the message of the calling thread's last failure.
 *
 * The packed byte layouts are the GGUF block layouts of the reference
 * (mini_llm/ops/quantized_weight.py:24-37,208-250); format ids follow the reference's CPU
 * library and Triton decoder (mini_llm/ops/native_packed_cpu.py:25-26,
 * mini_llm/ops/quantized_linear.py:34).
 */
#ifndef B200Q_H
#define B200Q_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* packed formats */
#define B200Q_Q8_0 0
#define B200Q_Q4_0 1
#define B200Q_Q4_K 2
#define B200Q_Q3_K 3
#define B200Q_Q5_K 4
#define B200Q_Q6_K 5
/* Q6_K re-ordered on the device into 16-row x 1-super-block tiles (b200q_q6k_retile): same size, same
 * values, 16-byte aligned pieces. Accepted by b200q_gemv and b200q_moe_down(_peer) only. */
#define B200Q_Q6_K_TILED 21
/* Q4_K re-ordered the same way (b200q_q4k_retile): a permutation of 16-byte pieces inside each
 * 16-row x 1-super-block tile. Accepted by b200q_gemv, b200q_swiglu, b200q_moe_gate_up and
 * b200q_moe_down(_peer); gate and up must share the layout. */
#define B200Q_Q4_K_TILED 22
/* Q8_0 in 16-row x 256-value tiles (b200q_q8_0_retile): codes stored +128, eight block scales per row
 * kept as fp16. Accepted by b200q_gemv and b200q_moe_down(_peer); K must be a multiple of 256. */
#define B200Q_Q8_0_TILED 23
/* Q5_K in the tile layout of Q4_K plus the rows' fifth bits (b200q_q5k_retile): same size, a permutation of
 * 16-byte pieces. Accepted where B200Q_Q4_K_TILED is. */
#define B200Q_Q5_K_TILED 24

/* activation / output element types */
#define B200Q_F32 0
#define B200Q_F16 1
#define B200Q_BF16 2

/* return codes */
#define B200Q_OK 0
#define B200Q_EINVAL 1
#define B200Q_ECUDA 2
#define B200Q_EUNSUPPORTED 3

/* Library / build identification; also proves the shared object loaded. */
int b200q_abi_version(void);
const char *b200q_last_error(void);

/* Device status word written by kernels whose bounded waits gave up (0 = healthy).
 * Reads the word with a blocking copy: not capturable. */
int b200q_device_status(int *status_out);
/* Sets the status word back to 0 (blocking), after the host has handled a reported give-up. */
int b200q_device_status_clear(void);

/* out[n,k] (fp32) = dequantised W. Replaces PackedGGUFWeight.dequantize_reference
 * (mini_llm/ops/quantized_weight.py:166-250) as a device kernel; bit-exact with it. */
int b200q_dequantize(const void *w, int fmt, int64_t n, int k, float *out, void *stream);

/* y[m,n] = x[m,k] @ W[n,k]^T, FP32 accumulation; W is read once for up to 8 tokens.
 * Replaces quantized_linear's device branch and its Triton kernel
 * (mini_llm/ops/quantized_linear.py:174-192,272-335) and has the argument order of the
 * reference's CPU ABI mylocal_packed_gemv (mini_llm/ops/native_packed_cpu.cpp:206-216). */
int b200q_gemv(const void *w, int fmt, int n, int k, const void *x, int x_dtype, int m, void *y,
               int y_dtype, void *stream);

/* b200q_residual_rmsnorm followed by b200q_gemv as ONE launch, for one-token decoder steps, where the norm of a
 * row of a few KB is a launch of its own: every CTA of the GEMV normalises the m <= 4 rows itself (residual +
 * alpha * branch, RMSNorm with `gamma`, rounded to act_dtype - the arithmetic of b200q_residual_rmsnorm), keeps
 * them in shared memory and multiplies; res_out receives the new FP32 residual stream. Same bits as the two calls.
 * Tile-layout Q6_K / Q8_0 weights, BF16 / FP16 activations (= the type of gamma); b200q_gemv_norm_supported answers
 * without a launch. Replaces RMSNormInference.forward_residual_add + quantized_linear of the reference's decoder
 * block (mini_llm/ops/rmsnorm_inference.py:228-252, mini_llm/ops/quantized_linear.py:174-192). */
int b200q_gemv_norm_supported(int fmt, int n, int k, int act_dtype, int m);
int b200q_gemv_norm(const void *w, int fmt, int n, int k, const float *residual, const void *branch,
                    int branch_dtype, float alpha, const void *gamma, int act_dtype, float eps, int m,
                    float *res_out, void *y, int y_dtype, void *stream);

/* y[m, n] = (silu(gate) * up) W^T with gate|up the stacked FP32 projection output [m, 2k] of the preceding launch:
 * b200q_silu_mul fused into the GEMV that consumes it (the down projection of the Llama MLP whose gate, up and
 * down matrices mini_llm/external/llama_model.py:125-130 wires, in a one-token step), same bits as the two launches. Tile-layout
 * Q6_K / Q8_0 weights, act_dtype (the type the activation is rounded to) F16 or BF16, at most 4 rows;
 * b200q_gemv_silu_supported tells whether a shape is covered. */
int b200q_gemv_silu_supported(int fmt, int n, int k, int act_dtype, int m);
int b200q_gemv_silu(const void *w, int fmt, int n, int k, const float *gate_up, int act_dtype, int m, void *y,
                    int y_dtype, void *stream);

/* The same product for many tokens (prefill, batched decode) on the tensor cores: W is read once per
 * call, decoded tile by tile to BF16 in shared memory and multiplied by tcgen05.mma with an FP32
 * accumulator in tensor memory; the activations arrive by TMA. Serves the any-M contract of
 * quantized_linear (mini_llm/ops/quantized_linear.py:272-335, grid M*N at :322-334) for M > 16.
 * Requirements (else 3 = unsupported, use b200q_gemv): native GGUF layout (Q8_0, Q4_K, Q5_K, Q6_K),
 * BF16 activations, 16-byte aligned x, K a multiple of 256. Precision: weights are rounded to BF16
 * after the reference's FP32 dequantisation (relative 2^-9 per weight), accumulation is FP32.
 * b200q_gemm_supported answers the shape / type part of the requirements (1 = yes) without a launch. */
int b200q_gemm(const void *w, int fmt, int n, int k, const void *x, int x_dtype, int m, void *y,
               int y_dtype, void *stream);
int b200q_gemm_supported(int fmt, int n, int k, int x_dtype, int m);
/* The same product with room for a split of K. Shapes with few weight-row tiles (e.g. [2048 x 8192] at 512
 * tokens: 32 CTAs) leave most SMs idle; given b200q_gemm_workspace_bytes(...) bytes of 16-byte aligned device
 * scratch, 2-8 CTAs share the K range of a tile, store FP32 partial results there, and a second small kernel adds
 * them in ascending order (deterministic) and rounds once. The query returns 0 when the shape is not split;
 * without (enough) workspace the call behaves like b200q_gemm. */
long long b200q_gemm_workspace_bytes(int fmt, int n, int k, int x_dtype, int m);
int b200q_gemm_ws(const void *w, int fmt, int n, int k, const void *x, int x_dtype, int m, void *y, int y_dtype,
                  void *workspace, long long workspace_bytes, void *stream);

/* ---- Integer-dot mode (opt-in; changes numerics): Q8_1 activations. ------------------------------
 * b200q_quantize_q8_1: x[rows, k] (fp32 / fp16 / bf16) -> rows * k/32 blocks of 36 bytes {fp16 d, fp16 sum,
 * 32 x int8}: d = max|x| / 127 of the block, codes = round-half-away(x / d) clamped to +-127 (0 for an
 * all-zero block), sum = sum of the block's inputs; IEEE arithmetic. Replaces the quantiser of
 * mini_llm/ops/q8_1_gpu.py:30-58 (its non-fast-math "ieee" variant).
 * b200q_gemv_q8_1: y[m, n] = dequant(xq)[m, k] @ W[n, k]^T with integer dots (dp4a) per sub-block and the
 * per-sub-block scaling of mini_llm/ops/mixed_q8_gpu.py:86-139 (q8_linear / k_part for Q4_K and Q5_K). W: Q4_K
 * or Q5_K in GGUF or tile layout (other formats: 3 = unsupported), K a multiple of 256; 1..4 tokens per pass over W. */
int b200q_quantize_q8_1(const void *x, int x_dtype, int rows, int k, void *out_blocks, void *stream);
int b200q_gemv_q8_1(const void *w, int fmt, int n, int k, const void *xq_blocks, int m, void *y, int y_dtype,
                    void *stream);

/* h[m,f] = silu(x @ G^T) * (x @ U^T); gate and up may use different formats.
 * Replaces quantized_swiglu and _packed_gate_up_swiglu_kernel
 * (mini_llm/ops/quantized_linear.py:194-221,338-400). */
int b200q_swiglu(const void *gate, int gate_fmt, const void *up, int up_fmt, int f, int k,
                 const void *x, int x_dtype, int m, void *h, int h_dtype, void *stream);

/* y = x * rsqrt(mean(x^2)+eps) * gamma; x fp32/bf16/fp16 rows of length d, gamma fp32 or the
 * output type. Replaces RMSNormInference.forward (mini_llm/ops/rmsnorm_inference.py:80-119,
 * 304-318). */
int b200q_rmsnorm(const void *x, int x_dtype, const void *gamma, int gamma_dtype, int rows, int d,
                  float eps, void *y, int y_dtype, void *stream);

/* res_out(fp32) = residual(fp32) + alpha*branch; y = rmsnorm(res_out)*gamma.
 * Replaces forward_residual_add / residual_add_rmsnorm_f32_bf16
 * (mini_llm/ops/rmsnorm_inference.py:228-252,525-539). res_out may alias residual. */
int b200q_residual_rmsnorm(const float *residual, const void *branch, int branch_dtype, float alpha,
                           const void *gamma, int gamma_dtype, int rows, int d, float eps,
                           float *res_out, void *y, int y_dtype, void *stream);

/* logits[t,e] (fp32) = x[t,d] @ Wr[d,e] + bias[e] (bias may be NULL); FP32 accumulation in
 * ascending d. Replaces the router logits product of RouterInference.forward
 * (mini_llm/ops/router_inference.py:38-46) and _vector_matmul
 * (mini_llm/ops/inference_matmul.py:17-41). */
int b200q_router_logits(const void *x, int x_dtype, int t, int d, const float *wr, const float *bias,
                        int e, float *logits, void *stream);

/* Same product with the weight stored [e, d] (the orientation GGUF files use for
 * ffn_gate_inp.weight): one warp per expert row, all SMs busy even for a single token. */
int b200q_router_logits_t(const void *x, int x_dtype, int t, int d, const float *wt, const float *bias,
                          int e, float *logits, void *stream);

/* scale[t] (fp32) = sigmoid(x[t,:] . gate[:]) - the admission weight of the shared expert
 * (mini_llm/external/qwen3next_moe.py:145-146). */
int b200q_shared_gate(const void *x, int x_dtype, int t, int d, const float *gate, float *scale,
                      void *stream);

/* Per row: softmax over all n logits, top-k by descending logit (ties -> lower id, NaN last),
 * weights = p[ids]; if renormalize != 0, divided by max(sum, floor_value).
 * Replaces expert_topk_forward + renormalisation (mini_llm/ops/router.py:21-43,
 * mini_llm/ops/router_inference.py:47-60) and the fused decode kernel normalized_topk
 * (mini_llm/ops/router_decode.py:16-96) for any number of rows. n <= 4096, k <= 32. */
int b200q_router_topk(const float *logits, int rows, int n, int k, int renormalize,
                      float floor_value, float *weights, int64_t *ids, void *stream);

/* b200q_router_topk that also appends one fixed assignment per row: outputs have k+1 entries, the
 * last being (extra_id, extra_weight[row] or 1 when extra_weight is NULL). Used to run an always-on
 * shared expert (mini_llm/external/qwen3next_moe.py:138-147) through the grouped expert kernels as
 * the highest expert id, so that it is added last. extra_id < 0 appends nothing. */
int b200q_router_topk_ex(const float *logits, int rows, int n, int k, int renormalize,
                         float floor_value, int extra_id, const float *extra_weight, float *weights,
                         int64_t *ids, void *stream);

/* Device routing plan: stable counting sort of the rows*k assignments by expert id.
 * Outputs (all device, caller-allocated):
 *   counts[e]            assignments per expert
 *   offsets[e+1]         exclusive prefix sum
 *   order[rows*k]        flat assignment index (row*k+slot) at each sorted position
 *   inv[rows*k]          sorted position of each flat assignment (inverse of order)
 *   seg_expert/seg_begin/seg_count[max_segments] + num_segments[1]
 *                        compacted list of active experts, ascending id, each split into
 *                        runs of at most seg_cap assignments
 *   status[1]            0; 1 if an id was outside [0,e) (it is then counted as expert 0);
 *                        2 if max_segments was too small (extra segments are dropped)
 * Replaces RoutingPlan.from_router_outputs (mini_llm/ops/routing_plan.py:52-118) and
 * plan_routes (mini_llm/ops/device_expert_plan.py:17-36) without the host round trip. */
int b200q_moe_plan(const void *ids, int ids_is_i64, int rows, int k, int e, int seg_cap,
                   int32_t *counts, int32_t *offsets, int32_t *order, int32_t *inv,
                   int32_t *seg_expert, int32_t *seg_begin, int32_t *seg_count,
                   int32_t *num_segments, int max_segments, int32_t *status, void *stream);

/* b200q_moe_plan with one expert id whose assignments are counted and sorted but get no segment, so
 * the grouped kernels never touch them (skip_expert < 0: none). Expert-parallel ranks map the
 * assignments that belong to other ranks to that id. (No counterpart in the reference, which has no
 * multi-GPU path.) */
int b200q_moe_plan_ex(const void *ids, int ids_is_i64, int rows, int k, int e, int skip_expert, int seg_cap,
                      int32_t *counts, int32_t *offsets, int32_t *order, int32_t *inv,
                      int32_t *seg_expert, int32_t *seg_begin, int32_t *seg_count,
                      int32_t *num_segments, int max_segments, int32_t *status, void *stream);

/* Grouped gate/up + SwiGLU over the plan's segments:
 *   hbuf[pos, f] (fp32) = silu(x[token(pos)] . G_e) * (x[token(pos)] . U_e)
 * for every sorted position pos of every segment; token(pos) = order[pos] / k.
 * Expert e's matrices start at gate_base + e*gate_stride (bytes) inside a contiguous bank, or, when
 * gate_table / up_table (device arrays of one address per expert, the reference's pointer table of
 * mini_llm/ops/grouped_quantized_experts.py:186-196) are given, at table[e]; tables_aligned16 != 0
 * promises that every table entry is 16-byte aligned (enables the tensor-core kernels).
 * Replaces _grouped_gate_up (mini_llm/ops/grouped_quantized_experts.py:31-43) and the
 * per-expert loop of ExpertsInference.forward (mini_llm/ops/experts_inference.py:293-310). */
int b200q_moe_gate_up(const void *gate_base, int64_t gate_stride, int gate_fmt, const void *up_base,
                      int64_t up_stride, int up_fmt, const uint64_t *gate_table, const uint64_t *up_table,
                      int tables_aligned16, int f, int d, const void *x, int x_dtype, int k,
                      const int32_t *order, const int32_t *seg_expert, const int32_t *seg_begin,
                      const int32_t *seg_count, const int32_t *num_segments, int max_segments,
                      float *hbuf, void *stream);

/* The same launch fed with per-token activation images. A token routed to k experts is otherwise converted
 * (scaled, split into FP16 fragments, summed per sub-block) once per expert segment it appears in;
 * b200q_moe_token_images does that conversion once per row of x [rows, d] and stores it, and
 * b200q_moe_gate_up_images lets every segment gather its tokens' images instead. The conversion code is
 * the same, so the results are the same bits as b200q_moe_gate_up's. `images` holds rows *
 * b200q_moe_token_image_bytes(d, x_dtype) bytes, 16-byte aligned; that function returns 0 when d has no
 * images (not a multiple of 256, or too large), and kernels that do not use images ignore the buffer.
 * No counterpart in the reference: its grouped op indexes the activations per expert
 * (mini_llm/ops/grouped_quantized_experts.py:31-43). */
int b200q_moe_token_image_bytes(int d, int x_dtype);
int b200q_moe_token_images(const void *x, int x_dtype, int rows, int d, void *images, void *stream);
int b200q_moe_gate_up_images(const void *gate_base, int64_t gate_stride, int gate_fmt, const void *up_base,
                             int64_t up_stride, int up_fmt, const uint64_t *gate_table, const uint64_t *up_table,
                             int tables_aligned16, int f, int d, const void *x, int x_dtype, const void *images,
                             int k, const int32_t *order, const int32_t *seg_expert, const int32_t *seg_begin,
                             const int32_t *seg_count, const int32_t *num_segments, int max_segments,
                             float *hbuf, void *stream);

/* Grouped down projection with the route weight applied and stored per assignment:
 *   terms[pos, d] (fp32) = (hbuf[pos] . D_e) * route[order[pos]]
 * With flat_rows != 0 the row index is order[pos] (the flat assignment index row*k+slot) instead of
 * pos - the layout an expert-parallel exchange needs, because it does not depend on the rank.
 * Replaces _grouped_down_weighted (mini_llm/ops/grouped_quantized_experts.py:45-68). */
int b200q_moe_down(const void *down_base, int64_t down_stride, int down_fmt, const uint64_t *down_table,
                   int tables_aligned16, int flat_rows, int d, int f, const float *hbuf, const float *route, const int32_t *order,
                   const int32_t *seg_expert, const int32_t *seg_begin, const int32_t *seg_count,
                   const int32_t *num_segments, int max_segments, float *terms, void *stream);

/* out[row, d] = sum over the row's k assignments of terms[pos], added one by one in
 * ascending expert id starting from zero (plain FP32 adds, no FMA, no tree), plus an optional
 * extra[row,d]*extra_scale[row] term added last (the shared expert). `inv` maps the flat
 * assignment index to its sorted position (inverse of `order`).
 * Replaces _ordered_reduce (mini_llm/ops/grouped_quantized_experts.py:70-79) and the ordered
 * scatter-add of ExpertsInference.forward (mini_llm/ops/experts_inference.py:293-310). */
int b200q_moe_combine(const float *terms, const int32_t *inv, int rows, int k, int d,
                      const float *extra, const float *extra_scale, void *out, int out_dtype,
                      void *stream);

/* b200q_moe_combine fused with the residual add and RMSNorm that follow it in a decoder layer
 * (b200q_residual_rmsnorm: mini_llm/ops/rmsnorm_inference.py:228-252 of the reference):
 *   branch = the ordered sum, rounded to branch_dtype (the type b200q_moe_combine would store);
 *   res_out = residual + alpha*branch (FP32);  y = rmsnorm(res_out)*gamma in y_dtype.
 * Same bits as the two calls; k <= 16 (else B200Q_EUNSUPPORTED); res_out must not alias residual. */
int b200q_moe_combine_norm(const float *terms, const int32_t *inv, int rows, int k, int d, const float *extra,
                           const float *extra_scale, int branch_dtype, const float *residual, float alpha,
                           const void *gamma, int gamma_dtype, float eps, float *res_out, void *y, int y_dtype,
                           void *stream);

/* b200q_router_topk_ex and b200q_moe_plan for ONE token row in one launch (the one-token decode
 * step): weights / ids as b200q_router_topk_ex (rows = 1), plan arrays as b200q_moe_plan for those
 * ids over `e` experts with one row per segment (counts [e], offsets [e+1], order / inv [k'],
 * seg_* [max_segments]). n <= 1024, k <= 31; an appended extra_id must be >= n (it is for the
 * shared expert, id n). */
int b200q_router_topk_plan_row(const float *logits, int n, int k, int renormalize, float floor_value, int extra_id,
                               const float *extra_weight, float *weights, int64_t *ids, int e, int32_t *counts,
                               int32_t *offsets, int32_t *order, int32_t *inv, int32_t *seg_expert, int32_t *seg_begin,
                               int32_t *seg_count, int32_t *num_segments, int max_segments, int32_t *status,
                               void *stream);

/* Ordered combine for terms stored at the flat assignment index: out[row] = sum of terms[row*k+slot]
 * in ascending (expert id, slot) order, plain FP32 adds from zero (same semantics as
 * b200q_moe_combine; used by the home rank of an expert-parallel layer). */
int b200q_moe_combine_ids(const float *terms, const void *ids, int ids_is_i64, int rows, int k, int d,
                          const float *extra, const float *extra_scale, void *out, int out_dtype, void *stream);

/* Lossless re-ordering of a native Q6_K matrix [rows, k] (rows % 16 == 0, k % 256 == 0; a bank of
 * experts is one matrix of E*rows_per_expert rows) into the tile layout and back. Out of place; the
 * tiled buffer must be 16-byte aligned. GGUF stores 210-byte Q6_K blocks, which no 128-bit load can
 * address; the tile layout is what the tensor-core kernel streams at full width. (No counterpart in
 * the reference, which reads native blocks byte by byte: mini_llm/ops/quantized_linear.py:139-158.) */
int b200q_q4k_retile(const void *native, void *tiled, int64_t rows, int k, void *stream);
int b200q_q4k_untile(const void *tiled, void *native, int64_t rows, int k, void *stream);
int b200q_q6k_retile(const void *native, void *tiled, int64_t rows, int k, void *stream);
int b200q_q5k_retile(const void *native, void *tiled, int64_t rows, int k, void *stream);
int b200q_q5k_untile(const void *tiled, void *native, int64_t rows, int k, void *stream);
int b200q_q8_0_retile(const void *native, void *tiled, int64_t rows, int k, void *stream);
int b200q_q8_0_untile(const void *tiled, void *native, int64_t rows, int k, void *stream);
int b200q_q6k_untile(const void *tiled, void *native, int64_t rows, int k, void *stream);

/* ---- Decode-step bookkeeping of the Llama path (the reference's graph decoder has NVRTC kernels of
 * the same role: qkv_rope_store_fp16_d64_dynamic / dense_attention_fp16_d64_dynamic,
 * mini_llm/external/cuda_graph_decode.py:64-260). ------------------------------------------------ */

/* Rotate-half RoPE of q (in place, FP32 [B,T,H,Dh]) and k, and store of rotated k and v (FP32
 * [B,T,Hkv,Dh]) into the caches [B,Hkv,horizon,Dh] (cache_dtype) at positions[t] (device int64 [T]);
 * *_row_stride = elements between consecutive (b,t) rows (q, k, v may be column slices of one fused
 * projection output); cos/sin tables are FP32 [table_rows, Dh/2] with theta_i = pos / base^(2i/Dh).
 * The positions are read on the device (a captured step advances them between replays), so the
 * kernel checks them itself: a position outside [0, min(horizon, table_rows)) reads no table entry,
 * leaves q and the caches as they are and stores 301 in the device status word. */
int b200q_rope_kv_store(float *q, const float *k, const float *v, int64_t q_row_stride, int64_t k_row_stride,
                        int64_t v_row_stride, const int64_t *positions, const float *cos_table,
                        const float *sin_table, int table_rows, int batch, int t, int heads, int kv_heads,
                        int head_dim, int horizon, void *k_cache, void *v_cache, int cache_dtype, void *stream);

/* act[m, f] = silu(gu[m, f]) * gu[m, F + f] for a stacked gate|up projection output gu [M, 2F] FP32
 * (the epilogue of b200q_swiglu as a separate step, for weights whose tile layout has no fused
 * SwiGLU kernel). */
int b200q_silu_mul(const float *gate_up, int m, int f, void *out, int out_dtype, void *stream);

/* Single-query attention: out[b, h*Dh..] = softmax(scale * q[b,h] . K[b,kv(h),0..pos]) V, with
 * pos = position[0] read on the device (graph-capturable); q FP32 [B,H,Dh] with q_row_stride elements
 * between batch rows; head_dim 64 or 128. */
int b200q_decode_attention(const float *q, int64_t q_row_stride, const void *k_cache, const void *v_cache,
                           int cache_dtype, const int64_t *position, int batch, int heads, int kv_heads, int head_dim,
                           int horizon, float scale, void *out, int out_dtype, void *stream);

/* The two calls above as one launch for a one-token step (t = 1): q, k, v are the raw FP32 projection outputs
 * ([B,H,Dh] / [B,Hkv,Dh] with their row strides); every CTA rotates its query head and the new key of its KV head,
 * the new key / value enter the softmax from registers (rounded through cache_dtype, as a load from the cache would
 * return them) and are written to the caches at position[0]; q is not modified. Results are bit-identical to
 * b200q_rope_kv_store followed by b200q_decode_attention (mini_llm/ops/cuda_graph_decode.py:379-449 runs those two
 * steps per layer); an out-of-range position behaves as in b200q_rope_kv_store (status 301). */
int b200q_rope_attention(const float *q, const float *k, const float *v, int64_t q_row_stride, int64_t k_row_stride,
                         int64_t v_row_stride, const int64_t *position, const float *cos_table, const float *sin_table,
                         int table_rows, int batch, int heads, int kv_heads, int head_dim, int horizon, void *k_cache,
                         void *v_cache, int cache_dtype, float scale, void *out, int out_dtype, void *stream);

/* ---- Expert-parallel execution over the GPUs of one node (no counterpart in the reference, which is
 * single-process; semantics = the single-GPU layer, bit for bit). ------------------------------- */

/* Routing plan of one rank: ids hold GLOBAL expert ids for the tokens of ALL ranks ([rows,k]).
 * Global ids first_expert..first_expert+n_local-1 become local experts 0..n_local-1; shared_id
 * (< 0: none) becomes local expert n_local for rows home_lo..home_hi-1 (the rows this rank is home
 * of); everything else is sorted last and gets no segment. counts/offsets have n_local+2 (+1)
 * entries. The id e_global itself marks a padding entry (rows a rank did not fill in its slot of
 * the gathered ids): it is legal and never executed. Ids outside [0, e_global] set *status = 1. */
int b200q_moe_plan_ep(const void *ids, int ids_is_i64, int rows, int k, int e_global, int first_expert, int n_local,
                      int shared_id, int home_lo, int home_hi, int seg_cap, int32_t *counts, int32_t *offsets,
                      int32_t *order, int32_t *inv, int32_t *seg_expert, int32_t *seg_begin, int32_t *seg_count,
                      int32_t *num_segments, int max_segments, int32_t *status, void *stream);

/* b200q_moe_down with the projection and the exchange in one kernel: the term row of flat assignment
 * i (= row*k + slot over all ranks' rows) is stored at row i - r*rows_per_rank of the buffer whose
 * address is term_tables[r], r = i / rows_per_rank - the home rank's arena, written through peer
 * memory. Each row has exactly one writer, so no reduction and no clearing is needed; a
 * b200q_peer_barrier must separate it from the home rank's combine. */
int b200q_moe_down_peer(const void *down_base, int64_t down_stride, int down_fmt, const uint64_t *down_table,
                        int tables_aligned16, int d, int f, const float *hbuf, const float *route,
                        const int32_t *order, const int32_t *seg_expert, const int32_t *seg_begin,
                        const int32_t *seg_count, const int32_t *num_segments, int max_segments,
                        const uint64_t *term_tables, int rows_per_rank, void *stream);

/* Peer arena: cudaMalloc'd, cleared, exported as a 64-byte CUDA IPC handle; peers map it with
 * b200q_peer_open (which also enables peer access). Setup-time calls, not for the decode loop. */
int b200q_peer_alloc(size_t bytes, void **ptr, unsigned char *handle64);
int b200q_peer_open(const unsigned char *handle64, void **ptr);
int b200q_peer_close(void *ptr);
int b200q_peer_free(void *ptr);

/* Barrier over the ranks' streams. pads: device array of `world` addresses, entry r = rank r's
 * signal pad (>= 128 zero-initialised bytes inside its arena). Returns when every rank has reached
 * its matching call, or after timeout_ms with 201 in the device status word (b200q_device_status).
 * One rank per GPU only: ranks sharing a GPU would wait on one another's unscheduled kernels. */
int b200q_peer_barrier(const uint64_t *pads, int rank, int world, int timeout_ms, void *stream);

/* All-gather by stores: copies `bytes` from src to dst_bases[p] + dst_offset_bytes for every p < world. */
int b200q_peer_push_rows(const void *src, size_t bytes, const uint64_t *dst_bases, size_t dst_offset_bytes,
                         int world, void *stream);
/* The same for up to three buffers in one launch (rows, routing weights, expert ids): buffer z goes
 * to dst_bases[p] + dst_offset_z for every p < world; a size of 0 skips a buffer. */
int b200q_peer_push3(const void *src0, size_t bytes0, size_t dst_offset0, const void *src1, size_t bytes1,
                     size_t dst_offset1, const void *src2, size_t bytes2, size_t dst_offset2,
                     const uint64_t *dst_bases, int world, void *stream);

/* One-token decode step of a whole stack of MoE layers (norm -> router -> top-k -> routed + shared experts ->
 * ordered combine -> residual add, per layer) as ONE persistent cooperative kernel: the stages the entry points
 * b200q_rmsnorm, b200q_router_logits_t, b200q_router_topk_plan_row, b200q_moe_gate_up, b200q_moe_down and
 * b200q_moe_combine_norm run as separate launches are walked by one grid with a bounded device-wide barrier
 * between them, and the result is bit-identical to that chain of launches. Replaces the per-layer launch
 * sequence the reference captures for one decode step (mini_llm/external/cuda_graph_decode.py:379-449).
 *   layers        device array of n_layers records of five 8-byte pointers: router weight [e, d] FP32
 *                 (expert-major, 16-byte aligned), gate / up / down pointer tables (e + 1 addresses each: the
 *                 routed experts, then the always-selected shared expert; 16-byte aligned matrices), and the
 *                 weight of the norm that FOLLOWS the layer (the last record: the final norm)
 *   gamma0        weight of the norm in front of the first layer; all norm weights have type act_dtype
 *   residual_in   FP32 [d]; residual_out FP32 [d] and hidden_out [d] (act_dtype) receive the residual stream
 *                 and the normalised activations after the last layer
 *   workspace     b200q_moe_decode_stack_workspace(d, f, e, k) bytes, 256-byte aligned, used by one step
 *                 at a time
 * Supported: gate/up Q4_K (native or tile layout), down in the Q6_K tile layout, BF16/FP16 activations,
 * e <= 1024, k <= 15, d and f multiples of 256; anything else returns 3 and the caller runs the separate
 * launches. A wait at the device-wide barrier that runs out (1 s) sets device status 401 and ends the step. */
long long b200q_moe_decode_stack_workspace(int d, int f, int e, int k);
int b200q_moe_decode_stack(const void *layers, int n_layers, int d, int f, int e, int k, int renormalize,
                           float floor_value, int gate_up_fmt, int down_fmt, const void *gamma0, int act_dtype,
                           float eps, const float *residual_in, float *residual_out, void *hidden_out,
                           void *workspace, long long workspace_bytes, void *stream);

/* One SwiGLU expert, y[m,d_model] = down( silu(x gate^T) * (x up^T) ), for callers that cannot
 * allocate device memory. (No counterpart in the reference: its expert FFN allocates the hidden
 * activations with CuPy.) The FP32 hidden activations [m, d_ff] between the two kernels live in a
 * fixed array inside the library (512 KiB on every GPU that loads it), so the call performs no
 * cudaMalloc/cudaFree and needs no framework allocator: meant for hosts without a device allocator
 * of their own and for loops where allocation is forbidden or would stall the device.
 *   - limit: m * d_ff <= 131072 (e.g. 8 tokens x 16384); larger requests return 3 with a message;
 *   - the first call on each device looks up the array's device address (cudaGetSymbolAddress, with
 *     that device current): make that first call before starting any stream capture;
 *   - every call on a device shares the one array: calls that can overlap on the GPU (different
 *     streams, or graphs replayed concurrently) race on it - serialise them. Nothing needs to be
 *     cleared between calls; each call overwrites all it reads. */
int b200q_expert_ffn_static(const void *gate, int gate_fmt, const void *up, int up_fmt, const void *down,
                            int down_fmt, int d_model, int d_ff, const void *x, int x_dtype, int m,
                            void *y, int y_dtype, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* B200Q_H */
