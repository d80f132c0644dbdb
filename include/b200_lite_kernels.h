/*
 * b200_lite_kernels.h -- C ABI of libb200lite.so, the B200 (sm_100a) kernel layer that stands in
 * for `lite_llama.kernels` (reference: /root/reference/lite_llama/kernels/__init__.py:11-39).
 *
 * The reference has no FFI: its boundary is Python name binding (`from ..kernels import ...`,
 * lite_llama/models/base.py:31-38, lite_llama/executor/model_runner.py:22,
 * lite_llama/models/quantization/methods/*.py).  Each entry point below is what a ctypes binding
 * for one of those names calls; lite_llama_b200/kernels/ holds that binding with the reference's
 * exact Python signatures, INTEGRATION.md shows how to bind them inside the unmodified reference.
 *
 * Conventions
 *   - every pointer is a DEVICE pointer unless stated otherwise; the caller owns all memory;
 *   - no entry point allocates, synchronises or touches the default stream: work is enqueued on
 *     `stream` (a cudaStream_t) and is CUDA-graph capturable;
 *   - strides are in ELEMENTS of the tensor's dtype; the innermost dimension must be contiguous;
 *   - `dtype`: B2L_F16 / B2L_BF16 activation dtype (the reference is fp16-only);
 *   - `*_width`: 4 or 8, byte width of an index vector (callers pass int32 or int64 vectors for
 *     b_seq_len / b_req_idx / b_start_loc);
 *   - return 0 on success, negative on error (B2L_ERR_*); b2l_last_error() returns a thread-local
 *     message.  The Python shim turns non-zero returns into ValueError, mirroring the reference's
 *     error behaviour (e.g. kernels/quantization/w4a16.py:174-184);
 *   - workspaces: `b2l_*_workspace_bytes` are pure functions of shapes (+ SM count), so the caller
 *     can size a torch.empty scratch buffer outside graph capture.  Split-K GEMMs additionally take a
 *     small int32 `counters` array that must be ZERO on entry; kernels leave it zero on exit.
 *     The QUANTISED GEMMs' workspace (b2l_w4a16_matmul*, b2l_w8a16_matmul) carries stream-K partial sums as
 *     tagged words (flag-in-data): it must be ZERO on entry as well and is left zero on exit, so keep ONE persistent,
 *     once-zeroed buffer per device (and one stream of launches), exactly like `counters`.
 */
#ifndef B200_LITE_KERNELS_H
#define B200_LITE_KERNELS_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B2L_F16 0
#define B2L_BF16 1
#define B2L_F32 2 /* true 32-bit activations and weights: accepted by the entry points that say so */

#define B2L_OK 0
#define B2L_ERR_INVALID (-1)
#define B2L_ERR_CUDA (-2)
#define B2L_ERR_UNSUPPORTED (-3)

/* quantised-weight kinds for b2l_quant_gemm_workspace_bytes */
#define B2L_Q_INT4 0
#define B2L_Q_FP8 1
#define B2L_Q_INT8 2

const char* b2l_last_error(void);
int b2l_version(void);
int b2l_device_info(int* sm_count, int* cc_major, int* cc_minor, int* max_smem_optin);
/* number of kernels this library has launched in this process (monotonic; bench.py's gpu_launches) */
int64_t b2l_launch_count(void);
/* Programmatic dependent launch (every kernel is launched so that the next one's set-up and weight prefetch
 * overlap it; see csrc/common.cuh).  Returns the previous setting.  Also: environment B2L_PDL=0 at load.
 * No reference counterpart: the reference launches every Triton kernel fully serialised. */
int b2l_set_pdl(int enabled);
/* Device-side hang watchdog (csrc/common.cuh): every barrier wait of the warp-specialised kernels traps after
 * B2L_HANG_MS milliseconds (environment, default 4000, 0 = off) instead of parking for ever, after writing a
 * host-pinned record.  out16 receives: [0] 0xB2D00DED when a record exists, [1] FNV-1a hash of the source file's
 * basename, [2] line of the wait, [3..5] blockIdx, [6] threadIdx.x, [7] shared address of the barrier, [8] parity,
 * [9] ms waited, [10..12] gridDim, [13] blockDim.x.  Readable after the CUDA context has died.  No reference
 * counterpart (Triton kernels have no cross-warp pipelines to dead-lock). */
int b2l_hang_report(int* out16);

/* skip_rmsnorm(X, residual, weight, eps) -- lite_llama/kernels/skip_rmsnorm.py:192-234.
 * residual (nullable) is updated in place with x + residual (rounded to dtype); y gets
 * round(sum_f32 * rrms) * weight. */
int b2l_skip_rmsnorm(void* y, const void* x, void* residual, const void* weight, int64_t rows, int64_t n,
                     int64_t x_row_stride, int64_t r_row_stride, int64_t y_row_stride, float eps, int dtype,
                     void* stream);

/* rope_emb_forward(q, k, cos, sin, batch_size, seq_len) -- lite_llama/kernels/rope_emb.py:86-134.
 * In place on q [B*S, n_qh, D] and k [B*S, n_kh, D]; cos/sin [B, S, >=D/2] (first D/2 entries read). */
int b2l_rope_emb(void* q, void* k, const void* cos, const void* sin, int64_t batch, int64_t seq_len, int n_qh,
                 int n_kh, int head_dim, int64_t q_tok_stride, int64_t q_head_stride, int64_t k_tok_stride,
                 int64_t k_head_stride, int64_t cs_batch_stride, int64_t cs_seq_stride, int dtype, void* stream);

/* swiglu_forward(a, b) -- lite_llama/kernels/swiglu.py:45-65; also fused_moe's _silu_and_mul
 * (lite_llama/kernels/fused_moe.py:296-313) by pointing b at the second half of each row. */
int b2l_swiglu(void* c, const void* a, const void* b, int64_t rows, int64_t n, int64_t a_row_stride,
               int64_t b_row_stride, int64_t c_row_stride, int dtype, void* stream);

/* update_kv_buffer(KV_Values, Select_Index, KV_Buffer) -- lite_llama/kernels/update_kv_buffer.py:55-89.
 * Heads [0, heads_a) of every destination row come from src_a, heads [heads_a, heads_a+heads_b) from
 * src_b (so K and V need no torch.cat, lite_llama/models/base.py:76); pass heads_b = 0 for one source.
 * 2-byte element dtype. */
int b2l_update_kv_buffer(const void* src_a, const void* src_b, const void* select_index, int index_width,
                         void* kv_buffer, int64_t tokens, int heads_a, int heads_b, int head_dim,
                         int64_t a_tok_stride, int64_t a_head_stride, int64_t b_tok_stride, int64_t b_head_stride,
                         int64_t d_tok_stride, int64_t d_head_stride, void* stream);

/* update_kv_index(req_to_token_indexs, b_req_idx, b_seq_len, select_index)
 * -- lite_llama/kernels/update_kv_index.py:51-88.  table is int32. */
int b2l_update_kv_index(void* table, const void* b_req_idx, int req_width, const void* b_seq_len, int len_width,
                        const void* select_index, int sel_width, int64_t n, int64_t stride_b, int64_t stride_s,
                        void* stream);

/* flash_decoding(q, k_cache, v_cache, qk_scale, b_req_tokens_table, b_req_idx, b_seq_len,
 * max_actual_seq_len) -- lite_llama/kernels/flashdecoding.py:316-380. */
int64_t b2l_flash_decoding_workspace_bytes(int64_t batch, int num_q_heads, int num_kv_heads, int head_dim,
                                           int64_t max_seq_len);
int b2l_flash_decoding(void* out, const void* q, const void* k_cache, const void* v_cache,
                       const void* b_req_tokens_table, const void* b_req_idx, int req_idx_width,
                       const void* b_seq_len, int seq_len_width, int64_t batch, int num_q_heads, int num_kv_heads,
                       int head_dim, int64_t max_seq_len, float qk_scale, int64_t q_batch_stride,
                       int64_t q_head_stride, int64_t k_token_stride, int64_t k_head_stride, int64_t v_token_stride,
                       int64_t v_head_stride, int64_t table_batch_stride, int64_t table_seq_stride,
                       int64_t o_batch_stride, int64_t o_head_stride, void* workspace, int64_t workspace_bytes,
                       void* tickets, int64_t num_tickets, int dtype, void* stream);

/* flash_attention2_no_pad(q, k, v, sm_scale, b_start_loc, b_seq_len, max_seq_len)
 * -- lite_llama/kernels/flashattention2_nopad.py:175-231.  sm_scale already carries log2(e).  total_tokens = q.shape[0]
 * (rows of q / k / v; bounds the TMA descriptors of the tcgen05 kernel, csrc/flash_attention_tc.cu, which takes
 * head_dim 128 with heads packed inside a token row; other shapes run the mma.sync kernel). */
int b2l_flash_attention2_no_pad(void* out, const void* q, const void* k, const void* v, const void* b_start_loc,
                                int start_loc_width, const void* b_seq_len, int seq_len_width, int64_t batch,
                                int num_q_heads, int num_kv_heads, int head_dim, int64_t max_seq_len,
                                int64_t total_tokens, float sm_scale_log2, int64_t q_tok_stride, int64_t q_head_stride,
                                int64_t k_tok_stride, int64_t k_head_stride, int64_t v_tok_stride,
                                int64_t v_head_stride, int64_t o_tok_stride, int64_t o_head_stride, int dtype,
                                void* stream);

/* rope_emb_forward + torch.cat + update_kv_buffer in ONE launch (lite_llama/kernels/rope_emb.py:86-134,
 * lite_llama/models/base.py:76-79, lite_llama/kernels/update_kv_buffer.py:55-89): rotates q [T, n_qh, D] and
 * k [T, n_kh, D] in place (same arithmetic as b2l_rope_emb), stores the rotated k rows and the v rows [T, n_kh, D] into
 * kv_buffer [max_tokens, 2 * n_kh, D] at rows select_index[t] (K heads first).  Strides in elements. */
int b2l_rope_kv_write(void* q, void* k, const void* v, const void* cos, const void* sin, const void* select_index,
                      int index_width, void* kv_buffer, int64_t batch, int64_t seq_len, int n_qh, int n_kh,
                      int head_dim, int64_t q_tok_stride, int64_t q_head_stride, int64_t k_tok_stride,
                      int64_t k_head_stride, int64_t v_tok_stride, int64_t v_head_stride, int64_t cs_batch_stride,
                      int64_t cs_seq_stride, int64_t d_tok_stride, int64_t d_head_stride, int dtype, void* stream);

/* Greedy sampling: out[r] = argmax_j x[r, j] (int64; ties -> lowest index).  Reference: temperature-0 path of the
 * Sampler, torch.argmax over the [batch, vocab] logits (lite_llama/engine/sampler.py, engine/llm_engine.py:172). */
int b2l_argmax_rows(void* out_index_i64, const void* x, int64_t rows, int64_t n, int64_t row_stride, int dtype,
                    void* stream);

/* Dense projection y = x @ w.T (+ bias): the reference's F.linear call sites
 * (lite_llama/models/quantization/methods/unquantized.py:21-22, lite_llama/models/base.py:489). */
int64_t b2l_linear_workspace_bytes(int64_t m, int64_t n, int64_t k, int elem_bytes);
int64_t b2l_linear_num_counters(int64_t m, int64_t n);
int b2l_linear(void* y, const void* x, const void* w, const void* bias, int64_t m, int64_t n, int64_t k,
               int64_t x_row_stride, int64_t w_row_stride, int64_t y_row_stride, void* workspace,
               int64_t workspace_bytes, void* counters, int64_t num_counters, int dtype, void* stream);

/* w4a16_matmul(x, qweight, scales, zeros, *, group_size, bias)
 * -- lite_llama/kernels/quantization/w4a16.py:152-207.  fp16 activations only (w4a16.py:174). */
int64_t b2l_quant_gemm_workspace_bytes(int kind, int64_t m, int64_t n, int64_t k, int64_t group_k);
int64_t b2l_quant_gemm_num_counters(int64_t m, int64_t n);
/* launch plan of a quantised GEMM, for tests and tools (no GPU work): out[10] = {stream-K CTAs (0 = tile x split
 * grid), workspace slots per tile, raw blocks per tile, weight-row tiles, splits, k-blocks per split, weight ring
 * depth, activation ring depth, shared-memory bytes, scale-table columns}.  The trailing argument is unused. */
int b2l_quant_gemm_plan(int kind, int64_t m, int64_t n, int64_t k, int64_t group_k, int* out, void* reserved);
int b2l_w4a16_matmul(void* y, const void* x, const void* qweight, const void* scales, const void* zeros,
                     const void* bias, int bias_is_f32, int64_t m, int64_t n, int64_t k, int group_size,
                     int64_t x_row_stride, int64_t qw_row_stride, int64_t s_row_stride, int64_t s_col_stride,
                     int64_t y_row_stride, void* workspace, int64_t workspace_bytes, void* counters,
                     int64_t num_counters, void* stream);

/* Load-time repack of the three W4A16 tensors into the kernel-native layout (the reference reserves this seam:
 * lite_llama/models/quantization/_layout/__init__.py:1-6; its own tensors stay as w4a16.py:9-12 defines them).
 * Bit-exact permutations, one pass each:
 *   qweight_packed int32 [N, K/8]: nibble position p of a word holds the K index [0,2,4,6,1,3,5,7][p] of that word
 *   table_packed   fp32 [ceil(N/128)][groups][128]: table_packed[t][g][r] = table[128 t + r][g], rows past N zero
 * b2l_w4a16_matmul_packed computes exactly b2l_w4a16_matmul's result from the repacked tensors; zeros_foldable = 1
 * promises that every zero point is an integer in [0, 1023] (checked once by the packer's caller).
 * epilogue = 1 fuses swiglu_forward (lite_llama/kernels/swiglu.py:45-65; models/base.py:259-264 runs gate_proj,
 * up_proj and swiglu as three launches): the packed rows must be interleaved (row 2i = gate_i, row 2i+1 = up_i);
 * y is [m, n/2] = silu(gate) * up with both projections rounded to fp16 first, bit-identical to the unfused path. */
int b2l_w4a16_pack_qweight(void* out, const void* in, int64_t n, int64_t k8, int64_t in_row_stride,
                           int64_t out_row_stride, void* stream);
int b2l_w4a16_pack_table(void* out, const void* in, int64_t n, int64_t groups, int64_t row_stride,
                         int64_t col_stride, void* stream);
int b2l_w4a16_matmul_packed(void* y, const void* x, const void* qweight_packed, const void* scales_packed,
                            const void* zeros_packed, const void* bias, int bias_is_f32, int64_t m, int64_t n,
                            int64_t k, int group_size, int zeros_foldable, int64_t x_row_stride,
                            int64_t qw_row_stride, int64_t y_row_stride, void* workspace, int64_t workspace_bytes,
                            void* counters, int64_t num_counters, int epilogue, void* stream);

/* w8a16_matmul(x, qweight, scales, *, group_n, group_k, bias)
 * -- lite_llama/kernels/quantization/w8a16.py:155-216.  qweight uint8 (fp8-e4m3 bits) or int8. */
int b2l_w8a16_matmul(void* y, const void* x, const void* qweight, int weight_is_fp8, const void* scales,
                     const void* bias, int bias_is_f32, int64_t m, int64_t n, int64_t k, int64_t group_n,
                     int64_t group_k, int64_t x_row_stride, int64_t qw_row_stride, int64_t s_row_stride,
                     int64_t s_col_stride, int64_t y_row_stride, void* workspace, int64_t workspace_bytes,
                     void* counters, int64_t num_counters, void* stream);

/* smoothquant_matmul(x, qweight, weight_scales, *, bias) -- lite_llama/kernels/quantization/w8a8.py:151-217
 * is two calls: per-token dynamic quantisation (w8a8.py:35-68), then the int8 GEMM (w8a8.py:75-130). */
int b2l_quantize_activations_int8(void* q, void* scales, const void* x, int64_t m, int64_t k, int64_t x_row_stride,
                                  int64_t q_row_stride, int dtype, void* stream);
/* skip_rmsnorm (skip_rmsnorm.py:192-234) followed by the per-token quantisation above (w8a8.py:35-68) in one
 * launch, for a norm whose only consumer is an int8 GEMM (models/base.py:307-312 under SmoothQuant): q / scales
 * are bit-identical to b2l_skip_rmsnorm + b2l_quantize_activations_int8; the fp16 norm output is never written.
 * Needs n % 8 == 0, n <= 16384, 16-byte aligned rows. */
int b2l_skip_rmsnorm_quant_int8(void* q, void* scales, const void* x, void* residual, const void* weight,
                                int64_t rows, int64_t n, int64_t x_row_stride, int64_t r_row_stride,
                                int64_t q_row_stride, float eps, int dtype, void* stream);
int b2l_w8a8_gemm(void* y, const void* xq, const void* wq, const void* a_scale, const void* b_scale,
                  const void* bias_f32, int64_t m, int64_t n, int64_t k, int64_t xq_row_stride,
                  int64_t wq_row_stride, int64_t y_row_stride, void* workspace, int64_t workspace_bytes,
                  void* counters, int64_t num_counters, int out_dtype, void* stream);

/* fused_moe(hidden_states, w1, w2, topk_weights, topk_ids, *, w1_scale, w2_scale, group_n, group_k)
 * -- lite_llama/kernels/fused_moe.py:352-438 -- is moe_align_block_size (:45-99), grouped GEMM1
 * (b2l_moe_gemm), silu_and_mul (b2l_swiglu on the two halves, :296-313), grouped GEMM2 with the routing
 * weight folded in (b2l_moe_gemm, :201-205) and moe_sum (:316-333).
 *
 * moe_align_block_size(topk_ids, block_size, num_experts): sorted_token_ids int32
 * [num_slots + E*(block-1)] (sentinel = num_slots), expert_ids int32 [ceil(that / block)],
 * num_tokens_post_padded int32 [1]; topk_ids int32 or int64. */
int b2l_moe_align_block_size(const void* topk_ids, int id_width, int64_t num_slots, int block_size, int num_experts,
                             void* sorted_token_ids, void* expert_ids, void* num_tokens_post_padded, void* stream);
/* C[slot, :] = A[slot / top_k, :] @ W[expert(block)].T (* topk_weights[slot] when non-null).  fp16 activations.
 * weight_kind: 0 = fp16 [E, N, K], B2L_Q_FP8 / B2L_Q_INT8 = 8-bit with fp32 scales
 * [E, ceil(N/group_n), ceil(K/group_k)] (element strides s_stride_*).  block_size in {16, 32, 64}. */
int b2l_moe_gemm(void* c, const void* a, const void* w, int weight_kind, const void* scales,
                 const void* topk_weights, const void* sorted_token_ids, const void* expert_ids,
                 const void* num_tokens_post_padded, int64_t em, int64_t num_valid_slots, int top_k, int block_size,
                 int num_experts, int64_t n, int64_t k, int64_t a_row_stride, int64_t w_row_stride,
                 int64_t c_row_stride, int64_t group_n, int64_t group_k, int64_t s_stride_e, int64_t s_stride_n,
                 int64_t s_stride_k, void* stream);
int b2l_moe_sum(void* out, const void* in, const void* addend, int64_t tokens, int64_t n, int top_k, int dtype,
                void* stream);
/* Router (lite_llama/models/qwen3_moe.py:94-100): fp32 softmax over all experts of the [tokens, E] logits,
 * top-k (ties -> lowest index), optional renormalisation; weights in the activation dtype, ids int64. */
int b2l_moe_route_topk(void* topk_weights, void* topk_ids_i64, const void* router_logits, int64_t row_stride,
                       int64_t tokens, int num_experts, int top_k, int renormalize, int dtype, void* stream);

/* ---- tensor-parallel exchange over NVLink peer memory (csrc/tp_comm.cu) ----
 * Replaces all_reduce_tp (lite_llama/distributed/parallel_state.py:208-213: in-place NCCL SUM of the [tokens, hidden]
 * partial after every row-parallel projection, lite_llama/models/linear.py:160-161, models/qwen3_moe.py:110) TOGETHER
 * WITH the skip_rmsnorm that follows every one of them (lite_llama/models/base.py:307,312,486): one kernel pushes this
 * rank's partial rows into every peer's receive buffer as 16-byte {6 values, epoch} packets (no fence, no separate
 * flag), polls the peers' packets in its own buffer, sums in rank order (fp32, rounded to
 * the activation dtype like the all-reduce output) and applies residual += sum; y = rmsnorm(residual) * weight.
 * One process per GPU: b2l_tp_comm_create allocates this rank's buffer (capacity max_rows x max_row_elems 16-bit
 * elements per peer) and returns an opaque handle (0 on error); b2l_tp_comm_get_handle exports its CUDA IPC handle
 * (b2l_tp_comm_handle_bytes() bytes); the caller all-gathers the handles (torch.distributed) and passes the rank-major
 * concatenation to b2l_tp_comm_open.  weight == NULL: plain all-reduce, y = sum.  Every rank must issue the same call
 * sequence.  Graph-capturable (the double-buffer epoch lives in device memory). */
int64_t b2l_tp_comm_create(int rank, int world, int max_rows, int64_t max_row_elems);
int b2l_tp_comm_handle_bytes(void);
int b2l_tp_comm_get_handle(int64_t comm, void* out, int64_t out_bytes);
int b2l_tp_comm_open(int64_t comm, const void* handles, int64_t handles_bytes);
int b2l_tp_comm_destroy(int64_t comm);
int b2l_tp_allreduce_skip_rmsnorm(int64_t comm, void* y, const void* x_partial, void* residual, const void* weight,
                                  int64_t rows, int64_t n, int64_t x_row_stride, int64_t r_row_stride,
                                  int64_t y_row_stride, float eps, int dtype, void* stream);

/* ---- layer-list models: fp32 residual stream, recurrent mixers, ragged steps -------------------------------------
 * No reference counterpart (the reference serves rotary-attention decoders only).  Every entry point below accepts
 * dtype B2L_F16 / B2L_BF16 / B2L_F32 for the activation AND weight element type; statistics, softmax, recurrent
 * state and the residual stream are fp32 in all of them.  A ragged step is described by int32 device vectors:
 * seq_start [num_seqs + 1] (token offsets into the flat batch), seq_ctx [num_seqs] (tokens the sequence already has
 * in its cache / state), seq_slot [num_seqs] (its row of the request table and its recurrent-state slot). */

/* y = x . w^T (+ bias) on the CUDA cores, fp32 accumulation in ascending k; any shape (csrc/gemm_simt.cu). */
int b2l_gemm_simt(void* y, const void* x, const void* w, const void* bias, int64_t m, int64_t n, int64_t k,
                  int64_t x_row_stride, int64_t w_row_stride, int64_t y_row_stride, int dtype, void* stream);

/* Norm kinds of the entry points below: 0 = RMS (x / sqrt(mean(x^2) + eps)), 1 = layer norm without bias
 * ((x - mean) / sqrt(mean((x - mean)^2) + eps)). */
/* residual[t] = scale * embed[token[t]] + pos_table[pos[t]] (pos_table nullable); act (nullable) gets the copy in dtype. */
int b2l_embed_positions(void* residual_f32, void* act, const void* tokens_i32, const void* pos_i32, const void* embed,
                        const void* pos_table, int64_t rows, int64_t n, int64_t vocab, int64_t max_pos, float scale,
                        int dtype, void* stream);
/* residual += norm(y) * (weight_offset + weight) * layer_scale (nullable): the norm sits on the sublayer OUTPUT.
 * act (nullable) gets the updated residual in dtype, or, with next_weight, the NEXT sublayer's input norm of it:
 * norm'(residual) * next_weight (kind next_norm_kind). */
int b2l_post_norm_residual(void* residual_f32, void* act, const void* y, const void* weight, const void* layer_scale,
                           const void* next_weight, int64_t rows, int64_t n, int64_t y_row_stride, float eps,
                           float weight_offset, int norm_kind, int next_norm_kind, int dtype, void* stream);
/* out[i] = norm(residual[rows[i]]) * (weight_offset + weight); rows_i32 nullable = identity. */
int b2l_rmsnorm_from_f32(void* out, const void* residual_f32, const void* rows_i32, const void* weight, int64_t rows,
                         int64_t n, float eps, float weight_offset, int norm_kind, int dtype, void* stream);
int b2l_relu_squared(void* out, const void* x, int64_t total, int dtype, void* stream);
/* out = gelu(x): exact (erf) form, or the tanh form 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3))). */
int b2l_gelu(void* out, const void* x, int64_t total, int tanh_form, int dtype, void* stream);
/* out_f32 = cap * tanh(scale * x / cap) (cap <= 0: scale * x) as fp32: scaled, soft-capped logits. */
int b2l_softcap_to_f32(void* out_f32, const void* x, int64_t total, float cap, float scale, int dtype, void* stream);
/* y[t, h, :] = W[h] . x[t, h, :] for W [heads, n, k] (csrc/gemm_simt.cu); x / y rows hold the heads side by side
 * (strides in elements); gate (nullable) [m, >= heads]: y[t, h, :] *= sigmoid(gate[t, h]). */
int b2l_head_linear(void* y, int64_t y_row_stride, int64_t y_head_stride, const void* x, int64_t x_row_stride,
                    int64_t x_head_stride, const void* w, const void* gate, int64_t gate_row_stride, int64_t m,
                    int heads, int64_t n, int64_t k, int dtype, void* stream);
/* Grouped product over expert-sorted slots (b2l_moe_align_block_size with block_size = b2l_moe_gemm_simt_block()):
 * c[s, :] = act(W[expert(s)] . a[s / top_k, :]) * slot_weight_f32[s] (nullable); act 0 = none, 1 = exact gelu;
 * W [experts, n, k] dense; every dtype of this section, fp32 sums in ascending k. */
int b2l_moe_gemm_simt_block(void);
int b2l_moe_gemm_simt(void* c, const void* a, const void* w, const void* slot_weight_f32,
                      const void* sorted_token_ids, const void* expert_ids, const void* num_tokens_post_padded,
                      int64_t em, int64_t num_valid_slots, int top_k, int64_t n, int64_t k, int64_t a_row_stride,
                      int64_t c_row_stride, int act, int dtype, void* stream);
/* Tensor-core (mma.sync, fp32 accumulators) versions of b2l_head_linear and b2l_moe_gemm_simt for 16-bit dtypes
 * (csrc/gemm_rows_mma.cu); b2l_rows_gemm_mma_ok says whether they take the operands (k and the x strides multiples
 * of 8 elements, 16-byte aligned bases).  b2l_moe_gemm_mma: block_size 16, 64 or 128 = the block size of the alignment. */
int b2l_rows_gemm_mma_ok(const void* x, const void* w, int64_t k, int64_t x_row_stride, int64_t x_head_stride,
                         int dtype);
int b2l_head_linear_mma(void* y, int64_t y_row_stride, int64_t y_head_stride, const void* x, int64_t x_row_stride,
                        int64_t x_head_stride, const void* w, const void* gate, int64_t gate_row_stride, int64_t m,
                        int heads, int64_t n, int64_t k, int dtype, void* stream);
int b2l_moe_gemm_mma(void* c, const void* a, const void* w, const void* slot_weight_f32, const void* sorted_token_ids,
                     const void* expert_ids, const void* num_tokens_post_padded, int64_t em, int64_t num_valid_slots,
                     int top_k, int block_size, int64_t n, int64_t k, int64_t a_row_stride, int64_t c_row_stride,
                     int act, int dtype, void* stream);
/* Sigmoid scores + selection bias + group-limited top-k (csrc/moe_routing.cu); the router product is done inside
 * unless logits_f32 [tokens, experts] (nullable) brings it:
 * z = router_w . x in fp32, s = sigmoid(z), choice = s + bias (nullable); `groups` equal runs of neighbouring experts,
 * group score = sum of its two largest choice scores, only the `keep` best groups are eligible; the top_k largest
 * choice scores win; weights_f32 [tokens, top_k] = s of the winners / (their sum + 1e-20), or with renormalize 0 the
 * winners' s themselves; ids_i32 [tokens, top_k]. */
int b2l_moe_route_sigmoid_groups(void* weights_f32, void* ids_i32, const void* x, int64_t x_row_stride,
                                 const void* router_w, const void* bias, const void* logits_f32, int64_t tokens,
                                 int num_experts, int64_t k, int top_k, int groups, int keep, int renormalize,
                                 int dtype, void* stream);
/* y_f32[m, n] = x[m, k] . w[n, k]^T: 16-bit operands on the tensor cores, the fp32 sums stored unrounded (router
 * logits); operands as b2l_rows_gemm_mma_ok asks. */
int b2l_linear_f32out_mma(void* y_f32, const void* x, const void* w, int64_t m, int64_t n, int64_t k,
                          int64_t x_row_stride, int64_t y_row_stride, int dtype, void* stream);
/* cos_sin_f32[t] = [cos(pos[t] f_i), i < rot_dims / 2 | sin(pos[t] f_i)] with f_i = base^(-2i / rot_dims), angles in
 * fp64 (csrc/latent_attention.cu); one table per step serves every layer with these rotary constants. */
int b2l_rope_table(void* cos_sin_f32, const void* pos_i32, int64_t tokens, int rot_dims, float rot_base, void* stream);
/* Latent attention, per token of the fused down-projection row [a: q_rank | b: kv_rank | r: rot_dim | ...]:
 * a <- rmsnorm(a) * q_norm_weight in place; pool row kv_rows[t] = [rmsnorm(b) * kv_norm_weight | r with its first
 * rot_dims entries rotated by the token's row of cos_sin_f32 (entry i pairs with i + rot_dims / 2)]. */
int b2l_latent_prepare(void* proj, int64_t proj_row_stride, void* pool, int64_t pool_row_stride,
                       const void* kv_rows_i32, const void* cos_sin_f32, const void* q_norm_weight,
                       const void* kv_norm_weight, int64_t tokens, int q_rank, int kv_rank, int rot_dim, int rot_dims,
                       float eps, int dtype, void* stream);
/* dst[t, h, :width] = src[t, h, :width], the first rot_dims entries rotated by the token's row of cos_sin_f32. */
int b2l_rope_heads(void* dst, int64_t dst_row_stride, int dst_head_stride, const void* src, int64_t src_row_stride,
                   int src_head_stride, const void* cos_sin_f32, int64_t tokens, int heads, int width, int rot_dims,
                   int dtype, void* stream);

/* Short causal convolution per channel + SiLU (activation 1; 0 = none) over a ragged step, and the slot's tail (last
 * taps-1 inputs) update.
 * in: [tokens, >= channels] with row stride; weight [channels, taps] (last column = current token); tail
 * [slots, taps - 1, channels] in dtype. */
int b2l_causal_conv_silu(void* out, const void* in, int64_t in_row_stride, const void* weight, const void* bias,
                         void* tail, const void* seq_start, const void* seq_ctx, const void* seq_slot, int64_t num_seqs,
                         int64_t tokens, int channels, int taps, int activation, int dtype, void* stream);
/* Scalar-decay state-space recurrence (csrc/ssm_scan.cu).  xbc rows = [x: heads*head_dim | B: groups*state | C: ...];
 * state_f32 [slots, heads, state, head_dim] fp32; y_f32 [tokens, heads*head_dim] fp32.  fixed_decay_f32 [heads]
 * (nullable): decayed linear attention S <- decay_h S + B x^T, y = S^T C with dt = 1 and no skip term (dt_raw, dt_bias,
 * a_log, d_skip unused); silu_inputs: SiLU on x, B and C as they are read. */
int b2l_ssm_scan(void* y_f32, void* state_f32, const void* xbc, int64_t xbc_row_stride, const void* dt_raw,
                 int64_t dt_row_stride, const void* dt_bias, const void* a_log, const void* d_skip,
                 const void* seq_start, const void* seq_ctx, const void* seq_slot, int64_t num_seqs, int heads,
                 int groups, int state_size, int head_dim, const void* fixed_decay_f32, int silu_inputs, int dtype,
                 void* stream);
/* The fixed-decay case of b2l_ssm_scan with SiLU inputs, over prompt portions in chunks of 64 tokens on the tensor
 * cores (csrc/decay_attention_mma.cu): same y_f32 and state_f32; x rows = [v: heads*head_dim | k: heads*state_size |
 * q: heads*state_size].  b2l_decay_attention_mma_ok: 16-bit dtype, both sizes in {32, 64, 128}, 16-byte aligned rows. */
int b2l_decay_attention_mma_ok(const void* x, int64_t x_row_stride, int state_size, int head_dim, int dtype);
int b2l_decay_attention_mma(void* y_f32, void* state_f32, const void* x, int64_t x_row_stride, const void* decay_f32,
                            const void* seq_start, const void* seq_ctx, const void* seq_slot, int64_t num_seqs, int heads,
                            int state_size, int head_dim, int dtype, void* stream);
/* out = unit_rms(y * silu(z)) * weight, the unit RMS taken in `groups` equal parts of the row. */
int b2l_gated_group_norm(void* out, const void* y_f32, const void* z, int64_t z_row_stride, const void* weight,
                         int64_t rows, int inner, int groups, float eps, int dtype, void* stream);

/* Per token of a fused [q | k | v] projection: whole-row RMS norm of q and k with plain weights (nullable = none),
 * query gain 1 + gain_coef * ln(floor((pos + 1) / gain_every) + 1) (gain_every <= 0: none), value mixing
 * v <- (1 - lambda) v + lambda v_first_in (nullable), copy of the unmixed v to v_first_out (nullable), and the
 * K|V write into pool row kv_rows[t].  q is updated in place. */
int b2l_attn_prepare(void* qkv, int64_t qkv_row_stride, void* kv_pool, int64_t kv_row_stride, const void* kv_rows_i32,
                     const void* pos_i32, const void* q_norm_weight, const void* k_norm_weight, const void* v_first_in,
                     void* v_first_out, const void* v_lambda, int64_t tokens, int q_cols, int k_cols, int v_cols,
                     float eps, float gain_coef, float gain_every, int dtype, void* stream);
/* Soft-capped attention with an optional per-head sink over the pool (csrc/attention_sink.cu).  num_splits == 0: tiled
 * mode for sequences of up to max_q_len new tokens; num_splits > 0: every listed sequence brings one token, its keys
 * (from the first one it sees) are cut into num_splits ranges of split_keys and merged (workspace:
 * b2l_sink_attention_workspace_bytes).  window > 0: token p sees keys p - window + 1 .. p only; block > 0 (window <= 0):
 * token p sees keys floor(p / block) * block .. p only.  v_col0 < 0: a pool
 * row is [keys | values]; v_col0 >= 0: the values start at that column (0: they are the keys' leading columns).
 * v_blocks > 1 (num_splits > 0 only): v_blocks neighbouring blocks of v_head_dim value columns in one call, each as
 * `heads` more results (out [v_blocks][heads][v_head_dim] per token; workspace for heads * v_blocks heads). */
int64_t b2l_sink_attention_workspace_bytes(int64_t num_seqs, int heads, int v_head_dim, int num_splits);
int b2l_sink_attention(void* out, int64_t out_row_stride, const void* q, int64_t q_row_stride, const void* kv_pool,
                       int64_t kv_row_stride, const void* table_i32, int64_t table_row_stride, const void* seq_start,
                       const void* seq_ctx, const void* seq_slot, const void* seq_list, int64_t num_seqs,
                       int max_q_len, const void* sink, int heads, int kv_heads, int head_dim, int v_head_dim,
                       float scale, float softcap, int window, int block, int v_col0, int v_head_stride,
                       int v_blocks, int num_splits, int split_keys, void* workspace, int64_t workspace_bytes, int dtype,
                       void* stream);
/* One new token per listed sequence, the heads' softmax weights mixed across heads before the values:
 * p'_h(j) = sum_g mix[h, g] p_g(j), out_h = sum_j p'_h(j) v_kv(h)(j).  mix [heads, heads] has q's element type.  max_keys
 * bounds the keys any listed token sees (window, or context + 1); the workspace holds num_seqs * heads * max_keys fp32
 * weights.  Mask and value-column arguments as in b2l_sink_attention. */
int64_t b2l_mixed_head_attention_workspace_bytes(int64_t num_seqs, int heads, int max_keys);
int b2l_mixed_head_attention(void* out, int64_t out_row_stride, const void* q, int64_t q_row_stride, const void* kv_pool,
                             int64_t kv_row_stride, const void* table_i32, int64_t table_row_stride, const void* seq_start,
                             const void* seq_ctx, const void* seq_slot, const void* seq_list, int64_t num_seqs,
                             const void* mix, int heads, int kv_heads, int head_dim, int v_head_dim, float scale,
                             float softcap, int window, int block, int v_col0, int max_keys, void* workspace,
                             int64_t workspace_bytes, int dtype, void* stream);

/* Parallel-block layer-list models with a depth-weighted residual stack (csrc/parallel_stream.cu).
 * embed_rmsnorm: residual_f32[t] = unit_rms(scale * embed[token[t]]) * (weight_offset + weight) (weight nullable).
 * depth_mix_norms: x = sum_j coef[j] * stack[j] over `count` levels `level_stride` floats apart (coef NULL: x = the last
 * level), written to x_out_f32 (nullable when n % 4 == 0 and n <= 8192), h1 = unit_rms(x) * (offset + w1), h2 likewise
 * (both nullable).  branch_sum_residual: residual += scale * a' + scale_b * b' + c with a' = unit_rms(a) * a_weight when
 * the weight is given, else a (b likewise; b, c nullable); act (nullable) = the new residual in dtype, or, with
 * next_weight, unit_rms(new residual) * next_weight (the input norm of the block that follows).
 * gelu_mul_gather: out[t, d] = gelu_tanh(z[t, d]) * table[token[t], col0 + d], d < dim. */
int b2l_embed_rmsnorm(void* residual_f32, const void* tokens_i32, const void* embed, const void* weight, int64_t rows,
                      int64_t n, int64_t vocab, float eps, float weight_offset, float scale, int dtype, void* stream);
int b2l_depth_mix_norms(void* x_out_f32, void* h1, void* h2, const void* stack_f32, int64_t level_stride,
                        const void* coef, int count, const void* w1, const void* w2, int64_t rows, int64_t n, float eps,
                        float weight_offset, int dtype, void* stream);
int b2l_branch_sum_residual(void* residual_f32, void* act, const void* a, int64_t a_row_stride, const void* a_weight,
                            const void* b, int64_t b_row_stride, const void* b_weight, const void* c,
                            int64_t c_row_stride, const void* next_weight, int64_t rows, int64_t n, float eps,
                            float scale, float scale_b, int dtype, void* stream);
int b2l_gelu_mul_gather(void* out, const void* z, int64_t z_row_stride, const void* tokens_i32, const void* table,
                        int64_t table_row_stride, int64_t vocab, int col0, int dim, int64_t rows, int dtype,
                        void* stream);

/* Element-wise gated recurrences S_t = a_t S_(t-1) + b_t, o_t = S_t g_t over a ragged step (csrc/gated_recurrence.cu).
 * mode 0 (minimal GRU): p0 / p1 / p2 = update-gate, candidate, output-gate pre-activations.  mode 1 (real-gated LRU):
 * p0 = recurrence input, p1 / p2 = recurrence- / input-gate pre-activations (+ bias_r / bias_i), p3 = pre-activation
 * of the gelu branch, a = exp(-decay_scale * r * softplus(lam)).  state_f32 [slots, width]. */
int b2l_gated_scan(void* out, int64_t out_row_stride, void* state_f32, const void* p0, int64_t p0_row_stride,
                   const void* p1, int64_t p1_row_stride, const void* p2, int64_t p2_row_stride, const void* p3,
                   int64_t p3_row_stride, const void* bias_r, const void* bias_i, const void* lam, float decay_scale,
                   const void* seq_start, const void* seq_ctx, const void* seq_slot, int64_t num_seqs, int width,
                   int mode, int dtype, void* stream);
/* out = unit_rms(y_f32) * weight * sigmoid(z) over whole rows of n. */
int b2l_norm_sigmoid_gate(void* out, const void* y_f32, const void* z, int64_t z_row_stride, const void* weight,
                          int64_t rows, int n, float eps, int dtype, void* stream);

/* Linear attention with data-dependent gates over a ragged step (csrc/gated_linear_attention.cu); state_f32 [slots,
 * heads, dim, vdim] is advanced in place, y_f32 [tokens, heads * vdim].
 * mode 0, forget-gate form: q [tokens, heads*dim] pre-activation (SiLU inside), k = forget-gate logits [tokens,
 * heads*dim], c0 = lower bounds [heads*dim]: f = c0 + (1 - c0) sigmoid(k); S[d,:] <- f[d] S[d,:] + (1 - f[d]) v; o = S^T q.
 * mode 1, gated delta rule: q, k [tokens, qk_heads*dim] (made unit vectors with unit_eps inside the root; q times
 * q_scale), p0 / p1 = write-strength and decay logits [tokens, heads], c0 = dt_bias, c1 = A_log [heads]:
 * g = exp(-exp(c1) softplus(p1 + c0)), S <- g S, u = sigmoid(p0) (v - S^T k), S <- S + k u^T, o = S^T q. */
int b2l_gated_linear_scan(void* y_f32, void* state_f32, const void* q, int64_t q_row_stride, const void* k,
                          int64_t k_row_stride, const void* v, int64_t v_row_stride, const void* p0,
                          int64_t p0_row_stride, const void* p1, int64_t p1_row_stride, const void* c0, const void* c1,
                          const void* seq_start, const void* seq_ctx, const void* seq_slot, int64_t num_seqs, int heads,
                          int qk_heads, int dim, int vdim, float q_scale, float unit_eps, int mode, int dtype,
                          void* stream);
/* out[t, h, :] = unit_rms(y_f32[t, h, :]) * weight[vdim] * silu(gate[t, h, :]) (gate nullable: no gate). */
int b2l_head_norm_gate(void* out, const void* y_f32, const void* gate, int64_t gate_row_stride, const void* weight,
                       int64_t rows, int heads, int vdim, float eps, int dtype, void* stream);
/* out[t, h, :] = sum_g mix[h, g] * wide[t, g, kv(h), :] for wide [rows, calls, heads, per_call, vdim] (kv head c of
 * query head g lies at call c / per_call, part c % per_call): softmax weights mixed across heads, on the outputs. */
int b2l_head_mix(void* out, const void* wide, int64_t wide_row_stride, const void* mix, int64_t rows, int heads,
                 int kv_heads, int per_call, int vdim, int dtype, void* stream);
/* out[r, :] = silu(s_r * gate[r, :]) * (s_r * up[r, :]) * sigmoid(z[r]); in_scale_f32 [rows] and z (one value per row,
 * row stride given) are nullable. */
int b2l_swiglu_scaled(void* out, int64_t out_row_stride, const void* gate, int64_t gate_row_stride, const void* up,
                      int64_t up_row_stride, const void* in_scale_f32, const void* z, int64_t z_row_stride, int64_t rows,
                      int64_t n, int dtype, void* stream);

/* Rotary table from given per-pair frequencies (csrc/rotary_heads.cu): cos_sin_f32[t] = magnitude * [cos(pos f_i) |
 * sin(pos f_i)], fp64 frequencies and angles.  head_norm_rope_prepare: per token of a fused [q | k | v] row, per-head RMS norm of q and
 * k with one [head_dim] weight each (nullable), rotation of the first rot_dims entries (pairing 0: neighbours 2i, 2i+1;
 * 1: i and i + rot_dims / 2), q in place, k and v into pool row kv_rows[t]. */
int b2l_rope_table_freqs(void* cos_sin_f32, const void* pos_i32, const void* freqs_f64, int64_t tokens, int rot_dims,
                         float magnitude, void* stream);
int b2l_head_norm_rope_prepare(void* qkv, int64_t qkv_row_stride, void* kv_pool, int64_t kv_row_stride,
                               const void* kv_rows_i32, const void* cos_sin_f32, const void* q_norm_weight,
                               const void* k_norm_weight, int64_t tokens, int heads, int kv_heads, int head_dim,
                               int v_head_dim, int rot_dims, int pairing, float eps, int dtype, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200_LITE_KERNELS_H */
