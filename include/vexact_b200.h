/*
 * libvexact_b200: C ABI of the B200 (sm_100a) rollout-forward kernels.
 *
 * Every function
 *   - takes raw device pointers, explicit sizes, element strides and a cudaStream_t
 *     (passed as void*; NULL = the legacy default stream),
 *   - launches on that stream, allocates nothing and does not synchronise
 *     (b200_status_read excepted), so it can be captured in a CUDA graph,
 *   - returns 0 when the work was launched and a negative code otherwise:
 *       -1 invalid argument, -2 unsupported shape, -3 CUDA launch error,
 *       -4 driver entry point (tensor-map encoder) unavailable.
 * Nothing is reported from the device except through the status word read by
 * b200_status_read (bounded waits that expired, out-of-range slot / expert ids).
 *
 * bf16 tensors are `__nv_bfloat16`, row-major with the innermost dimension
 * contiguous unless a stride says otherwise.  Strides are in elements.
 *
 * Each declaration names the reference interface (path inside verl-project/vexact)
 * that it stands in for.
 */
#ifndef VEXACT_B200_H
#define VEXACT_B200_H

#ifdef __cplusplus
extern "C" {
#endif

/* Changes whenever an exported signature changes or an entry point is added (currently 4). */
int b200_abi_version(void);

/* Hash of the sources and compiler flags the binary was built from: the Python loader compares it with
 * the sources next to it, so that a library left over from an older checkout is never bound to newer
 * argument lists.  No counterpart in the reference (it ships no compiled code). */
const char* b200_source_hash(void);

/* Self-test of the bounded device wait: one CTA waits limit_us microseconds (1..1000000) on an mbarrier that
 * nothing completes; the wait must expire, put {1 (wait expired), 999, ...} into the status word and let the
 * kernel return.  out_flag_device[0] (int32, device) becomes 1.  No counterpart in the reference. */
int b200_selftest_wait_expiry(int limit_us, int* out_flag_device, void* stream);

/* Reads {code, detail, block, spare} of the device status word into host_out4 and clears it.
 * Synchronises `stream`.  code: 0 ok, 1 a bounded wait expired, 2 an index was out of range. */
int b200_status_read(int* host_out4, void* stream);

/* ---- vexact/batch_invariant_ops/batch_invariant_ops.py:159 matmul_persistent(a, b, bias),
 *      :476 mm_batch_invariant, :480 addmm_batch_invariant.
 * out[T, N] = x[T, K] @ w[N, K]^T (+ bias[N] in fp32 before the cast).  `w` is the
 * nn.Linear weight itself ([N, K], K contiguous): the reference receives weight.t().
 * K and the row strides must be multiples of 8 elements; pointers 16-byte aligned.
 * out_dtype: 0 = bf16, 1 = fp32. */
int b200_gemm_bf16(const void* x, const void* w, const void* bias, void* out, long long T, int N, int K,
                   long long x_row_stride, long long w_row_stride, long long out_row_stride, int out_dtype,
                   void* stream);
/* The same GEMM on fp16 tensors (matmul_persistent serves bf16, fp16 and fp32, batch_invariant_ops.py:181-189):
 * fp32 accumulation in the same K order, bias (fp16) added in fp32, one rounding.  out_dtype 0 = f16, 1 = f32. */
int b200_gemm_f16(const void* x, const void* w, const void* bias, void* out, long long T, int N, int K,
                  long long x_row_stride, long long w_row_stride, long long out_row_stride, int out_dtype,
                  void* stream);

/* fp32 variant for the DeepSeek-V3 router (vexact/models/deepseek_v3/modeling_deepseek_v3.py:97-100,
 * F.linear in fp32, reaching matmul_persistent with fp32 operands).  Exact fp32 FMA arithmetic. */
int b200_gemm_f32(const void* x, const void* w, const void* bias, void* out, long long T, int N, int K,
                  long long x_row_stride, long long w_row_stride, long long out_row_stride, void* stream);

/* Same product on bf16 tensors widened to fp32 on the fly: bit-identical to b200_gemm_f32 on x.float(),
 * w.float() (the router module's casts), without the fp32 copies. */
int b200_gemm_f32_from_bf16(const void* x, const void* w, void* out, long long T, int N, int K,
                            long long x_row_stride, long long w_row_stride, long long out_row_stride, void* stream);

/* ---- vexact/batch_invariant_ops/batch_invariant_ops.py:728 batch_invariant_rms_norm (mode 0:
 *      fp32 math, one rounding) and the HF eager RMSNorm the reference reaches through its
 *      aten::mean.dim override, :619 mean_batch_invariant (mode 1: x*rsqrt(var+eps) rounded to
 *      bf16, then multiplied by the weight). */
int b200_rmsnorm(const void* x, const void* weight, void* out, long long rows, int n, long long x_row_stride,
                 long long out_row_stride, float eps, int mode, void* stream);

/* ---- vexact/batch_invariant_ops/batch_invariant_ops.py:701-725 BatchInvariantRMSNormFunction.backward (the
 *      training-side twin of mode 0): grad_in = inv * (d - normed * mean(d * normed)) with d = grad_out * w,
 *      grad_weight = sum over rows of grad_out * normed, reduced in a fixed order (64-row partials, then the
 *      partials ascending).  All tensors bf16 contiguous; scratch_f32 holds rows + ceil(rows / 64) * n floats. */
int b200_rmsnorm_backward(const void* x, const void* weight, const void* grad_out, void* grad_in, void* grad_weight,
                          void* scratch_f32, long long rows, int n, float eps, void* stream);

/* sum_out = bf16(residual + x); out = rmsnorm(sum_out).  All tensors [rows, n] contiguous.
 * The decoder layer's "residual add, then norm" (HF Qwen3DecoderLayer.forward) in one pass. */
int b200_add_rmsnorm(const void* x, const void* residual, const void* weight, void* sum_out, void* out,
                     long long rows, int n, float eps, int mode, void* stream);

/* ---- vexact/batch_invariant_ops/batch_invariant_ops.py:385 mean_dim (last dimension only).
 * dtype: 0 = fp32, 1 = bf16 (input and output). */
int b200_mean_lastdim(const void* x, void* out, long long rows, int n, long long x_row_stride, int dtype,
                      void* stream);

/* ---- vexact/batch_invariant_ops/batch_invariant_ops.py:295 log_softmax (fp32, last dim). */
int b200_log_softmax_f32(const void* x, void* out, long long rows, int n, long long x_row_stride,
                         long long out_row_stride, void* stream);

/* ---- vexact/batch_invariant_ops/standalone_logprobs.py:28 logprobs_from_logits_flash_attn.
 * out[r] = logits[r, labels[r]] - logsumexp(logits[r, :]) in fp32; 0 where labels[r] == ignore_index.
 * labels are int64.  dtype of logits: 0 = fp32, 1 = bf16. */
int b200_gather_logprob(const void* logits, const void* labels, void* out, long long rows, int n,
                        long long row_stride, int dtype, long long ignore_index, void* stream);

/* Gradient of b200_gather_logprob with respect to the logits (the backward of flash-attn's cross_entropy_loss, which
 * standalone_logprobs.py:28 wraps, with a log-probability's sign): dlogits[r, i] = grad_out[r] * ((i == label[r]) -
 * softmax(logits[r])[i]), in the logits' dtype, a zero row for an ignored label.  dlogits may be logits itself
 * (`inplace_backward=True`). */
int b200_gather_logprob_backward(const void* logits, const void* labels, const void* grad_out_f32, void* dlogits,
                                 long long rows, int n, long long row_stride, long long d_row_stride, int dtype,
                                 long long ignore_index, void* stream);

/* ---- vexact/inferencer/inferencer.py:393-449 _select_tokens for greedy decoding: the argmax of each
 *      row of logits (lowest index on ties) and that token's log-probability (the value
 *      logprobs_from_logits_flash_attn returns for it), in one pass.  tokens int64, logprobs fp32. */
int b200_greedy_logprob(const void* logits, void* tokens_i64, void* logprobs_f32, long long rows, int n,
                        long long row_stride, int dtype, void* stream);

/* ---- vexact/inferencer/inferencer.py:393-449 _select_tokens for greedy requests, fused with the lm_head
 *      projection (model_loader.py:267-268): tokens[t] = argmax_v(bf16(x[t] . w[v])) (lowest index on ties),
 *      logprobs[t] = that logit's log-softmax, without storing the [T, V] logits.  `partials` is scratch of
 *      T * ceil(V / 128) * 16 bytes (device).  Two launches: the GEMM with a reducing epilogue, then a fold
 *      per token in a fixed order (results do not depend on T).  Same token as b200_gemm_bf16 +
 *      b200_greedy_logprob; log-probability within 2e-5 of theirs. */
int b200_lm_head_greedy(const void* x, const void* w, void* partials, void* tokens_i64, void* logprobs_f32,
                        long long T, int V, int K, long long x_row_stride, long long w_row_stride, void* stream);

/* ---- vexact/inferencer/sampler.py:32-87 Sampler.batch_sample_token with uniform sampling
 *      parameters (temperature, top-k :168-173, top-p :175-181, arg-max of probs / q :146), fused
 *      with the chosen token's log-probability on the raw logits (inferencer.py:436-441).
 * noise_q_f32 [rows, n]: one draw of Exp(1) per logit (torch's exponential_(), as the reference
 * makes); NULL, temperature <= 0 or top_p <= 0 select the arg-max path (= b200_greedy_logprob).
 * top_k <= 0 or >= n: no top-k; top_p >= 1: no top-p.  tokens int64, logprobs fp32.
 * dtype of logits: 0 = fp32, 1 = bf16 (cast to fp32 first, as the reference does). */
int b200_sample_token(const void* logits, const void* noise_q_f32, void* tokens_i64, void* logprobs_f32,
                      long long rows, int n, long long row_stride, long long q_row_stride, int dtype,
                      float temperature, int top_k, float top_p, void* stream);

/* ---- vexact/inferencer/sampler.py:146-186 apply_top_k_top_p as an operator of its own: out[r, i] =
 *      logits[r, i] / temperature where token i survives top-k (ties with the k-th value kept) and top-p
 *      (ascending cumulative mass <= 1 - p masked, at least one kept), -inf elsewhere; fp32 [rows, n].
 *      Same thresholds as b200_sample_token.  top_k <= 0 / top_p >= 1 switch the respective cut off. */
int b200_apply_top_k_top_p(const void* logits, void* out_f32, long long rows, int n, long long row_stride,
                           long long out_row_stride, int dtype, float temperature, int top_k, float top_p,
                           void* stream);

/* ---- modeling_qwen3_moe.py:128-134 routing + fused_moe.py:268-292 index math in two launches instead of three:
 *      b200_moe_route_plan_softmax_topk routes like b200_moe_route_softmax_topk and also gives every selected
 *      (token, expert) its rank inside the expert's group (an atomic counter per expert) and, from the last CTA to
 *      finish, cu_seqlens and the token-tile table; b200_moe_scatter_ranked then writes the expert-sorted copy,
 *      row_scale and scatter_index.  Rows keep no particular order inside an expert's group (it varies from run
 *      to run), which changes no output of the MoE; the reference's index arrays are reproduced by
 *      b200_moe_permute.  counters_i32: 257 int32, zero before the first call, left zero by every call; calls
 *      sharing it must not overlap on the GPU. */
int b200_moe_route_plan_softmax_topk(const void* logits, int logits_dtype, long long row_stride, void* weights_bf16,
                                     void* experts_i64, void* rank_i32, void* counters_i32, void* cu_seqlens,
                                     void* tile_table, void* tile_count, long long T, int E, int topk, int renorm,
                                     int tile_rows, int max_tiles, void* stream);
int b200_moe_scatter_ranked(const void* x, long long x_row_stride, const void* experts_i64, const void* weights_bf16,
                            const void* rank_i32, const void* cu_seqlens, void* scatter_index, void* x_perm,
                            void* row_scale, long long T, int topk, int E, int H, void* stream);

/* ---- HF nn.Embedding on input_ids, and vexact/inferencer/inferencer.py:403-404 (each sequence's last-token row:
 *      hidden[query_start_loc[1:] - 1]) as one row-gather kernel instead of torch indexing kernels:
 *      out[t, :] = src[ids[t], :] (ids int64), or with ids_i64 == NULL src[max(query_start_loc[t + 1] - 1, 0), :].
 *      src rows src_row_stride elements apart, out [T, H] contiguous bf16, H % 8 == 0.  An index outside
 *      [0, src_rows) is reported in the status word (code 2) and reads row 0. */
int b200_gather_rows(const void* src, long long src_rows, long long src_row_stride, const void* ids_i64,
                     const void* query_start_loc_i32, void* out, long long T, int H, void* stream);

/* ---- vexact/inferencer/sampler.py:57-63, 90-118 seeded sampling (per-request seed, keyed by token position):
 *      fills noise_q_f32 [rows, n] with Exp(1) draws from Philox4x32-10 (key = seeds[r], counter = (column / 4,
 *      positions[r], 0)), to be passed to b200_sample_token.  A request's draws depend on its seed, the position
 *      and the column only.  Same construction as the vLLM kernel the reference calls, not the same stream. */
int b200_seeded_exponential(void* noise_q_f32, const void* seeds_i64, const void* positions_i64, long long rows,
                            int n, long long q_row_stride, void* stream);

/* ---- vexact/inferencer/inferencer.py:193-291 Inferencer._prepare_gen_ctx and :293-349
 *      _prepare_input_buffers_from_gen_ctx: one scheduler step's padded input buffers, built on the
 *      device from per-request counters instead of per-token host loops.
 * Per request i (device arrays): num_computed_tokens[i] (= context length after this step),
 * tokens_this_step[i], row i of block_tables_in [num_seqs, max_blocks] (-1 beyond the request's
 * blocks), prefill_offset[i] = offset of the request's first token of this step in prefill_ids
 * (int64, packed) or -1 for a decode request, which feeds last_tokens[i] (int64, e.g. the previous
 * step's sampled tokens, still on the device).  prefill_ids / prefill_offset / last_tokens may be NULL.
 * Outputs (all sizes are the captured graph's): input_ids, position_ids int64 [capture_tokens]
 * (0 beyond the step's tokens), slot_mapping int32 [capture_tokens] (-1 beyond), context_lens
 * [graph_num_seqs] (0 for padded requests), query_start_loc [graph_num_seqs + 1] (padded entries =
 * total tokens), block_tables_out [graph_num_seqs, max_blocks] (padded rows 0), step_info[2] =
 * {total tokens, max tokens_this_step}.  num_seqs <= 8192.  A request whose block is missing or whose
 * start is negative gets slot -1 and sets the status word (b200_status_read). */
int b200_prepare_step(const int* num_computed_tokens, const int* tokens_this_step, const int* block_tables_in,
                      const long long* prefill_ids, const int* prefill_offset, const long long* last_tokens,
                      int num_seqs, int graph_num_seqs, int capture_tokens, int max_blocks, int page_size,
                      long long* input_ids, long long* position_ids, int* slot_mapping, int* context_lens,
                      int* query_start_loc, int* block_tables_out, int* step_info, void* stream);

/* ---- vexact/batch_invariant_ops/kv_cache_context.py:294 store_kvcache.
 * key [T, heads, dk], value [T, heads, dv] (token strides given, heads*dim contiguous);
 * caches [blocks, page, heads, d] contiguous; slot_mapping int32 [T], -1 = skip.
 * num_slots = blocks * page bounds the slot ids. */
int b200_kv_store(const void* key, const void* value, void* k_cache, void* v_cache, const void* slot_mapping,
                  long long num_tokens, int num_kv_heads, int k_head_dim, int v_head_dim,
                  long long k_token_stride, long long v_token_stride, long long num_slots, void* stream);

/* Fused per-head q/k RMSNorm (optional, HF formula) + rotary embedding + KV-cache store for
 * head_dim 128: what HF Qwen3Attention / Qwen2Attention.forward does between the QKV
 * projection and the attention call, followed by store_kvcache (kv_cache_context.py:294).
 * qkv [T, (q_heads + 2 kv_heads) * 128] bf16; positions int64 [T]; inv_freq fp32 [64]. */
int b200_qknorm_rope_store(const void* qkv, long long qkv_token_stride, const void* positions,
                           const void* slot_mapping, const void* q_norm_weight, const void* k_norm_weight,
                           const void* inv_freq, void* q_out, void* k_cache, void* v_cache,
                           long long num_tokens, int num_q_heads, int num_kv_heads, int head_dim,
                           long long num_slots, float eps, void* stream);

/* ---- vexact/models/deepseek_v3/modeling_deepseek_v3.py:225-283 deepseek_v3_attention_forward, the part
 *      between the projections and the attention call (split nope / rope, interleaved rotary embedding
 *      with the deterministic cos/sin of :409-436, k_rot expanded to every head, concat) followed by
 *      store_kvcache.  q [T, heads, nope + 64]; kvb [T, heads, nope + dv] (kv_b_proj output);
 *      k_rot [T, 64]; positions int64; inv_freq fp32 [32]; caches [blocks, page, heads, nope + 64 | dv]. */
int b200_mla_rope_store(const void* q, long long q_token_stride, const void* kvb, long long kvb_token_stride,
                        const void* k_rot, long long k_rot_token_stride, const void* positions,
                        const void* slot_mapping, const void* inv_freq, void* q_out, void* k_cache,
                        void* v_cache, long long num_tokens, int num_heads, int qk_nope_dim, int qk_rope_dim,
                        int v_dim, long long num_slots, void* stream);

/* ---- vexact/batch_invariant_ops/triton_invariant_attention.py:905 flash_attn_varlen_func with a
 *      page table (:605 _PagedFlashAttentionVarlen, kernel :434) and the FA3 / FA4 calls of
 *      vexact/batch_invariant_ops/flash_attention.py:142-178.  Causal only.
 * (dk, dv) in {(128,128), (192,128), (64,64)}; page_size a multiple of 8 that divides, or is a
 * multiple of, 64; query heads per KV head <= 8 or a multiple of 8. */
int b200_paged_attn_fwd(const void* q, const void* k_cache, const void* v_cache, void* out,
                        const void* cu_seqlens_q, const void* seqused_k, const void* page_table, int num_seqs,
                        int max_seqlen_q, int num_q_heads, int num_kv_heads, int dk, int dv, int num_blocks,
                        int page_size, int max_pages, long long page_table_stride, long long q_tok_stride,
                        long long q_head_stride, long long o_tok_stride, long long o_head_stride,
                        long long kc_block_stride, long long kc_page_stride, long long kc_head_stride,
                        long long vc_block_stride, long long vc_page_stride, long long vc_head_stride,
                        float softmax_scale, void* stream);

/* Same call with a processing order for ragged batches: seq_order (int32 [num_seqs], a permutation,
 * typically sequences by descending context length; may be NULL) names the sequence each group of
 * tiles belongs to.  The persistent tcgen05 kernel deals tiles to its CTAs round by round, so a
 * longest-first order keeps the CTAs' totals within about one tile of each other.  Results do not
 * depend on the order.  No counterpart in the reference (its grid is one program per head and tile).
 * total_q: number of rows of q (0 = not known); with it, tiles of 128 queries fetch their queries by TMA
 * (rows past total_q read as zeros) instead of through a loader warp.  Results do not depend on it either. */
int b200_paged_attn_fwd_ordered(const void* q, const void* k_cache, const void* v_cache, void* out,
                                const void* cu_seqlens_q, const void* seqused_k, const void* page_table,
                                int num_seqs, int max_seqlen_q, int num_q_heads, int num_kv_heads, int dk, int dv,
                                int num_blocks, int page_size, int max_pages, long long page_table_stride,
                                long long q_tok_stride, long long q_head_stride, long long o_tok_stride,
                                long long o_head_stride, long long kc_block_stride, long long kc_page_stride,
                                long long kc_head_stride, long long vc_block_stride, long long vc_page_stride,
                                long long vc_head_stride, float softmax_scale, const void* seq_order,
                                long long total_q, void* stream);

/* ---- vexact/batch_invariant_ops/triton_invariant_attention.py:194-431 (_varlen_attn_bwd_dq_kernel,
 *      _varlen_attn_bwd_dkv_kernel): dq, dk, dv of the packed (non-paged) causal varlen attention.  All tensors
 *      bf16 and contiguous: q / dq [total_q, hq, dk_dim], k / dk [total_k, hkv, dk_dim], v / dv [total_k, hkv,
 *      dv_dim], out / dout [total_q, hq, dv_dim]; cu_seqlens_q / _k [num_seqs + 1] int32; lse / delta: fp32
 *      scratch [total_q, hq] each (the log-sum-exp is recomputed here, the forward does not save it).
 *      (dk_dim, dv_dim) in {(64, 64), (128, 128), (192, 128)}.  p and ds are rounded to bf16 before their
 *      products as in the reference; fp32 accumulation in a fixed order, no atomics.  A training-side operator
 *      on mma.sync tensor-core instructions (B200_ATTN_BWD_SIMT=1: the CUDA-core form).  Pass zero-filled dq /
 *      dk / dv: rows of no sequence are not written. */
int b200_varlen_attn_backward(const void* q, const void* k, const void* v, const void* out, const void* dout,
                              const void* cu_seqlens_q, const void* cu_seqlens_k, void* dq, void* dk, void* dv,
                              void* lse_scratch_f32, void* delta_scratch_f32, int num_seqs, int max_seqlen_q,
                              int max_seqlen_k, long long total_q, long long total_k, int num_q_heads,
                              int num_kv_heads, int dk_dim, int dv_dim, float softmax_scale, void* stream);

/* ---- vexact/models/qwen3_moe/modeling_qwen3_moe.py:128-134 (softmax, top-k, renormalise, cast).
 * logits_dtype: 0 = fp32, 1 = bf16.  Any of the four outputs may be NULL except that one weight
 * and one expert output are required. */
int b200_moe_route_softmax_topk(const void* logits, int logits_dtype, long long row_stride, void* weights_bf16,
                                void* weights_f32, void* experts_i32, void* experts_i64, long long T, int E,
                                int topk, int renorm, void* stream);

/* ---- vexact/models/deepseek_v3/modeling_deepseek_v3.py:185-208 route_tokens_to_experts. */
int b200_moe_route_sigmoid_group_topk(const void* logits_f32, long long row_stride, const void* bias_f32,
                                      void* weights_f32, void* experts_i32, void* experts_i64, long long T,
                                      int E, int n_group, int topk_group, int topk, int renorm, float scale,
                                      void* stream);

/* ---- vexact/batch_invariant_ops/fused_moe.py:268 _build_moe_indices and
 *      group_gemm/kernel/moe.py:304 moe_scatter.  Outputs are caller-provided scratch:
 *      scatter_index [T*topk] i32, cu_seqlens [E+1] i32, x_perm [T*topk, H] bf16,
 *      row_scale [T*topk] bf16, tile_table [max_tiles] int4, tile_count [1] i32. */
int b200_moe_permute(const void* experts, int experts_dtype, const void* weights_bf16, const void* x,
                     long long x_row_stride, void* scatter_index, void* cu_seqlens, void* x_perm,
                     void* row_scale, void* tile_table, void* tile_count, long long T, int topk, int E, int H,
                     int tile_rows, int max_tiles, void* stream);

/* ---- vexact/batch_invariant_ops/fused_moe.py:319-339 (quack gemm with cu_seqlens_m) /
 *      group_gemm/kernel/group_gemm.py:156 group_gemm_same_nk.
 * mode 0: out[r, :] = x[r, :] @ w[g(r)]^T, w [G, n_out, K].
 * mode 1: out[r, i] = silu(x.w[g, i]) * (x.w[g, n_out + i]) * row_scale[r], w [G, 2*n_out, K]
 *         (gate rows first), each intermediate rounded to bf16 as in fused_moe.py:325-336. */
int b200_moe_grouped_gemm(const void* x, const void* w, const void* row_scale, void* out,
                          const void* tile_table, const void* tile_count, long long x_rows, int num_groups,
                          int n_out, int K, long long out_row_stride, int max_tiles, int tile_rows_max, int mode,
                          void* stream);

/* ---- vexact/batch_invariant_ops/fused_moe.py:268-292 _build_moe_indices + :319-322 quack gemm(A, ..., A_idx=):
 *      the permutation without the permuted copy.  b200_moe_permute_index writes scatter_index, cu_seqlens and
 *      the tile table like b200_moe_permute, plus gather_index [T*topk] i32 (sorted row -> token: the
 *      reference's A_idx) and row_scale [T*topk] bf16 (routing weight of each sorted row; may be null), in one
 *      launch.  b200_moe_grouped_gemm_gather is b200_moe_grouped_gemm reading sorted row r from
 *      x[gather_index[r]] of the unpermuted x [T, K] (rows x_row_stride elements apart); same bits as the
 *      GEMM on the permuted copy.  tile_rows_max <= 128. */
int b200_moe_permute_index(const void* experts, int experts_dtype, const void* weights_bf16, void* scatter_index,
                           void* cu_seqlens, void* gather_index, void* row_scale, void* tile_table,
                           void* tile_count, long long T, int topk, int E, int tile_rows, int max_tiles,
                           void* stream);
int b200_moe_grouped_gemm_gather(const void* x, long long T, long long x_row_stride, const void* gather_index,
                                 const void* w, const void* row_scale, void* out, const void* tile_table,
                                 const void* tile_count, int num_groups, int n_out, int K,
                                 long long out_row_stride, int max_tiles, int tile_rows_max, int mode,
                                 void* stream);

/* No counterpart in the reference.  b200_moe_grouped_gemm for callers that cannot allocate device
 * memory (a C/C++ host with statically owned buffers, a thread barred from cudaMalloc while a
 * stream capture is open, a service with a fixed memory budget): rows already sorted by group
 * plus cu_seqlens [num_groups + 1] (int32, device), as quack's varlen GEMM takes them.  The token-
 * tile table lives in a fixed ~64 KiB device array inside the library, shared by all calls (calls
 * that overlap on the GPU race on it).  Limits: num_groups <= 1024 and
 * num_groups + x_rows / 64 <= 4095; larger problems return -2.  The first call on a device looks
 * up the array's address and should be made before any stream capture. */
int b200_moe_grouped_gemm_noalloc(const void* x, const void* w, const void* row_scale, void* out,
                                  const void* cu_seqlens, long long x_rows, int num_groups, int n_out, int K,
                                  long long out_row_stride, int mode, void* stream);

/* ---- vexact/batch_invariant_ops/fused_moe.py:325-336 for split gate / up weights. */
int b200_swiglu_scale(const void* gate, const void* up, const void* row_scale, void* out, long long rows,
                      int I, void* stream);

/* Same with gate and up read from rows in_row_stride elements apart (e.g. the two column halves of one
 * [rows, 2I] GEMM output); out is [rows, I] contiguous. */
int b200_swiglu_scale_strided(const void* gate, const void* up, const void* row_scale, void* out, long long rows,
                              int I, long long in_row_stride, void* stream);

/* ---- vexact/batch_invariant_ops/group_gemm/kernel/moe.py:131 moe_gather
 *      (+ optional bf16 add of `addend` [T, H] afterwards, e.g. the shared experts'
 *      output of modeling_deepseek_v3.py:217). */
int b200_moe_unpermute_reduce(const void* y, const void* scatter_index, const void* addend, void* out,
                              long long T, int topk, int H, void* stream);

/* ---- vexact/batch_invariant_ops/group_gemm/kernel/moe.py:304 moe_scatter and :131 moe_gather as operators
 *      over an index array the CALLER supplies (index [T, topk] int32, element strides given):
 *      scatter: out[index[t, k]] = x[t] (any 2-byte element type; out [out_rows, H] contiguous);
 *      gather:  out[t] = bf16(sum over k, ascending, of fp32(x[index[t, k]])) (x [x_rows, H] bf16 contiguous).
 *      H a multiple of 8, 16-byte aligned rows.  An index outside the row count is skipped and reported through
 *      the status word (code 2), where the reference has a device assert. */
int b200_moe_scatter(const void* x, long long x_row_stride, const void* index_i32, long long index_stride_t,
                     long long index_stride_k, void* out, long long out_rows, long long T, int topk, int H,
                     void* stream);
int b200_moe_gather(const void* x, long long x_rows, const void* index_i32, long long index_stride_t,
                    long long index_stride_k, void* out, long long T, int topk, int H, void* stream);

/* No counterpart in the reference (its Triton GEMM reads either layout): out[g, c, r] = x[g, r, c] for 2-byte
 * elements, x [G, R, C] and out [G, C, R] contiguous, R and C multiples of 8, 16-byte aligned.  Used to hand the
 * expert weights to the dgrad form of the grouped GEMM (group_gemm.py:156 with transpose_b=False). */
int b200_transpose_last2(const void* x, void* out, int G, int R, int C, void* stream);

/* ---- vexact/batch_invariant_ops/group_gemm/kernel/group_gemm.py:360 group_gemm_same_mn(transpose_a=True): the
 *      weight gradient of a grouped GEMM, c[g] = a[rows of g]^T @ b[rows of g] with the rows of group g being
 *      [cu_seqlens[g], cu_seqlens[g + 1]).  a [rows, M], b [rows, N], c [num_groups, M, N], all bf16 contiguous;
 *      fp32 accumulation in ascending row order, one rounding; an empty group gets zeros.  M, N multiples of 4.
 *      A training-side operator: mma.sync tensor-core kernel when M and N are multiples of 8 and the pointers
 *      16-byte aligned (sum over 16-row steps in ascending order), a CUDA-core kernel otherwise. */
int b200_moe_grouped_wgrad(const void* a, const void* b, void* c, const void* cu_seqlens, long long rows,
                           int num_groups, int M, int N, void* stream);

/* b200_moe_unpermute_reduce followed by b200_add_rmsnorm (the residual add and input RMSNorm the next
 * decoder layer starts with) in one launch, with that pair's arithmetic element for element:
 * sum_out[t] = bf16(residual[t] + moe[t]), out[t] = rmsnorm(sum_out[t]) * weight (mode as b200_rmsnorm).
 * H a multiple of 8 in 1032..8192; all pointers 16-byte aligned.  No counterpart in the reference
 * (there: moe_gather, a torch add and the RMSNorm module are separate ops). */
int b200_moe_unpermute_add_rmsnorm(const void* y, const void* scatter_index, const void* addend,
                                   const void* residual, const void* weight, void* sum_out, void* out,
                                   long long T, int topk, int H, float eps, int mode, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* VEXACT_B200_H */
