/*
 * b200tts.h - C ABI of libb200tts.so: the Qwen3-TTS decode hot path as hand-written
 * sm_100a CUDA kernels (paged KV write, paged GQA attention for decode and varlen
 * prefill, RMSNorm, q/k-norm + RoPE, SiLU*mul, top-k sampler, frame-loop gathers).
 *
 * The reference (tsdocode/nano-qwen3tts-vllm) has no FFI: its "operator API" for this
 * path is a set of Python callables.  Each entry point below replaces the arithmetic
 * of one of them; citations are file:line under /root/reference/nano-qwen3tts-vllm/.
 * The Python modules in nano-qwen3tts-vllm_b200/layers/ keep the reference's names and
 * signatures and call these through ctypes.
 *
 * Contract common to every entry point
 *   - plain pointers and sizes only; every pointer is a DEVICE pointer unless named host_*;
 *   - bf16 tensors are `const void*` / `void*` to 2-byte bfloat16, row-major, innermost
 *     stride 1; `*_stride` arguments are in ELEMENTS;
 *   - `stream` is a cudaStream_t passed as void* (NULL = legacy default stream);
 *   - no allocation, no synchronisation, no host read of device memory: every call is
 *     capturable in a CUDA graph; scratch comes from the caller (`*_workspace_bytes`);
 *   - returns B2TTS_OK or a negative B2TTS_E* code; b2tts_last_error() gives a
 *     thread-local message.  Nothing throws, nothing calls exit().
 *   - rows with slot -1 / context length 0 are CUDA-graph padding and are skipped
 *     (talker_mode_runner.py:97-100, base.py:166-170).
 */
#ifndef B200TTS_H
#define B200TTS_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define B2TTS_API __attribute__((visibility("default")))
#else
#define B2TTS_API
#endif

#define B2TTS_OK            0
#define B2TTS_EINVAL       -1   /* bad size / null pointer / inconsistent arguments      */
#define B2TTS_EALIGN       -2   /* pointer or stride not 16-byte aligned                 */
#define B2TTS_EUNSUPPORTED -3   /* shape outside what the sm_100a kernels are built for  */
#define B2TTS_ECUDA        -4   /* CUDA launch error (message carries cudaGetErrorString) */
#define B2TTS_EWORKSPACE   -5   /* workspace too small                                   */

/* rounding modes of the element-wise kernels (see DESIGN.md "rounding points") */
#define B2TTS_ROUND_EAGER 0   /* the reference's Python source evaluated op by op in bf16 */
#define B2TTS_ROUND_FUSED 1   /* what torch-inductor emits for the same source on a GPU:
                                  fp32 throughout, one rounding at the store            */

B2TTS_API int         b2tts_version(void);                 /* ABI version, bumped on any signature change */
B2TTS_API const char* b2tts_last_error(void);              /* thread-local, never NULL */
/* Kernels launched (or recorded into a CUDA graph under capture) by this library in this process. */
B2TTS_API unsigned long long b2tts_launch_count(void);
/* SM count / max dynamic smem of the current device (host query, cached). */
B2TTS_API int         b2tts_device_info(int* sm_count, int* max_smem_bytes, int* cc_major, int* cc_minor);

/* ---- a1: paged KV write --------------------------------------------------------------
 * replaces store_kvcache_kernel / store_kvcache          layers/attention.py:10-30, 33-54
 * key,value [n_tokens, kv_dim] with row strides; caches [num_slots, kv_dim] contiguous
 * (the reference asserts k_cache.stride(1) == D, :52); slot_mapping[i] == -1 skips row i. */
B2TTS_API int b2tts_store_kvcache(const void* key, const void* value,
                        int64_t key_row_stride, int64_t value_row_stride,
                        void* k_cache, void* v_cache, const int32_t* slot_mapping,
                        int n_tokens, int kv_dim, void* stream);

/* ---- a2: paged GQA decode attention ---------------------------------------------------
 * replaces flash_attn_with_kvcache(q.unsqueeze(1), k_cache, v_cache, cache_seqlens,
 *          block_table, softmax_scale, causal=True)        layers/attention.py:92-95
 * q [batch, num_heads, head_dim] (row stride q_row_stride), caches
 * [num_pages, page_size, num_kv_heads, head_dim], block_table [batch, bt_stride] int32
 * (entries beyond ceil(len/page) are never read, -1 allowed), context_lens [batch] int32
 * INCLUDING the token written this step.  out [batch, num_heads, head_dim] bf16.
 * max_ctx bounds the split-KV grid (capacity of the block table in tokens). */
B2TTS_API size_t b2tts_paged_attn_decode_workspace_bytes(int batch, int num_heads, int head_dim, int max_ctx);
B2TTS_API int b2tts_paged_attn_decode(const void* q, int64_t q_row_stride,
                            const void* k_cache, const void* v_cache,
                            const int32_t* block_table, int bt_stride,
                            const int32_t* context_lens,
                            void* out, void* workspace, size_t workspace_bytes,
                            int batch, int num_heads, int num_kv_heads, int head_dim,
                            int page_size, float scale, int max_ctx, void* stream);

/* The same operation with the split-KV partial sums in a file-scope device array inside the library instead of a
 * caller-provided workspace: the call allocates nothing (no cudaMalloc / cudaFree, no allocating library routine), for
 * callers that cannot allocate - code under CUDA-graph capture, tight serving loops, harnesses that forbid it.
 * NO COUNTERPART IN THE REFERENCE: added at the request of the run's operators.
 * Limit: the array holds b2tts_paged_attn_decode_static_max_bytes() = 8 MiB, held by every GPU that loads the library until
 * the process exits; shapes whose b2tts_paged_attn_decode_workspace_bytes(...) exceeds it are rejected with
 * B2TTS_EWORKSPACE (use b2tts_paged_attn_decode with your own workspace).  All calls share the array, which keeps the last
 * call's contents (nothing in it needs clearing: every partial is written before it is read): calls that can overlap on
 * the GPU - different streams, parallel graph branches - race on it.  Arguments and results as b2tts_paged_attn_decode. */
B2TTS_API size_t b2tts_paged_attn_decode_static_max_bytes(void);
B2TTS_API int b2tts_paged_attn_decode_static(const void* q, int64_t q_row_stride,
                            const void* k_cache, const void* v_cache,
                            const int32_t* block_table, int bt_stride,
                            const int32_t* context_lens, void* out,
                            int batch, int num_heads, int num_kv_heads, int head_dim,
                            int page_size, float scale, int max_ctx, void* stream);

/* ---- a3: varlen causal prefill attention ----------------------------------------------
 * replaces flash_attn_varlen_func(q, k, v, cu_seqlens_q/k, max_seqlen_q/k, softmax_scale,
 *          causal=True, block_table)                       layers/attention.py:78-91
 * q [total_q, num_heads, head_dim], k,v [total_k, num_kv_heads, head_dim] packed, row
 * strides in elements; cu_seqlens_* [num_seqs+1] int32.  Causal mask is bottom-right
 * aligned (query i of a sequence sees keys 0 .. len_k-len_q+i).  When block_table is
 * non-NULL (prefix-cache hit, attention.py:79-80) k,v are the paged caches
 * [num_pages, page_size, kv_heads, head_dim] and are read through block_table.
 * total_k = rows of the packed k/v (ignored with a block table).  max_seqlen_q >= 128 (packed k/v) runs the
 * tcgen05 tile kernel: 128-query x 128-key tiles, QK^T and PV on the tensor cores with TMEM accumulators, K/V by
 * TMA, causal tile skipping; shorter prompts run one CTA per query token. */
B2TTS_API int b2tts_varlen_attn_prefill(const void* q, int64_t q_row_stride,
                              const void* k, int64_t k_row_stride,
                              const void* v, int64_t v_row_stride,
                              const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k,
                              void* out, int num_seqs, int total_q, int total_k,
                              int max_seqlen_q, int max_seqlen_k,
                              int num_heads, int num_kv_heads, int head_dim, float scale,
                              const int32_t* block_table, int bt_stride, int page_size,
                              void* stream);

/* ---- a4: RMSNorm ----------------------------------------------------------------------
 * replaces Qwen3TTSRMSNorm.rms_forward / add_rms_forward    layers/layernorm.py:18-27, 30-41
 * x [rows, cols] (row stride x_row_stride), w [cols]; y [rows, cols] contiguous.
 * add variant: sum = f32(x)+f32(res); res_out = bf16(sum); norm uses the fp32 sum
 * (layernorm.py:35-38) or, with round_sum_first != 0, the bf16-rounded sum - which is
 * what the decoder layer's `residual + hidden` followed by rms_forward computes
 * (models/qwen3_tts_share.py:171-173).  y/res_out may alias x/res. */
B2TTS_API int b2tts_rmsnorm(const void* x, int64_t x_row_stride, const void* w, void* y,
                  int rows, int cols, float eps, int rounding, void* stream);
B2TTS_API int b2tts_add_rmsnorm(const void* x, const void* res, const void* w, void* y, void* res_out,
                      int rows, int cols, float eps, int rounding, int round_sum_first,
                      void* stream);

/* ---- a4+a5+a1 fused: per-head q/k RMSNorm + RoPE (+ paged KV write) ---------------------
 * replaces q_norm, k_norm, rotary_emb and store_kvcache as called from
 * Qwen3TTSAttention.forward                       models/qwen3_tts_share.py:96-106
 *   RotaryEmbedding.forward / TalkerRotaryEmbedding.forward / apply_*_rotary_pos_emb
 *                                                 layers/rotary_embedding.py:11-212
 * q [n, heads, 128], k,v [n, kv_heads, 128] with row strides (they may be slices of one
 * fused QKV GEMM output).  q_out [n, heads*128] and k_out [n, kv_heads*128] contiguous
 * (may alias q / k when the strides match).  q_weight/k_weight NULL skips the norm
 * (plain RoPE, the rotary_emb.forward surface).  positions int64 [3 or 1][n]
 * (pos_row_stride = 0 for 1-D); inv_freq fp32 [head_dim/2]; modality int32 [head_dim]
 * selects the position row per cos/sin column (NULL = row 0; columns f and head_dim/2+f share
 * frequency f but may read different rows, rotary_embedding.py:73-80).  cos/sin are computed in fp32,
 * scaled by attention_scaling, rounded to bf16, and the rotation is three bf16-rounded
 * ops exactly as the reference's eager expression (rotary_embedding.py:33-34).
 * slot_mapping NULL skips the cache write; otherwise K (normed+rotated) and V (raw) rows
 * go to k_cache/v_cache[slot] and slot -1 is skipped. */
B2TTS_API int b2tts_qknorm_rope_kvwrite(const void* q, int64_t q_row_stride,
                              const void* k, int64_t k_row_stride,
                              const void* v, int64_t v_row_stride,
                              void* q_out, void* k_out,
                              const void* q_weight, const void* k_weight, float eps,
                              const int64_t* positions, int64_t pos_row_stride,
                              const float* inv_freq, const int32_t* modality,
                              float attention_scaling,
                              const int32_t* slot_mapping, void* k_cache, void* v_cache,
                              int n_tokens, int num_heads, int num_kv_heads, int head_dim,
                              int rounding, void* stream);

/* ---- a6: SiLU and the gated product ------------------------------------------------------
 * replaces Silu.forward (layers/activation.py:12-13) and `act_fn(gate) * up`
 * (models/qwen3_tts_share.py:131-135).  gate, up [rows, inter] with a common row stride
 * (two halves of a fused gate_up GEMM output); up == NULL computes silu(gate) only. */
B2TTS_API int b2tts_silu_and_mul(const void* gate, const void* up, int64_t in_row_stride,
                       void* out, int rows, int inter, int rounding, void* stream);

/* ---- a8: sampler ---------------------------------------------------------------------------
 * replaces Sampler.forward                                  layers/sampler.py:15-24
 * logits [batch, vocab] bf16 (or fp32 when logits_fp32 != 0), temperatures [batch] fp32,
 * noise [batch, vocab] fp32 = the Exp(1) draws torch.multinomial makes
 * (`empty_like(probs).exponential_(1)`), out_index [batch] int64 = argmax(softmax(topk-masked
 * logits / T) / noise).  Values tied with the k-th largest are kept (`logits < kth`).
 * top_p is accepted and, like the reference, ignored unless apply_top_p != 0.
 * probs_out (optional, fp32 [batch, vocab]) receives the softmax for inspection. */
B2TTS_API int b2tts_topk_sample(const void* logits, int64_t logits_row_stride, int logits_fp32,
                      const float* temperatures, const float* noise,
                      int64_t* out_index, float* probs_out,
                      int batch, int vocab, int top_k, float top_p, int apply_top_p,
                      void* stream);
/* The same sampler followed, in the same launch, by the gather of the next predictor pass's input embedding:
 * embed_out[i, :] = embed_table[out_index[i], :]   (bf16 rows of embed_cols)
 * replaces Sampler.forward + codec_embedding[g-1](id)   layers/sampler.py:15-24, models/qwen3_tts_predictor.py:94-95
 * vocab <= 4096 and a multiple of 8. */
B2TTS_API int b2tts_topk_sample_embed(const void* logits, int64_t logits_row_stride, int logits_fp32,
                            const float* temperatures, const float* noise,
                            int64_t* out_index, int batch, int vocab, int top_k,
                            const void* embed_table, int embed_cols, void* embed_out,
                            int64_t embed_out_row_stride, void* stream);

/* ---- a9 / frame-loop gathers ------------------------------------------------------------------
 * b2tts_gather_rows: out[i] = tables[table_index[i]][row_index[i]]  (bf16 rows of `cols`)
 *   replaces the per-sequence loop codec_embedding[g_i-1](id_i)   models/qwen3_tts_predictor.py:94-98
 *   tables = base pointer of a stacked [num_tables, rows_per_table, cols] tensor;
 *   table_index NULL = table 0; an index < 0 writes a zero row.
 * b2tts_codec_embed_sum: out[i] = bf16(sum_{c<ncb} f32(E_c[codes[i,c]])) + extra[extra_index ? extra_index[i] : i]
 *   replaces the 16-codebook gather-sum + trailing-text add        interface.py:1276-1286
 *   (extra_index selects trailing_text_hiddens[:, generation_step] or the tts_pad_embed row per stream) */
B2TTS_API int b2tts_gather_rows(const void* tables, int64_t table_stride, int rows_per_table,
                      const int64_t* row_index, const int32_t* table_index,
                      void* out, int64_t out_row_stride, int n, int cols, void* stream);
B2TTS_API int b2tts_codec_embed_sum(const void* table0, const void* tables_rest, int64_t table_stride,
                          const int64_t* codes, int64_t codes_row_stride,
                          const void* extra, int64_t extra_row_stride, const int64_t* extra_index,
                          void* out, int n, int num_codebooks, int cols, void* stream);

/* ---- a12 on the device: decode batch layout -------------------------------------------------------
 * replaces the host loops of prepare_decode / prepare_decode_talker
 *                          engine/model_runner/base.py:218-234, talker_mode_runner.py:116-140
 * seq_lens [n] int32 (device) = tokens of each stream INCLUDING the one decoded this step, 0 =
 * inactive row.  Writes context_lens = len, slot = block_table[i][(len-1)/page]*page + (len-1)%page,
 * positions = len-1+position_offset (1 = talker quirk, 0 = predictor); inactive rows - and rows whose
 * token would fall beyond the bt_width pages of their table row - get slot -1, context 0.
 * advance != 0 then adds `advance` to the active seq_lens (next step's length). */
B2TTS_API int b2tts_decode_layout(int32_t* seq_lens, const int32_t* block_table, int bt_stride, int bt_width,
                        int page_size, int position_offset, int advance, int64_t* positions,
                        int32_t* slot_mapping, int32_t* context_lens, int n, void* stream);

/* ---- f1: per-frame stream state of the on-device frame loop ---------------------------------------
 * replaces the host bookkeeping of generate_async                      interface.py:1233-1239, 1282-1285
 * code0 [n] int64 = the talker code sampled for this frame.  A stream whose code0 == eos_id (2150; eos_id < 0
 * ignores EOS) or that has produced max_frames frames goes inactive BEFORE the frame is produced: active[i] = 0,
 * seq_lens[i] = 0 (a padding row for b2tts_decode_layout from now on).  extra_row[i] = i*(trail_rows+1) +
 * min(gen_step[i], trail_rows) indexes a [n, trail_rows+1, H] buffer whose row trail_rows holds tts_pad_embed
 * (b2tts_codec_embed_sum's extra_index).  Active streams then count the frame: gen_step += 1, frames_done += 1. */
B2TTS_API int b2tts_frame_advance(const int64_t* code0, int eos_id, int32_t* active, int32_t* seq_lens,
                        int32_t* gen_step, int32_t* frames_done, int64_t* extra_row, int trail_rows,
                        int max_frames, int n, void* stream);

/* ---- a7: the projections (weight-streaming tcgen05 GEMM) -------------------------------------------
 * replaces F.linear in ColumnParallelLinear / RowParallelLinear.forward   layers/linear.py:72-73, 149-153
 *   (q/k/v and gate/up as ONE GEMM each over a merged weight: models/qwen3_tts_share.py:85-87, 126-134),
 *   nn.Linear small_to_mtp_projection / lm_head[g]                 models/qwen3_tts_predictor.py:54-61,
 *   ParallelLMHead's F.linear                                      layers/embed_head.py:61
 * y[m, n] = x[m, k] @ W[n, k]^T, bf16 in/out, fp32 accumulate in TMEM, m >= 1 (rows beyond 128 run as
 * 128-row chunks inside the same launch), n % 128 == 0, k % 64 == 0.  W is passed PRE-PACKED: b2tts_gemm_pack_weight() re-tiles a row-major [n, k] weight
 * once at load time into [n/128][k/64] tiles of 16 KiB (the K-major SWIZZLE_128B shared-memory image
 * of a UMMA operand), b2tts_gemm_packed_bytes(n, k) bytes.  B2TTS_PACK_GATE_UP packs a merged
 * [gate; up] weight (n = 2 * intermediate) so that every 8 consecutive tile rows hold 4 gate features
 * and the 4 matching up features - required by the SiLU*mul epilogue.
 * epilogue: B2TTS_GEMM_BIAS      out[m, n]   = bf16(acc + bias)              (bias may be NULL)
 *           B2TTS_GEMM_RESIDUAL  out[m, n]   = bf16(bf16(acc) + residual)    (qwen3_tts_share.py:171,175;
 *                                              out may alias residual)
 *           B2TTS_GEMM_SILU_MUL  out[m, n/2] = silu(bf16(gate)) * bf16(up)   (qwen3_tts_share.py:131-135;
 *                                              `rounding` as b2tts_silu_and_mul)
 *           B2TTS_GEMM_RELU_SQ   out[m, n]   = bf16(max(bf16(acc), 0)^2)      (squared-ReLU feed-forwards; single-GEMM
 *                                              entry points only)
 * splits: K-split = cluster size (1,2,4,8,16; 0 = choose so that tiles * splits fill the SMs); the
 * partial sums are exchanged through distributed shared memory and added in a fixed order.
 * splits = -2 / -4: the cluster splits the BATCH instead (m padded to 16 must be a multiple of 32 / 64, m <= 128):
 * every CTA runs the whole K range for its 16 - 48 rows and each weight tile is fetched once per cluster (1 / |splits|
 * per CTA, multicast to all) - no partial sums, no exchange.  splits = 0 never picks it unless B2TTS_GEMM_BSPLIT=1
 * (then for K <= 1024): in the decode frame it is slower than the K split.
 * pdl != 0 launches with programmatic stream serialization: the weight stream starts while the
 * previous kernel on the stream is still running (every kernel of this library that is launched
 * this way executes griddepcontrol.wait before touching its inputs/outputs). */
#define B2TTS_GEMM_BIAS     0
#define B2TTS_GEMM_RESIDUAL 1
#define B2TTS_GEMM_SILU_MUL 2
#define B2TTS_GEMM_RELU_SQ  3
#define B2TTS_PACK_PLAIN    0
#define B2TTS_PACK_GATE_UP  1
B2TTS_API int    b2tts_gemm_bf16_supported(int m, int n, int k);
B2TTS_API size_t b2tts_gemm_packed_bytes(int n, int k);
B2TTS_API int    b2tts_gemm_pack_weight(const void* weight, int64_t weight_row_stride, void* packed,
                                        int n, int k, int mode, void* stream);
B2TTS_API int    b2tts_gemm_bf16(const void* x, int64_t x_row_stride, const void* w_packed,
                                 const void* bias, const void* residual, int64_t residual_row_stride,
                                 void* out, int64_t out_row_stride, int m, int n, int k,
                                 int epilogue, int rounding, int splits, int pdl, void* stream);


/* ---- a4 fused into a7: input RMSNorm in the GEMM's x producers, row sums of squares out of its epilogue ----
 * replaces `hidden = layernorm(residual)` followed by the projection that reads it
 *                                          models/qwen3_tts_share.py:166-167,172-174, layers/layernorm.py:18-27
 * As b2tts_gemm_bf16, plus:
 *   norm_weight != NULL: x is the residual stream; the GEMM multiplies norm(x)[m, k] =
 *     rounding(x[m, k] * rstd[m], norm_weight[k]) (same rounding points as b2tts_rmsnorm) with
 *     rstd[m] = 1/sqrt(sum_j ssq_in[m, j] / k + eps), j < ssq_in_slots summed in a fixed order.
 *   ssq_out != NULL (bias / residual epilogues): ssq_out[m, slot] = sum of squares of the bf16 values this
 *     call stored in out[m, :] over slot's 128-feature tile; slots per row = b2tts_gemm_ssq_slots(m, n, k, splits)
 *     = n / 128 (the K-split CTAs of a tile combine their sums inside the cluster, in rank order).
 *     The next b2tts_gemm_norm_bf16 over `out` takes it as ssq_in: the decoder layer's two norm launches
 *     disappear, and the normalised activations never reach HBM. */
B2TTS_API int    b2tts_gemm_ssq_slots(int m, int n, int k, int splits);
B2TTS_API int    b2tts_gemm_norm_bf16(const void* x, int64_t x_row_stride, const void* w_packed,
                                      const void* bias, const void* residual, int64_t residual_row_stride,
                                      void* out, int64_t out_row_stride, int m, int n, int k,
                                      int epilogue, int rounding, int splits, int pdl,
                                      const void* norm_weight, const float* ssq_in, int ssq_in_slots, float eps,
                                      float* ssq_out, void* stream);

/* b2tts_gemm_norm_bf16 plus an L2 prefetch of the NEXT projection's packed weights (prefetch_next, prefetch_bytes =
 * b2tts_gemm_packed_bytes of that weight, or NULL / 0): weights do not depend on activations, and a decode step is a
 * chain of latency-bound launches during which HBM idles most of the time - every CTA pulls its slice of the next
 * weight image into the 126 MB L2 (cp.async.bulk.prefetch.L2) so the next launch streams from L2 while HBM already
 * fetches the launch after it.  Results are identical to b2tts_gemm_norm_bf16. */
B2TTS_API int    b2tts_gemm_prefetch_bf16(const void* x, int64_t x_row_stride, const void* w_packed,
                                          const void* bias, const void* residual, int64_t residual_row_stride,
                                          void* out, int64_t out_row_stride, int m, int n, int k,
                                          int epilogue, int rounding, int splits, int pdl,
                                          const void* norm_weight, const float* ssq_in, int ssq_in_slots, float eps,
                                          float* ssq_out, const void* prefetch_next, size_t prefetch_bytes, void* stream);

/* ---- a7 x 4 in one launch: the persistent GEMM chain of the decoder layer ------------------------------------
 * replaces the four dependent projections between two attention calls
 *     o_proj (+ residual add) -> gate_up_proj (post_attention_layernorm in, SiLU*mul out) -> down_proj (+ residual add)
 *     -> the next layer's qkv_proj (input_layernorm in)                      models/qwen3_tts_share.py:163-176
 * with ONE persistent kernel (one CTA per SM) whose weight stream never stops at a GEMM boundary: a producer
 * thread keeps a deep shared-memory ring of packed weight tiles full across the whole chain while the CTAs
 * reduce split-K partials through L2 and cross a grid barrier between GEMMs.  Every op is a b2tts_gemm_norm_bf16
 * (same packed weights, epilogues, fused input norm and rounding points); op i+1 may read what op i wrote
 * (x, residual, ssq_in).  ssq_out of an op has b2tts_gemm_chain_ssq_slots(n) = n/128 slots per row.
 * 1 <= nops <= 4, 1 <= m <= 128.  workspace: b2tts_gemm_chain_workspace_bytes(...) bytes, ZERO-FILLED once by the
 * caller (the kernel leaves its barrier counters zero); one workspace must not be used by two launches that
 * can run concurrently.  The grid needs every SM of the device: do not run two chains concurrently. */
typedef struct b2tts_gemm_op {
  const void* x;            int64_t x_row_stride;         /* [m, k] bf16 */
  const void* w_packed;                                   /* b2tts_gemm_pack_weight image of W[n, k] */
  const void* residual;     int64_t residual_row_stride;  /* B2TTS_GEMM_RESIDUAL */
  void* out;                int64_t out_row_stride;       /* [m, n] (or [m, n/2] for SiLU*mul); may alias residual */
  const void* norm_weight;  const float* ssq_in;          /* fused input RMSNorm (or NULL) */
  float* ssq_out;                                         /* [m, n/128] partial row sums of squares (or NULL) */
  int n, k, epilogue, ssq_in_slots;
} b2tts_gemm_op;
B2TTS_API int    b2tts_gemm_chain_ssq_slots(int n);
B2TTS_API size_t b2tts_gemm_chain_workspace_bytes(int m, const int* n, const int* k, int nops);
B2TTS_API int    b2tts_gemm_chain(const b2tts_gemm_op* ops, int nops, int m, float eps, int rounding,
                                  void* workspace, size_t workspace_bytes, int pdl, void* stream);

/* ---- a5 + a4 + a1 + a2 in one launch: the decode step of Qwen3TTSAttention.forward ------------------------
 * replaces q_norm, k_norm, rotary_emb, store_kvcache and flash_attn_with_kvcache as called per decode token
 *                                       models/qwen3_tts_share.py:96-109, layers/attention.py:33-54, 92-95
 * q/k/v are the rows of the QKV projection (one new token per sequence).  The kernel normalises + rotates q
 * and k (arguments as b2tts_qknorm_rope_kvwrite), writes K (normed + rotated) and V (raw) of the new token
 * to cache[slot_mapping[i]], attends over context_lens[i] cached tokens INCLUDING the new one
 * (arguments as b2tts_paged_attn_decode) and folds the split-KV partials itself (the last CTA of a
 * sequence to finish does it, in split order).  K cache bytes and attention outputs equal those of the
 * separate calls.  workspace: b2tts_fused_decode_attn_workspace_bytes(...) bytes, ZERO-FILLED once by the
 * caller before the first launch (the kernel leaves its tickets zero).  The tickets occupy a fixed span at the
 * start of the workspace, so ONE workspace sized for the largest batch serves launches of every smaller batch
 * (batch <= 4096).  pdl as b2tts_gemm_bf16. */
B2TTS_API size_t b2tts_fused_decode_attn_workspace_bytes(int batch, int num_heads, int head_dim, int max_ctx);
B2TTS_API int b2tts_fused_decode_attn(const void* q, int64_t q_row_stride, const void* k, int64_t k_row_stride,
                            const void* v, int64_t v_row_stride,
                            const void* q_weight, const void* k_weight, float eps,
                            const int64_t* positions, int64_t pos_row_stride,
                            const float* inv_freq, const int32_t* modality, float attention_scaling,
                            const int32_t* slot_mapping, void* k_cache, void* v_cache,
                            const int32_t* block_table, int bt_stride, const int32_t* context_lens,
                            void* out, void* workspace, size_t workspace_bytes,
                            int batch, int num_heads, int num_kv_heads, int head_dim, int page_size,
                            float scale, int max_ctx, int rounding, int pdl, void* stream);

/* ---- f3: prompt-prep embedding assembly -------------------------------------------------------------------
 * replaces the per-request tensor ops of prepare_inputs / generate_icl_prompt   utils/generation.py:18-379, 412-515
 * (torch.cat / expand / `+` of projected text rows, codec-tag rows, the speaker row and the ICL reference frames,
 * then pad_sequence into the left-padded batch, :329-377).  The host plans every row of every request of a batch;
 * one launch writes  out[r] = a[a_index[r]] (+) b[b_index[r]]  (bf16 rows of `cols`; the add is bf16(f32 + f32),
 * torch's bf16 tensor add; an index < 0 = that side absent, both absent = a zero padding row).
 * a = the projected text rows text_projection(text_embedding(ids)), b = codec-side rows; indices are NOT range-checked
 * on the device (a_rows / b_rows are validated by the host wrapper). */
B2TTS_API int b2tts_prompt_assemble(const void* a, int64_t a_row_stride, int a_rows, const void* b, int64_t b_row_stride,
                                    int b_rows, const int32_t* a_index, const int32_t* b_index, void* out,
                                    int64_t out_row_stride, int rows, int cols, void* stream);

/* ---- f4 (tail): decoded waveform -> PCM16 ----------------------------------------------------------------------
 * replaces _float_to_pcm16 / _apply_volume_pcm16                                    examples/server.py:338-349
 *   out[i] = (int16) trunc(clip(wav[i], -1, 1) * 32767);  volume != 1: out[i] = clip(rint(out[i] * volume), -32768, 32767)
 * (the vocoder itself - qwen_tts 0.0.5, not part of the reference tree - is out of reach). */
B2TTS_API int b2tts_float_to_pcm16(const float* wav, int16_t* out, int64_t n, float volume, void* stream);

/* ---- a10 in one launch: the decode pass of a whole (small) decoder stack ----------------------------------------
 * replaces, for one decode step of up to 64 sequences, the layer loop of Qwen3TTSCodePredictorModel.forward /
 * Qwen3TTSTalkerModel.forward                          models/qwen3_tts_predictor.py:30-44, qwen3_tts_talker.py:53-62
 * over Qwen3TTSDecoderLayer.forward                    models/qwen3_tts_share.py:163-176 (and :79-113, :131-135)
 * i.e. per layer: input RMSNorm, QKV projection, q/k head norm + RoPE + paged KV write + paged GQA attention,
 * o projection + residual add, post-attention RMSNorm, gate_up projection + SiLU*mul, down projection + residual
 * add; then the final RMSNorm.  ONE persistent dataflow kernel (one CTA per SM): every CTA owns one (projection,
 * 128-feature tile, K split) job in every layer and prefetches its packed weights ahead of the activations; phases
 * are linked by arrival counters in the workspace instead of kernel boundaries (csrc/decoder_stack.cu).  Same packed
 * weights (b2tts_gemm_pack_weight; gate_up in B2TTS_PACK_GATE_UP mode), rounding points and summation orders as
 * b2tts_rmsnorm -> b2tts_gemm_bf16 -> b2tts_fused_decode_attn -> b2tts_gemm_bf16(RESIDUAL, splits = o_splits) ->
 * b2tts_rmsnorm -> b2tts_gemm_bf16(SILU_MUL) -> b2tts_gemm_bf16(RESIDUAL, splits = down_splits): bit-identical.
 * x [m, hidden] is the residual stream entering layer 0 (left intact), out [m, hidden] the normalised final hidden
 * states.  positions [m] int64 (1-D RoPE), slot_mapping / block_table / context_lens as b2tts_fused_decode_attn.
 * 1 <= m <= 64, 1 <= num_layers <= 8, head_dim 128, num_heads == 2 * num_kv_heads, hidden <= 2048, and the jobs must
 * fit one per SM (b2tts_decoder_stack_plan returns 0 otherwise).  workspace: b2tts_decoder_stack_workspace_bytes(...)
 * bytes, 256-byte aligned, ZERO-FILLED once by the caller; one workspace must not be used by two launches that can
 * run concurrently, and the grid needs every SM of the device.  A dependency that fails to resolve within 4 s traps
 * (CUDA launch failure) rather than hanging the device. */
typedef struct b2tts_stack_layer {
  const void *qkv_w, *o_w, *gate_up_w, *down_w;                      /* packed weights */
  const void *input_norm_w, *post_norm_w, *q_norm_w, *k_norm_w;       /* bf16 norm weights [hidden] / [128] */
  void *k_cache, *v_cache;                                            /* [pages, page, kv_heads, 128] bf16 */
} b2tts_stack_layer;
B2TTS_API int    b2tts_decoder_stack_plan(int hidden, int q_size, int kv_size, int intermediate,
                                          int* o_splits, int* down_splits);
B2TTS_API size_t b2tts_decoder_stack_workspace_bytes(int hidden, int q_size, int kv_size, int intermediate);
B2TTS_API int    b2tts_decoder_stack_decode(const void* x, int64_t x_row_stride, void* out, int64_t out_row_stride,
                                            const b2tts_stack_layer* layers, int num_layers, const void* final_norm_weight,
                                            int m, int hidden, int num_heads, int num_kv_heads, int head_dim,
                                            int intermediate, float eps, int rounding,
                                            const int64_t* positions, const float* inv_freq, float attention_scaling,
                                            const int32_t* slot_mapping, const int32_t* block_table, int bt_stride,
                                            const int32_t* context_lens, int page_size, float scale,
                                            void* workspace, size_t workspace_bytes, void* stream);

/* ---- token-id decoder models with a 32-bit residual stream -------------------------------------
 * (no counterpart in the reference, whose models take embeddings and keep a bf16 residual)
 * `dtype` selects the activation / cache / table type of the void* tensors: bf16 for serving, float for the
 * all-32-bit mode.  The residual stream x, every norm, the router, the per-head constants and the convolution
 * weights are float in both.  Rows whose slot is -1 and sequences whose length is 0 are CUDA-graph padding. */
#define B2TTS_DTYPE_BF16 0
#define B2TTS_DTYPE_F32  1

/* x[r] = embed[tokens[r]] + pos_table[positions[r]] (float sum); h[r] = T(x[r] / sqrt(mean(x[r]^2) + eps) * gain[0])
 * when h != NULL ("gain norm": one gain for all coordinates). */
B2TTS_API int b2tts_embed_pos_norm(const int32_t* tokens, const int32_t* positions, const void* embed, const void* pos_table,
                                   float* x, void* h, const float* gain, int rows, int cols, int vocab, int max_pos,
                                   float eps, int dtype, void* stream);
/* The residual update of a layer whose sublayers all read one norm, fused with the next norm:
 * x[r] += mult * (a[r] + b[r] + sum_k zw[r, k] * z[r * top + k]) (each term optional, k in ascending order);
 * h[r] = gain norm of the new x[r] when h != NULL. */
B2TTS_API int b2tts_residual_norm(float* x, const void* a, const void* b, const void* z, const float* zw, int top, float mult,
                                  void* h, const float* gain, int rows, int cols, float eps, int dtype, void* stream);
/* out[i] = gain norm of x[rows_idx[i]] (rows_idx NULL = row i). */
B2TTS_API int b2tts_gather_gain_norm(const float* x, const int32_t* rows_idx, void* out, const float* gain, int rows, int cols,
                                     float eps, int dtype, void* stream);
/* y <- max(y, 0)^2 in place. */
B2TTS_API int b2tts_relu_sq(void* y, int64_t n, int dtype, void* stream);
/* Short causal convolution over time on every channel of the merged projection u [n, C] = [q | k | v]
 * (C = heads*dim + kv_heads*dim + kv_heads*vdim; conv_w [C, taps] float, tap taps-1 is the token itself), then RMS norm
 * per head over dim with q_norm_w / k_norm_w [dim] for q and k; q goes to q_out [n, heads*dim], k and v to their cache
 * slot (slot_mapping[n]).  Token n belongs to batch row tok_seq[n] at position positions[n]; row b brings seq_len[b]
 * tokens starting at batch index seq_start[b] and position seq_pos0[b], and owns state slot seq_slot[b]:
 * state [slots, taps-1, C] holds the last taps-1 projections of the sequence (oldest first) and is advanced by this
 * call.  Positions before 0 read as zero whatever the slot holds, so a slot needs no clearing between owners. */
B2TTS_API int b2tts_conv_headnorm_kvwrite(const void* u, int64_t u_stride, const float* conv_w, void* state,
                                          const int32_t* tok_seq, const int32_t* positions, const int32_t* seq_start,
                                          const int32_t* seq_pos0, const int32_t* seq_len, const int32_t* seq_slot,
                                          const int32_t* slot_mapping, const float* q_norm_w, const float* k_norm_w,
                                          void* q_out, void* k_cache, void* v_cache, int n_tokens, int n_seqs, int heads,
                                          int kv_heads, int dim, int vdim, int taps, float eps, int dtype, void* stream);
/* Sliding-window attention with un-normalised sigmoid weights and a logarithmic distance bias over the paged cache:
 * out[i, h] = sum_{0 <= i-j < window} sigmoid(q_ih . k_jg * scale - r1[h] * ln(1 + r2[h] * (i-j)) + pb[h]) * v_jg.
 * q [n, heads*dim], caches [slots, kv_heads*dim] / [slots, kv_heads*vdim], out [n, heads*vdim]; key j of batch row b lives
 * in slot block_tables[b, j / page] * page + j % page (this step's keys included: write them first).  max_new >= every
 * seq_len[b] sizes the grid. */
B2TTS_API int b2tts_window_sigmoid_attn(const void* q, const void* k_cache, const void* v_cache, void* out,
                                        const int32_t* seq_start, const int32_t* seq_pos0, const int32_t* seq_len,
                                        const int32_t* block_tables, int bt_stride, const float* r1, const float* r2,
                                        const float* pb, int n_seqs, int max_new, int heads, int kv_heads, int dim, int vdim,
                                        int page, int window, float scale, int dtype, void* stream);
/* Top-k router, in float.  mode 0: scores = sigmoid(h router^T), top_w = score / (sum of the chosen + 1e-20) * scale.
 * mode 1: scores = h router^T + bias (bias may be null), top_w = softmax over the chosen scores only, * scale.
 * mode 2: scores = softmax(h router^T) over all experts, the choice is made on score + bias, top_w = the chosen scores
 * * scale (not renormalised).  top_idx [n, top] the `top` largest (ties: lower index); then the (token, choice) pairs grouped by expert:
 * offsets [experts + 1], sorted_pair [n * top] (pair = token * top + choice; order inside a group unspecified). */
B2TTS_API int b2tts_moe_route(const void* h, const float* router, int32_t* top_idx, float* top_w, int32_t* offsets,
                              int32_t* sorted_pair, int n_tokens, int cols, int experts, int top, float scale,
                              const float* bias, int mode, int dtype, void* stream);
/* C[out_row(s), :] = act(A[in_row(s), :] W[e]^T) for s in offsets[e] .. offsets[e+1], W [experts, n, k];
 * in_row(s) = sorted_pair[s] / top if in_by_token else s; out_row(s) = sorted_pair[s] if out_by_pair else s;
 * act 0 = none, 1 = squared ReLU; float accumulation. */
B2TTS_API int b2tts_grouped_gemm(const void* a, int64_t lda, const void* w, void* c, int64_t ldc, const int32_t* offsets,
                                 const int32_t* sorted_pair, int n_pairs, int experts, int n, int k, int top, int in_by_token,
                                 int out_by_pair, int act, int dtype, void* stream);

/* ---- decoders with latent attention, token shift and a norm on each sublayer's output (csrc/latent_ops.cu, latent_attn.cu).
 * `dtype` is the activation / cache type (B2TTS_DTYPE_*); x is the float residual stream [rows, cols]. */
/* x[i] = embed[tokens[i]] * scale. */
B2TTS_API int b2tts_embed_scale(const int32_t* tokens, const void* embed, float* x, int rows, int cols, int vocab, float scale,
                                int dtype, void* stream);
/* out[t] = x[t] + (prev - x[t]) * mu; prev = x[t-1] inside a sequence's portion, state[seq_slot] at its first token, zero at
 * position 0; then state[seq_slot] = the sequence's last row of this step.  Rows of sequences with seq_len 0 give zeros. */
B2TTS_API int b2tts_token_shift(const float* x, const float* mu, float* state, const int32_t* tok_seq, const int32_t* positions,
                                const int32_t* seq_start, const int32_t* seq_len, const int32_t* seq_slot, void* out,
                                int n_tokens, int cols, int dtype, void* stream);
/* Row t of the merged projection u (row stride ldu): cq[t] = rms_norm(u[t, q_off : q_off + q_rank]) * q_norm_w (skipped when
 * q_rank == 0); cache[slot_mapping[t]] = [rms_norm(u[t, kv_off : +kv_rank]) * kv_norm_w | rotate(u[t, kv_off + kv_rank : +rot_dim])],
 * pair (2i, 2i+1), i < rot_dims / 2, turned by positions[t] * freq[i], cos and sin times rot_mult.  Slot -1: no cache write. */
B2TTS_API int b2tts_latent_prep(const void* u, int64_t ldu, int q_off, int kv_off, void* cq, const float* q_norm_w,
                                const float* kv_norm_w, const float* freq, float rot_mult, const int32_t* positions,
                                const int32_t* slot_mapping, void* cache, int n_tokens, int q_rank, int kv_rank, int rot_dim,
                                int rot_dims, float eps, int dtype, void* stream);
/* Multi-query softmax attention over cached rows [c | kr] with a sink in the denominator; see csrc/latent_attn.cu.
 * sink null: an ordinary softmax.  ql: absorbed queries (element (t, h, :) at ql + t * ql_tok + h * ql_head, kv_rank numbers), qr: rotary query parts, not yet
 * turned (rot_dim numbers), out: weighted latent sums (kv_rank numbers), strides in elements.  window 0 = every earlier key.
 * path 0 = choose, 1 = the plain kernel, 2 = the tensor-core kernel with two key stages (bf16; fails if the sizes do not
 * fit it), 3 = the tensor-core kernel with one key stage and two CTAs per SM. */
B2TTS_API int b2tts_latent_attn(const void* ql, int64_t ql_tok, int64_t ql_head, const void* qr, int64_t qr_tok, int64_t qr_head,
                                const void* cache, void* out, int64_t o_tok, int64_t o_head, const float* sink, const float* freq,
                                float rot_mult, int rot_dims, const int32_t* seq_start, const int32_t* seq_pos0,
                                const int32_t* seq_len, const int32_t* block_tables, int64_t bt_stride, int n_seqs, int max_new,
                                int heads, int kv_rank, int rot_dim, int page, int window, float scale, int dtype, int path,
                                int splits, float* ws, void* stream);
/* splits > 1 (tensor-core kernel only): each query tile's keys are cut into that many ranges, run by CTAs of their own,
 * and merged by a second launch; ws holds b2tts_latent_attn_workspace_floats() floats.  b2tts_latent_attn_splits() proposes
 * a count that fills the GPU for a decode step (1 for anything else). */
B2TTS_API int b2tts_latent_attn_splits(int n_seqs, int max_new, int heads);
B2TTS_API size_t b2tts_latent_attn_workspace_floats(int n_seqs, int max_new, int heads, int kv_rank, int splits);
/* How many bounded waits for a key tile ran out inside the tensor-core kernel since load (0 in a healthy run); synchronises. */
B2TTS_API int b2tts_latent_attn_timeouts(void);
/* out[t, h * vdim + d] = v[t * v_tok + h * v_head + d] * sigmoid(gate[t * ldg + h * vdim + d]) (gate null: the copy alone). */
B2TTS_API int b2tts_gate_heads(const void* v, int64_t v_tok, int64_t v_head, const void* gate, int64_t ldg, void* out, int n,
                               int heads, int vdim, int dtype, void* stream);
/* y = a + sum_k zw[:, k] z[:, k] (a or z may be null); x += w * y / sqrt(mean over the group (y^2) + eps), the row cut into
 * `groups` equal consecutive parts; copy (optional) = the new x in the activation type. */
B2TTS_API int b2tts_group_norm_residual(float* x, const void* a, const void* z, const float* zw, int top, const float* w, int groups,
                                        float eps, void* copy, int rows, int cols, int dtype, void* stream);
/* out[i] = group RMS norm of x[rows_idx[i]] times w (rows_idx null: row i; w null: the conversion alone). */
B2TTS_API int b2tts_gather_group_norm(const float* x, const int32_t* rows_idx, void* out, const float* w, int groups, float eps,
                                      int rows, int cols, int dtype, void* stream);
/* In place: z = y + bias (bias [cols] or null); y = z > 0 ? softplus(pq[0]) z^2 + z/2 : (1/2 + softplus(pq[1])) (e^z - 1 - z) + z/2. */
B2TTS_API int b2tts_xielu(void* y, const void* bias, const float* pq, int64_t rows, int cols, int dtype, void* stream);
/* y[r, c] = silu(gu[r, c]) * gu[r, ff + c], gu [rows, 2 ff]. */
B2TTS_API int b2tts_silu_mul(const void* gu, void* y, int64_t rows, int ff, int dtype, void* stream);

/* ---- decoders with several residual streams and mixers that pair an attention branch with a recurrent branch
 * (csrc/hybrid_ops.cu, sink_attn.cu, recurrent.cu).  `dtype` is the activation / cache type (B2TTS_DTYPE_*); xs is the float
 * stream tensor [rows, streams, cols].  The per-sequence arrays (seq_start, seq_pos0, seq_len, seq_slot) and the per-token
 * arrays (tok_seq, positions, slot_mapping) describe the step as everywhere in this library; seq_len 0 / slot -1 is padding. */
/* xs[i, s, :] = embed[tokens[i]] + bigram[row_i] for every stream s; row_i = (prev_tokens[i] * mul_prev + tokens[i] * mul_cur)
 * mod buckets, or row `buckets` (the table's last) where prev_tokens[i] < 0.  bigram null: the token embedding alone. */
B2TTS_API int b2tts_embed_bigram_streams(const int32_t* tokens, const int32_t* prev_tokens, const void* embed, const void* bigram,
                                         float* xs, int rows, int cols, int streams, int vocab, int buckets, int mul_prev,
                                         int mul_cur, int dtype, void* stream);
/* y1 given: x_t <- sum_s mix[s, t] x_s + out_w[t] * (c1 * y1 + c2 * y2) for all streams t at once from the old ones (y2 may be
 * null).  h given: h = rms_norm(sum_s in_w[s] x_s) * norm_w (in_w null: the plain sum), over the updated streams. */
B2TTS_API int b2tts_stream_mix_norm(float* xs, const void* y1, const void* y2, float c1, float c2, const float* mix,
                                    const float* out_w, const float* in_w, const float* norm_w, void* h, int rows, int cols,
                                    int streams, float eps, int dtype, void* stream);
/* out[i] = rms_norm(sum_s in_w[s] xs[rows_idx[i], s]) * norm_w (rows_idx null: row i; in_w null: the plain sum). */
B2TTS_API int b2tts_stream_gather_norm(const float* xs, const int32_t* rows_idx, const float* in_w, const float* norm_w, void* out,
                                       int rows, int cols, int streams, float eps, int dtype, void* stream);
/* Row t of the merged projection u (row stride ldu): q = u[q_off : +heads*dim] + q_bias, k = u[k_off : +kv_heads*dim] + k_bias,
 * v = u[v_off : +kv_heads*vdim] + v_bias, or v = k as it stands here when v_off < 0 (biases may be null).  With q_norm_w and
 * k_norm_w, q and k are divided by the root mean square of their whole projection and multiplied by the weights.  With
 * rot_dims > 0, coordinate i < rot_dims/2 of every head is paired with i + rot_dims/2 (interleaved != 0: coordinate 2i with
 * 2i + 1) and turned by positions[t] * freq[i].  q -> q_out[t]; k, v -> the caches at slot_mapping[t]; with both caches null
 * only q is made (a layer that reads the keys and values another layer wrote).  v_heads: value heads projected and cached
 * (kv_heads unless several key maps share one set of values). */
B2TTS_API int b2tts_attn_prep(const void* u, int64_t ldu, int q_off, int k_off, int v_off, const float* q_bias, const float* k_bias,
                              const float* v_bias, const float* q_norm_w, const float* k_norm_w, const float* freq, int rot_dims,
                              const int32_t* positions, const int32_t* slot_mapping, void* q_out, void* k_cache, void* v_cache,
                              int n_tokens, int heads, int kv_heads, int dim, int vdim, float eps, int interleaved, int v_heads,
                              int dtype, void* stream);
/* Softmax attention with exp(sink[h]) added to the denominator (sink null: none) over the paged cache, this step's keys
 * included.  Token i sees key j <= i with j >= max(0, i - mask + 1) (mask_kind 0, a sliding window) or j >= floor(i / mask) *
 * mask (mask_kind 1, chunks counted from position 0); mask <= 0: every j <= i.  keep_first F > 0: keys j < F stay visible
 * behind the mask.  softcap c > 0: a scaled score s becomes c tanh(s / c).  v_heads: value heads in v_cache, key head g reads
 * value head g mod v_heads (v_heads == kv_heads: one each).  out_f32 != 0 with bf16 inputs: out is a float tensor (results not
 * rounded to 16 bits).  gate (optional): element (t, h) at
 * gate[t * ldg + h]; the head's output is multiplied by its sigmoid.  q [n, heads*dim], out [n, heads*vdim].  max_new >= every
 * seq_len[b].  path 0 = choose (bf16 prompt portions with head sizes the tensor-core kernel is built for run there, everything
 * else in the plain kernel), 1 = the plain kernel, 2 = the tensor-core kernel for prompt portions (fails if the sizes do not fit). */
B2TTS_API int b2tts_sink_attn(const void* q, const void* k_cache, const void* v_cache, void* out, const int32_t* tok_seq,
                              const int32_t* positions, const int32_t* seq_start, const int32_t* seq_pos0, const int32_t* seq_len,
                              const int32_t* block_tables, int64_t bt_stride, const float* sink, const void* gate, int64_t ldg,
                              int n_tokens, int n_seqs, int max_new, int heads, int kv_heads, int v_heads, int dim, int vdim,
                              int page, int mask_kind, int mask, int keep_first, float softcap, float scale, int dtype, int path,
                              int out_f32, void* stream);
/* out[t, c] = act(bias[c] + sum_j w[c, j] * u(position(t) - taps + 1 + j)[c_off + c]) for c < channels (act 0: none, 1: SiLU;
 * bias may be null).  Earlier positions come from this step's rows, from state [slots, taps-1, channels] (the sequence's last
 * rows, oldest first, advanced by this call) or are zero before position 0.  max_new >= every seq_len[b] (0: unknown). */
B2TTS_API int b2tts_short_conv_act(const void* u, int64_t ldu, int c_off, const float* w, const float* bias, void* state,
                                   const int32_t* tok_seq, const int32_t* positions, const int32_t* seq_start,
                                   const int32_t* seq_pos0, const int32_t* seq_len, const int32_t* seq_slot, void* out, int64_t ldo,
                                   int n_tokens, int n_seqs, int max_new, int channels, int taps, int act, int dtype, void* stream);
/* Row y [cols] (float) in `groups` equal parts, each divided by its root mean square, times w[c mod w_len]; the gate
 * (sigmoid for gate_act 0, SiLU for 1, of gate[r * ldg + c]; null: none) multiplies y before the norm (gate_first) or after. */
B2TTS_API int b2tts_gated_group_norm(const float* y, const void* gate, int64_t ldg, const float* w, int w_len, int groups,
                                     int gate_act, int gate_first, float eps, void* out, int rows, int cols, int dtype, void* stream);
/* State-space recurrence per head h (group g = h / (heads / groups)), state [slots, heads, dim, vdim] float:
 * dt = softplus(dt_in[t, h] + dt_bias[h]); S <- exp(-exp(a_log[h]) dt) S + dt B_t x_t^T; out[t, h] = S^T C_t + d_skip[h] x_t, with
 * row t of xbc = [x: heads*vdim | B: groups*dim | C: groups*dim] (after its convolution and activation).  out [rows, heads*vdim];
 * coef [rows, heads, 3] float is scratch (the per-token scalars, computed by a kernel in front of the recurrence). */
B2TTS_API int b2tts_ssm_scan(const void* xbc, int64_t ldx, const void* dt, int64_t lddt, const float* dt_bias, const float* a_log,
                             const float* d_skip, float* state, float* coef, float* out, const int32_t* seq_start,
                             const int32_t* seq_pos0, const int32_t* seq_len, const int32_t* seq_slot, int n_tokens, int n_seqs,
                             int heads, int groups, int vdim, int dim, int dtype, void* stream);
/* Delta rule per head, state [slots, heads, dim, vdim] float: row t of qkv = [q: kv_heads*dim | k: kv_heads*dim | v: heads*vdim];
 * q and k are made unit vectors (x / sqrt(sum x^2 + 1e-6)), q also times dim^(-1/2); g = exp(-exp(a_log[h]) softplus(a_in[t, h] +
 * dt_bias[h])), beta = sigmoid(beta_in[t, h]); S <- g S; u = beta (v - S^T k); S <- S + k u^T; out[t, h] = S^T q.
 * coef [rows, heads, 3] float is scratch. */
B2TTS_API int b2tts_delta_rule_scan(const void* qkv, int64_t ldq, const void* beta, const void* a_in, int64_t ldu, const float* a_log,
                                    const float* dt_bias, float* state, float* coef, float* out, const int32_t* seq_start,
                                    const int32_t* seq_pos0, const int32_t* seq_len, const int32_t* seq_slot, int n_tokens, int n_seqs,
                                    int heads, int kv_heads, int dim, int vdim, int dtype, void* stream);
/* Matrix memory with exponential gates per head: i = cap tanh((ig[t, h] + i_bias[h]) / cap), f = logsigmoid(cap tanh((fg[t, h] +
 * f_bias[h]) / cap)); m' = max(f + m, i) (m starts at 0); S <- exp(f + m - m') S + exp(i - m') k v^T, n likewise with k alone;
 * out[t, h] = S^T q / (max(|n . q|, exp(-m')) + 1e-6) with q times dim^(-1/2).  q, k [rows, heads*dim] and v [rows, heads*vdim]
 * share the row stride ldu with ig and fg.  state [slots, heads, dim, vdim], state_nm [slots, heads, dim + 1] (n, then m), both
 * float; gates [rows, heads, 3] float is scratch. */
B2TTS_API int b2tts_matrix_memory_scan(const void* q, const void* k, const void* v, const void* ig, const void* fg, int64_t ldu,
                                       const float* i_bias, const float* f_bias, float cap, float* state, float* state_nm,
                                       float* gates, float* out, const int32_t* seq_start, const int32_t* seq_pos0,
                                       const int32_t* seq_len, const int32_t* seq_slot, int n_tokens, int n_seqs, int heads, int dim,
                                       int vdim, int dtype, void* stream);

/* Gated linear attention per head, state [slots, heads, dim, vdim] float: decay[t, h, i] = sigmoid(z[t, h * dim + i] + z_bias[h * dim
 * + i])^(1 / tau) (in float; z_bias may be null); S[i, :] <- decay[i] S[i, :] + k[i] v^T; out[t, h] = S^T q * dim^(-1/2).  q, k, z
 * [rows, heads*dim] and v [rows, heads*vdim] with their own row strides; decay [rows, heads*dim] float is scratch. */
B2TTS_API int b2tts_gated_linear_scan(const void* q, int64_t ldq, const void* k, int64_t ldk, const void* v, int64_t ldv, const void* z,
                                      int64_t ldz, const float* z_bias, float tau, float* decay, float* state, float* out,
                                      const int32_t* seq_start, const int32_t* seq_pos0, const int32_t* seq_len,
                                      const int32_t* seq_slot, int n_tokens, int n_seqs, int heads, int dim, int vdim, int dtype,
                                      void* stream);

/* ---- decoders whose sublayers are normed on the way in and on the way out with single-gain RMS norms (csrc/sandwich_ops.cu).
 * x[r] (init != 0: starting from zero) += g_out[0] * N(y[r]); h[r] = g_in[0] * N(x[r]) when h != null; N(v) = v / sqrt(mean(v^2) + eps).
 * y = a[a_index ? a_index[r] : r] (a table of a_rows rows when indexed), or, with wa and wb, branch_scale * (N(a) * wa + N(b) * wb);
 * plus sum_k zw[r, k] * (z_idx == null || z_idx[r, k] < n_real ? z[r * top + k] : hin[r]) in ascending k. */
B2TTS_API int b2tts_sandwich_residual(float* x, const void* a, const int32_t* a_index, int a_rows, const void* b, const float* wa,
                                      const float* wb, float branch_scale, const void* z, const float* zw, const int32_t* z_idx,
                                      int top, int n_real, const void* hin, const float* g_out, const float* g_in, void* h,
                                      int rows, int cols, int init, float eps, int dtype, void* stream);
/* In place on rows of y: coef[0] N(y) + coef[1] N(y^2) + coef[2] N(y^3) + coef[3], powers element by element. */
B2TTS_API int b2tts_polynorm(void* y, const float* coef, int rows, int cols, float eps, int dtype, void* stream);
/* maps [rows, 2, heads, vdim]: out[r, h] = (maps[r, 0, h] - lambda * maps[r, 1, h]) / sqrt(mean over vdim of its square + eps) * mult.
 * maps_f32 != 0: the maps are floats whatever `dtype` (the type of out) is. */
B2TTS_API int b2tts_diff_combine(const void* maps, void* out, float lambda, float mult, int rows, int heads, int vdim, float eps,
                                 int maps_f32, int dtype, void* stream);
/* In place: y <- cap * tanh(y / cap). */
B2TTS_API int b2tts_tanh_cap(float* y, int64_t n, float cap, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200TTS_H */
