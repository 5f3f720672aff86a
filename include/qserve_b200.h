/* qserve_b200 -- C ABI of the Blackwell (sm_100a) W4A8KV4 kernel library.
 *
 * Drop-in boundary for the seven `qserve_backend.*` torch-extension modules of mit-han-lab/qserve
 * (kernels/setup.py:158-245).  The reference has no C ABI: its boundary is pybind11 functions taking
 * torch::Tensor.  Every entry point below is the plain-pointer form of one such function; the reference-side
 * binding (a ten-line pybind11 / ctypes stub per function) is shown in INTEGRATION.md, and the shipped Python
 * package `qserve_backend/` is exactly that stub written with ctypes.
 *
 * Conventions
 *   - all pointers are DEVICE pointers unless stated otherwise; `stream` is a cudaStream_t (0 = legacy default);
 *   - fp16 tensors are passed as `const void*` / `void*` to IEEE binary16 data ("half");
 *   - every function returns 0 on success and a negative qs_status otherwise; qs_last_error() returns a
 *     thread-local, NUL-terminated description of the last failure (the Python layer raises RuntimeError with it,
 *     matching the reference's TORCH_CHECK behaviour, fused_attention.cpp:168-199);
 *   - nothing here allocates device memory: outputs and workspaces are caller-owned, so every call is
 *     CUDA-graph capturable; launches go to the caller's stream (the reference GEMMs use the legacy default
 *     stream, gemm_cuda.cu:53 -- using the current stream is a superset);
 *   - there is no CPU fallback: without a CUDA device the launches fail with QS_ERR_CUDA.
 */
#ifndef QSERVE_B200_H_
#define QSERVE_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define QS_ABI_VERSION 1
#if defined(__GNUC__)
#define QS_API __attribute__((visibility("default")))
#else
#define QS_API
#endif

typedef enum qs_status {
  QS_OK = 0,
  QS_ERR_INVALID = -1,
  QS_ERR_CUDA = -2,
  QS_ERR_WORKSPACE = -3,
  QS_ERR_UNSUPPORTED = -4
} qs_status;

QS_API int qs_abi_version(void);
QS_API const char* qs_last_error(void);
/* Enable (1) / disable (0) programmatic dependent launch for all subsequent launches; returns the previous value.
 * With PDL on (default) every kernel runs `griddepcontrol.launch_dependents` at entry and reads STATIC operands -- weights, weight scales,
 * level-2 parameters, the page-pointer table, length_per_sample -- BEFORE `griddepcontrol.wait`, so that its prologue overlaps the previous
 * kernel.  Those tensors must therefore not be written by a kernel of the same stream inside a chain of back-to-back library calls (update block
 * tables / context lengths from the host, as the reference's ModelRunner does, or behind a non-library kernel).  The controls of this header
 * (qs_set_pdl, qs_gemm_force_*, ...) are process-wide and unsynchronised; qs_last_error() is thread-local.  Host-side caches (kernel
 * attributes, SM count, tensor maps) are keyed by the CURRENT device: make the tensors' device current before calling (the Python mirror does). */
QS_API int qs_set_pdl(int enabled);

/* ---------------------------------------------------------------------------------------------------------
 * qserve_backend.qgemm_w4a8_per_chn.gemm_forward_cuda           kernels/csrc/qgemm/w4a8_per_chn/gemm_cuda.cu:596-652
 *   out[m,n] = half( float(sum_k in[m,k]*q[n,k]) * wscales[n] * ascales[m] - w_szs[n] * a_ssums[m] )
 *   in_feats int8 [M,K]; kernel packed uint4 [N,K/2] in the checkpoint layout (w4a8_linear.py:292-322);
 *   wscales, w_szs fp16 [N]; ascales, a_ssums fp16 [M]; out fp16 [M,N].  N % 128 == 0, K % 128 == 0.
 *   workspace: reserved (split-K partial tiles are exchanged through distributed shared memory inside a thread-block
 *   cluster, no global scratch is needed); pass NULL / 0 or a buffer of qs_gemm_workspace_bytes() bytes.
 *   acc_out (optional, may be NULL): raw INT32 accumulators [M,N] for bit-exact parity checks.
 * --------------------------------------------------------------------------------------------------------- */
QS_API int qs_w4a8_gemm_per_chn(const int8_t* in_feats, const int8_t* kernel, const void* wscales, const void* ascales, const void* w_szs,
                         const void* a_ssums, void* out_feats, int32_t* acc_out, int M, int N, int K, void* workspace,
                         size_t workspace_bytes, void* stream);

/* qserve_backend.qgemm_w4a8_per_group.gemm_forward_cuda         kernels/csrc/qgemm/w4a8_per_group/gemm_cuda.cu:630-702
 *   w8[n,k] = (q[n,k]*s2[k/128,n] + z2[k/128,n]) mod 256 as int8 ;  out = half( float(acc) * (wscales[n]*ascales[m]) )
 *   zeros, scales_i8: int8 [K/128, N] with the checkpoint's per-32-column shuffle (w4a8_linear.py:231-277).          */
QS_API int qs_w4a8_gemm_per_group(const int8_t* in_feats, const int8_t* kernel, const int8_t* zeros, const int8_t* scales_i8,
                           const void* wscales, const void* ascales, void* out_feats, int32_t* acc_out, int M, int N, int K,
                           void* workspace, size_t workspace_bytes, void* stream);

/* qserve_backend.qgemm_w8a8.w8a8_gemm_forward_cuda              kernels/csrc/qgemm/w8a8/w8a8_gemm_cuda.cu:532-577
 *   kernel int8 [N,K] row-major;  out = half( float(acc) * (wscales[n]*ascales[m]) )                                  */
QS_API int qs_w8a8_gemm(const int8_t* in_feats, const int8_t* kernel, const void* wscales, const void* ascales, void* out_feats,
                 int32_t* acc_out, int M, int N, int K, void* workspace, size_t workspace_bytes, void* stream);

QS_API size_t qs_gemm_workspace_bytes(void);
/* test hook: force the cluster split-K factor (1, 2, 4 or 8) of the next GEMM calls; 0 = automatic */
QS_API int qs_gemm_force_split(int split);
/* test / tuning hook: force the tokens-per-tile of the GEMMs (32, 64, 128; 0 = automatic: 32 / 64 / 128 by M, and CTA-pair
 * 256-token tiles (cta_group::2) for W4A8 at M >= 512); returns the previous value */
QS_API int qs_gemm_force_tile_tokens(int nt);
/* profiling hook: device buffer of 16 x uint64 per CTA receiving %globaltimer stamps of the GEMM phases; NULL disables */
QS_API int qs_gemm_set_profile_buffer(void* dev_buffer);
/* step tracing: u64 buffer [0] = record count (zero it), then `capacity_records` x (kernel_id << 8 | phase, %globaltimer);
 * block 0 of every kernel logs entry (0), dependency resolved (1) and exit (2); NULL disables (tools/step_timeline.py) */
QS_API int qs_set_trace_buffer(void* dev_buffer, unsigned capacity_records);

/* ---------------------------------------------------------------------------------------------------------
 * qserve_backend.fused_attention.single_query_attention         kernels/csrc/fused_attention/fused_attention.cpp:150-240
 *   q fp16 [B,Hq,D] with row stride q_stride (elements); k, v fp16 [B,Hkv,D] with row strides k_stride, v_stride
 *   (stride(1) == D, stride(2) == 1, fused_attention.cpp:179-180); kv_pointers int64 [B,2,max_blocks] absolute
 *   device addresses of the K then V pages (kvCacheUtils.h:84-90); length_per_sample int32 [B] = context length
 *   INCLUDING the token being decoded (may be NULL: then `timestep` is used); out fp16 [B,Hq,D] contiguous.
 *   Side effect: RoPE(k) and v of the new token are quantised and appended at index length-1.
 *   D must be 128, kv_cache_with_zeros must be 1 (ZINT4 / ZINT8), rotary_embedding_dim must equal D.
 *   workspace (optional): qs_attention_workspace_bytes(...) bytes, zero-initialised once; enables context splits.  */
QS_API int qs_single_query_attention(const void* q, const void* k, const void* v, int64_t q_stride, int64_t k_stride, int64_t v_stride,
                              const int64_t* kv_pointers, const int32_t* length_per_sample, void* out, int batch, int num_heads,
                              int num_kv_heads, int head_dim, int max_blocks_per_seq, int memory_max_seqlen, int tokens_per_block,
                              int size_per_token, int timestep, int rotary_embedding_dim, float rotary_base, int neox_rotary_style,
                              int int4_kv_cache, int kv_cache_with_zeros, void* workspace, size_t workspace_bytes, void* stream);
QS_API size_t qs_attention_workspace_bytes(int batch, int num_heads, int head_dim);

/* qserve_backend.fused_attention.apply_bias_rope_update_kv_cache    kernels/csrc/fused_attention/update_kv_cache.cu:20-108
 *   qkv fp16 [T,(Hq+2Hkv)*D]: q and k are rotated IN PLACE (NeoX), K/V quantised per (token, kv head) into the pages.
 *   kv_pointers may be NULL (rotate only).                                                                          */
QS_API int qs_apply_bias_rope_update_kv_cache(void* qkv, const int32_t* seq_lens, const int32_t* padding_offset, const int64_t* kv_pointers,
                                       int batch, int num_tokens, int max_blocks_per_seq, int head_num, int kv_head_num, int head_dim,
                                       int seq_len, int tokens_per_block, int size_per_token, int rotary_embedding_dim,
                                       float rotary_embedding_base, int rotary_embedding_max_positions, int neox_rotary_style,
                                       int int4_kv_cache, int kv_cache_with_zeros, void* stream);

/* Prompt-phase attention: replaces the third-party call flash_attn.flash_attn_varlen_func(q, k, v, cu_seqlens, cu_seqlens, max_seqlen,
 *   max_seqlen, dropout_p=0.0, causal=True) at qserve/modeling/models/llama_w4a8_unpad.py:232-242.
 *   q [T,Hq,128], k / v [T,Hkv,128] fp16: strided views of the qkv buffer apply_bias_rope_update_kv_cache has rotated in place (row strides in
 *   halfs, multiples of 8); cu_seqlens int32 [batch+1] shared by queries and keys; out fp16 [T,Hq,128].  Causal, no dropout, GQA by
 *   Hq / Hkv.  fp32 softmax, P rounded to fp16 before the second MMA (as flash-attn does); tcgen05 kind::f16, sm_100a only.
 *   max_seqlen must be >= the longest sequence (as for flash-attn: query blocks beyond it are not launched).                          */
QS_API int qs_prefill_attention(const void* q, const void* k, const void* v, int64_t q_stride, int64_t k_stride, int64_t v_stride, void* out,
                         int64_t out_stride, const int32_t* cu_seqlens, int batch, int num_tokens, int max_seqlen, int num_heads,
                         int num_kv_heads, int head_dim, float softmax_scale, void* stream);

/* qserve_backend.fused_attention.compute_padding_offsets         kernels/csrc/fused_attention/input_metadata_helper.cu:33-45 */
QS_API int qs_compute_padding_offsets(int32_t* padding_offsets, const int32_t* cu_seqlens, int batch, int max_seqlen, void* stream);

/* ---------------------------------------------------------------------------------------------------------
 * qserve_backend.layernorm_ops                                   kernels/csrc/layernorm.cpp:47-72
 * --------------------------------------------------------------------------------------------------------- */
/* rms_norm(out, input, weight, epsilon, use_quant): out fp16 (use_quant=0) or int8 (use_quant=1)                   */
QS_API int qs_rms_norm(void* out, const void* input, const void* weight, float epsilon, int use_quant, int tokens, int hidden, void* stream);
/* rms_norm_general(out int8, input, weight, scaling fp16 [tokens] (out) | [1] (in), epsilon, use_per_token_quant)   */
QS_API int qs_rms_norm_general(int8_t* out, const void* input, const void* weight, void* scaling, float epsilon, int use_per_token_quant,
                        int tokens, int hidden, void* stream);
/* rms_norm_general_fuse_sum(out, input, weight, input_sum fp16 [tokens] (out), scaling, epsilon, use_per_token_quant) */
QS_API int qs_rms_norm_general_fuse_sum(int8_t* out, const void* input, const void* weight, void* input_sum, void* scaling, float epsilon,
                                 int use_per_token_quant, int tokens, int hidden, void* stream);
/* invoke_dequant_add_residual_rms_norm_quant: scale_vec fp16 [tokens] or NULL (then scalar `scale`); residual updated in place */
QS_API int qs_dequant_add_residual_rms_norm_quant(int8_t* out, const int32_t* input, void* residual, const void* gamma, const void* scale_vec,
                                           float scale, float epsilon, int tokens, int hidden, void* stream);

/* ---------------------------------------------------------------------------------------------------------
 * qserve_backend.fused_kernels                                   kernels/csrc/fused.cpp:47-70
 * --------------------------------------------------------------------------------------------------------- */
QS_API int qs_invoke_quant(int8_t* out, const void* input, void* scale /* fp16 [tokens] out */, int tokens, int hidden, void* stream);
QS_API int qs_invoke_quant_scalar(int8_t* out, const void* input, float scale, int tokens, int hidden, void* stream);
QS_API int qs_invoke_quant_fuse_sum(int8_t* out, const void* input, void* input_sum, void* scale, int tokens, int hidden, void* stream);
/* Tensor-parallel extension (no reference counterpart: the reference has tp_size = 1 hard-coded, llama_w4a8_unpad.py:115).
 * SURVEY.md 8e parity rule: all ranks quantise their K shard of a token with the same scale.  qs_row_absmax writes the local
 * per-token max |x| (fp32 [tokens]); the caller max-all-reduces it; qs_invoke_quant_given_amax then does the arithmetic of
 * invoke_quant[_fuse_sum] with that amax (input_sum, may be null, is the LOCAL shard's row sum). */
/* Tensor-parallel extension: the sum-all-reduce of a row-parallel GEMM output fused into its consumer ("fused into
 * the GEMM epilogue ... over NVLink").  delta_ptrs[r] = address, valid in THIS process, of rank r's fp16 partial [tokens, hidden] of this
 * phase (peer-mapped symmetric memory); flag_ptrs[r] = rank r's flag pad (16 x u32, zero-initialised, peer-mapped); state = 4 x u32 of
 * local device memory, zero-initialised, owned by the library afterwards.  phase 0 / 1 = o_proj / down_proj (two buffers: see DESIGN.md 6).
 * Semantics: delta = fp16(sum over ranks, fp32, rank order) ; then exactly qs_add_rms_norm_general(out, hidden_out, x, delta, ...).
 * All ranks must issue the same sequence of peer calls. */
QS_API int qs_add_rms_norm_general_peer(int8_t* out, void* hidden_out, const void* x, const void* const* delta_ptrs, void* const* flag_ptrs, void* state,
                                        int world, int rank, int phase, const void* gamma, void* input_sum, void* scaling, float epsilon, int tokens,
                                        int hidden, void* stream);
QS_API int qs_row_absmax(float* amax_out, const void* input, int tokens, int hidden, void* stream);
QS_API int qs_invoke_quant_given_amax(int8_t* out, const void* input, const float* amax, void* input_sum, void* scale, int tokens, int hidden,
                                      void* stream);
QS_API int qs_invoke_dequant_add_residual(void* out, const int32_t* input, const void* residual, const void* scale_vec, float scale, int tokens,
                                   int hidden, void* stream);
QS_API int qs_invoke_dequant(void* out, const int32_t* input, float scale, int tokens, int hidden, int input_stride, int out_stride, void* stream);

/* ---------------------------------------------------------------------------------------------------------
 * qserve_backend.activation_ops                                  kernels/csrc/activation.cpp:25-39
 * --------------------------------------------------------------------------------------------------------- */
QS_API int qs_silu_and_mul(void* out, const void* input, int tokens, int d, void* stream);
QS_API int qs_gelu_new(void* out, const void* input, int tokens, int d, void* stream);
QS_API int qs_gelu_fast(void* out, const void* input, int tokens, int d, void* stream);
/* scale_out_vec float [tokens] (out) and tmp float [tokens,d] select the per-token overload; both NULL = scalar scale_out */
QS_API int qs_dequant_silu_and_mul_quant(int8_t* out, const int32_t* input, float scale_gate, float scale_up, float scale_out,
                                  float* scale_out_vec, float* tmp, int tokens, int d, void* stream);

/* ---------------------------------------------------------------------------------------------------------
 * Fused extensions (NOT part of the reference surface; bit-identical to the op sequences they replace).
 * Used by qserve_b200/decode.py to cut the launch count of the decode step.
 * --------------------------------------------------------------------------------------------------------- */
/* hidden_out = half(x + delta)   [the torch `residual + out_buf` of llama_w4a8_unpad.py:348,360]
 * followed by rms_norm_general[_fuse_sum](out, hidden_out, weight, input_sum | NULL, scaling, epsilon, per_token=1)      */
QS_API int qs_add_rms_norm_general(int8_t* out, void* hidden_out, const void* x, const void* delta, const void* weight, void* input_sum,
                                   void* scaling, float epsilon, int tokens, int hidden, void* stream);
/* single_query_attention followed by invoke_quant[_fuse_sum] of the [B, Hq*D] result: out_q int8 [B, Hq*D], out_scale fp16 [B],
 * out_sum fp16 [B] or NULL.  The fp16 attention row stays in `workspace` (>= qs_attention_workspace_bytes, zero-initialised
 * once, L2 resident); the last CTA of a token to finish quantises it, so the result is bit-identical to the two-op sequence. */
QS_API int qs_single_query_attention_quant(const void* q, const void* k, const void* v, int64_t q_stride, int64_t k_stride, int64_t v_stride,
                                           const int64_t* kv_pointers, const int32_t* length_per_sample, int8_t* out_q, void* out_scale,
                                           void* out_sum, int batch, int num_heads, int num_kv_heads, int head_dim, int max_blocks_per_seq,
                                           int memory_max_seqlen, int tokens_per_block, int size_per_token, int timestep,
                                           int rotary_embedding_dim, float rotary_base, int int4_kv_cache, int kv_cache_with_zeros, void* workspace,
                                           size_t workspace_bytes, void* stream);
/* silu_and_mul(input [tokens, 2d]) followed by invoke_quant[_fuse_sum](out, act, input_sum | NULL, scale)                 */
/* greedy sampling helper for the decode runner: out[r] = index of the first maximum of logits[r, :] (fp16, NaN = maximum), as
 * torch.argmax(logits, -1) does in the reference's sampler */
QS_API int qs_argmax_rows(int64_t* out, const void* logits, int rows, int vocab, void* stream);
QS_API int qs_silu_and_mul_quant(int8_t* out, const void* input, void* input_sum, void* scale, int tokens, int d, void* stream);

/* ---------------------------------------------------------------------------------------------------------
 * Unquantised hybrid decoders (qserve_b200/hybrid.py): attention layers and recurrent layers in one stack over an fp32
 * residual stream.  Not part of the reference surface.  `dtype` is the storage type of activations, weights tables and
 * the key/value cache; norms, scores, softmax weights, rotary angles, decays, the recurrent state and the stream are fp32.
 * All kernels take a FLAT batch of tokens with per-token tables (slot of the sequence, position) and, for the recurrent
 * layer, per-entry tables (first row, length, slot, position of the first token of each sequence's run of tokens).
 * --------------------------------------------------------------------------------------------------------- */
#define QS_DTYPE_BF16 0
#define QS_DTYPE_F32 1
/* out[t, c] (c < copies: out is [tokens, copies, width]) = table[tokens[t]] * scale + pair_table[prev[t] < 0 ? buckets : (prev[t] * mul_prev + tokens[t] * mul_cur) % buckets]; pair_table may be NULL */
QS_API int qs_hyb_embed(float* out, const int32_t* tokens, const int32_t* prev, const void* table, const void* pair_table, int tokens_n,
                        int width, int buckets, int64_t mul_prev, int64_t mul_cur, float scale, int copies, int dtype, void* stream);
/* [x <- x + add (storage type, may be NULL);]  out_k = x * rsqrt(mean(x^2) + eps) * (offset + w_k), k = 1, 2 (out2 / w2 may be NULL);
 * x fp32 [tokens, width] (updated in place when add is given), w fp32 */
QS_API int qs_hyb_rms_norm(void* out1, void* out2, float* x, const void* add, const float* w1, const float* w2, float offset, float eps,
                           int tokens_n, int width, int dtype, void* stream);
/* x[i] += y[i] (x fp32, y in the storage type) */
QS_API int qs_hyb_residual_add(float* x, const void* y, int64_t n, int dtype, void* stream);
/* out[t, i] = gelu_tanh(in[t, i]) * in[t, ff + i]; out rows of out_stride elements */
QS_API int qs_hyb_gelu_tanh_mul(void* out, int64_t out_stride, const void* in, int tokens_n, int ff, int dtype, void* stream);
/* interleaved rotary embedding (angle = position * inv_freq[pair], cos / sin times `amplitude`) of the first rot_dims entries of every
 * query / key map of the projection rows [H*maps*dim q | G*maps*dim k | G*vdim v] (q in place), keys and values appended to the pages
 * K [page][page_size][G][maps*dim], V [page][page_size][G][vdim] through block_table [slots, max_blocks] */
QS_API int qs_hyb_rope_append(void* proj, int64_t stride, const int32_t* tok_slot, const int32_t* tok_pos, const int32_t* block_table,
                              int max_blocks, void* kpool, void* vpool, const float* inv_freq, float amplitude, int tokens_n, int heads,
                              int kv_heads, int maps, int dim, int vdim, int rot_dims, int page_size, int dtype, void* stream);
/* Optional parts of qs_hyb_attention / qs_hyb_attention_fast (a NULL pointer: none of them).
 * keep_first: with a window (and no chunks), positions < keep_first of the sequence stay visible to every later query.
 * slopes (fp32 [heads], may be NULL): slopes[h] * (query position - key position) is taken off head h's scaled score.
 * gate (storage type, may be NULL): head h's output of token t is multiplied by sigmoid(gate[t * gate_stride + h]). */
typedef struct {
  int keep_first;
  const float* slopes;
  const void* gate;
  int64_t gate_stride;
} qs_attn_extra;
/* causal attention of every token over positions first..tok_pos of its sequence in the paged cache, `maps` (1 or 2) softmax maps per head
 * over shared values: o = a1 [- lambda a2]; head_norm: o *= rsqrt(mean(o^2) + eps); o *= out_scale.  out [tokens, heads*vdim].
 * first = start of the position's chunk of `chunk` positions (0: no chunks; chunks count from position 0 of the sequence), and at least
 * tok_pos - window + 1 (0: no window).  sinks (fp32 [heads], may be NULL): one more term exp(sinks[head]) in every softmax denominator of
 * the head, without a value and outside `scale`. */
QS_API int qs_hyb_attention(void* out, int64_t out_stride, const void* q, int64_t q_stride, const void* kpool, const void* vpool,
                            const int32_t* tok_slot, const int32_t* tok_pos, const int32_t* block_table, int max_blocks, int tokens_n,
                            int heads, int kv_heads, int maps, int dim, int vdim, float scale, float lambda, float out_scale, float eps,
                            int head_norm, int page_size, int chunk, int window, const float* sinks, const qs_attn_extra* extra, int dtype,
                            void* stream);
/* The same attention on the fast kernels (bfloat16 storage, dim and vdim multiples of 16, vdim in {32, 64, 96, 128, 256}, heads / kv_heads <= 16):
 * entries of at least 16 tokens run as 64-row tiles on the tensor cores (tile_entry / tile_row0: entry and first row within it of every tile;
 * long_tokens: their token rows), the tokens listed in short_tokens one by one, the query heads of a key/value head as the rows of a
 * tensor-core tile and the keys shared out over several blocks.  scratch: fp32, qs_hyb_attention_scratch_floats elements.
 * qs_hyb_attention_fast_supported returns 1 if the shape qualifies. */
QS_API int qs_hyb_attention_fast_supported(int dtype, int heads, int kv_heads, int maps, int dim, int vdim, int64_t q_stride);
/* fp32 elements of scratch that qs_hyb_attention_fast needs for a step of `tokens` tokens */
QS_API int64_t qs_hyb_attention_scratch_floats(int tokens, int heads, int kv_heads, int maps, int vdim);
QS_API int qs_hyb_attention_fast(void* out, int64_t out_stride, const void* q, int64_t q_stride, const void* kpool, const void* vpool,
                                 const int32_t* tok_slot, const int32_t* tok_pos, const int32_t* block_table, int max_blocks,
                                 const int32_t* tile_entry, const int32_t* tile_row0, int n_tiles, const int32_t* long_tokens, int n_long,
                                 const int32_t* short_tokens, int n_short, const int32_t* entry_start, const int32_t* entry_len,
                                 const int32_t* entry_slot, const int32_t* entry_pos0, float* scratch, int heads, int kv_heads, int maps, int dim,
                                 int vdim, float scale, float lambda, float out_scale, float eps, int head_norm, int page_size, int chunk,
                                 int window, const float* sinks, const qs_attn_extra* extra, int dtype, void* stream);
/* gated delta rule over projection rows [G*dim q | G*dim k | H*vdim v | H*vdim gate | H b | H a]: short convolution (taps) + silu on
 * q | k | v, unit q (times dim^-1/2) and k, beta = sigmoid(b), decay = exp(-exp(a_log) softplus(a + dt_bias)), then per head
 * S <- decay S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q; out = o * rsqrt(mean(o^2) + eps) * norm_w * silu(gate).
 * state fp32 [slots, H, dim, vdim], conv_state fp32 [slots, taps-1, 2 G dim + H vdim]; a run that starts at position 0 starts from zero.
 * prep fp32 [tokens, 2 G dim + H vdim + 2 H] and o_raw fp32 [tokens, H vdim] are scratch. */
QS_API int qs_hyb_gated_delta(void* out, int64_t out_stride, float* prep, float* o_raw, const void* proj, int64_t stride, const float* conv_w,
                              float* conv_state, float* state, const float* a_log, const float* dt_bias, const float* norm_w,
                              const int32_t* tok_entry, const int32_t* tok_pos, const int32_t* entry_start, const int32_t* entry_len,
                              const int32_t* entry_slot, const int32_t* entry_pos0, int tokens_n, int entries, int heads, int kv_heads,
                              int dim, int vdim, int taps, float unit_eps, float eps, int dtype, void* stream);

/* Residual streams x fp32 [tokens, streams, width], streams <= 16 (hyper-connections; streams = 1 with all coefficients 1 is the plain
 * residual).  In order:
 * (upd != NULL) every stream at once from the old ones: x_t <- sum_s upd_mix[s, t] x_s + upd_out[t] upd (upd: [tokens, width], fp32 if
 * upd_f32, else storage type);  u = sum_s in_coef[s] x_s (in_coef NULL: the plain sum);  (out_sum != NULL) out_sum <- u (fp32);
 * (out_h != NULL) out_h <- u brought to unit RMS in `groups` equal consecutive parts, times (offset + w) (storage type; w fp32 [width]). */
QS_API int qs_hyb_stream_norm(void* out_h, float* out_sum, float* x, int streams, const void* upd, int upd_f32, const float* upd_mix,
                              const float* upd_out, const float* in_coef, const float* w, int groups, float offset, float eps, int tokens_n,
                              int width, int dtype, void* stream);
/* y = scale (a rsqrt(mean(a^2) + eps) wa + b rsqrt(mean(b^2) + eps) wb) per row; a, b storage type [tokens, width], y fp32 */
QS_API int qs_hyb_branch_norm_mean(float* y, const void* a, const void* b, const float* wa, const float* wb, float scale, float eps, int tokens_n,
                                   int width, int dtype, void* stream);
/* Query / key preparation and cache append for one softmax map per head.  Projection rows [H*dim q | G*dim k | G*vdim v]; bias (fp32, same
 * layout) and q_factor (fp32 [H]) may be NULL.  Per head: + bias; (unit_rms) x *= rsqrt(mean(x^2) + eps); rotary on the first rot_dims
 * entries (rot_layout 0: pairs (2i, 2i+1); 1: pairs (i, i + rot_dims/2); angle = position * inv_freq[i]; rot_dims 0: none); queries times
 * q_factor[head], in place.  Keys and values (+ bias) go to the pages K [page][page_size][G][dim], V [page][page_size][G][vdim].
 * q_gain / k_gain (fp32 [dim], may be NULL): gains of the unit-RMS heads, shared by the heads.  tied_values: the rows have no v part, a key
 * head's value is that key head as projected (+ bias), not yet normed (vdim == dim). */
QS_API int qs_hyb_qk_prepare_append(void* proj, int64_t stride, const float* bias, const float* q_factor, const int32_t* tok_slot,
                                    const int32_t* tok_pos, const int32_t* block_table, int max_blocks, void* kpool, void* vpool,
                                    const float* inv_freq, int rot_layout, int rot_dims, int unit_rms, float eps, int tokens_n, int heads,
                                    int kv_heads, int dim, int vdim, int page_size, const float* q_gain, const float* k_gain, int tied_values,
                                    int dtype, void* stream);
/* Gate recurrence (HGRN2) over projection rows [H*dim q | H*dim f | H*vdim v]: q <- silu(q), f <- lower + (1 - lower) sigmoid(f + f_bias)
 * (fp32 [H*dim] each), per head S <- diag(f) S + (1 - f) v^T, o = S^T q, out = o rsqrt(mean(o^2) + eps) norm_w (fp32 [vdim], may be NULL).
 * state fp32 [slots, H, dim, vdim]; a run that starts at position 0 starts from zero.  prep fp32 [tokens, 2 H dim + H vdim] and o_raw fp32
 * [tokens, H vdim] are scratch. */
QS_API int qs_hyb_gate_recurrence(void* out, int64_t out_stride, float* prep, float* o_raw, const void* proj, int64_t stride, const float* f_bias,
                                  const float* lower, const float* norm_w, float* state, const int32_t* entry_start, const int32_t* entry_len,
                                  const int32_t* entry_slot, const int32_t* entry_pos0, int tokens_n, int entries, int heads, int dim, int vdim,
                                  float eps, int dtype, void* stream);
/* Retention over projection rows [H*dim q | H*dim k | H*vdim v | H*vdim gate]: q and k rotated on their first rot_dims entries (entry i
 * paired with i + rot_dims/2, angle = position * inv_freq[i]), k times k_scale, per head S <- head_decay[h] S + k v^T, o = S^T q,
 * out = o rsqrt(mean(o^2) + eps) [silu(gate) if gated].  state, prep and o_raw as for the gate recurrence. */
QS_API int qs_hyb_retention(void* out, int64_t out_stride, float* prep, float* o_raw, const void* proj, int64_t stride, const float* head_decay,
                            const float* inv_freq, int rot_dims, float k_scale, int gated, float* state, const int32_t* tok_pos,
                            const int32_t* entry_start, const int32_t* entry_len, const int32_t* entry_slot, const int32_t* entry_pos0,
                            int tokens_n, int entries, int heads, int dim, int vdim, float eps, int dtype, void* stream);
/* Gated linear attention over projection rows [H*dim q | H*dim k | H*vdim v | H*vdim gate | ...] and decay logits z fp32 [tokens, H*dim]
 * (+ z_bias fp32 [H*dim], may be NULL): q times dim^-1/2, a = sigmoid(z)^(1/tau) per head and row, per head S <- diag(a) S + k v^T, o = S^T q,
 * out = o rsqrt(mean(o^2) + eps) norm_w (fp32 [vdim], may be NULL) silu(gate).  state fp32 [slots, H, dim, vdim]; a run that starts at position 0
 * starts from zero.  prep fp32 [tokens, 3 H dim + H vdim] and o_raw fp32 [tokens, H vdim] are scratch. */
QS_API int qs_hyb_gated_linear(void* out, int64_t out_stride, float* prep, float* o_raw, const void* proj, int64_t stride, const float* z,
                               const float* z_bias, float tau, const float* norm_w, float* state, const int32_t* entry_start,
                               const int32_t* entry_len, const int32_t* entry_slot, const int32_t* entry_pos0, int tokens_n, int entries, int heads,
                               int dim, int vdim, float eps, int dtype, void* stream);
/* Mixture-of-experts router: fp32 logits z = w_router [experts, width] h.  route fp32 [tokens, experts] (weight of a chosen expert, 0
 * elsewhere), top_idx int32 / top_w fp32 [tokens, top], best first (ties: the lower index).
 * QS_ROUTER_SOFTMAX: scores softmax(z) over all experts, the `top` largest kept as they are (correction, groups, keep unused).
 * QS_ROUTER_SIGMOID_GROUPS: scores s = sigmoid(z); the choice is made on s + correction (fp32 [experts], may be NULL): the experts form
 * `groups` equal runs of neighbours, a group's score is the sum of its two largest choice scores, only experts of the `keep` best groups can
 * be chosen, the `top` largest choice scores win; weights s / (sum of the winners' s + 1e-20). */
#define QS_ROUTER_SOFTMAX 0
#define QS_ROUTER_SIGMOID_GROUPS 1
QS_API int qs_hyb_moe_router(float* route, int32_t* top_idx, float* top_w, const void* h, const float* w_router, int tokens_n, int width,
                             int experts, int top, int mode, const float* correction, int groups, int keep, int dtype, void* stream);
/* Activation of all experts' columns of a token: in rows [F gate | F up], F = experts * ff + ff_shared (the shared expert's columns last);
 * g = min(gate, limit), u = clamp(up, -limit, limit), out = route[t, expert] g sigmoid(alpha g) (u + shift); shared columns: weight 1 and
 * limit_shared.  limit = +inf, alpha = 1, shift = 0 is silu(gate) * up.  out [tokens, F]. */
QS_API int qs_hyb_moe_act(void* out, const void* in, const float* route, int tokens_n, int experts, int ff, float limit, int ff_shared,
                          float limit_shared, float alpha, float shift, int dtype, void* stream);
/* Expert-sorted rows of a mixture of experts.  Entry i = token * top + choice of top_idx [tokens, top]; the sorted order holds expert 0's
 * entries first, then expert 1's, ..., each in token order.  row_of [tokens * top]: the entry's sorted row; src_token [tokens * top]: the token of
 * a sorted row; ends [experts]: one past the last row of each expert.  work: int32, qs_hyb_moe_plan_work_ints(experts) elements. */
QS_API int qs_hyb_moe_plan(int32_t* ends, int32_t* row_of, int32_t* src_token, int32_t* work, const int32_t* top_idx, int tokens_n, int experts,
                           int top, void* stream);
QS_API int64_t qs_hyb_moe_plan_work_ints(int experts);
/* xs[row] = h[src_token[row]] (storage type rows of `width`) */
QS_API int qs_hyb_moe_gather(void* xs, const void* h, const int32_t* src_token, int rows, int width, int dtype, void* stream);
/* y[t] = shared[t] + sum_k top_w[t, k] rows[row_of[t * top + k]]; y fp32 [tokens, width]; rows, shared (may be NULL) storage type */
QS_API int qs_hyb_moe_combine(float* y, const void* rows, const void* shared, const int32_t* row_of, const float* top_w, int tokens_n, int top,
                              int width, int dtype, void* stream);

/* Residual update and norm of a plain fp32 stream x [tokens, width]: x <- x + add1 + add2 + add_bias (each may be NULL; add1 / add2 rows fp32
 * if their flag is set, else of the storage type; add_bias fp32 [width]); cat_out (may be NULL) <- [x | x0] per token in the storage type;
 * out_h (may be NULL) <- norm of x: QS_NORM_RMS x rsqrt(mean x^2 + eps) w, QS_NORM_LAYER (x - mean) rsqrt(var + eps) w + b (b may be NULL). */
#define QS_NORM_RMS 1
#define QS_NORM_LAYER 2
QS_API int qs_hyb_stream_update_norm(void* out_h, void* cat_out, float* x, const float* x0, const void* add1, int add1_f32, const void* add2,
                                     int add2_f32, const float* add_bias, const float* w, const float* b, int kind, float eps, int tokens_n,
                                     int width, int dtype, void* stream);
/* out[t, i] = gelu_tanh(in[t, i] + bias[i]) (bias fp32, may be NULL); rows of in_stride / out_stride elements */
QS_API int qs_hyb_bias_gelu_tanh(void* out, int64_t out_stride, const void* in, int64_t in_stride, const float* bias, int tokens_n, int ff,
                                 int dtype, void* stream);
/* Post-norm residual update: y = add (+ add_bias, fp32 [width], may be NULL); x <- x + y rsqrt(mean(y^2) + eps) (offset + w) (* ls, fp32
 * [width], may be NULL); out_h (may be NULL) <- x in the storage type.  add rows: fp32 if add_f32, else storage type; x fp32 [tokens, width]. */
QS_API int qs_hyb_post_norm_update(void* out_h, float* x, const void* add, int add_f32, const float* add_bias, const float* w, const float* ls,
                                   float offset, float eps, int tokens_n, int width, int dtype, void* stream);
/* out[i] = x[i] in the storage type (x fp32) */
QS_API int qs_hyb_cast_rows(void* out, const float* x, int64_t n, int dtype, void* stream);
/* out[t, i] = act(in[t, i] + bias[i]) * (in[t, ff + i] + bias[ff + i]) (bias fp32 [2 ff], may be NULL); rows of in_stride / out_stride elements */
#define QS_ACT_GELU_TANH 0
#define QS_ACT_SILU 1
QS_API int qs_hyb_bias_gated_act(void* out, int64_t out_stride, const void* in, int64_t in_stride, const float* bias, int tokens_n, int ff, int act,
                                 int dtype, void* stream);
/* x[i] <- cap tanh(x[i] / cap), fp32 in place */
QS_API int qs_hyb_softcap(float* x, int64_t n, float cap, void* stream);

/* Latent attention (csrc/hybrid_latent.cu): the pages hold, per position, kv_rank numbers of a normed latent and rot_dim numbers of a rotated
 * key part shared by all heads: pool [page][page_size][kv_rank + rot_dim].
 * qs_hyb_latent_prepare: from the rows of the first projection (query latent at column col_q, q_rank wide; key/value latent and rotated part
 * at col_kv, kv_rank + rot_dim wide): cq [tokens, q_rank] = unit-RMS query latent times gain_q; the token's cell = [unit-RMS latent times
 * gain_kv | rotated part].  Rotation: rot_layout 1 pairs entry i < rot_dims/2 with entry i + rot_dims/2, rot_layout 0 pairs entries
 * (2i, 2i + 1); angle = position * inv_freq[i], cos and sin times `amplitude`.  q_rank 0: there is no query latent (cq, gain_q may be NULL). */
QS_API int qs_hyb_latent_prepare(void* cq, const void* proj, int64_t stride, int col_q, int col_kv, const float* gain_q, const float* gain_kv,
                                 const float* inv_freq, int rot_dims, const int32_t* tok_slot, const int32_t* tok_pos,
                                 const int32_t* block_table, int max_blocks, void* pool, int tokens_n, int q_rank, int kv_rank, int rot_dim,
                                 int page_size, float eps, int rot_layout, float amplitude, int dtype, void* stream);
/* qa [tokens, heads, kv_rank + rot_dim] = [qlat[head, token, :] | rotated q[token, head * (dim + rot_dim) + dim ...]]: the queries as they are
 * scored against the cells (qlat [heads, tokens, kv_rank]: the unrotated query parts taken through the heads' key up-projections).  qa may be
 * NULL.  rotate_back: the rotated part also replaces q's own. */
QS_API int qs_hyb_latent_query(void* qa, const void* qlat, void* q, int64_t q_stride, const float* inv_freq, int rot_dims, const int32_t* tok_pos,
                               int tokens_n, int heads, int dim, int kv_rank, int rot_dim, int rotate_back, int rot_layout, float amplitude, int dtype,
                               void* stream);
/* out [heads, tokens, kv_rank] = softmax-weighted sum of the cells' first kv_rank numbers over positions first..tok_pos (first as in
 * qs_hyb_attention), scores scale * qa . cell in fp32.  Any shape with kv_rank <= 512.  sinks (fp32 [heads], may be NULL): one more term
 * exp(sinks[head]) in the head's softmax denominators, without a value and outside `scale`. */
QS_API int qs_hyb_latent_attention(void* out, const void* qa, const void* pool, const int32_t* tok_slot, const int32_t* tok_pos,
                                   const int32_t* block_table, int max_blocks, int tokens_n, int heads, int kv_rank, int rot_dim, float scale,
                                   int page_size, int chunk, int window, const float* sinks, int dtype, void* stream);
/* The same on the tensor cores where qs_hyb_latent_attention_fast_supported returns 1 (bfloat16 storage, kv_rank in {32, 64, 128, 256, 512},
 * kv_rank + rot_dim a multiple of 8): the 64 rows of a tile are (token, head) pairs of one sequence.  Entries of at least 16 tokens run by the
 * tile tables of the batch (tile_entry / tile_row0: entry and first row of every span of 64 tokens), the tokens listed in short_tokens one
 * by one with their cells shared out over several blocks.  scratch: fp32, qs_hyb_latent_attention_scratch_floats elements. */
QS_API int qs_hyb_latent_attention_fast_supported(int dtype, int heads, int kv_rank, int rot_dim);
QS_API int64_t qs_hyb_latent_attention_scratch_floats(int tokens, int heads, int kv_rank);
QS_API int qs_hyb_latent_attention_fast(void* out, const void* qa, const void* pool, const int32_t* tok_slot, const int32_t* tok_pos,
                                        const int32_t* block_table, int max_blocks, const int32_t* tile_entry, const int32_t* tile_row0,
                                        int n_tiles, const int32_t* short_tokens, int n_short, const int32_t* entry_start,
                                        const int32_t* entry_len, const int32_t* entry_slot, const int32_t* entry_pos0, int tokens_n,
                                        float* scratch, int heads, int kv_rank, int rot_dim, float scale, int page_size, int chunk, int window,
                                        const float* sinks, int dtype, void* stream);
/* out[t, h * vdim + j] = o * sigmoid(gate[t, col_g + h]) (gate may be NULL: no gate; gate_wide: gate[t, col_g + h * vdim + j]); o = ov[h, t, j] (ov [heads, tokens, vdim]) or, for tokens
 * of entries of at least min_long tokens when alt is given, alt[t, h * vdim + j] */
QS_API int qs_hyb_latent_gate_out(void* out, int64_t out_stride, const void* ov, const void* alt, int64_t alt_stride, const int32_t* tok_entry,
                                  const int32_t* entry_len, int min_long, const void* gate, int64_t gate_stride, int col_g, int tokens_n, int heads,
                                  int vdim, int gate_wide, int dtype, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* QSERVE_B200_H_ */
