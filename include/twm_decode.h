/*
 * twm_decode.h — the kernels either side of the W4A16 GEMMs in one decode step, so that a whole
 * step (forward_decode_tw_marlin_graph, crates/kernels/src/generate.rs:2124-2211) can be enqueued
 * through this ABI and captured in one CUDA graph.  Same conventions as twmarlin.h: device
 * pointers owned by the caller, enqueue only, nothing allocated, status returned.  Position and
 * sequence length are read from device buffers (generate.rs:1413-1416), never from launch
 * parameters.  `flags` takes TWM_FLAG_PDL.
 */
#ifndef TWM_DECODE_H
#define TWM_DECODE_H

#include "twmarlin.h"

#ifdef __cplusplus
extern "C" {
#endif

/* x[r][:] (f32) = table[tokens[r]][:] (f16 table [vocab][hidden]); replaces warp_embedding
 * (crates/kernels/src/sampling.rs:16-32). */
twm_status twm_embed(float* x, const void* table_f16, const int* tokens, int rows, int hidden, int flags, void* stream);

/* y (f16) = x * rsqrt(mean(x^2) + eps) * gamma; replaces rmsnorm / fused_residual_rmsnorm
 * (crates/kernels/src/ops.rs:302-336, 928-962; the residual add is the GEMM's TWM_FLAG_ACCUMULATE). */
twm_status twm_rmsnorm(void* y_f16, const float* x, const float* gamma, int rows, int hidden, float eps, int flags,
                       void* stream);

/* x += add, then y = rmsnorm(x) as above (fused_residual_rmsnorm, ops.rs:928-962).  y_f16 may be
 * NULL: only the addition is done.  Used where a row-parallel GEMM's all-reduced output joins the
 * residual stream. */
twm_status twm_add_rmsnorm(void* y_f16, float* x, const float* add, const float* gamma, int rows, int hidden,
                           float eps, int flags, void* stream);

/* Bias + rotate-half RoPE on q and k, bias on v, append k/v at pos_buf[0]; input is the fused QKV
 * GEMM output [q | k | v] (f16), so split_qkv (ops.rs:2300-2345) disappears.  Replaces
 * fused_bias_rope_append_device_pos (ops.rs:2601-2680).  Caches: f16 [max_seq][kv_heads*head_dim].
 * bias may be NULL.  rows > 1 = that many sequences decoding in lock step: qkv [rows][q|k|v],
 * q_out [rows][q], one cache per row ([rows][max_seq][kv_dim]), one shared position. */
twm_status twm_rope_append(void* q_out_f16, void* k_cache_f16, void* v_cache_f16, const void* qkv_f16,
                           const float* bias, int rows, int num_heads, int num_kv_heads, int head_dim,
                           const int* pos_buf, int max_seq, float rope_base, int flags, void* stream);

/* Bytes of scratch twm_attn_decode needs for (rows, num_heads, max_seq). */
size_t twm_attn_scratch_bytes(int rows, int num_heads, int head_dim, int max_seq);

/* Decode attention over the cache, length len_buf[0] (device), split over 128-token chunks and
 * merged; grouped-query heads share their kv head's rows.  Replaces
 * decode_attention_flash_device_len (crates/kernels/src/kv_cache.rs:951-1134; that one allocates
 * its scratch inside the call, this one takes it).  head_dim must be 128. */
twm_status twm_attn_decode(void* out_f16, const void* q_f16, const void* k_cache_f16, const void* v_cache_f16,
                           int rows, int num_heads, int num_kv_heads, int head_dim, const int* len_buf, int max_seq,
                           void* scratch, size_t scratch_bytes, int flags, void* stream);

/* The two passes above as one: the attention kernel takes the fused QKV GEMM output [rows][q | k | v]
 * itself, rotates q on the way in, and the CTA whose chunk holds position pos_buf[0] rotates and
 * appends the new k row and the new v row (bias added) before using them.  Same bits as
 * twm_rope_append followed by twm_attn_decode, one launch less per layer.  rope_table = cos
 * [head_dim/2] then sin [head_dim/2] of pos_buf[0], written once per decode step by twm_rope_table
 * (the freq/theta formulas of ops.rs:2601-2650); it must be the table of the same position. */
twm_status twm_rope_table(float* table, const int* pos_buf, int head_dim, float rope_base, int flags, void* stream);
twm_status twm_attn_decode_rope(void* out_f16, const void* qkv_f16, const float* bias, const float* rope_table,
                                void* k_cache_f16, void* v_cache_f16, int rows, int num_heads, int num_kv_heads,
                                int head_dim, const int* pos_buf, const int* len_buf, int max_seq, void* scratch,
                                size_t scratch_bytes, int flags, void* stream);

/* act (f16 [rows][ffn]) = silu(gate) * up on the fused gate+up GEMM output [rows][gate | up];
 * replaces split_gate_up + fused_silu_mul (ops.rs:2255-2298, 966-977). */
twm_status twm_silu_mul(void* act_f16, const void* gate_up_f16, int rows, int ffn, int flags, void* stream);

/* logits (f32 [vocab]) = W (f16 [vocab][hidden]) . x (f16 [hidden]); the LM head
 * (generate.rs:1727-1735 uses cuBLAS SGEMM on f32).  hidden % 8 == 0. */
twm_status twm_lm_head(float* logits, const void* x_f16, const void* w_f16, int hidden, int vocab, int flags,
                       void* stream);

/* Bytes of scratch twm_argmax_advance needs. */
size_t twm_argmax_scratch_bytes(void);

/* token_out[0] = argmax(logits) (ties: smallest index; 0 when no logit is a number);
 * history[step_buf[0]] = token when step_buf[0] < history_capacity (history may be NULL: a full
 * list is simply not written past its end); then step_buf[0]++, pos_buf[0]++, len_buf[0]++.
 * Replaces the host-side sampling after a full-logits copy (generate.rs:2514, 2531-2534) for
 * greedy decoding. */
twm_status twm_argmax_advance(int* token_out, int* history, int history_capacity, int* pos_buf, int* len_buf,
                              int* step_buf, const float* logits, int n, void* scratch, size_t scratch_bytes, int flags,
                              void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TWM_DECODE_H */
