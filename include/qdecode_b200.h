/* qdecode_b200.h -- the small kernels a decode step runs BETWEEN the packed GEMVs of a Llama / Qwen2
 * style decoder layer, for one new token per sequence (B200, sm_100a).  Part of libqgemv_b200.so.
 *
 * The reference project leaves this work to the framework: its decode loop is the Hugging Face model
 * under torch.compile(mode='reduce-overhead') (ai_accel_lab/runtime_v5.py:7-23), i.e. generated
 * element-wise kernels between its Triton GEMVs.  Here each step between two GEMVs is ONE hand-written
 * kernel, so a layer is about a dozen launches and a CUDA graph of the whole step stays short:
 *
 *   qdec_rmsnorm       residual update + RMS normalisation            (2 per layer + 1 final)
 *   qdec_rope_append   rotary embedding of q and k, k / v appended to the cache
 *   qdec_attention     one query token per sequence over the cache (grouped-query, split over the sequence)
 *   qdec_silu_mul      silu(gate) * up, where the two projections could not be fused into one GEMV
 *
 * Arithmetic follows what a 16-bit framework computes operator by operator: values are rounded to
 * the activation type (fp16 or bf16; `dtype` is a qgemv_dtype) wherever a separate operator would
 * store them, sums and softmax run in fp32.  All tensors are row-major with unit inner stride;
 * every pointer is device memory; nothing allocates, synchronises or waits on another CTA; all
 * entry points are capturable in a CUDA graph.  Return codes and qgemv_error_string() as in
 * qgemv_b200.h.
 */
#ifndef QDECODE_B200_H
#define QDECODE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* h[m, :] = r(h[m, :] + delta[m, :]) in place when delta != NULL, then
 * y[m, :] = r(weight[:] * r(h[m, :] * rsqrt(mean(h[m, :]^2) + eps))).
 * hidden: a multiple of 8, at most 16384; h, delta, y: [rows, hidden] with leading dimensions ldh,
 * ldd, ldy (elements) and 16-byte aligned rows; weight: [hidden] of the activation type. */
int qdec_rmsnorm(void* h, int64_t ldh, const void* delta, int64_t ldd, const void* weight, void* y, int64_t ldy,
                 int rows, int hidden, float eps, int dtype, void* stream);

/* Rotary embedding (rotate-half convention) of the new token's queries and keys, and the append of
 * its keys and values to the cache, at position *pos (a device int64, so a captured graph can be
 * replayed for every token):
 *   q[b, h, :]            <- r(r(q * cos) + r(rot(q) * sin))           in place, h < q_heads
 *   kcache[b, h, *pos, :] <- the same of k[b, h, :];   vcache[b, h, *pos, :] <- v[b, h, :]
 * q: [batch, q_heads * head_dim] (ldq), k / v: [batch, kv_heads * head_dim] (ldk, ldv);
 * cos / sin: [table_rows, head_dim] of the activation type, row *pos is used;
 * kcache / vcache: [batch, kv_heads, max_len, head_dim] contiguous.  head_dim: even, at most 256.
 * A position outside [0, min(max_len, table_rows)) writes nothing and raises *status (a device
 * int32, may be NULL) to 1. */
int qdec_rope_append(void* q, int64_t ldq, const void* k, int64_t ldk, const void* v, int64_t ldv,
                     const void* cos_table, const void* sin_table, int table_rows, const int64_t* pos,
                     void* kcache, void* vcache, int batch, int q_heads, int kv_heads, int head_dim, int max_len,
                     int32_t* status, int dtype, void* stream);

/* Scratch of qdec_attention for these sizes, in bytes (256-byte aligned device memory, zero before
 * the first call; it is left ready for the next call). */
size_t qdec_attention_workspace_bytes(int batch, int q_heads, int kv_heads, int head_dim, int max_len);

/* out[b, h, :] = softmax_j(scale * q[b, h, :] . K[b, h / group, j, :]) . V[b, h / group, j, :] over the cache
 * positions j = 0 .. *pos (inclusive: the new token's own key was appended first), group = q_heads /
 * kv_heads (1..8, q_heads a multiple of kv_heads), head_dim 64 or 128.
 * q: [batch, q_heads * head_dim] (ldq); out the same shape (ldo), rounded to the activation type.
 * The sequence is cut into slices handled by different CTAs; the last CTA to finish a (sequence,
 * kv head) merges the slices (arrival counter in the workspace, no waiting). */
int qdec_attention(const void* q, int64_t ldq, const void* kcache, const void* vcache, const int64_t* pos,
                   void* out, int64_t ldo, int batch, int q_heads, int kv_heads, int head_dim, int max_len,
                   float scale, void* workspace, size_t workspace_bytes, int dtype, void* stream);

/* y[i] = r(r(silu(gate[i])) * up[i]) for [rows, width] tensors (leading dimensions in elements). */
int qdec_silu_mul(const void* gate, int64_t ldg, const void* up, int64_t ldu, void* y, int64_t ldy,
                  int rows, int width, int dtype, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* QDECODE_B200_H */
