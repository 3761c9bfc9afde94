// Launchers of the decoder-layer glue kernels (decoder_ops.cu). All asynchronous on the
// context's stream; activations fp32, token-major. The *_planes forms (and attention with hi/lo
// given) write their result as the two bf16 planes the tensor-core projection reads, instead of
// fp32: hi = bf16(v), lo = bf16(v - hi), same element order.
#pragma once

#include <cuda_bf16.h>

#include <cstddef>
#include <cstdint>

struct csdr_context;

namespace csdr {

void op_rmsnorm(csdr_context* ctx, const float* x, const float* w, uint32_t T, uint32_t H, float eps, float* out);
void op_rmsnorm_planes(csdr_context* ctx, const float* x, const float* w, uint32_t T, uint32_t H, float eps,
                       __nv_bfloat16* hi, __nv_bfloat16* lo);
// RMS normalisation in two halves for hidden states split over tensor-parallel ranks (H = this
// rank's slice): planes of w*x plus per-token sums of squares; and the normalised values once
// the sums over the whole width are known.
void op_scale_sumsq_planes(csdr_context* ctx, const float* x, const float* w, uint32_t T, uint32_t H,
                           __nv_bfloat16* hi, __nv_bfloat16* lo, float* sumsq);
void op_norm_from_sumsq(csdr_context* ctx, const float* x, const float* w, const float* sumsq, uint32_t T,
                        uint32_t H, uint32_t full_width, float eps, float* out);
void op_add_rmsnorm(csdr_context* ctx, float* hidden, const float* delta, const float* w, uint32_t T,
                    uint32_t H, float eps, float* out);
// kc, vc: the layer's cache, fp32 or bf16 as kv_dtype (CSDR_DTYPE_*) says.
void op_rope_cache(csdr_context* ctx, float* q, const float* k, const float* v, void* kc, void* vc, int kv_dtype,
                   const int32_t* seq_of, const int32_t* pos_of, uint32_t T, uint32_t QH, uint32_t KVH,
                   uint32_t HD, uint32_t max_seq, float theta);
void op_attention(csdr_context* ctx, const float* q, const void* kc, const void* vc, int kv_dtype, const int32_t* seq_of,
                  const int32_t* pos_of, uint32_t T, uint32_t QH, uint32_t KVH, uint32_t HD, uint32_t max_seq,
                  float* out, __nv_bfloat16* hi = nullptr, __nv_bfloat16* lo = nullptr);
// A decode step (every token of a different sequence): rotary embedding of q and of the new
// keys, the cache write of the new keys and values, and attention in ONE launch. q, k_new, v_new
// are the projection outputs as they stand (not rotated); the kernel takes a sequence's newest
// key and value from them, rounded as the cache holds them, and files them in the cache.
// head_dim 64, 128 or 256 (attention_step_supported).
bool attention_step_supported(uint32_t HD);
void op_attention_step(csdr_context* ctx, const float* q, const float* k_new, const float* v_new, float theta, void* kc,
                       void* vc, int kv_dtype, const int32_t* seq_of, const int32_t* pos_of, uint32_t T, uint32_t QH,
                       uint32_t KVH, uint32_t HD, uint32_t max_seq, float* out, __nv_bfloat16* hi = nullptr,
                       __nv_bfloat16* lo = nullptr);
void op_silu_mul(csdr_context* ctx, const float* gate, const float* up, size_t n, float* out);
void op_silu_mul_planes(csdr_context* ctx, const float* gate, const float* up, size_t n, __nv_bfloat16* hi,
                        __nv_bfloat16* lo);
void op_add(csdr_context* ctx, float* a, const float* b, size_t n);
void op_unshard(csdr_context* ctx, const float* staged, uint32_t P, uint32_t T, uint32_t W, float* out, bool add);
void op_gather_rows(csdr_context* ctx, const float* table, uint32_t n_rows, uint32_t H, const int32_t* ids,
                    uint32_t T, float* out);
void op_argmax(csdr_context* ctx, const float* logits, uint32_t rows, uint32_t V, int32_t* out);
// The reference's token selection (select_best_from_logits, api/cortex_sdk.cpp:1005-1030) per
// row: logit / temperature (<= 0: unscaled), non-finite scores skipped, 1.5 off for tokens whose
// bit is set in the row's bitmap (seen: [rows][seen_words] words), first maximum wins, -1 when
// nothing is selectable; the pick's bit is set.
void op_select(csdr_context* ctx, const float* logits, uint32_t rows, uint32_t V, int32_t* out, float temperature,
               uint32_t* seen, uint32_t seen_words);
void op_mark_seen(csdr_context* ctx, uint32_t* seen_row, const int32_t* tokens_dev, uint32_t n, uint32_t V);
void op_step_positions(csdr_context* ctx, int32_t* pos, uint32_t B, int32_t* seq_of, int32_t* pos_of);

}  // namespace csdr
