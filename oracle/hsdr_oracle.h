/* TEST INFRASTRUCTURE ONLY — a CPU restatement, in plain C, of the reference's
 * HSDR decode / fused-matmul / dequantisation path and of its decoder-layer
 * arithmetic. Only tests, the smoke check and the bench's CPU-baseline leg may
 * call it; the product library never does.
 *
 * Parity status: PINNED. tests/test_oracle_golden.py checks every function here
 * against (a) the known-answer k-quant vectors of the reference's own
 * src/test_hsdr_kquants.cpp, (b) fixtures under tests/golden/ produced by running
 * the unmodified reference (oracle/_ref) on the seeds and shapes of its own tests,
 * and (c), where the reference tree is present, the reference library live.
 * Exception: the decoder-layer functions (decoder_oracle.c) restate code the
 * reference never executes with default settings and no reference test covers:
 * for those parity is UNPINNED beyond primitive-level checks (attention is pinned
 * against the reference's attention kernel).
 *
 * All citations are paths inside the reference tree.
 */
#ifndef HSDR_ORACLE_H
#define HSDR_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Parsed view of an "HSDR" (dictionary embedded) or "HSDC" (codes only) payload.
 * Layouts: strategies/HierarchicalSDRStrategy.cpp:49-66 (HSDR v2, 36 bytes) and
 * :675-692 (HSDC v1, 32 bytes). */
typedef struct {
    int kind;               /* 0 = HSDR, 1 = HSDC */
    uint32_t rows, cols, n_tiles;
    uint16_t tile_rows, tile_cols, n_atoms;
    uint8_t n_stages, k;
    float decay;
    uint32_t edge_bytes;
    size_t off_scales, off_dict, off_codes, off_edges; /* byte offsets; 0 when absent */
} orc_hsdr_view;

/* Return 0 on success, negative on malformed input (truncated, bad magic/version). */
int orc_hsdr_parse(const uint8_t* payload, size_t n, orc_hsdr_view* v);

/* unpackIndexSign, strategies/HierarchicalSDRStrategy.cpp:81-84. */
void orc_unpack_codes(const uint16_t* packed, size_t n, int32_t* idx, int8_t* sign);

/* matmulRowMajor, strategies/HierarchicalSDRStrategy.cpp:1257-1338.
 * x is (C x batch) row-major, y is (R x batch) row-major. -2 for 2-D tiles etc. */
int orc_hsdr_matmul(const uint8_t* payload, size_t n, const float* x, size_t batch, float* y);

/* matmulWithExternalDictionary, :1830-1883 (+ parseCodesStream :1766-1801). */
int orc_hsdc_matmul(const uint8_t* codes, size_t n, const float* atoms, const float* scales,
                    uint16_t d_tile_rows, uint16_t d_tile_cols, uint16_t d_atoms,
                    uint8_t d_stages, uint8_t d_k, const float* x, size_t batch, float* y);

/* decompress, :1340-1440 (decodeAllTiles :612-634, reassembleTiles :119-135, edge
 * strips :1412-1438). out holds rows*cols floats. */
int orc_hsdr_decompress(const uint8_t* payload, size_t n, float* out);

/* The encoder's coding pass: hierarchicalBinaryCode :219-262 over every tile (as encode_all,
 * :552-566), packed with packIndexSign :76-80. tiles holds n_tiles x T floats in extractTiles
 * order (:95-116); packed receives n_tiles*S*k codes, tile-major, then stage, then slot. Per
 * step: project the residual on every atom (atoms already used in this stage count as 0), take
 * the FIRST atom with the largest |projection| (sign + when the projection is >= 0), subtract
 * gamma_l * sign * atom. The dictionary fit around it (:494-607) is not restated. */
void orc_hsdr_code_tiles(const float* tiles, size_t n_tiles, size_t T, const float* D, uint16_t K,
                         uint8_t S, uint8_t k, const float* gammas, uint16_t* packed);

/* The encoder in its fast mode (ksvd_iters = 0): compress :1068-1236 with fitHierarchicalKSVD
 * :494-571 reduced to its first encode. gamma_l = decay^l; atom j = tile number
 * uniform_int_distribution(0, n_tiles-1)(mt19937(0xC0DE)) (libstdc++: Lemire's multiply-shift
 * draw with rejection), normalised to unit length and scaled by mean tile norm / max(1,
 * sqrt(S*k)); codes by the coding pass above; edge strips verbatim. Writes an HSDR v2 payload
 * into out (capacity cap) and returns its size, or a negative number: -1 no full tile,
 * -2 fewer tiles than atoms, -3 capacity, -10 memory. The reference build reorders the float
 * sums of the normalisation (-ffast-math), so atoms agree with its payloads to rounding, not
 * bit for bit. The caller passes the tile shape configFor (:1024-1065) would choose: a row
 * tile (tile_rows == 1) always spans the whole row. */
/* The fit of the encoder on a pool of tiles (n_tiles x T): dictionary D (K x T), stage scales gam
 * (S) and the pool's codes (n_tiles x S x k) out. fitHierarchicalKSVD, :494-607; what
 * fitSharedDictionary (:1446-1469) runs on the pooled tiles of several tensors. */
int orc_hsdr_fit_tiles(const float* tiles, uint32_t n_tiles, size_t T, uint16_t K, uint8_t S, uint8_t k, float decay,
                       uint8_t ksvd_iters, float* D, float* gam, uint16_t* codes);
long orc_hsdr_encode_fast(const float* W, uint32_t R, uint32_t C, uint16_t tile_rows, uint16_t tile_cols,
                          uint16_t K, uint8_t S, uint8_t k, float decay, uint8_t* out, size_t cap);

/* The same with ksvd_iters rounds of (atomUpdateStep :281-489, encode again) between the first
 * encode and the serialisation, and the final sweep that zeroes non-finite atoms (:598-604).
 * Sums that the reference takes across OpenMP threads or reorders under -ffast-math are taken
 * in index order here. */
long orc_hsdr_encode(const float* W, uint32_t R, uint32_t C, uint16_t tile_rows, uint16_t tile_cols,
                     uint16_t K, uint8_t S, uint8_t k, float decay, uint8_t ksvd_iters, uint8_t* out, size_t cap);

/* decompressWithExternalDictionary, :1804-1828. */
int orc_hsdc_decompress(const uint8_t* codes, size_t n, const float* atoms, const float* scales,
                        uint16_t d_tile_rows, uint16_t d_tile_cols, uint16_t d_atoms,
                        uint8_t d_stages, uint8_t d_k, float* out);

/* Same arithmetic as decompress+dense in one pass, for any tile geometry:
 * y (R x batch) = W_reconstructed (R x C) * x (C x batch). Used as the ground truth
 * for 2-D tile matmuls, which the reference only reaches via decompress() +
 * SDRInferenceEngine::matmulForLayer's dense loop (SparseInferenceEngine.cpp:1301-1310). */
int orc_dense_matmul(const float* W, size_t R, size_t C, const float* x, size_t batch, float* y);

/* dequantizeSegmentToFP32, :713-989. fmt is one of
 * "f32","f16","bf16","i8","q4_0","q8_0","q4_k","q5_k","q6_k".
 * Returns number of floats written, negative on size errors. */
long orc_dequantize(const char* fmt, const uint8_t* data, size_t nbytes, float scale,
                    float zero_point, float* out, size_t out_cap);

/* SparseInferenceEngine.cpp:276-469 (decodeSupportedGGUFQuantized): how the INFERENCE side
 * widens a stored-raw tensor in a GGUF block format - ggml's element order, not the encoder's:
 * q4_k 32 low nibbles then 32 high nibbles per 64-element group (:362-383); q6_k four runs of
 * 32 per 128-element half, d * (float)(scale * q) with scales [0],[2],[4],[6] of the half
 * (:329-360); q5_k through the generic bit-field fallback (:437-463: 5-bit fields from byte 16,
 * (q - 16) * d); q4_0 and q8_0 sequential. fmt: "q4_0","q8_0","q4_k","q5_k","q6_k".
 * Returns number of floats written (min(n_elements, what the blocks hold)), negative on errors. */
long orc_dequantize_inference(const char* fmt, const uint8_t* data, size_t nbytes, size_t n_elements,
                              float* out, size_t out_cap);

float orc_fp16_to_fp32(uint16_t h); /* utils/fp16_convert.hpp:26-60 */

/* ---- decoder-layer arithmetic (decoder_oracle.c) ---- */

/* api/cortex_sdk.cpp:1208-1232 */
void orc_rms_norm(const float* in, const float* w, size_t tokens, size_t hidden, float eps,
                  float* out);
/* api/cortex_sdk.cpp:1363-1423; tensor is (seq, heads, head_dim); position of row t is pos0+t */
void orc_rope(float* t, size_t seq, size_t heads, size_t head_dim, float theta, size_t pos0);
/* api/cortex_sdk.cpp:1245-1256 */
void orc_silu_mul(const float* gate, const float* up, size_t n, float* out);
int orc_select_best_from_logits(const float* logits, size_t n, const unsigned char* generated, float temperature);
/* kernels/attention_kernels.cpp:26-113 + kernels/simd_kernels.cpp:198-217, causal, with
 * the kv heads shared by q_heads/kv_heads query heads (cortex_sdk.cpp:1453-1478).
 * q (seq, q_heads, hd); k, v (seq, kv_heads, hd); out (seq, q_heads*hd). */
void orc_attention(const float* q, const float* k, const float* v, size_t seq, size_t q_heads,
                   size_t kv_heads, size_t head_dim, float* out);

typedef struct {
    uint32_t n_layers, hidden, q_heads, kv_heads, head_dim, inter, vocab;
    float eps, theta;
} orc_decoder_cfg;

/* Dense fp32 weights of one block, all (out x in) row-major, as decompress() yields. */
typedef struct {
    const float *attn_norm, *wq, *wk, *wv, *wo, *ffn_norm, *w_gate, *w_up, *w_down;
} orc_block_weights;

/* run_transformer_decode, api/cortex_sdk.cpp:1543-1696, over the whole `tokens`
 * sequence (no KV cache, as the reference). hidden_out receives the final-normed
 * hidden state of EVERY position (seq x hidden); logits_out (may be NULL) the
 * logits of the LAST position: dot of its hidden with each row of lm_head
 * (SparseInferenceEngine.cpp:2310-2320). */
int orc_decoder_forward(const orc_decoder_cfg* cfg, const float* tok_embd,
                        const orc_block_weights* blocks, const float* out_norm,
                        const float* lm_head, const int32_t* tokens, size_t seq,
                        float* hidden_out, float* logits_out);

#ifdef __cplusplus
}
#endif
#endif
