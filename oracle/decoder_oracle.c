/* TEST INFRASTRUCTURE ONLY — see hsdr_oracle.h. Restates the decoder-layer
 * arithmetic of the reference's run_transformer_decode (api/cortex_sdk.cpp:1543-1696)
 * primitive by primitive. The reference reaches this code only when a flag that is
 * never set is false, and none of its tests covers it: parity for this file is
 * UNPINNED, except orc_attention, which is checked against the reference's own attention
 * kernel (kernels/attention_kernels.cpp, compiled into oracle/_ref): the other primitives sit
 * in an anonymous namespace of a file that does not link without the ONNX parser.
 * Two parameters the reference hard-codes or guesses are explicit here: eps (its
 * default is 1e-5, cortex_sdk.cpp:1212) and head_dim (it guesses from
 * {128,64,256,32,16}, cortex_sdk.cpp:1335). */
#include "hsdr_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

/* rms_norm: api/cortex_sdk.cpp:1208-1232 */
void orc_rms_norm(const float* in, const float* w, size_t tokens, size_t hidden, float eps,
                  float* out) {
    for (size_t t = 0; t < tokens; ++t) {
        const float* src = in + t * hidden;
        float* dst = out + t * hidden;
        float ms = 0.0f;
        for (size_t i = 0; i < hidden; ++i) ms += src[i] * src[i];
        ms /= (float)hidden;
        const float inv = 1.0f / sqrtf(ms + eps);
        for (size_t i = 0; i < hidden; ++i) dst[i] = src[i] * inv * w[i];
    }
}

/* get_rope_cache + apply_rope_inplace: api/cortex_sdk.cpp:1363-1423. Adjacent pairs
 * (2i, 2i+1); freq = theta^(-i/head_dim) with i the even index; odd head_dim leaves
 * the last element untouched (rotary_dim = head_dim - head_dim % 2). */
void orc_rope(float* t, size_t seq, size_t heads, size_t head_dim, float theta, size_t pos0) {
    const size_t rotary = head_dim - (head_dim % 2);
    for (size_t p = 0; p < seq; ++p) {
        for (size_t h = 0; h < heads; ++h) {
            float* base = t + (p * heads + h) * head_dim;
            for (size_t i = 0; i < rotary; i += 2) {
                const float exponent = (float)i / (float)head_dim;
                const float freq = powf(theta, -exponent);
                const float angle = (float)(pos0 + p) * freq;
                const float c = cosf(angle), s = sinf(angle);
                const float x0 = base[i], x1 = base[i + 1];
                base[i] = x0 * c - x1 * s;
                base[i + 1] = x0 * s + x1 * c;
            }
        }
    }
}

/* silu_mul: api/cortex_sdk.cpp:1245-1256 */
void orc_silu_mul(const float* gate, const float* up, size_t n, float* out) {
    for (size_t i = 0; i < n; ++i) {
        const float x = gate[i];
        const float sig = 1.0f / (1.0f + expf(-x));
        out[i] = (x * sig) * up[i];
    }
}

/* multi_head_attention(causal) per head: kernels/attention_kernels.cpp:26-113;
 * scores = q.k * (1/sqrt(hd)), upper triangle -inf, softmax with max subtraction
 * (kernels/simd_kernels.cpp:198-217), out = P.V. Query head h reads kv head
 * h / (q_heads/kv_heads): repeat_kv_heads, api/cortex_sdk.cpp:1453-1478. */
void orc_attention(const float* q, const float* k, const float* v, size_t seq, size_t q_heads,
                   size_t kv_heads, size_t hd, float* out) {
    const size_t rep = q_heads / kv_heads;
    const float scale = 1.0f / sqrtf((float)hd);
    #pragma omp parallel
    {
        float* sc = (float*)malloc(seq * sizeof(float));
        #pragma omp for collapse(2) schedule(dynamic, 8)
        for (long h = 0; h < (long)q_heads; ++h) {
            for (long i = 0; i < (long)seq; ++i) {
                const size_t kvh = (size_t)h / rep;
                const float* qi = q + ((size_t)i * q_heads + h) * hd;
                float mx = -INFINITY;
                for (long j = 0; j <= i; ++j) {
                    const float* kj = k + ((size_t)j * kv_heads + kvh) * hd;
                    float s = 0.0f;
                    for (size_t d = 0; d < hd; ++d) s += qi[d] * kj[d];
                    s *= scale;
                    sc[j] = s;
                    if (s > mx) mx = s;
                }
                float sum = 0.0f;
                for (long j = 0; j <= i; ++j) { sc[j] = expf(sc[j] - mx); sum += sc[j]; }
                const float inv = 1.0f / sum;
                float* o = out + ((size_t)i * q_heads + h) * hd;
                for (size_t d = 0; d < hd; ++d) o[d] = 0.0f;
                for (long j = 0; j <= i; ++j) {
                    const float pj = sc[j] * inv;
                    const float* vj = v + ((size_t)j * kv_heads + kvh) * hd;
                    for (size_t d = 0; d < hd; ++d) o[d] += pj * vj[d];
                }
            }
        }
        free(sc);
    }
}

/* Kernels::linear_forward semantics (kernels/blas_kernels.cpp:264-293): token-major
 * input (tokens x in), weights (out x in), output (tokens x out). */
static void linear(const float* in, const float* W, size_t tokens, size_t n_in, size_t n_out,
                   float* out) {
    #pragma omp parallel for collapse(2) schedule(static)
    for (long t = 0; t < (long)tokens; ++t)
        for (long o = 0; o < (long)n_out; ++o) {
            const float* w = W + (size_t)o * n_in;
            const float* x = in + (size_t)t * n_in;
            float s = 0.0f;
            for (size_t i = 0; i < n_in; ++i) s += x[i] * w[i];
            out[(size_t)t * n_out + o] = s;
        }
}

/* run_transformer_decode: api/cortex_sdk.cpp:1543-1696; block order :1569-1679;
 * final norm :1681-1687; logits SparseInferenceEngine.cpp:2310-2320. */
int orc_decoder_forward(const orc_decoder_cfg* c, const float* tok_embd,
                        const orc_block_weights* blocks, const float* out_norm,
                        const float* lm_head, const int32_t* tokens, size_t seq,
                        float* hidden_out, float* logits_out) {
    const size_t H = c->hidden, QD = (size_t)c->q_heads * c->head_dim,
                 KD = (size_t)c->kv_heads * c->head_dim, I = c->inter;
    float* hidden = (float*)malloc(seq * H * sizeof(float));
    float* normed = (float*)malloc(seq * H * sizeof(float));
    float* q = (float*)malloc(seq * QD * sizeof(float));
    float* k = (float*)malloc(seq * KD * sizeof(float));
    float* v = (float*)malloc(seq * KD * sizeof(float));
    float* att = (float*)malloc(seq * QD * sizeof(float));
    float* proj = (float*)malloc(seq * H * sizeof(float));
    float* gate = (float*)malloc(seq * I * sizeof(float));
    float* up = (float*)malloc(seq * I * sizeof(float));
    if (!hidden || !normed || !q || !k || !v || !att || !proj || !gate || !up) return -10;
    for (size_t t = 0; t < seq; ++t) {
        if (tokens[t] < 0 || (uint32_t)tokens[t] >= c->vocab) return -11;
        memcpy(hidden + t * H, tok_embd + (size_t)tokens[t] * H, H * sizeof(float));
    }
    for (uint32_t b = 0; b < c->n_layers; ++b) {
        const orc_block_weights* w = &blocks[b];
        orc_rms_norm(hidden, w->attn_norm, seq, H, c->eps, normed);
        linear(normed, w->wq, seq, H, QD, q);
        linear(normed, w->wk, seq, H, KD, k);
        linear(normed, w->wv, seq, H, KD, v);
        orc_rope(q, seq, c->q_heads, c->head_dim, c->theta, 0);
        orc_rope(k, seq, c->kv_heads, c->head_dim, c->theta, 0);
        orc_attention(q, k, v, seq, c->q_heads, c->kv_heads, c->head_dim, att);
        linear(att, w->wo, seq, QD, H, proj);
        for (size_t i = 0; i < seq * H; ++i) hidden[i] = hidden[i] + proj[i];
        orc_rms_norm(hidden, w->ffn_norm, seq, H, c->eps, normed);
        linear(normed, w->w_gate, seq, H, I, gate);
        linear(normed, w->w_up, seq, H, I, up);
        orc_silu_mul(gate, up, seq * I, gate);
        linear(gate, w->w_down, seq, I, H, proj);
        for (size_t i = 0; i < seq * H; ++i) hidden[i] = hidden[i] + proj[i];
    }
    if (out_norm) orc_rms_norm(hidden, out_norm, seq, H, c->eps, hidden_out);
    else memcpy(hidden_out, hidden, seq * H * sizeof(float));
    if (logits_out && lm_head) linear(hidden_out + (seq - 1) * H, lm_head, 1, H, c->vocab, logits_out);
    free(hidden); free(normed); free(q); free(k); free(v); free(att); free(proj); free(gate); free(up);
    return 0;
}

/* select_best_from_logits, api/cortex_sdk.cpp:1005-1030 (token_is_repeated :946-948): score =
 * logit * (temperature > 0 ? 1/temperature : 1); non-finite scores are skipped; 1.5 is taken off
 * tokens already generated (generated[t] != 0); the first strictly greater score wins; -1 when no
 * score is finite or the row is empty. */
int orc_select_best_from_logits(const float* logits, size_t n, const unsigned char* generated, float temperature) {
    const float temp_scale = temperature > 0.0f ? (1.0f / temperature) : 1.0f;
    float best_score = -INFINITY;
    int best_token = -1;
    for (size_t t = 0; t < n; ++t) {
        float score = logits[t] * temp_scale;
        if (!isfinite(score)) continue;
        if (generated && generated[t]) score -= 1.5f;
        if (score > best_score) {
            best_score = score;
            best_token = (int)t;
        }
    }
    return best_token;
}
