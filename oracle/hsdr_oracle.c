/* TEST INFRASTRUCTURE ONLY — see hsdr_oracle.h. Plain-C restatement of the
 * reference's HSDR decode side. Each function names the reference lines it follows
 * (paths inside the reference tree). Loop order and fp32 accumulation order follow
 * the reference so that differences stay at rounding level. */
#include "hsdr_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

#define HSDR_HDR 36u
#define HSDC_HDR 32u

static uint32_t rd32(const uint8_t* p) { uint32_t v; memcpy(&v, p, 4); return v; }
static uint16_t rd16(const uint8_t* p) { uint16_t v; memcpy(&v, p, 2); return v; }
static float rdf(const uint8_t* p) { float v; memcpy(&v, p, 4); return v; }

/* HSDRHeader / HSDRCodesHeader: strategies/HierarchicalSDRStrategy.cpp:49-66, :675-692;
 * stream order after the header: scales, dictionary, codes, edges (:1222-1235). */
int orc_hsdr_parse(const uint8_t* p, size_t n, orc_hsdr_view* v) {
    memset(v, 0, sizeof(*v));
    if (n < HSDC_HDR) return -1;
    if (memcmp(p, "HSDR", 4) == 0) v->kind = 0;
    else if (memcmp(p, "HSDC", 4) == 0) v->kind = 1;
    else return -2;
    const uint32_t ver = rd32(p + 4);
    if (v->kind == 0 && (n < HSDR_HDR || ver != 2)) return -3;
    if (v->kind == 1 && ver != 1) return -3;
    v->rows = rd32(p + 8);
    v->cols = rd32(p + 12);
    v->n_tiles = rd32(p + 16);
    v->tile_rows = rd16(p + 20);
    v->tile_cols = rd16(p + 22);
    v->n_atoms = rd16(p + 24);
    v->n_stages = p[26];
    v->k = p[27];
    v->decay = rdf(p + 28);
    const size_t tile_dim = (size_t)v->tile_rows * v->tile_cols;
    const size_t n_codes = (size_t)v->n_tiles * v->n_stages * v->k;
    if (v->kind == 0) {
        v->edge_bytes = rd32(p + 32);
        v->off_scales = HSDR_HDR;
        v->off_dict = v->off_scales + 4u * v->n_stages;
        v->off_codes = v->off_dict + 4u * (size_t)v->n_atoms * tile_dim;
        v->off_edges = v->off_codes + 2u * n_codes;
        if (v->off_edges + v->edge_bytes > n) return -4;
    } else {
        v->off_codes = HSDC_HDR;
        if (v->off_codes + 2u * n_codes > n) return -4;
    }
    return 0;
}

/* unpackIndexSign: :81-84 */
void orc_unpack_codes(const uint16_t* packed, size_t n, int32_t* idx, int8_t* sign) {
    for (size_t i = 0; i < n; ++i) {
        idx[i] = (int32_t)(packed[i] & 0x7FFFu);
        sign[i] = (packed[i] & 0x8000u) ? -1 : 1;
    }
}

/* hierarchicalBinaryCode :219-262 per tile + packIndexSign :76-80; see the header. */
void orc_hsdr_code_tiles(const float* tiles, size_t n_tiles, size_t T, const float* D, uint16_t K,
                         uint8_t S, uint8_t k, const float* gammas, uint16_t* packed) {
    float* r = (float*)malloc(T * sizeof(float));
    float* proj = (float*)malloc((size_t)K * sizeof(float));
    uint8_t* used = (uint8_t*)malloc(K);
    if (!r || !proj || !used) {
        free(r); free(proj); free(used);
        return;
    }
    for (size_t t = 0; t < n_tiles; ++t) {
        memcpy(r, tiles + t * T, T * sizeof(float));
        for (uint8_t l = 0; l < S; ++l) {
            memset(used, 0, K);
            for (uint8_t step = 0; step < k; ++step) {
                for (uint16_t j = 0; j < K; ++j) {
                    const float* atom = D + (size_t)j * T;
                    float s = 0.0f;
                    for (size_t c = 0; c < T; ++c) s += atom[c] * r[c];
                    proj[j] = used[j] ? 0.0f : s;
                }
                uint16_t best = 0;
                float best_abs = 0.0f;
                for (uint16_t j = 0; j < K; ++j) {
                    const float a = fabsf(proj[j]);
                    if (a > best_abs) { best_abs = a; best = j; }
                }
                const int neg = !(proj[best] >= 0.0f);
                packed[(t * S + l) * k + step] = (uint16_t)((best & 0x7FFFu) | (neg ? 0x8000u : 0u));
                used[best] = 1;
                const float scale = neg ? -gammas[l] : gammas[l];
                const float* atom = D + (size_t)best * T;
                for (size_t c = 0; c < T; ++c) r[c] -= scale * atom[c];
            }
        }
    }
    free(r); free(proj); free(used);
}

/* MT19937 (Matsumoto & Nishimura 1998) as std::mt19937 seeds and tempers it. */
typedef struct { uint32_t mt[624]; int i; } orc_mt;
static void mt_seed(orc_mt* g, uint32_t seed) {
    g->mt[0] = seed;
    for (int i = 1; i < 624; ++i) g->mt[i] = 1812433253u * (g->mt[i - 1] ^ (g->mt[i - 1] >> 30)) + (uint32_t)i;
    g->i = 624;
}
static uint32_t mt_next(orc_mt* g) {
    if (g->i >= 624) {
        for (int i = 0; i < 624; ++i) {
            const uint32_t y = (g->mt[i] & 0x80000000u) | (g->mt[(i + 1) % 624] & 0x7FFFFFFFu);
            g->mt[i] = g->mt[(i + 397) % 624] ^ (y >> 1) ^ ((y & 1u) ? 0x9908B0DFu : 0u);
        }
        g->i = 0;
    }
    uint32_t y = g->mt[g->i++];
    y ^= y >> 11;
    y ^= (y << 7) & 0x9D2C5680u;
    y ^= (y << 15) & 0xEFC60000u;
    y ^= y >> 18;
    return y;
}
/* uniform draw from [0, range) out of a 32-bit generator: Lemire's multiply-shift with
 * rejection of the biased low products, the method libstdc++ (GCC 11 and later) uses. */
static uint32_t mt_below(orc_mt* g, uint32_t range) {
    uint64_t prod = (uint64_t)mt_next(g) * range;
    uint32_t low = (uint32_t)prod;
    if (low < range) {
        const uint32_t threshold = (uint32_t)(0u - range) % range;
        while (low < threshold) {
            prod = (uint64_t)mt_next(g) * range;
            low = (uint32_t)prod;
        }
    }
    return (uint32_t)(prod >> 32);
}

static void wr32(uint8_t* p, uint32_t v) { memcpy(p, &v, 4); }
static void wr16(uint8_t* p, uint16_t v) { memcpy(p, &v, 2); }

/* atomUpdateStep :281-489: every atom moves half a least-squares step toward the residuals of
 * the tiles that use it (all atoms from the same residual, doubles for the sums), is rescaled
 * to the target norm when it grows past 1.5 times it, and is replaced by a random tile when
 * nothing uses it. One generator draw per call seeds the replacements. The user list packs
 * (tile << 16 | slot), so the reference folds tile numbers above 65535; kept. */
static int atom_update(const float* tiles, uint32_t n_tiles, size_t T, float* D, uint16_t K,
                       const uint16_t* packed, uint8_t S, uint8_t k, const float* gam, orc_mt* g) {
    const uint32_t slots = (uint32_t)S * k;
    float* resid = (float*)malloc((size_t)n_tiles * T * sizeof(float));
    double* corr = (double*)malloc(T * sizeof(double));
    if (!resid || !corr) { free(resid); free(corr); return -10; }
    double norm_sum = 0.0;
    for (uint32_t i = 0; i < n_tiles; ++i) {
        float* r = resid + (size_t)i * T;
        for (size_t c = 0; c < T; ++c) r[c] = 0.0f;                 /* reconstruction first ... */
        for (uint32_t s_ = 0; s_ < slots; ++s_) {
            const uint16_t code = packed[(size_t)i * slots + s_];
            const float scale = (code & 0x8000u) ? -gam[s_ / k] : gam[s_ / k];
            const float* atom = D + (size_t)(code & 0x7FFFu) * T;
            for (size_t c = 0; c < T; ++c) r[c] += scale * atom[c];
        }
        double sq = 0.0;
        for (size_t c = 0; c < T; ++c) {
            const float t = tiles[(size_t)i * T + c];
            r[c] = t - r[c];                                          /* ... then the residual */
            sq += (double)t * t;
        }
        norm_sum += sqrt(sq);
    }
    const double mean = norm_sum / (double)(n_tiles ? n_tiles : 1u);
    double target = mean / sqrt((double)slots);
    if (target < 1e-6) target = 1e-6;
    const double cap = 1.5 * target;
    const uint64_t base_seed = (uint64_t)mt_next(g) ^ 0xA0B1C2D3u;
    for (uint32_t j = 0; j < K; ++j) {
        float* atom = D + (size_t)j * T;
        for (size_t c = 0; c < T; ++c) corr[c] = 0.0;
        double wsum = 0.0;
        int users = 0;
        for (uint32_t i = 0; i < n_tiles; ++i)
            for (uint32_t s_ = 0; s_ < slots; ++s_) {
                const uint16_t code = packed[(size_t)i * slots + s_];
                if ((uint32_t)(code & 0x7FFFu) != j) continue;
                ++users;
                const uint32_t it = (uint32_t)(i << 16) >> 16;       /* the packed user entry */
                const uint16_t own = packed[(size_t)it * slots + s_];
                const double gamma = (double)gam[s_ / k];
                const double sg = ((own & 0x8000u) ? -1.0 : 1.0) * gamma;
                const float* r = resid + (size_t)it * T;
                for (size_t c = 0; c < T; ++c) corr[c] += sg * (double)r[c];
                wsum += gamma * gamma;
            }
        int reseed = 0;
        uint32_t salt = 0x9E3779B1u;
        if (!users) reseed = 1;
        else if (wsum <= 1e-12) continue;
        else {
            const double inv_w = 0.5 / wsum;
            double new_sq = 0.0;
            for (size_t c = 0; c < T; ++c) {
                const double v = (double)atom[c] + corr[c] * inv_w;
                const float vf = (float)v;
                if (!isfinite(v) || !isfinite(vf)) { reseed = 1; break; }
                atom[c] = vf;
                new_sq += (double)vf * (double)vf;
            }
            if (!reseed && !isfinite(new_sq)) reseed = 1;
            if (reseed) salt = 0xB7E15163u;
            else {
                const double nn = sqrt(new_sq);
                if (nn > cap) {
                    const double sc = target / nn;
                    for (size_t c = 0; c < T; ++c) atom[c] = (float)((double)atom[c] * sc);
                }
            }
        }
        if (reseed) {
            orc_mt local;
            mt_seed(&local, (uint32_t)(base_seed ^ (uint64_t)(uint32_t)(j * salt)));
            const float* src = tiles + (size_t)mt_below(&local, n_tiles) * T;
            double sq = 0.0;
            for (size_t c = 0; c < T; ++c) sq += (double)src[c] * src[c];
            const double sc = target / sqrt(sq > 1e-30 ? sq : 1e-30);
            for (size_t c = 0; c < T; ++c) atom[c] = (float)(src[c] * sc);
        }
    }
    free(resid); free(corr);
    return 0;
}

long orc_hsdr_encode_fast(const float* W, uint32_t R, uint32_t C, uint16_t tile_rows, uint16_t tile_cols,
                          uint16_t K, uint8_t S, uint8_t k, float decay, uint8_t* out, size_t cap) {
    return orc_hsdr_encode(W, R, C, tile_rows, tile_cols, K, S, k, decay, 0, out, cap);
}

/* fitHierarchicalKSVD :494-607 on a pool of tiles (one tensor's, or several tensors' pooled by
 * fitSharedDictionary :1446-1469): stage scales :507-509, dictionary init :511-538 (tiles picked
 * by mt19937(0xC0DE), normalised, scaled by the mean tile norm over sqrt(S * k)), a coding pass
 * :552-567, ksvd_iters rounds of atom update + coding pass :573-577, the non-finite sweep
 * :598-604. D (K x T), gam (S) and codes (n_tiles x S x k, the last pass's) are outputs. */
int orc_hsdr_fit_tiles(const float* tiles, uint32_t n_tiles, size_t T, uint16_t K, uint8_t S, uint8_t k, float decay,
                       uint8_t ksvd_iters, float* D, float* gam, uint16_t* codes) {
    if (n_tiles < K) return -2;
    for (uint8_t l = 0; l < S; ++l) gam[l] = powf(decay, (float)l);          /* :507-509 */
    orc_mt g;
    mt_seed(&g, 0xC0DEu);
    for (uint16_t j = 0; j < K; ++j) {
        const float* src = tiles + (size_t)mt_below(&g, n_tiles) * T;
        float* atom = D + (size_t)j * T;
        float sq = 0.0f;
        for (size_t c = 0; c < T; ++c) sq += src[c] * src[c];
        const float norm = sqrtf(sq > 1e-24f ? sq : 1e-24f);
        for (size_t c = 0; c < T; ++c) atom[c] = src[c] / norm;
    }
    double norm_sum = 0.0;
    for (uint32_t i = 0; i < n_tiles; ++i) {
        double sq = 0.0;
        for (size_t c = 0; c < T; ++c) sq += (double)tiles[i * T + c] * tiles[i * T + c];
        norm_sum += sqrt(sq);
    }
    const float mean = (float)(norm_sum / (double)(n_tiles ? n_tiles : 1u));
    const float root = sqrtf((float)((uint32_t)S * k));
    const float init_scale = mean / (root > 1.0f ? root : 1.0f);
    for (size_t i = 0; i < (size_t)K * T; ++i) D[i] *= init_scale;
    orc_hsdr_code_tiles(tiles, n_tiles, T, D, K, S, k, gam, codes);          /* encode_all :552-567 */
    for (uint8_t it = 0; it < ksvd_iters; ++it) {                          /* :573-577 */
        if (atom_update(tiles, n_tiles, T, D, K, codes, S, k, gam, &g)) return -10;
        orc_hsdr_code_tiles(tiles, n_tiles, T, D, K, S, k, gam, codes);
    }
    for (size_t i = 0; i < (size_t)K * T; ++i)                              /* :598-604 */
        if (!isfinite(D[i])) D[i] = 0.0f;
    return 0;
}

/* compress :1068-1236 around fitHierarchicalKSVD :494-607; see the header. */
long orc_hsdr_encode(const float* W, uint32_t R, uint32_t C, uint16_t tile_rows, uint16_t tile_cols,
                     uint16_t K, uint8_t S, uint8_t k, float decay, uint8_t ksvd_iters, uint8_t* out, size_t cap) {
    const uint32_t R_full = (R / tile_rows) * tile_rows, C_full = (C / tile_cols) * tile_cols;
    if (!R_full || !C_full) return -1;
    const uint32_t n_rt = R_full / tile_rows, n_ct = C_full / tile_cols, n_tiles = n_rt * n_ct;
    const size_t T = (size_t)tile_rows * tile_cols;
    if (n_tiles < K) return -2;
    const size_t n_codes = (size_t)n_tiles * S * k;
    const size_t edge_floats = (size_t)R_full * (C - C_full) + (size_t)(R - R_full) * C;
    const size_t total = HSDR_HDR + 4u * S + 4u * (size_t)K * T + 2u * n_codes + 4u * edge_floats;
    if (total > cap) return -3;
    float* tiles = (float*)malloc((size_t)n_tiles * T * sizeof(float));
    if (!tiles) return -10;
    /* extractTiles :95-116 over the aligned top-left block */
    for (uint32_t br = 0; br < n_rt; ++br)
        for (uint32_t bc = 0; bc < n_ct; ++bc)
            for (uint32_t r = 0; r < tile_rows; ++r)
                memcpy(tiles + ((size_t)br * n_ct + bc) * T + (size_t)r * tile_cols,
                       W + (size_t)(br * tile_rows + r) * C + (size_t)bc * tile_cols, sizeof(float) * tile_cols);
    memset(out, 0, HSDR_HDR);
    memcpy(out, "HSDR", 4);
    wr32(out + 4, 2u); wr32(out + 8, R); wr32(out + 12, C); wr32(out + 16, n_tiles);
    wr16(out + 20, tile_rows); wr16(out + 22, tile_cols); wr16(out + 24, K);
    out[26] = S; out[27] = k;
    memcpy(out + 28, &decay, 4);
    wr32(out + 32, (uint32_t)(4u * edge_floats));
    float* gam = (float*)(out + HSDR_HDR);            /* 36 and 36+4S are multiples of 4 */
    float* D = (float*)(out + HSDR_HDR + 4u * S);
    /* the code stream may sit on an odd 16-bit boundary only if 4S+4KT is odd, which it never is */
    uint16_t* codes = (uint16_t*)(out + HSDR_HDR + 4u * S + 4u * (size_t)K * T);
    if (orc_hsdr_fit_tiles(tiles, n_tiles, T, K, S, k, decay, ksvd_iters, D, gam, codes)) { free(tiles); return -10; }
    free(tiles);
    /* edge strips :1185-1197: top-right, then bottom */
    uint8_t* e = out + total - 4u * edge_floats;
    for (uint32_t r = 0; r < R_full; ++r, e += 4u * (C - C_full))
        memcpy(e, W + (size_t)r * C + C_full, 4u * (size_t)(C - C_full));
    for (uint32_t r = R_full; r < R; ++r, e += 4u * (size_t)C)
        memcpy(e, W + (size_t)r * C, 4u * (size_t)C);
    return (long)total;
}

/* Shared body of matmulRowMajor (:1301-1337) and matmulWithExternalDictionary
 * (:1853-1882): Dx = D*x, then per-row signed gather scaled per stage. */
static int fused_matmul(const float* D, const float* scales, const uint8_t* codes_bytes,
                        uint32_t R, uint32_t C, uint16_t K, uint8_t S, uint8_t k,
                        const float* x, size_t batch, float* y) {
    float* Dx = (float*)calloc((size_t)K * batch, sizeof(float));
    if (!Dx) return -10;
    for (uint32_t a = 0; a < K; ++a) {
        const float* atom = D + (size_t)a * C;
        float* out_row = Dx + (size_t)a * batch;
        for (uint32_t c = 0; c < C; ++c) {
            const float av = atom[c];
            const float* xrow = x + (size_t)c * batch;
            for (size_t b = 0; b < batch; ++b) out_row[b] += av * xrow[b];
        }
    }
    const uint32_t slots = (uint32_t)S * k;
    memset(y, 0, (size_t)R * batch * sizeof(float));
    for (uint32_t r = 0; r < R; ++r) {
        float* y_row = y + (size_t)r * batch;
        for (uint8_t l = 0; l < S; ++l) {
            const float gamma = scales[l];
            for (uint8_t kk = 0; kk < k; ++kk) {
                const uint16_t pk = rd16(codes_bytes + 2u * ((size_t)r * slots + (size_t)l * k + kk));
                const uint16_t a = pk & 0x7FFFu;
                const float scale = gamma * ((pk & 0x8000u) ? -1.0f : 1.0f);
                if (a >= K) { free(Dx); return -11; }
                const float* dx_row = Dx + (size_t)a * batch;
                for (size_t b = 0; b < batch; ++b) y_row[b] += scale * dx_row[b];
            }
        }
    }
    free(Dx);
    return 0;
}

/* matmulRowMajor: :1257-1338 (geometry checks :1273-1289). */
int orc_hsdr_matmul(const uint8_t* p, size_t n, const float* x, size_t batch, float* y) {
    orc_hsdr_view v;
    int rc = orc_hsdr_parse(p, n, &v);
    if (rc) return rc;
    if (v.kind != 0) return -2;
    if (v.tile_rows != 1) return -20;           /* "fused matmul requires tile_rows == 1" */
    if (v.tile_cols != v.cols) return -21;      /* "must have tile_cols == original_cols" */
    if (v.n_tiles != v.rows) return -22;        /* "tile count must equal row count" */
    const size_t dict_bytes = 4u * (size_t)v.n_atoms * v.cols;
    float* D = (float*)malloc(dict_bytes);
    float scales[256];
    if (!D) return -10;
    memcpy(D, p + v.off_dict, dict_bytes);
    memcpy(scales, p + v.off_scales, 4u * v.n_stages);
    rc = fused_matmul(D, scales, p + v.off_codes, v.rows, v.cols, v.n_atoms, v.n_stages, v.k,
                      x, batch, y);
    free(D);
    return rc;
}

static int check_dict_geometry(const orc_hsdr_view* v, uint16_t tr, uint16_t tc, uint16_t K,
                               uint8_t S, uint8_t k) {
    /* parseCodesStream: :1781-1787 */
    return (v->tile_rows == tr && v->tile_cols == tc && v->n_atoms == K && v->n_stages == S &&
            v->k == k) ? 0 : -30;
}

/* matmulWithExternalDictionary: :1830-1883 */
int orc_hsdc_matmul(const uint8_t* p, size_t n, const float* atoms, const float* scales,
                    uint16_t tr, uint16_t tc, uint16_t K, uint8_t S, uint8_t k,
                    const float* x, size_t batch, float* y) {
    orc_hsdr_view v;
    int rc = orc_hsdr_parse(p, n, &v);
    if (rc) return rc;
    if (v.kind != 1) return -2;
    if ((rc = check_dict_geometry(&v, tr, tc, K, S, k))) return rc;
    if (v.tile_rows != 1) return -20;
    if (v.tile_cols != v.cols) return -21;
    if (v.n_tiles != v.rows) return -22;
    return fused_matmul(atoms, scales, p + v.off_codes, v.rows, v.cols, K, S, k, x, batch, y);
}

/* decodeAllTiles (:612-634) followed by reassembleTiles (:119-135) into a matrix with
 * leading dimension ld (= C for the aligned fast path and for the edge-splice path,
 * whose intermediate aligned block is copied row by row into the same place, :1416-1424). */
static int decode_tiles_into(const float* D, const float* scales, const uint8_t* codes_bytes,
                             uint32_t n_tiles, uint16_t tr, uint16_t tc, uint16_t K, uint8_t S,
                             uint8_t k, uint32_t n_col_tiles, float* out, size_t ld) {
    const size_t T = (size_t)tr * tc;
    const uint32_t slots = (uint32_t)S * k;
    float* t = (float*)malloc(T * sizeof(float));
    if (!t) return -10;
    for (uint32_t i = 0; i < n_tiles; ++i) {
        for (size_t c = 0; c < T; ++c) t[c] = 0.0f;
        for (uint8_t l = 0; l < S; ++l) {
            const float gamma = scales[l];
            for (uint8_t kk = 0; kk < k; ++kk) {
                const uint16_t pk = rd16(codes_bytes + 2u * ((size_t)i * slots + (size_t)l * k + kk));
                const uint16_t a = pk & 0x7FFFu;
                if (a >= K) { free(t); return -11; }
                const float scale = gamma * ((pk & 0x8000u) ? -1.0f : 1.0f);
                const float* atom = D + (size_t)a * T;
                for (size_t c = 0; c < T; ++c) t[c] += scale * atom[c];
            }
        }
        const uint32_t br = i / n_col_tiles, bc = i % n_col_tiles;
        for (uint16_t r = 0; r < tr; ++r)
            memcpy(out + ((size_t)br * tr + r) * ld + (size_t)bc * tc, t + (size_t)r * tc,
                   sizeof(float) * tc);
    }
    free(t);
    return 0;
}

/* decompress: :1340-1440 */
int orc_hsdr_decompress(const uint8_t* p, size_t n, float* out) {
    orc_hsdr_view v;
    int rc = orc_hsdr_parse(p, n, &v);
    if (rc) return rc;
    if (v.kind != 0) return -2;
    if (v.tile_rows == 0 || v.tile_cols == 0) return -5;
    const uint32_t R = v.rows, C = v.cols;
    const uint32_t R_full = (R / v.tile_rows) * v.tile_rows;
    const uint32_t C_full = (C / v.tile_cols) * v.tile_cols;
    const uint32_t n_col_tiles = C_full / v.tile_cols;
    if (n_col_tiles == 0 || v.n_tiles != (R_full / v.tile_rows) * n_col_tiles) return -6;
    const size_t T = (size_t)v.tile_rows * v.tile_cols;
    float* D = (float*)malloc(4u * (size_t)v.n_atoms * T);
    float scales[256];
    if (!D) return -10;
    memcpy(D, p + v.off_dict, 4u * (size_t)v.n_atoms * T);
    memcpy(scales, p + v.off_scales, 4u * v.n_stages);
    rc = decode_tiles_into(D, scales, p + v.off_codes, v.n_tiles, v.tile_rows, v.tile_cols,
                           v.n_atoms, v.n_stages, v.k, n_col_tiles, out, C);
    free(D);
    if (rc) return rc;
    /* edge strips, :1425-1437: top-right rows[0,R_full) x cols[C_full,C), then bottom rows */
    const size_t need = 4u * ((size_t)R_full * (C - C_full) + (size_t)(R - R_full) * C);
    if (need != v.edge_bytes) return -7;
    const uint8_t* e = p + v.off_edges;
    for (uint32_t r = 0; r < R_full; ++r)
        for (uint32_t c = C_full; c < C; ++c) { out[(size_t)r * C + c] = rdf(e); e += 4; }
    for (uint32_t r = R_full; r < R; ++r)
        for (uint32_t c = 0; c < C; ++c) { out[(size_t)r * C + c] = rdf(e); e += 4; }
    return 0;
}

/* decompressWithExternalDictionary: :1804-1828 */
int orc_hsdc_decompress(const uint8_t* p, size_t n, const float* atoms, const float* scales,
                        uint16_t tr, uint16_t tc, uint16_t K, uint8_t S, uint8_t k, float* out) {
    orc_hsdr_view v;
    int rc = orc_hsdr_parse(p, n, &v);
    if (rc) return rc;
    if (v.kind != 1) return -2;
    if ((rc = check_dict_geometry(&v, tr, tc, K, S, k))) return rc;
    if (v.rows % tr || v.cols % tc) return -6;
    const uint32_t n_col_tiles = v.cols / tc;
    if (v.n_tiles != (v.rows / tr) * n_col_tiles) return -6;
    return decode_tiles_into(atoms, scales, p + v.off_codes, v.n_tiles, tr, tc, K, S, k,
                             n_col_tiles, out, v.cols);
}

/* SDRInferenceEngine::matmulForLayer dense fallback, SparseInferenceEngine.cpp:1301-1310 */
int orc_dense_matmul(const float* W, size_t R, size_t C, const float* x, size_t batch, float* y) {
    memset(y, 0, R * batch * sizeof(float));
    #pragma omp parallel for schedule(static)
    for (long r = 0; r < (long)R; ++r)
        for (size_t c = 0; c < C; ++c) {
            const float w = W[(size_t)r * C + c];
            for (size_t b = 0; b < batch; ++b) y[(size_t)r * batch + b] += w * x[c * batch + b];
        }
    return 0;
}

/* fp16_to_fp32, utils/fp16_convert.hpp:26-60 (bit-manipulation branch) */
float orc_fp16_to_fp32(uint16_t h) {
    const uint32_t sign = (h >> 15) & 1u;
    uint32_t exponent = (h >> 10) & 0x1Fu;
    uint32_t mantissa = h & 0x3FFu;
    uint32_t f;
    if (exponent == 0) {
        if (mantissa == 0) {
            f = sign << 31;
        } else {
            int e = 1;
            while ((mantissa & 0x400u) == 0) { mantissa <<= 1; --e; }
            mantissa &= 0x3FFu;
            f = (sign << 31) | ((uint32_t)(e + (127 - 15)) << 23) | (mantissa << 13);
        }
    } else if (exponent == 0x1F) {
        f = (sign << 31) | 0x7F800000u | (mantissa << 13);
    } else {
        f = (sign << 31) | ((exponent + (127 - 15)) << 23) | (mantissa << 13);
    }
    float out;
    memcpy(&out, &f, 4);
    return out;
}

/* 6-bit scale/min unpack shared by Q4_K and Q5_K: :802-814 */
static void unpack_k_scales_mins(const uint8_t* s12, uint8_t* sc, uint8_t* mn) {
    for (int is = 0; is < 4; ++is) {
        sc[is] = s12[is] & 0x3F;
        mn[is] = s12[is + 4] & 0x3F;
    }
    for (int is = 4; is < 8; ++is) {
        sc[is] = (uint8_t)((s12[is + 4] & 0x0F) | ((s12[is - 4] >> 6) << 4));
        mn[is] = (uint8_t)((s12[is + 4] >> 4) | ((s12[is] >> 6) << 4));
    }
}

/* dequantizeSegmentToFP32: :713-989 */
long orc_dequantize(const char* fmt, const uint8_t* p, size_t nbytes, float scale,
                    float zero_point, float* out, size_t cap) {
    if (!strcmp(fmt, "f32")) {                                   /* :943-952 */
        if (nbytes % 4) return -1;
        if (nbytes / 4 > cap) return -2;
        memcpy(out, p, nbytes);
        return (long)(nbytes / 4);
    }
    if (!strcmp(fmt, "bf16")) {                                  /* :725-737 */
        if (nbytes % 2) return -1;
        const size_t n = nbytes / 2;
        if (n > cap) return -2;
        for (size_t i = 0; i < n; ++i) {
            const uint32_t bits = (uint32_t)rd16(p + 2 * i) << 16;
            memcpy(&out[i], &bits, 4);
        }
        return (long)n;
    }
    if (!strcmp(fmt, "f16")) {                                   /* :955-965 */
        if (nbytes % 2) return -1;
        const size_t n = nbytes / 2;
        if (n > cap) return -2;
        for (size_t i = 0; i < n; ++i) out[i] = orc_fp16_to_fp32(rd16(p + 2 * i));
        return (long)n;
    }
    if (!strcmp(fmt, "i8")) {                                    /* :968-982 */
        if (nbytes > cap) return -2;
        for (size_t i = 0; i < nbytes; ++i) out[i] = ((float)(int8_t)p[i] - zero_point) * scale;
        return (long)nbytes;
    }
    if (!strcmp(fmt, "q4_0")) {                                  /* :742-767 */
        if (nbytes % 18) return -1;
        const size_t nb = nbytes / 18;
        if (nb * 32 > cap) return -2;
        for (size_t b = 0; b < nb; ++b, p += 18) {
            const float d = orc_fp16_to_fp32(rd16(p));
            for (size_t j = 0; j < 16; ++j) {
                const uint8_t byte = p[2 + j];
                out[b * 32 + 2 * j] = (float)((int)(byte & 0x0F) - 8) * d;
                out[b * 32 + 2 * j + 1] = (float)((int)(byte >> 4) - 8) * d;
            }
        }
        return (long)(nb * 32);
    }
    if (!strcmp(fmt, "q8_0")) {                                  /* :769-790 */
        if (nbytes % 34) return -1;
        const size_t nb = nbytes / 34;
        if (nb * 32 > cap) return -2;
        for (size_t b = 0; b < nb; ++b, p += 34) {
            const float d = orc_fp16_to_fp32(rd16(p));
            for (size_t j = 0; j < 32; ++j) out[b * 32 + j] = (float)(int8_t)p[2 + j] * d;
        }
        return (long)(nb * 32);
    }
    if (!strcmp(fmt, "q4_k") || !strcmp(fmt, "q5_k")) {          /* :816-849, :851-887 */
        const int q5 = fmt[1] == '5';
        const size_t bb = q5 ? 176 : 144;
        if (nbytes % bb) return -1;
        const size_t nb = nbytes / bb;
        if (nb * 256 > cap) return -2;
        uint8_t sc[8], mn[8];
        for (size_t b = 0; b < nb; ++b, p += bb) {
            const float d = orc_fp16_to_fp32(rd16(p));
            const float dmin = orc_fp16_to_fp32(rd16(p + 2));
            const uint8_t* qh = p + 16;
            const uint8_t* qs = q5 ? qh + 32 : p + 16;
            unpack_k_scales_mins(p + 4, sc, mn);
            for (int is = 0; is < 8; ++is) {
                const float ds = d * (float)sc[is];
                const float dm = dmin * (float)mn[is];
                for (int j = 0; j < 32; ++j) {
                    const int idx = is * 32 + j;
                    const uint8_t byte = qs[idx / 2];
                    uint8_t q = (idx & 1) ? (uint8_t)(byte >> 4) : (uint8_t)(byte & 0x0F);
                    if (q5) q |= (uint8_t)(((qh[idx / 8] >> (idx % 8)) & 1) << 4);
                    out[b * 256 + idx] = (float)q * ds - dm;
                }
            }
        }
        return (long)(nb * 256);
    }
    if (!strcmp(fmt, "q6_k")) {                                  /* :889-940 */
        if (nbytes % 210) return -1;
        const size_t nb = nbytes / 210;
        if (nb * 256 > cap) return -2;
        for (size_t b = 0; b < nb; ++b, p += 210) {
            const uint8_t* ql = p;
            const uint8_t* qh = p + 128;
            const int8_t* scales = (const int8_t*)(p + 192);
            const float d = orc_fp16_to_fp32(rd16(p + 208));
            for (int half = 0; half < 2; ++half) {
                const uint8_t* ql_h = ql + half * 64;
                const uint8_t* qh_h = qh + half * 32;
                for (int sub = 0; sub < 8; ++sub) {
                    const float ds = d * (float)scales[half * 8 + sub];
                    for (int j = 0; j < 16; ++j) {
                        const int e = sub * 16 + j;
                        const uint8_t lb = ql_h[e / 2];
                        const uint8_t lo = (e & 1) ? (uint8_t)(lb >> 4) : (uint8_t)(lb & 0x0F);
                        const uint8_t hi = (uint8_t)((qh_h[e / 4] >> ((e % 4) * 2)) & 3);
                        const int q = (int)((hi << 4) | lo) - 32;
                        out[b * 256 + half * 128 + e] = (float)q * ds;
                    }
                }
            }
        }
        return (long)(nb * 256);
    }
    return -3;
}

/* ---- SparseInferenceEngine.cpp:252-469: stored-raw GGUF block formats as the inference side
 * decodes them ---- */
static void gguf_scale_min_q4k(const uint8_t* scales, size_t j, uint8_t* sc, uint8_t* mn) {   /* :262-273 */
    if (j < 4) {
        *sc = (uint8_t)(scales[j] & 0x3F);
        *mn = (uint8_t)(scales[j + 4] & 0x3F);
    } else {
        *sc = (uint8_t)((scales[j + 4] & 0x0F) | ((scales[j - 4] >> 6) << 4));
        *mn = (uint8_t)((scales[j + 4] >> 4) | ((scales[j] >> 6) << 4));
    }
}

static uint32_t read_bits_lsb(const uint8_t* bytes, size_t bit_offset, size_t bit_count) {     /* :250-260 */
    uint32_t v = 0;
    for (size_t b = 0; b < bit_count; ++b) {
        const size_t a = bit_offset + b;
        v |= (uint32_t)((bytes[a / 8] >> (a % 8)) & 1u) << b;
    }
    return v;
}

long orc_dequantize_inference(const char* fmt, const uint8_t* data, size_t nbytes, size_t n_elements,
                              float* out, size_t cap) {
    size_t bb = 0, be = 0;
    if (!strcmp(fmt, "q4_0")) { bb = 18; be = 32; }
    else if (!strcmp(fmt, "q8_0")) { bb = 34; be = 32; }
    else if (!strcmp(fmt, "q4_k")) { bb = 144; be = 256; }
    else if (!strcmp(fmt, "q5_k")) { bb = 176; be = 256; }
    else if (!strcmp(fmt, "q6_k")) { bb = 210; be = 256; }
    else return -3;
    if (nbytes < bb) return -1;                                   /* :289-291 */
    const size_t blocks = nbytes / bb;
    size_t count = blocks * be;
    if (n_elements < count) count = n_elements;                   /* :305 */
    if (count > cap) return -2;
    size_t o = 0;
    for (size_t bi = 0; bi < blocks && o < count; ++bi) {
        const uint8_t* blk = data + bi * bb;
        if (bb == 34) {                                           /* q8_0 :311-318 */
            const float d = orc_fp16_to_fp32(rd16(blk));
            for (size_t i = 0; i < 32 && o < count; ++i) out[o++] = (float)(int8_t)blk[2 + i] * d;
        } else if (bb == 210) {                                   /* q6_k :329-360 */
            const uint8_t* ql = blk;
            const uint8_t* qh = blk + 128;
            const int8_t* scales = (const int8_t*)(blk + 192);
            const float d = orc_fp16_to_fp32(rd16(blk + 208));
            for (size_t half = 0; half < 2 && o < count; ++half) {
                const uint8_t* qlh = ql + half * 64;
                const uint8_t* qhh = qh + half * 32;
                const int8_t* sch = scales + half * 8;
                for (size_t l = 0; l < 32 && o < count; ++l) {
                    const int q = (int)((qlh[l] & 0x0F) | (((qhh[l] >> 0) & 3) << 4)) - 32;
                    out[o++] = d * (float)(sch[0] * q);
                }
                for (size_t l = 0; l < 32 && o < count; ++l) {
                    const int q = (int)((qlh[l + 32] & 0x0F) | (((qhh[l] >> 2) & 3) << 4)) - 32;
                    out[o++] = d * (float)(sch[2] * q);
                }
                for (size_t l = 0; l < 32 && o < count; ++l) {
                    const int q = (int)(((qlh[l] >> 4) & 0x0F) | (((qhh[l] >> 4) & 3) << 4)) - 32;
                    out[o++] = d * (float)(sch[4] * q);
                }
                for (size_t l = 0; l < 32 && o < count; ++l) {
                    const int q = (int)(((qlh[l + 32] >> 4) & 0x0F) | (((qhh[l] >> 6) & 3) << 4)) - 32;
                    out[o++] = d * (float)(sch[6] * q);
                }
            }
        } else if (bb == 144) {                                   /* q4_k :362-383 */
            const float d = orc_fp16_to_fp32(rd16(blk));
            const float dmin = orc_fp16_to_fp32(rd16(blk + 2));
            const uint8_t* scales = blk + 4;
            const uint8_t* qs = blk + 16;
            for (size_t g = 0; g < 4 && o < count; ++g) {
                uint8_t s0, m0, s1, m1;
                gguf_scale_min_q4k(scales, g * 2, &s0, &m0);
                gguf_scale_min_q4k(scales, g * 2 + 1, &s1, &m1);
                const float d0 = d * (float)s0, mm0 = dmin * (float)m0;
                const float d1 = d * (float)s1, mm1 = dmin * (float)m1;
                const uint8_t* qg = qs + g * 32;
                for (size_t i = 0; i < 32 && o < count; ++i) out[o++] = d0 * (float)(qg[i] & 0x0F) - mm0;
                for (size_t i = 0; i < 32 && o < count; ++i) out[o++] = d1 * (float)(qg[i] >> 4) - mm1;
            }
        } else if (bb == 18) {                                    /* q4_0 :397-405 */
            const float d = orc_fp16_to_fp32(rd16(blk));
            for (size_t i = 0; i < 32 && o < count; ++i) {
                const uint8_t nib = (i & 1) == 0 ? (blk[2 + i / 2] & 0x0F) : (blk[2 + i / 2] >> 4);
                out[o++] = ((float)nib - 8.0f) * d;
            }
        } else {                                                  /* q5_k: generic fallback :437-463 */
            const size_t bits = 5, packed_bytes = (be * bits + 7) / 8;
            const uint8_t* packed = blk + (bb - packed_bytes);
            float d = orc_fp16_to_fp32(rd16(blk));
            if (!isfinite(d) || fabsf(d) < 1e-12f) d = 1.0f;
            for (size_t i = 0; i < be && o < count; ++i) {
                const int32_t q = (int32_t)read_bits_lsb(packed, i * bits, bits) - 16;
                out[o++] = (float)q * d;
            }
        }
    }
    return (long)o;
}
