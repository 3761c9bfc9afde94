// HSDR encoder on the device (strategies/HierarchicalSDRStrategy.cpp:494-607 inside compress,
// :1068-1236): the dictionary starts as a scaled sample of the tiles, the tensor is coded against
// it, and every further round (ksvd_iters of them; 0 is the mode the reference calls fast) moves
// the atoms toward the residuals of their users and codes again.
//
//   extractTiles (:95-116)              extract_tiles_kernel: W -> [n_tiles][T]
//   dictionary init (:511-538)          the tile picks come from std::mt19937(0xC0DE) with
//                                       libstdc++'s uniform_int_distribution (host, encoder.cpp);
//                                       init_atoms_kernel normalises the picked tiles and scales
//                                       them by mean tile norm / sqrt(S * k)
//   hierarchicalBinaryCode (:219-262)   the coding pass in its Gram form. The reference subtracts
//                                       gamma_l * sign * atom from a residual and projects the
//                                       residual on all K atoms again, n_tiles * S * k times -
//                                       1.1 TFLOP for an 11008 x 4096 row-tile tensor. Here the
//                                       projections are computed once, P = tiles * D^T, with the
//                                       Gram matrix G = D * D^T beside them (both on the tensor
//                                       cores when the shapes allow it: the TMA-fed tcgen05
//                                       projection with the tiles in the role of the tokens, fp32
//                                       operands as three bf16 products), and a round is
//                                       "first largest |P| among the atoms this stage has not used;
//                                       P -= gamma_l * sign * G[best]" - one warp per tile, P in
//                                       registers. Equal in exact arithmetic; in fp32 the two differ
//                                       in rounding, so a round whose two best candidates tie within
//                                       rounding may pick the other atom.
//   atomUpdateStep (:281-489)           residual_kernel, atom_correct_kernel (one CTA per atom and
//                                       block of 2048 columns walks the code stream in order,
//                                       compacts the atom's users and adds their signed residual
//                                       rows up in double), atom_commit_kernel (the keep / rescale /
//                                       replace decision per atom); the replacement tiles are drawn
//                                       on the host with the reference's per-atom generators.
#include <cuda_runtime.h>

#include <algorithm>

#include "../internal.hpp"
#include "encode.hpp"
#include "gemm_tcgen05.hpp"

namespace csdr {

namespace {

__global__ void __launch_bounds__(256)
extract_tiles_kernel(const float* __restrict__ W, uint32_t C, uint32_t tr, uint32_t tc, uint32_t n_ct, size_t n_elems,
                     float* __restrict__ tiles) {
    const size_t T = static_cast<size_t>(tr) * tc;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n_elems;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const size_t tile = i / T, e = i - tile * T;
        const uint32_t r = static_cast<uint32_t>(e / tc), c = static_cast<uint32_t>(e - static_cast<size_t>(r) * tc);
        const uint32_t br = static_cast<uint32_t>(tile / n_ct), bc = static_cast<uint32_t>(tile - static_cast<size_t>(br) * n_ct);
        tiles[i] = W[(static_cast<size_t>(br) * tr + r) * C + static_cast<size_t>(bc) * tc + c];
    }
}

__device__ __forceinline__ float block_sum(float v, float* red) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, off);
    if ((threadIdx.x & 31u) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = 0.0f;
    for (uint32_t i = 0; i < (blockDim.x >> 5); ++i) t += red[i];
    __syncthreads();
    return t;
}

// One CTA per tile: sum over tiles of the tile's Euclidean norm, in double (:527-533).
__global__ void __launch_bounds__(256)
tile_norm_kernel(const float* __restrict__ tiles, uint32_t n_tiles, uint32_t T, double* __restrict__ norms) {
    __shared__ float red[8];
    for (uint32_t t = blockIdx.x; t < n_tiles; t += gridDim.x) {
        const float* src = tiles + static_cast<size_t>(t) * T;
        float sq = 0.0f;
        for (uint32_t c = threadIdx.x; c < T; c += 256) sq = fmaf(src[c], src[c], sq);
        const float total = block_sum(sq, red);
        if (threadIdx.x == 0) norms[t] = sqrt(static_cast<double>(total));
    }
}

// One CTA per atom: the picked tile, normalised, times the common scale (:515-538).
__global__ void __launch_bounds__(256)
init_atoms_kernel(const float* __restrict__ tiles, const uint32_t* __restrict__ picks, uint32_t T, float init_scale,
                  float* __restrict__ D) {
    __shared__ float red[8];
    const float* src = tiles + static_cast<size_t>(picks[blockIdx.x]) * T;
    float* atom = D + static_cast<size_t>(blockIdx.x) * T;
    float sq = 0.0f;
    for (uint32_t c = threadIdx.x; c < T; c += 256) sq = fmaf(src[c], src[c], sq);
    const float total = block_sum(sq, red);
    const float norm = sqrtf(fmaxf(total, 1e-24f));
    for (uint32_t c = threadIdx.x; c < T; c += 256) atom[c] = (src[c] / norm) * init_scale;
}

// C[m][n] = sum_t A[m][t] * B[n][t] on the CUDA cores, for shapes the tensor-core kernel does not
// take (atoms not a multiple of 128, tile width not a multiple of 8). 64 x 64 tile, 16 x 16 threads.
constexpr int kTile = 64, kStep = 16;
__global__ void __launch_bounds__(256) abt_kernel(const float* __restrict__ A, const float* __restrict__ B,
                                                  float* __restrict__ Cm, uint32_t M, uint32_t N, uint32_t T) {
    __shared__ float As[kStep][kTile + 1];
    __shared__ float Bs[kStep][kTile + 1];
    const uint32_t tx = threadIdx.x & 15u, ty = threadIdx.x >> 4;
    const uint32_t m0 = blockIdx.y * kTile, n0 = blockIdx.x * kTile;
    float acc[4][4] = {};
    for (uint32_t t0 = 0; t0 < T; t0 += kStep) {
        for (uint32_t i = threadIdx.x; i < kTile * kStep; i += 256u) {
            const uint32_t r = i / kStep, c = i % kStep;
            const uint32_t t = t0 + c;
            As[c][r] = (m0 + r < M && t < T) ? A[static_cast<size_t>(m0 + r) * T + t] : 0.f;
            Bs[c][r] = (n0 + r < N && t < T) ? B[static_cast<size_t>(n0 + r) * T + t] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int c = 0; c < kStep; ++c) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                a[i] = As[c][ty * 4 + i];
                b[i] = Bs[c][tx * 4 + i];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
            if (m < M && n < N) Cm[static_cast<size_t>(m) * N + n] = acc[i][j];
        }
}

// The greedy rounds. One warp per tile; lane holds the projections on atoms lane + 32 * i.
// Pt is the projection matrix atom-major: Pt[atom * stride + tile]; G is K x K.
template <int PER_LANE>
__global__ void __launch_bounds__(128)
greedy_kernel(const float* __restrict__ Pt, size_t stride, const float* __restrict__ G, const float* __restrict__ gammas,
              uint16_t* __restrict__ codes, uint32_t n_tiles, uint32_t K, uint32_t S, uint32_t k) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t tile = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (tile >= n_tiles) return;                 // the whole warp leaves together
    float p[PER_LANE];
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
        const uint32_t j = lane + 32u * i;
        p[i] = j < K ? Pt[static_cast<size_t>(j) * stride + tile] : 0.f;
    }
    for (uint32_t l = 0; l < S; ++l) {
        const float gamma = gammas[l];
        uint32_t used = 0;                       // bit i: atom lane + 32 * i taken in this stage
        for (uint32_t s = 0; s < k; ++s) {
            float best_abs = 0.f, best_val = 0.f;
            uint32_t best = 0xFFFFFFFFu;         // none yet: every value was 0 or taken
#pragma unroll
            for (int i = 0; i < PER_LANE; ++i) {
                const uint32_t j = lane + 32u * i;
                const float v = (((used >> i) & 1u) || j >= K) ? 0.f : p[i];
                const float a = fabsf(v);
                if (a > best_abs) {              // strict: inside a lane the lowest atom wins a tie
                    best_abs = a;
                    best = j;
                    best_val = v;
                }
            }
            // across lanes: the larger |v|, the lower atom on a tie (the reference scans atoms upwards)
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) {
                const float oa = __shfl_xor_sync(0xFFFFFFFFu, best_abs, off);
                const uint32_t ob = __shfl_xor_sync(0xFFFFFFFFu, best, off);
                const float ov = __shfl_xor_sync(0xFFFFFFFFu, best_val, off);
                if (oa > best_abs || (oa == best_abs && ob < best)) {
                    best_abs = oa;
                    best = ob;
                    best_val = ov;
                }
            }
            if (best == 0xFFFFFFFFu) {           // all zero: the reference keeps atom 0 with a plus sign
                best = 0;
                best_val = 0.f;
            }
            const bool neg = !(best_val >= 0.f);
            if (lane == 0)
                codes[(static_cast<size_t>(tile) * S + l) * k + s] = static_cast<uint16_t>((best & 0x7FFFu) | (neg ? 0x8000u : 0u));
            if ((best & 31u) == lane) used |= 1u << (best >> 5);
            const float scale = neg ? -gamma : gamma;
            const float* g = G + static_cast<size_t>(best) * K;
#pragma unroll
            for (int i = 0; i < PER_LANE; ++i) {
                const uint32_t j = lane + 32u * i;
                if (j < K) p[i] = fmaf(-scale, __ldg(g + j), p[i]);
            }
        }
    }
}


// ---- dictionary update (atomUpdateStep, :281-489) ----
// residual[i] = tile[i] - sum over its codes of (+-gamma_l) * atom, codes in stream order.
__global__ void __launch_bounds__(256)
residual_kernel(const float* __restrict__ tiles, const float* __restrict__ D, const uint16_t* __restrict__ codes,
                const float* __restrict__ gammas, uint32_t n_tiles, uint32_t T, uint32_t S, uint32_t k,
                float* __restrict__ resid) {
    const uint32_t slots = S * k;
    for (uint32_t i = blockIdx.x; i < n_tiles; i += gridDim.x) {
        const uint16_t* cs = codes + static_cast<size_t>(i) * slots;
        for (uint32_t c = threadIdx.x; c < T; c += 256u) {
            float r = 0.0f;
            for (uint32_t s = 0; s < slots; ++s) {
                const uint32_t code = cs[s];
                const float g = gammas[s / k];
                r = __fadd_rn(r, __fmul_rn((code & 0x8000u) ? -g : g, D[static_cast<size_t>(code & 0x7FFFu) * T + c]));
            }
            resid[static_cast<size_t>(i) * T + c] = tiles[static_cast<size_t>(i) * T + c] - r;
        }
    }
}

constexpr uint32_t kUpdCols = 2048;   // columns of an atom one CTA corrects: eight doubles per thread

struct AtomPartial {
    double new_sq;       // sum of squares of the candidate over this CTA's columns
    double wsum;         // sum of gamma^2 over the atom's users (the same in every column block)
    uint32_t users;
    uint32_t nonfinite;
};

// grid (atom, column block). The CTA walks the whole code stream in order, 256 codes at a time;
// the codes that name its atom are compacted in stream order (tile-major, slot-minor: the order
// of the reference's user list) and their residual rows are added up, signed and scaled, in
// double. The reference packs a user as (tile << 16 | slot) in 32 bits, so a tile number above
// 65535 folds onto its low 16 bits, for the residual row and for the sign alike; kept.
// Then the candidate atom + corr / (2 * wsum), as a float, into cand, with this block's share of
// its squared norm.
__global__ void __launch_bounds__(256)
atom_correct_kernel(const float* __restrict__ resid, const float* __restrict__ D, const uint16_t* __restrict__ codes,
                    const float* __restrict__ gammas, uint32_t n_tiles, uint32_t T, uint32_t S, uint32_t k,
                    float* __restrict__ cand, AtomPartial* __restrict__ partial) {
    constexpr uint32_t PER = kUpdCols / 256u;
    __shared__ uint32_t list_s[256];          // (flat code position) of this chunk's users, in order
    __shared__ uint32_t warp_count[8];
    __shared__ double red_s[8];
    __shared__ uint32_t flag_s;
    const uint32_t j = blockIdx.x, cb = blockIdx.y;
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t slots = S * k;
    const size_t n_codes = static_cast<size_t>(n_tiles) * slots;
    const uint32_t c0 = cb * kUpdCols;
    double corr[PER];
#pragma unroll
    for (uint32_t q = 0; q < PER; ++q) corr[q] = 0.0;
    double wsum = 0.0;
    uint32_t users = 0;
    if (tid == 0) flag_s = 0;
    for (size_t base = 0; base < n_codes; base += 256u) {
        const size_t pos = base + tid;
        const bool hit = pos < n_codes && (codes[pos] & 0x7FFFu) == j;
        const uint32_t ballot = __ballot_sync(0xFFFFFFFFu, hit);
        if (lane == 0) warp_count[warp] = __popc(ballot);
        __syncthreads();
        uint32_t before = 0, total = 0;
#pragma unroll
        for (uint32_t w = 0; w < 8u; ++w) {
            const uint32_t n = warp_count[w];
            before += w < warp ? n : 0u;
            total += n;
        }
        if (hit) list_s[before + __popc(ballot & ((1u << lane) - 1u))] = static_cast<uint32_t>(pos - base);
        __syncthreads();
        for (uint32_t u = 0; u < total; ++u) {
            const size_t p = base + list_s[u];
            const uint32_t i = static_cast<uint32_t>(p / slots), s_ = static_cast<uint32_t>(p - static_cast<size_t>(i) * slots);
            const uint32_t it = i & 0xFFFFu;
            const uint32_t own = codes[static_cast<size_t>(it) * slots + s_];
            const double gamma = static_cast<double>(gammas[s_ / k]);
            const double sg = (own & 0x8000u) ? -gamma : gamma;
            const float* r = resid + static_cast<size_t>(it) * T + c0;
#pragma unroll
            for (uint32_t q = 0; q < PER; ++q) {
                const uint32_t c = tid + q * 256u;
                if (c0 + c < T) corr[q] += sg * static_cast<double>(r[c]);
            }
            wsum += gamma * gamma;
        }
        users += total;
        // list_s is rewritten only behind the next chunk's first barrier
    }
    double sq = 0.0;
    bool bad = false;
    if (users && wsum > 1e-12) {
        const double inv_w = 0.5 / wsum;
#pragma unroll
        for (uint32_t q = 0; q < PER; ++q) {
            const uint32_t c = c0 + tid + q * 256u;
            if (c < T) {
                const double v = static_cast<double>(D[static_cast<size_t>(j) * T + c]) + corr[q] * inv_w;
                const float vf = static_cast<float>(v);
                if (!isfinite(v) || !isfinite(vf)) bad = true;
                cand[static_cast<size_t>(j) * T + c] = vf;
                sq += static_cast<double>(vf) * static_cast<double>(vf);
            }
        }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) sq += __shfl_xor_sync(0xFFFFFFFFu, sq, off);
    if (lane == 0) red_s[warp] = sq;
    if (bad) atomicOr(&flag_s, 1u);
    __syncthreads();
    if (tid == 0) {
        double t = 0.0;
        for (uint32_t w = 0; w < 8u; ++w) t += red_s[w];
        partial[static_cast<size_t>(j) * gridDim.y + cb] = AtomPartial{t, wsum, users, flag_s};
    }
}

// One CTA per atom: the decision of :404-487 from the column blocks' partials. No user: the atom
// becomes a random tile scaled to the target norm; weights that vanish: it stays; a non-finite
// candidate: random tile again (another salt); else the candidate, pulled back to the target norm
// when it has grown past 1.5 times it.
__global__ void __launch_bounds__(256)
atom_commit_kernel(const float* __restrict__ tiles, const float* __restrict__ cand, const AtomPartial* __restrict__ partial,
                   uint32_t n_blocks, const uint32_t* __restrict__ pick_unused, const uint32_t* __restrict__ pick_nonfinite,
                   uint32_t T, double target, float* __restrict__ D) {
    __shared__ double red_s[8];
    const uint32_t j = blockIdx.x, tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    double new_sq = 0.0;
    uint32_t nonfinite = 0;
    for (uint32_t b = 0; b < n_blocks; ++b) {
        const AtomPartial& p = partial[static_cast<size_t>(j) * n_blocks + b];
        new_sq += p.new_sq;
        nonfinite |= p.nonfinite;
    }
    const AtomPartial& p0 = partial[static_cast<size_t>(j) * n_blocks];
    float* atom = D + static_cast<size_t>(j) * T;
    const float* src = nullptr;
    if (p0.users == 0u) {
        src = tiles + static_cast<size_t>(pick_unused[j]) * T;
    } else if (p0.wsum <= 1e-12) {
        return;
    } else if (nonfinite || !isfinite(new_sq)) {
        src = tiles + static_cast<size_t>(pick_nonfinite[j]) * T;
    }
    if (!src) {
        const double nn = sqrt(new_sq);
        const bool shrink = nn > 1.5 * target;
        const double sc = shrink ? target / nn : 1.0;
        for (uint32_t c = tid; c < T; c += 256u) {
            const float v = cand[static_cast<size_t>(j) * T + c];
            atom[c] = shrink ? static_cast<float>(static_cast<double>(v) * sc) : v;
        }
        return;
    }
    double sq = 0.0;
    for (uint32_t c = tid; c < T; c += 256u) sq += static_cast<double>(src[c]) * static_cast<double>(src[c]);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) sq += __shfl_xor_sync(0xFFFFFFFFu, sq, off);
    if (lane == 0) red_s[warp] = sq;
    __syncthreads();
    double total = 0.0;
    for (uint32_t w = 0; w < 8u; ++w) total += red_s[w];
    const double sc = target / sqrt(total > 1e-30 ? total : 1e-30);
    for (uint32_t c = tid; c < T; c += 256u) atom[c] = static_cast<float>(static_cast<double>(src[c]) * sc);
}

// The sweep behind the last round (:598-604): values that are not finite become 0.
__global__ void __launch_bounds__(256) finite_sweep_kernel(float* __restrict__ D, size_t n) {
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n; i += static_cast<size_t>(gridDim.x) * blockDim.x)
        if (!isfinite(D[i])) D[i] = 0.0f;
}

}  // namespace

void launch_extract_tiles(csdr_context* ctx, const float* W, uint32_t C, uint32_t tr, uint32_t tc, uint32_t n_rt,
                          uint32_t n_ct, float* tiles) {
    const size_t n = static_cast<size_t>(n_rt) * n_ct * tr * tc;
    if (!n) return;
    LaunchScope ls(ctx, KC_ENCODE);
    extract_tiles_kernel<<<static_cast<unsigned>(std::min<size_t>((n + 255) / 256, static_cast<size_t>(ctx->sm_count) * 16)), 256, 0,
                           ctx->stream>>>(W, C, tr, tc, n_ct, n, tiles);
    ls.done("extract_tiles_kernel");
}

void launch_tile_norms(csdr_context* ctx, const float* tiles, uint32_t n_tiles, uint32_t T, double* norms) {
    LaunchScope ls(ctx, KC_ENCODE);
    tile_norm_kernel<<<std::min<uint32_t>(n_tiles, static_cast<uint32_t>(ctx->sm_count) * 8u), 256, 0, ctx->stream>>>(tiles, n_tiles, T,
                                                                                                                    norms);
    ls.done("tile_norm_kernel");
}

void launch_init_atoms(csdr_context* ctx, const float* tiles, const uint32_t* picks_dev, uint32_t K, uint32_t T, float init_scale,
                       float* D) {
    LaunchScope ls(ctx, KC_ENCODE);
    init_atoms_kernel<<<K, 256, 0, ctx->stream>>>(tiles, picks_dev, T, init_scale, D);
    ls.done("init_atoms_kernel");
}

void launch_code_tiles(csdr_context* ctx, const float* tiles, uint32_t n_tiles, uint32_t T, const DevPtr& D, uint32_t K,
                       uint32_t S, uint32_t k, const float* gammas_dev, uint16_t* codes_dev) {
    if (K == 0 || K > 1024u) throw Error(CSDR_ERR_LIMIT, "encoder: dictionaries of 1 to 1024 atoms");
    // projections atom-major, Pt[K][n_tiles], then the Gram matrix G[K][K]
    const size_t pt_floats = static_cast<size_t>(K) * n_tiles, g_floats = static_cast<size_t>(K) * K;
    // buffers of their own: the projection kernel below uses (and may regrow) the context's scratch
    DeviceBuffer work((pt_floats + g_floats) * sizeof(float), ctx->device);
    float* Pt = static_cast<float*>(work.ptr);
    float* G = Pt + pt_floats;
    // the dictionary in the role of a row-tile segment's atoms, the tiles in the role of the tokens
    csdr_segment dict{};
    dict.ctx = ctx;
    dict.g.rows = dict.g.rows_full = dict.g.n_tiles = 1;
    dict.g.cols = dict.g.cols_full = dict.g.tile_cols = T;
    dict.g.tile_rows = dict.g.n_col_tiles = 1;
    dict.g.n_atoms = K;
    dict.g.n_stages = dict.g.k = 1;
    dict.atoms = D;
    if (ctx->tensor_cores && dx_tma_supported(ctx, &dict, n_tiles) && n_tiles >= 16u) {
        MatmulArgs a;
        a.x = tiles;
        a.x_dtype = CSDR_DTYPE_F32;
        a.x_layout = CSDR_LAYOUT_TOKEN_MAJOR;
        a.batch = n_tiles;
        launch_dx_tma(ctx, &dict, a, Pt, n_tiles);
        a.x = D->ptr;
        a.batch = K;
        launch_dx_tma(ctx, &dict, a, G, K);
        // the planes cached on the dictionary buffer belong to these values only
        CSDR_CUDA(cudaStreamSynchronize(ctx->stream));
        D->aux.reset();
    } else {
        LaunchScope ls(ctx, KC_ENCODE);
        abt_kernel<<<dim3((n_tiles + kTile - 1) / kTile, (K + kTile - 1) / kTile), 256, 0, ctx->stream>>>(
            static_cast<const float*>(D->ptr), tiles, Pt, K, n_tiles, T);
        abt_kernel<<<dim3((K + kTile - 1) / kTile, (K + kTile - 1) / kTile), 256, 0, ctx->stream>>>(
            static_cast<const float*>(D->ptr), static_cast<const float*>(D->ptr), G, K, K, T);
        ls.done("abt_kernel");
    }
    LaunchScope ls(ctx, KC_ENCODE);
    const dim3 grid((n_tiles + 3u) / 4u);
    if (K <= 128) greedy_kernel<4><<<grid, 128, 0, ctx->stream>>>(Pt, n_tiles, G, gammas_dev, codes_dev, n_tiles, K, S, k);
    else if (K <= 256) greedy_kernel<8><<<grid, 128, 0, ctx->stream>>>(Pt, n_tiles, G, gammas_dev, codes_dev, n_tiles, K, S, k);
    else if (K <= 512) greedy_kernel<16><<<grid, 128, 0, ctx->stream>>>(Pt, n_tiles, G, gammas_dev, codes_dev, n_tiles, K, S, k);
    else greedy_kernel<32><<<grid, 128, 0, ctx->stream>>>(Pt, n_tiles, G, gammas_dev, codes_dev, n_tiles, K, S, k);
    ls.done("greedy_kernel");
    CSDR_CUDA(cudaStreamSynchronize(ctx->stream));   // `work` goes away with this scope
}

}  // namespace csdr

namespace csdr {

void launch_atom_update(csdr_context* ctx, const float* tiles, uint32_t n_tiles, uint32_t T, float* D, uint32_t K,
                        uint32_t S, uint32_t k, const float* gammas_dev, const uint16_t* codes_dev, double target,
                        const uint32_t* pick_unused_dev, const uint32_t* pick_nonfinite_dev) {
    const uint32_t n_blocks = (T + kUpdCols - 1u) / kUpdCols;
    DeviceBuffer resid(static_cast<size_t>(n_tiles) * T * sizeof(float), ctx->device);
    DeviceBuffer cand(static_cast<size_t>(K) * T * sizeof(float), ctx->device);
    DeviceBuffer partial(static_cast<size_t>(K) * n_blocks * sizeof(AtomPartial), ctx->device);
    LaunchScope ls(ctx, KC_ENCODE);
    residual_kernel<<<std::min<uint32_t>(n_tiles, static_cast<uint32_t>(ctx->sm_count) * 8u), 256, 0, ctx->stream>>>(
        tiles, D, codes_dev, gammas_dev, n_tiles, T, S, k, static_cast<float*>(resid.ptr));
    atom_correct_kernel<<<dim3(K, n_blocks), 256, 0, ctx->stream>>>(static_cast<const float*>(resid.ptr), D, codes_dev, gammas_dev,
                                                                    n_tiles, T, S, k, static_cast<float*>(cand.ptr),
                                                                    static_cast<AtomPartial*>(partial.ptr));
    atom_commit_kernel<<<K, 256, 0, ctx->stream>>>(tiles, static_cast<const float*>(cand.ptr),
                                                   static_cast<const AtomPartial*>(partial.ptr), n_blocks, pick_unused_dev,
                                                   pick_nonfinite_dev, T, target, D);
    ls.done("atom update kernels");
    CSDR_CUDA(cudaStreamSynchronize(ctx->stream));   // the work buffers go away with this scope
}

void launch_finite_sweep(csdr_context* ctx, float* D, size_t n) {
    if (!n) return;
    LaunchScope ls(ctx, KC_ENCODE);
    finite_sweep_kernel<<<static_cast<unsigned>(std::min<size_t>((n + 255) / 256, static_cast<size_t>(ctx->sm_count) * 16)), 256, 0,
                          ctx->stream>>>(D, n);
    ls.done("finite_sweep_kernel");
}

}  // namespace csdr
