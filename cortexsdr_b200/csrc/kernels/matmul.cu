// Fused HSDR matmul kernels for sm_100a: sparse-code unpack, the 1-D row-tile
// decode path (dictionary projection Dx = D*x, then a signed gather over Dx), the
// factored path for 2-D tiles, raw edge strips, and a dense fallback.
//
// What each kernel stands in for, in the reference tree (src/ai_compression/):
//   hsdr_unpack_kernel      unpackIndexSign, strategies/HierarchicalSDRStrategy.cpp:81-84
//   hsdr_dx_kernel          the Dx loop of matmulRowMajor, :1304-1315 (and :1854-1863)
//   hsdr_gather_kernel      the gather loop of matmulRowMajor, :1318-1336 (and :1866-1881)
//   hsdr_tile_project/_tile_gather/_edge kernels
//                           decompress (:1340-1440) followed by the dense product of
//                           SDRInferenceEngine::matmulForLayer (SparseInferenceEngine.cpp:1301-1310),
//                           computed in factored form so the weight never exists in memory
//   dense_rows_kernel       the same dense product for stored-raw fp32 segments
#include <cooperative_groups.h>
#include <cuda_bf16.h>

#include <algorithm>

#include "../internal.hpp"
#include "gemm_tcgen05.hpp"
#include "gemv_fused.hpp"
#include "gemv_queue.hpp"
#include "views.cuh"

namespace cg = cooperative_groups;

namespace csdr {

namespace {

// ---------------------------------------------------------------------------
// helpers
// ---------------------------------------------------------------------------

// ---------------------------------------------------------------------------
// K1: unpack. 8 codes per 128-bit load; indices leave as two 128-bit stores, signs
// as one 64-bit store.
// ---------------------------------------------------------------------------
__global__ void hsdr_unpack_kernel(const uint16_t* __restrict__ codes, size_t n,
                                   int32_t* __restrict__ idx, int8_t* __restrict__ sign) {
    const size_t n8 = n / 8;
    const size_t t = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (size_t i = t; i < n8; i += stride) {
        const uint4 v = reinterpret_cast<const uint4*>(codes)[i];
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
        int32_t id[8];
        uint32_t sg[2] = {0u, 0u};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t lo = w[j] & 0xFFFFu, hi = w[j] >> 16;
            id[2 * j] = static_cast<int32_t>(lo & 0x7FFFu);
            id[2 * j + 1] = static_cast<int32_t>(hi & 0x7FFFu);
            const uint32_t s0 = (lo & 0x8000u) ? 0xFFu : 0x01u;
            const uint32_t s1 = (hi & 0x8000u) ? 0xFFu : 0x01u;
            const int e = 2 * j;
            sg[e / 4] |= s0 << (8 * (e % 4));
            sg[(e + 1) / 4] |= s1 << (8 * ((e + 1) % 4));
        }
        reinterpret_cast<int4*>(idx)[2 * i] = make_int4(id[0], id[1], id[2], id[3]);
        reinterpret_cast<int4*>(idx)[2 * i + 1] = make_int4(id[4], id[5], id[6], id[7]);
        reinterpret_cast<uint2*>(sign)[i] = make_uint2(sg[0], sg[1]);
    }
    for (size_t i = n8 * 8 + t; i < n; i += stride) {
        const uint16_t c = codes[i];
        idx[i] = static_cast<int32_t>(c & 0x7FFFu);
        sign[i] = (c & 0x8000u) ? -1 : 1;
    }
}

// ---------------------------------------------------------------------------
// K2: Dx[a][b] = sum_c D[a][c] * x[c][b] for 1-D row tiles.
//
// Grid (nsplit, ceil(K / (8*A))), cluster (nsplit,1,1). A CTA owns 8*A atoms and one
// column slab; its x slab sits in shared memory token-major; each warp streams A
// dictionary rows with 128-bit loads, U*A of them in flight per lane, and keeps
// A*MT accumulators in registers. The column-split partials meet in distributed
// shared memory and are summed by the cluster's first CTA in a fixed order, so the
// result does not depend on scheduling.
// ---------------------------------------------------------------------------
template <int MT, int A, int U>
__global__ void __launch_bounds__(256)
hsdr_dx_kernel(const float* __restrict__ D, uint32_t K, uint32_t C, uint32_t slab, XView xv,
               float* __restrict__ dx, int nsplit) {
    extern __shared__ __align__(16) float smem[];
    float* xs = smem;                      // [MT][slab]
    float* part = smem + MT * slab;        // [8*A][MT]
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t c0 = blockIdx.x * slab;
    const uint32_t cw = c0 < C ? min(slab, C - c0) : 0u;

    for (uint32_t i = tid; i < MT * slab; i += 256) {
        const uint32_t b = i / slab, c = i - b * slab;
        xs[i] = (b < xv.M && c < cw) ? load_x(xv, c0 + c, b) : 0.0f;
    }
    __syncthreads();

    const uint32_t atom0 = (blockIdx.y * 8u + warp) * A;
    const uint32_t slab4 = slab >> 2, cw4 = cw >> 2;
    const float4* xs4 = reinterpret_cast<const float4*>(xs);
    const float4* drow[A];
    bool valid[A];
#pragma unroll
    for (int a = 0; a < A; ++a) {
        valid[a] = atom0 + a < K;
        drow[a] = reinterpret_cast<const float4*>(
            D + static_cast<size_t>(valid[a] ? atom0 + a : 0u) * C + c0);
    }
    float acc[A][MT];
#pragma unroll
    for (int a = 0; a < A; ++a)
#pragma unroll
        for (int b = 0; b < MT; ++b) acc[a][b] = 0.0f;

    for (uint32_t base = 0; base < cw4; base += 32u * U) {
        float4 d[U][A];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const uint32_t c4 = base + u * 32u + lane;
#pragma unroll
            for (int a = 0; a < A; ++a)
                d[u][a] = (c4 < cw4 && valid[a]) ? ldg_stream_f4(drow[a] + c4)
                                                 : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const uint32_t c4 = base + u * 32u + lane;
            if (c4 < cw4) {
#pragma unroll
                for (int b = 0; b < MT; ++b) {
                    const float4 x4 = xs4[b * slab4 + c4];
#pragma unroll
                    for (int a = 0; a < A; ++a) {
                        acc[a][b] = fmaf(d[u][a].x, x4.x, acc[a][b]);
                        acc[a][b] = fmaf(d[u][a].y, x4.y, acc[a][b]);
                        acc[a][b] = fmaf(d[u][a].z, x4.z, acc[a][b]);
                        acc[a][b] = fmaf(d[u][a].w, x4.w, acc[a][b]);
                    }
                }
            }
        }
    }
#pragma unroll
    for (int a = 0; a < A; ++a)
#pragma unroll
        for (int b = 0; b < MT; ++b) {
            float v = acc[a][b];
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, off);
            if (lane == 0) part[(warp * A + a) * MT + b] = v;
        }
    __syncthreads();

    const uint32_t n_out = 8u * A * MT;
    if (nsplit == 1) {
        for (uint32_t t = tid; t < n_out; t += 256) {
            const uint32_t atom = blockIdx.y * 8u * A + t / MT;
            if (atom < K) dx[static_cast<size_t>(atom) * MT + t % MT] = part[t];
        }
    } else {
        cg::cluster_group cluster = cg::this_cluster();
        cluster.sync();
        if (cluster.block_rank() == 0) {
            for (uint32_t t = tid; t < n_out; t += 256) {
                float s = 0.0f;
                for (int r = 0; r < nsplit; ++r) s += cluster.map_shared_rank(part, r)[t];
                const uint32_t atom = blockIdx.y * 8u * A + t / MT;
                if (atom < K) dx[static_cast<size_t>(atom) * MT + t % MT] = s;
            }
        }
        cluster.sync();  // peers' shared memory must outlive the reads above
    }
}

// ---------------------------------------------------------------------------
// K3: y[r][b] = sum_l gamma_l * sum_k sign * Dx[idx][b], in the reference's order
// (stage-major, slot-minor), one multiply and one add per code as its source has it.
// The CTA's slice of the code stream enters shared memory through 128-bit loads.
// ---------------------------------------------------------------------------
constexpr int kGatherThreads = 128;

template <int MT>
__global__ void __launch_bounds__(kGatherThreads)
hsdr_gather_kernel(const uint16_t* __restrict__ codes, uint32_t R, uint32_t S, uint32_t k,
                   const float* __restrict__ scales, const float* __restrict__ dx, uint32_t K,
                   uint32_t rows_per_cta, int dx_in_smem, YView yv, int* status) {
    extern __shared__ __align__(16) unsigned char gsm[];
    const uint32_t slots = S * k;
    const uint32_t tid = threadIdx.x;
    const uint32_t row0 = blockIdx.x * rows_per_cta;
    if (row0 >= R) return;
    const uint32_t rows_here = min(rows_per_cta, R - row0);

    // layout: codes (16-byte units) | scales | Dx
    const size_t code_byte0 = static_cast<size_t>(row0) * slots * 2u;
    const size_t aligned0 = code_byte0 & ~static_cast<size_t>(15);
    const uint32_t skip = static_cast<uint32_t>(code_byte0 - aligned0) >> 1;
    const uint32_t n_codes = rows_here * slots;
    const uint32_t n16 = (skip * 2u + n_codes * 2u + 15u) >> 4;
    const uint32_t cap16 = (rows_per_cta * slots * 2u + 15u + 16u) >> 4;
    uint4* cs16 = reinterpret_cast<uint4*>(gsm);
    float* sc = reinterpret_cast<float*>(gsm + static_cast<size_t>(cap16) * 16u);
    float* dxs = sc + ((S + 3u) & ~3u);

    const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const unsigned char*>(codes) + aligned0);
    for (uint32_t i = tid; i < n16; i += kGatherThreads) cs16[i] = src[i];
    for (uint32_t i = tid; i < S; i += kGatherThreads) sc[i] = scales[i];
    if (dx_in_smem) {
        const uint32_t n4 = (K * MT) >> 2;
        const float4* g4 = reinterpret_cast<const float4*>(dx);
        for (uint32_t i = tid; i < n4; i += kGatherThreads) reinterpret_cast<float4*>(dxs)[i] = g4[i];
        for (uint32_t i = (n4 << 2) + tid; i < K * MT; i += kGatherThreads) dxs[i] = dx[i];
    }
    __syncthreads();
    const uint16_t* cs = reinterpret_cast<const uint16_t*>(cs16) + skip;
    const float* dxp = dx_in_smem ? dxs : dx;

    const uint32_t b = tid % MT;
    constexpr uint32_t RP = kGatherThreads / MT;
    bool bad = false;
    for (uint32_t rl = tid / MT; rl < rows_here; rl += RP) {
        const uint16_t* rc = cs + rl * slots;
        float acc = 0.0f;
        for (uint32_t l = 0; l < S; ++l) {
            const float gamma = sc[l];
            for (uint32_t kk = 0; kk < k; ++kk) {
                const uint32_t code = rc[l * k + kk];
                const uint32_t atom = code & 0x7FFFu;
                const float scale = (code & 0x8000u) ? -gamma : gamma;
                // a code naming an atom the dictionary does not have contributes nothing and is
                // reported: images made by this library are checked on the host, raw device
                // streams handed to the allocation-free entry point are not
                const float v = atom < K ? dxp[atom * MT + b] : 0.0f;
                bad |= atom >= K;
                acc = __fadd_rn(acc, __fmul_rn(scale, v));
            }
        }
        if (b < yv.M) {
            const uint32_t r = row0 + rl;
            if (yv.bias) acc += yv.bias[r];
            yv.y[y_index(yv, r, b)] = acc;
        }
    }
    if (bad && status) atomicExch(status, 2);
}

// ---------------------------------------------------------------------------
// 2-D tiles, phase 1: P[a][bc][j][b] = sum_i D[a][j][i] * x[bc*Tc + i][b].
// The dictionary is one matrix of K*Tr "virtual rows" of Tc floats; the CTA stages 64
// of them in shared memory (row stride Tc+4 keeps 128-bit reads conflict-free), lane =
// virtual row, each warp walks its column tiles 8 at a time with x broadcast from
// shared memory. Writes are contiguous in j.
// ---------------------------------------------------------------------------
constexpr int kProjRows = 64;

template <int MT>
__global__ void __launch_bounds__(256)
hsdr_tile_project_kernel(const float* __restrict__ D, uint32_t VR /* K*Tr */, uint32_t Tr,
                         uint32_t Tc, uint32_t n_ct, XView xv, float* __restrict__ P) {
    extern __shared__ __align__(16) float psm[];
    const uint32_t dstride = Tc + 4u;
    float* dt = psm;                               // [64][Tc+4]
    float* xs = psm + kProjRows * dstride;         // [MT][n_ct][Tc]
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t vr0 = blockIdx.x * kProjRows;
    const uint32_t Tc4 = Tc >> 2;

    for (uint32_t i = tid; i < kProjRows * Tc4; i += 256) {
        const uint32_t r = i / Tc4, c4 = i - r * Tc4;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (vr0 + r < VR)
            v = ldg_stream_f4(reinterpret_cast<const float4*>(D + static_cast<size_t>(vr0 + r) * Tc) + c4);
        *reinterpret_cast<float4*>(dt + r * dstride + c4 * 4u) = v;
    }
    const uint32_t Cf = n_ct * Tc;
    for (uint32_t i = tid; i < MT * Cf; i += 256) {
        const uint32_t b = i / Cf, c = i - b * Cf;
        xs[i] = b < xv.M ? load_x(xv, c, b) : 0.0f;
    }
    __syncthreads();

    const uint32_t rg = warp & 1u;                 // which 32-row group
    const uint32_t vr = vr0 + rg * 32u + lane;
    const float* drow = dt + (rg * 32u + lane) * dstride;
    const uint32_t a = vr / Tr, j = vr - a * Tr;
    for (uint32_t bc0 = (warp >> 1) * 8u; bc0 < n_ct; bc0 += 32u) {
        float acc[8][MT];
#pragma unroll
        for (int q = 0; q < 8; ++q)
#pragma unroll
            for (int b = 0; b < MT; ++b) acc[q][b] = 0.0f;
        for (uint32_t i4 = 0; i4 < Tc4; ++i4) {
            const float4 d4 = *reinterpret_cast<const float4*>(drow + i4 * 4u);
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                if (bc0 + q < n_ct) {
#pragma unroll
                    for (int b = 0; b < MT; ++b) {
                        const float4 x4 = *reinterpret_cast<const float4*>(
                            xs + (static_cast<size_t>(b) * n_ct + bc0 + q) * Tc + i4 * 4u);
                        acc[q][b] = fmaf(d4.x, x4.x, acc[q][b]);
                        acc[q][b] = fmaf(d4.y, x4.y, acc[q][b]);
                        acc[q][b] = fmaf(d4.z, x4.z, acc[q][b]);
                        acc[q][b] = fmaf(d4.w, x4.w, acc[q][b]);
                    }
                }
            }
        }
        if (vr < VR) {
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                if (bc0 + q < n_ct) {
                    float* dst = P + ((static_cast<size_t>(a) * n_ct + bc0 + q) * Tr + j) * MT;
#pragma unroll
                    for (int b = 0; b < MT; ++b) dst[b] = acc[q][b];
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------
// 2-D tiles, phase 2: y[br*Tr + j][b] = sum_bc sum_codes sign*gamma * P[a][bc][j][b].
// CTA = (32 rows j) x (8 column-tile groups); group partials are summed through
// shared memory in a fixed order.
// ---------------------------------------------------------------------------
// Where the tile products P[atom][column tile][row in tile][token] sit, in floats: the CUDA-core
// projection writes them in that order; the tensor-core projection writes token-major rows
// [token * n_ct + column tile][atom * Tr + row].
struct TileProductStrides {
    size_t atom, col_tile, row, token;
};

template <int MT>
__global__ void __launch_bounds__(256)
hsdr_tile_gather_kernel(const uint16_t* __restrict__ codes, uint32_t Tr, uint32_t n_ct,
                        uint32_t n_jchunks, uint32_t S, uint32_t k,
                        const float* __restrict__ scales, const float* __restrict__ P, TileProductStrides ps, YView yv) {
    extern __shared__ __align__(16) unsigned char tsm[];
    const uint32_t slots = S * k;
    const uint32_t tid = threadIdx.x;
    const uint32_t br = blockIdx.x / n_jchunks, jc = blockIdx.x - br * n_jchunks;
    const uint32_t n_codes = n_ct * slots;

    const size_t code_byte0 = static_cast<size_t>(br) * n_codes * 2u;
    const size_t aligned0 = code_byte0 & ~static_cast<size_t>(15);
    const uint32_t skip = static_cast<uint32_t>(code_byte0 - aligned0) >> 1;
    const uint32_t n16 = (skip * 2u + n_codes * 2u + 15u) >> 4;
    const uint32_t cap16 = (n_codes * 2u + 15u + 16u) >> 4;
    uint4* cs16 = reinterpret_cast<uint4*>(tsm);
    float* sc = reinterpret_cast<float*>(tsm + static_cast<size_t>(cap16) * 16u);
    float* red = sc + ((S + 3u) & ~3u);            // [8][32][MT]
    float* mine = red + 8u * 32u * MT;             // [32][MT]: this CTA's sums, for the cluster's first CTA
    // grid y = cluster size: the column tiles of a row tile are dealt to the CTAs of a cluster when
    // there are too few row tiles to fill the GPU
    const uint32_t crank = blockIdx.y, csize = gridDim.y;
    const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const unsigned char*>(codes) + aligned0);
    for (uint32_t i = tid; i < n16; i += 256) cs16[i] = src[i];
    for (uint32_t i = tid; i < S; i += 256) sc[i] = scales[i];
    __syncthreads();
    const uint16_t* cs = reinterpret_cast<const uint16_t*>(cs16) + skip;

    const uint32_t jl = tid & 31u, grp = tid >> 5;
    const uint32_t j = jc * 32u + jl;
    float acc[MT];
#pragma unroll
    for (int b = 0; b < MT; ++b) acc[b] = 0.0f;
    if (j < Tr) {
        for (uint32_t bc = crank * 8u + grp; bc < n_ct; bc += 8u * csize) {
            const uint16_t* tc = cs + bc * slots;
            const float* pb = P + static_cast<size_t>(bc) * ps.col_tile + static_cast<size_t>(j) * ps.row;
            // eight codes at a time: their products are L2 round trips and must be in flight
            // together; the adds follow in slot order
            for (uint32_t s0 = 0; s0 < slots; s0 += 8u) {
                float v[8][MT], scale[8];
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    const uint32_t s_ = min(s0 + q, slots - 1u);
                    const uint32_t code = tc[s_];
                    const float gamma = sc[s_ / k];
                    scale[q] = s0 + q < slots ? ((code & 0x8000u) ? -gamma : gamma) : 0.0f;
                    const float* p = pb + static_cast<size_t>(code & 0x7FFFu) * ps.atom;
#pragma unroll
                    for (int b = 0; b < MT; ++b) v[q][b] = __ldg(p + static_cast<size_t>(b) * ps.token);
                }
#pragma unroll
                for (int q = 0; q < 8; ++q)
#pragma unroll
                    for (int b = 0; b < MT; ++b) acc[b] = fmaf(scale[q], v[q][b], acc[b]);
            }
        }
    }
#pragma unroll
    for (int b = 0; b < MT; ++b) red[(grp * 32u + jl) * MT + b] = acc[b];
    __syncthreads();
    for (uint32_t t = tid; t < 32u * MT; t += 256) {
        const uint32_t jj = t / MT, b = t - jj * MT;
        float s = 0.0f;
#pragma unroll
        for (int g = 0; g < 8; ++g) s += red[(g * 32u + jj) * MT + b];
        mine[t] = s;
    }
    if (csize > 1u) cg::this_cluster().sync();
    else __syncthreads();
    if (crank == 0u) {
        for (uint32_t t = tid; t < 32u * MT; t += 256) {
            const uint32_t jj = t / MT, b = t - jj * MT;
            float s = mine[t];
            for (uint32_t r = 1; r < csize; ++r) s += cg::this_cluster().map_shared_rank(mine, r)[t];   // rank order
            const uint32_t jr = jc * 32u + jj;
            if (jr < Tr && b < yv.M) {
                const uint32_t row = br * Tr + jr;
                if (yv.bias) s += yv.bias[row];
                yv.y[y_index(yv, row, b)] = s;
            }
        }
    }
    if (csize > 1u) cg::this_cluster().sync();   // the peers' shared memory must outlive the reads above
}

// One launch of the gather over tile products laid out as `ps` says.
template <int MT>
void launch_tile_gather(csdr_context* ctx, const csdr_segment* seg, const float* P, const TileProductStrides& ps, const YView& yv);

// ---------------------------------------------------------------------------
// Raw edge strips (stored fp32 verbatim): rows < R_full add their top-right strip's
// contribution to y; rows >= R_full are plain dense rows. One warp per row.
// ---------------------------------------------------------------------------
template <int MT>
__global__ void __launch_bounds__(256)
hsdr_edge_kernel(const float* __restrict__ edges, uint32_t R, uint32_t C, uint32_t Rf,
                 uint32_t Cf, XView xv, YView yv) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t r = blockIdx.x * 8u + (threadIdx.x >> 5);
    if (r >= R) return;
    const bool top = r < Rf;
    const uint32_t wc = top ? C - Cf : C;       // strip width
    if (wc == 0) return;
    const float* e = top ? edges + static_cast<size_t>(r) * (C - Cf)
                         : edges + static_cast<size_t>(Rf) * (C - Cf) + static_cast<size_t>(r - Rf) * C;
    const uint32_t cbase = top ? Cf : 0u;
    float acc[MT];
#pragma unroll
    for (int b = 0; b < MT; ++b) acc[b] = 0.0f;
    for (uint32_t c = lane; c < wc; c += 32u) {
        const float w = e[c];
#pragma unroll
        for (int b = 0; b < MT; ++b)
            if (b < xv.M) acc[b] = fmaf(w, load_x(xv, cbase + c, b), acc[b]);
    }
#pragma unroll
    for (int b = 0; b < MT; ++b) {
        float v = acc[b];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, off);
        if (lane == 0 && b < yv.M) {
            const size_t yi = y_index(yv, r, b);
            if (top) yv.y[yi] += v;
            else yv.y[yi] = v + (yv.bias ? yv.bias[r] : 0.0f);
        }
    }
}

// ---------------------------------------------------------------------------
// Dense rows: y[r][b] = sum_c W[r][c] * x[c][b]. One warp per row.
// ---------------------------------------------------------------------------
template <int MT>
__global__ void __launch_bounds__(256)
dense_rows_kernel(const float* __restrict__ W, uint32_t R, uint32_t C, XView xv, YView yv) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t r = blockIdx.x * 8u + (threadIdx.x >> 5);
    if (r >= R) return;
    const float* w = W + static_cast<size_t>(r) * C;
    float acc[MT];
#pragma unroll
    for (int b = 0; b < MT; ++b) acc[b] = 0.0f;
    for (uint32_t c = lane; c < C; c += 32u) {
        const float wv = w[c];
#pragma unroll
        for (int b = 0; b < MT; ++b)
            if (b < xv.M) acc[b] = fmaf(wv, load_x(xv, c, b), acc[b]);
    }
#pragma unroll
    for (int b = 0; b < MT; ++b) {
        float v = acc[b];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, off);
        if (lane == 0 && b < yv.M) yv.y[y_index(yv, r, b)] = v + (yv.bias ? yv.bias[r] : 0.0f);
    }
}

// y (token-major or feature-major, + bias) from a feature-major product t[r][stride].
__global__ void __launch_bounds__(256)
retile_bias_kernel(const float* __restrict__ t, uint32_t R, uint32_t M, uint32_t stride, YView yv) {
    __shared__ float tile[32][33];
    const uint32_t r0 = blockIdx.x * 32u, b0 = blockIdx.y * 32u;
    const uint32_t tx = threadIdx.x & 31u, ty = threadIdx.x >> 5;
    for (uint32_t j = ty; j < 32u; j += 8u) {
        const uint32_t r = r0 + j, b = b0 + tx;
        tile[j][tx] = (r < R && b < M) ? t[static_cast<size_t>(r) * stride + b] : 0.0f;
    }
    __syncthreads();
    for (uint32_t j = ty; j < 32u; j += 8u) {
        const uint32_t b = b0 + j, r = r0 + tx;
        if (r < R && b < M) yv.y[y_index(yv, r, b)] = tile[tx][j] + (yv.bias ? yv.bias[r] : 0.0f);
    }
}

// ---------------------------------------------------------------------------
// host-side dispatch
// ---------------------------------------------------------------------------
template <typename Kern>
void ensure_smem(Kern kern, size_t bytes) {
    if (bytes > 48 * 1024)
        CSDR_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(bytes)));
}

int pick_mt(size_t m) { return m <= 1 ? 1 : m <= 2 ? 2 : m <= 4 ? 4 : m <= 8 ? 8 : 16; }

template <int MT, int A, int U>
void launch_dx_t(csdr_context* ctx, const csdr_segment* seg, const XView& xv, float* dx,
                 uint32_t nsplit, uint32_t slab) {
    const Geometry& g = seg->g;
    auto kern = hsdr_dx_kernel<MT, A, U>;
    const size_t smem = (static_cast<size_t>(MT) * slab + 8u * A * MT) * sizeof(float);
    ensure_smem(kern, smem);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(nsplit, (g.n_atoms + 8u * A - 1u) / (8u * A), 1);
    cfg.blockDim = dim3(256, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = nsplit;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    LaunchScope ls(ctx, KC_DX);
    CSDR_CUDA(cudaLaunchKernelEx(&cfg, kern, static_cast<const float*>(seg->atoms->ptr), g.n_atoms,
                                 g.cols, slab, xv, dx, static_cast<int>(nsplit)));
    ls.done("hsdr_dx_kernel");
}

template <int MT>
void launch_gather_t(csdr_context* ctx, const csdr_segment* seg, const float* dx, const YView& yv) {
    const Geometry& g = seg->g;
    constexpr uint32_t RP = kGatherThreads / MT;
    // Every CTA stages the whole Dx block (n_atoms x MT floats): with wide tiles fewer, larger
    // CTAs keep that staging a small share of the traffic.
    const uint32_t ctas = (MT >= 8 ? 1u : 4u) * static_cast<uint32_t>(ctx->sm_count);
    uint32_t rows_per_cta = (g.rows + ctas - 1u) / ctas;
    rows_per_cta = std::max(RP, (rows_per_cta + RP - 1u) / RP * RP);
    const uint32_t slots = g.slots();
    const size_t cap16 = (static_cast<size_t>(rows_per_cta) * slots * 2u + 31u) >> 4;
    const size_t base = cap16 * 16u + ((g.n_stages + 3u) & ~3u) * sizeof(float);
    const size_t dx_bytes = static_cast<size_t>(g.n_atoms) * MT * sizeof(float);
    const int dx_in_smem = base + dx_bytes <= 160u * 1024u;
    const size_t smem = base + (dx_in_smem ? dx_bytes : 0u);
    auto kern = hsdr_gather_kernel<MT>;
    ensure_smem(kern, smem);
    const uint32_t grid = (g.rows + rows_per_cta - 1u) / rows_per_cta;
    LaunchScope ls(ctx, KC_GATHER);
    kern<<<grid, kGatherThreads, smem, ctx->stream>>>(
        seg->codes_ptr(), g.rows, g.n_stages, g.k, static_cast<const float*>(seg->scales->ptr), dx,
        g.n_atoms, rows_per_cta, dx_in_smem, yv, ctx->status_word);
    ls.done("hsdr_gather_kernel");
}

template <int MT>
void matmul_rowtiles_chunk(csdr_context* ctx, const csdr_segment* seg, const XView& xv,
                           const YView& yv) {
    const Geometry& g = seg->g;
    // Column split: slabs of about 1024 floats, at most 8 CTAs per cluster (the portable
    // limit), each slab a multiple of 4 floats.
    uint32_t nsplit = std::min<uint32_t>(8u, std::max<uint32_t>(1u, (g.cols + 1023u) / 1024u));
    uint32_t slab = ((g.cols + nsplit - 1u) / nsplit + 3u) & ~3u;
    nsplit = (g.cols + slab - 1u) / slab;
    float* dx = static_cast<float*>(
        ctx->scratch_get(0, static_cast<size_t>(g.n_atoms) * 16u * sizeof(float)));
    if constexpr (MT == 1) launch_dx_t<1, 1, 8>(ctx, seg, xv, dx, nsplit, slab);
    else if constexpr (MT == 2) launch_dx_t<2, 1, 8>(ctx, seg, xv, dx, nsplit, slab);
    else if constexpr (MT == 4) launch_dx_t<4, 2, 4>(ctx, seg, xv, dx, nsplit, slab);
    else if constexpr (MT == 8) launch_dx_t<8, 4, 2>(ctx, seg, xv, dx, nsplit, slab);
    else launch_dx_t<16, 4, 2>(ctx, seg, xv, dx, nsplit, slab);
    launch_gather_t<MT>(ctx, seg, dx, yv);
}

template <int MT>
void launch_tile_gather(csdr_context* ctx, const csdr_segment* seg, const float* P, const TileProductStrides& ps, const YView& yv) {
    const Geometry& g = seg->g;
    auto kern = hsdr_tile_gather_kernel<MT>;
    const uint32_t n_jchunks = (g.tile_rows + 31u) / 32u;
    const uint32_t n_row_tiles = g.rows_full / g.tile_rows;
    const size_t cap16 = (static_cast<size_t>(g.n_col_tiles) * g.slots() * 2u + 31u) >> 4;
    const size_t smem = cap16 * 16u + ((g.n_stages + 3u) & ~3u) * sizeof(float) + 9u * 32u * MT * sizeof(float);
    ensure_smem(kern, smem);
    const uint32_t ctas = n_row_tiles * n_jchunks, sms = static_cast<uint32_t>(ctx->sm_count);
    uint32_t csplit = 1;
    while (csplit < 8u && ctas * csplit < 2u * sms && g.n_col_tiles >= 16u * csplit) csplit *= 2u;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(ctas, csplit, 1);
    cfg.blockDim = dim3(256, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = csplit;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = csplit > 1u ? 1 : 0;
    LaunchScope ls(ctx, KC_TILE_GATHER);
    CSDR_CUDA(cudaLaunchKernelEx(&cfg, kern, seg->codes_ptr(), static_cast<uint32_t>(g.tile_rows), static_cast<uint32_t>(g.n_col_tiles),
                                 n_jchunks, static_cast<uint32_t>(g.n_stages), static_cast<uint32_t>(g.k),
                                 static_cast<const float*>(seg->scales->ptr), P, ps, yv));
    ls.done("hsdr_tile_gather_kernel");
}

template <int MT>
void matmul_tiles_chunk(csdr_context* ctx, const csdr_segment* seg, const XView& xv,
                        const YView& yv) {
    const Geometry& g = seg->g;
    const uint32_t VR = g.n_atoms * g.tile_rows;
    const size_t p_bytes = static_cast<size_t>(VR) * g.n_col_tiles * MT * sizeof(float);
    float* P = static_cast<float*>(ctx->scratch_get(1, p_bytes));
    {
        auto kern = hsdr_tile_project_kernel<MT>;
        const size_t smem = (static_cast<size_t>(kProjRows) * (g.tile_cols + 4u) +
                             static_cast<size_t>(MT) * g.cols_full) * sizeof(float);
        ensure_smem(kern, smem);
        LaunchScope ls(ctx, KC_TILE_PROJECT);
        kern<<<(VR + kProjRows - 1u) / kProjRows, 256, smem, ctx->stream>>>(
            static_cast<const float*>(seg->atoms->ptr), VR, g.tile_rows, g.tile_cols, g.n_col_tiles,
            xv, P);
        ls.done("hsdr_tile_project_kernel");
    }
    launch_tile_gather<MT>(ctx, seg, P,
                           TileProductStrides{static_cast<size_t>(g.n_col_tiles) * g.tile_rows * MT, static_cast<size_t>(g.tile_rows) * MT, MT, 1},
                           yv);
    if (seg->edges) {
        LaunchScope ls(ctx, KC_EDGE);
        hsdr_edge_kernel<MT><<<(g.rows + 7u) / 8u, 256, 0, ctx->stream>>>(
            static_cast<const float*>(seg->edges->ptr), g.rows, g.cols, g.rows_full, g.cols_full, xv, yv);
        ls.done("hsdr_edge_kernel");
    }
}

// Tokens [b0, b0 + m) of a 2-D tile product whose tile products came from the tensor-core
// projection: P_T[(token * n_ct + column tile)][atom * Tr + row].
template <int MT>
void tiles_gather_token_major(csdr_context* ctx, const csdr_segment* seg, const float* P_T, uint32_t b0, const XView& xv,
                              const YView& yv) {
    const Geometry& g = seg->g;
    const size_t row_floats = static_cast<size_t>(g.n_atoms) * g.tile_rows;
    launch_tile_gather<MT>(ctx, seg, P_T + static_cast<size_t>(b0) * g.n_col_tiles * row_floats,
                           TileProductStrides{g.tile_rows, row_floats, 1, static_cast<size_t>(g.n_col_tiles) * row_floats}, yv);
    if (seg->edges) {
        LaunchScope ls(ctx, KC_EDGE);
        hsdr_edge_kernel<MT><<<(g.rows + 7u) / 8u, 256, 0, ctx->stream>>>(
            static_cast<const float*>(seg->edges->ptr), g.rows, g.cols, g.rows_full, g.cols_full, xv, yv);
        ls.done("hsdr_edge_kernel");
    }
}

// Largest token tile (a power of two <= 16) whose shared-memory need fits.
int fit_mt(int want, size_t fixed_bytes, size_t per_token_bytes, size_t budget) {
    int mt = want;
    while (mt > 1 && fixed_bytes + per_token_bytes * mt > budget) mt >>= 1;
    if (fixed_bytes + per_token_bytes * mt > budget) return 0;
    return mt;
}

template <typename F>
void dispatch_mt(int mt, F&& f) {
    switch (mt) {
        case 1: f(std::integral_constant<int, 1>{}); break;
        case 2: f(std::integral_constant<int, 2>{}); break;
        case 4: f(std::integral_constant<int, 4>{}); break;
        case 8: f(std::integral_constant<int, 8>{}); break;
        default: f(std::integral_constant<int, 16>{}); break;
    }
}

}  // namespace

void launch_gather_tile(csdr_context* ctx, const csdr_segment* seg, const float* dx, int mt, float* y, int y_layout,
                        uint32_t m_total, uint32_t b0, uint32_t m, const float* bias) {
    YView yv{y, y_layout, seg->g.rows, m_total, b0, m, bias};
    dispatch_mt(mt, [&](auto mtc) { launch_gather_t<decltype(mtc)::value>(ctx, seg, dx, yv); });
}

void launch_unpack(csdr_context* ctx, const uint16_t* codes, size_t n, int32_t* idx, int8_t* sign) {
    if (n == 0) return;
    const size_t blocks = std::min<size_t>((n / 8 + 255) / 256 + 1, static_cast<size_t>(ctx->sm_count) * 8);
    LaunchScope ls(ctx, KC_UNPACK);
    hsdr_unpack_kernel<<<static_cast<unsigned>(blocks), 256, 0, ctx->stream>>>(codes, n, idx, sign);
    ls.done("hsdr_unpack_kernel");
}

void launch_dense_matmul(csdr_context* ctx, const float* W, uint32_t R, uint32_t C,
                         const MatmulArgs& a) {
    for (size_t b0 = 0; b0 < a.batch; b0 += 16) {
        const uint32_t m = static_cast<uint32_t>(std::min<size_t>(16, a.batch - b0));
        XView xv{a.x, a.x_dtype, a.x_layout, C, static_cast<uint32_t>(a.batch), static_cast<uint32_t>(b0), m};
        YView yv{a.y, a.y_layout, R, static_cast<uint32_t>(a.batch), static_cast<uint32_t>(b0), m, a.bias};
        dispatch_mt(pick_mt(m), [&](auto mt) {
            LaunchScope ls(ctx, KC_DENSE);
            dense_rows_kernel<decltype(mt)::value><<<(R + 7u) / 8u, 256, 0, ctx->stream>>>(W, R, C, xv, yv);
            ls.done("dense_rows_kernel");
        });
    }
}

void launch_matmul(csdr_context* ctx, const csdr_segment* seg, const MatmulArgs& a) {
    const Geometry& g = seg->g;
    if (a.batch == 0) return;
    if (a.batch > 0xFFFFFFFFull) throw Error(CSDR_ERR_LIMIT, "batch too large");
    if (tcgen05_supported(ctx, seg, a.batch)) {
        launch_matmul_tcgen05(ctx, seg, a);
        return;
    }
    if (ctx->gemv_queue_single) {
        // a list of one: the persistent kernel's streaming loader without the column split
        const QueueItem item{seg, a.x, a.x_dtype, a.x_layout, a.batch, a.y, a.y_layout, a.bias};
        if (gemv_queue_supported(ctx, &item, 1)) {
            launch_gemv_queue(ctx, &item, 1);
            return;
        }
    }
    if (!g.row_tiles() && ctx->cache_2d && ctx->tensor_cores && a.batch >= 16 && g.rows % 128u == 0 && g.cols % 8u == 0 &&
        g.rows <= 0x7FFFu * 128u) {
        // 2-D tiles at a wide batch: what the reference does (decompress once, keep the layer, dense
        // product - SparseInferenceEngine.cpp:1301-1310 behind its layer cache), on the tensor cores:
        // the weight is rebuilt once by the bit-exact decode kernel, split into bf16 hi/lo planes that
        // stay with the segment (4 bytes per element, as the reference's cached fp32 layer), and every
        // wide product is the TMA-fed tcgen05 kernel over those planes with one "atom" per output row.
        // Rebuilding tiles in shared memory per product instead would re-read S*k atoms of 64 KB per
        // tile from L2 - 4 to 5 GB per product at the 7B shapes, whatever the batch.
        if (!seg->dense) {
            auto dn = std::make_shared<csdr_segment>();
            dn->ctx = ctx;
            dn->g.rows = dn->g.n_tiles = dn->g.rows_full = g.rows;   // not used by the projection
            dn->g.cols = dn->g.cols_full = dn->g.tile_cols = g.cols;
            dn->g.tile_rows = 1;
            dn->g.n_col_tiles = 1;
            dn->g.n_atoms = g.rows;
            dn->g.n_stages = dn->g.k = 1;
            dn->atoms = std::make_shared<DeviceBuffer>(static_cast<size_t>(g.rows) * g.cols * 4u, ctx->device);
            launch_decode_rows(ctx, seg, nullptr, g.rows, static_cast<float*>(dn->atoms->ptr));
            if (!dx_tma_supported(ctx, dn.get(), a.batch)) throw Error(CSDR_ERR_UNSUPPORTED, "tensor maps unavailable");
            dx_tma_prepare(ctx, dn.get());
            CSDR_CUDA(cudaStreamSynchronize(ctx->stream));
            dn->atoms->release_data();                               // the planes hang on the buffer object
            seg->dense = dn;
        }
        const uint32_t M = static_cast<uint32_t>(a.batch);
        const bool direct = a.y_layout == CSDR_LAYOUT_FEATURE_MAJOR && !a.bias;
        float* out = direct ? a.y
                            : static_cast<float*>(ctx->scratch_get(7, static_cast<size_t>(g.rows) * M * sizeof(float)));
        launch_dx_tma(ctx, seg->dense.get(), a, out, M);
        if (!direct) {
            YView yv{a.y, a.y_layout, g.rows, M, 0u, M, a.bias};
            LaunchScope ls(ctx, KC_DECODER_OP);
            retile_bias_kernel<<<dim3((g.rows + 31u) / 32u, (M + 31u) / 32u), 256, 0, ctx->stream>>>(out, g.rows, M, M, yv);
            ls.done("retile_bias_kernel");
        }
        return;
    }
    const size_t budget = std::min<size_t>(ctx->smem_optin, 200u * 1024u);
    const bool fast_rows = g.row_tiles() && (g.cols % 4u == 0);
    const bool fast_tiles = !fast_rows && (g.tile_cols % 4u == 0);
    if (!fast_rows && ctx->tile_tc && ctx->tensor_cores && ctx->tma && g.cols == g.cols_full && g.tile_cols % 8u == 0 &&
        (static_cast<size_t>(g.n_atoms) * g.tile_rows) % 128u == 0 &&
        a.batch * g.n_col_tiles >= ctx->tc_min_batch &&
        a.batch * g.n_col_tiles * g.n_atoms * static_cast<size_t>(g.tile_rows) * 4u <= (1ull << 30)) {
        // 2-D tiles, a few tokens: the tile products are ONE GEMM - the dictionary read as
        // K * Tr rows of Tc columns against the activations read as batch * n_ct tokens of Tc
        // columns (a token-major activation row IS its n_ct column tiles one after the other) -
        // on the tensor cores, out in token-major rows the gather reads with unit stride.
        if (!seg->tile_view) {
            auto tv = std::make_shared<csdr_segment>();
            tv->ctx = ctx;
            tv->g.rows = tv->g.rows_full = tv->g.n_tiles = 1;
            tv->g.cols = tv->g.cols_full = tv->g.tile_cols = g.tile_cols;
            tv->g.tile_rows = tv->g.n_col_tiles = 1;
            tv->g.n_atoms = g.n_atoms * g.tile_rows;
            tv->g.n_stages = tv->g.k = 1;
            tv->atoms = seg->atoms;
            seg->tile_view = tv;
        }
        const csdr_segment* tv = seg->tile_view.get();
        if (dx_tma_supported(ctx, tv, a.batch * g.n_col_tiles)) {
            const uint32_t M = static_cast<uint32_t>(a.batch), n_tok = M * g.n_col_tiles;
            const XPlanesView xp = make_x_planes(ctx, a.x, a.x_dtype, a.x_layout, M, g.cols);
            float* P_T = static_cast<float*>(ctx->scratch_get(7, static_cast<size_t>(n_tok) * tv->g.n_atoms * sizeof(float)));
            launch_dx_tma_group(ctx, &tv, 1, xp, n_tok, &P_T, tv->g.n_atoms, nullptr, nullptr, nullptr, true);
            for (size_t b0 = 0; b0 < a.batch; b0 += 4) {
                const uint32_t m = static_cast<uint32_t>(std::min<size_t>(4, a.batch - b0));
                XView xv{a.x, a.x_dtype, a.x_layout, g.cols, M, static_cast<uint32_t>(b0), m};
                YView yv{a.y, a.y_layout, g.rows, M, static_cast<uint32_t>(b0), m, a.bias};
                dispatch_mt(pick_mt(m), [&](auto mt) {
                    constexpr int MT = decltype(mt)::value;
                    if constexpr (MT <= 4) tiles_gather_token_major<MT>(ctx, seg, P_T, static_cast<uint32_t>(b0), xv, yv);
                });
            }
            return;
        }
    }
    int mt_cap = 0;
    if (fast_rows) {
        uint32_t nsplit = std::min<uint32_t>(8u, std::max<uint32_t>(1u, (g.cols + 1023u) / 1024u));
        const uint32_t slab = ((g.cols + nsplit - 1u) / nsplit + 3u) & ~3u;
        mt_cap = fit_mt(16, 0, (static_cast<size_t>(slab) + 32u) * sizeof(float), budget);
    } else if (fast_tiles) {
        mt_cap = fit_mt(4, static_cast<size_t>(kProjRows) * (g.tile_cols + 4u) * sizeof(float),
                        static_cast<size_t>(g.cols_full) * sizeof(float), budget);
        const size_t gather_fixed = ((static_cast<size_t>(g.n_col_tiles) * g.slots() * 2u + 31u) & ~15u) +
                                    ((g.n_stages + 3u) & ~3u) * sizeof(float);
        if (gather_fixed + 8u * 32u * 16u * sizeof(float) > budget) mt_cap = 0;
    }
    if (mt_cap == 0) {
        // Odd geometry: materialise W once into scratch, then a dense product — what the
        // reference does for every 2-D encoding (decompress + dense).
        float* W = static_cast<float*>(
            ctx->scratch_get(2, static_cast<size_t>(g.rows) * g.cols * sizeof(float)));
        launch_decode_rows(ctx, seg, nullptr, g.rows, W);
        launch_dense_matmul(ctx, W, g.rows, g.cols, a);
        return;
    }
    for (size_t b0 = 0; b0 < a.batch; b0 += mt_cap) {
        const uint32_t m = static_cast<uint32_t>(std::min<size_t>(mt_cap, a.batch - b0));
        XView xv{a.x, a.x_dtype, a.x_layout, g.cols, static_cast<uint32_t>(a.batch),
                 static_cast<uint32_t>(b0), m};
        YView yv{a.y, a.y_layout, g.rows, static_cast<uint32_t>(a.batch), static_cast<uint32_t>(b0), m, a.bias};
        dispatch_mt(pick_mt(m), [&](auto mt) {
            constexpr int MT = decltype(mt)::value;
            if (fast_rows && gemv_fused_supported(ctx, &seg, 1, MT)) {
                float* yp = a.y;
                const float* bp = a.bias;
                launch_gemv_fused(ctx, &seg, 1, a.x, a.x_dtype, a.x_layout, static_cast<uint32_t>(a.batch),
                                  static_cast<uint32_t>(b0), m, &yp, a.y_layout, a.bias ? &bp : nullptr, MT);
            } else if (fast_rows) matmul_rowtiles_chunk<MT>(ctx, seg, xv, yv);
            else if constexpr (MT <= 4) matmul_tiles_chunk<MT>(ctx, seg, xv, yv);
        });
    }
}

}  // namespace csdr

// ---------------------------------------------------------------------------
// Allocation-free entry point.
//
// Some hosts of this library may not call cudaMalloc at all once they are running: a
// real-time or safety-certified process that fixes its device memory map at start-up, a
// plug-in living inside another runtime's memory pool, or a service whose own arena already
// holds all device memory. csdr_matmul_rowtiles_noalloc serves them:
// the row-tile product through the two-kernel path (projection, then gather), with the one
// piece of scratch that path needs - Dx, n_atoms x 16 floats - in a fixed array that lives
// in the library's device image instead of coming from the allocator.
// ---------------------------------------------------------------------------
namespace csdr {
namespace {

constexpr uint32_t kNoAllocMaxAtoms = 4096;  // 4096 atoms x 16 tokens x 4 B = 256 KiB per GPU
constexpr uint32_t kNoAllocTokens = 16;
constexpr int kNoAllocMaxDevices = 64;

// Held by every GPU that loads the library, until the process exits. Host code may name
// this array only to ask for its address: the symbol itself is not a device pointer.
static __device__ __align__(256) float g_noalloc_dx[kNoAllocMaxAtoms * kNoAllocTokens];
// Set to 2 by the gather when a code named an atom >= n_atoms (the code contributed nothing);
// read and cleared by csdr_matmul_rowtiles_noalloc_status.
static __device__ int g_noalloc_status;

struct NoAllocScratch {
    float* dx = nullptr;
    int* status = nullptr;
};

// Device addresses of the two symbols on `device`, which must be current. Looked up once per device.
NoAllocScratch noalloc_scratch(int device) {
    static NoAllocScratch addr[kNoAllocMaxDevices] = {};
    static std::mutex mu;
    if (device < 0 || device >= kNoAllocMaxDevices) throw Error(CSDR_ERR_LIMIT, "device index beyond 63");
    std::lock_guard<std::mutex> lk(mu);
    if (!addr[device].dx) {
        float* p = nullptr;
        int* q = nullptr;
        cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_dx);
        if (e == cudaSuccess) e = cudaGetSymbolAddress(reinterpret_cast<void**>(&q), g_noalloc_status);
        if (e != cudaSuccess || !p || !q)
            throw Error(CSDR_ERR_CUDA, std::string("cudaGetSymbolAddress(scratch): ") + cudaGetErrorString(e));
        addr[device].status = q;
        addr[device].dx = p;
    }
    return addr[device];
}

template <typename Kern>
void noalloc_smem(Kern kern, size_t bytes) {
    if (bytes > 48 * 1024) {
        const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                   static_cast<int>(bytes));
        if (e != cudaSuccess) throw Error(CSDR_ERR_CUDA, std::string("cudaFuncSetAttribute: ") + cudaGetErrorString(e));
    }
}

void noalloc_check(const char* what) {
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) throw Error(CSDR_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e));
}

template <int MT, int A, int U>
void noalloc_chunk(const float* D, const uint16_t* codes, const float* scales, uint32_t R, uint32_t C,
                   uint32_t K, uint32_t S, uint32_t k, const XView& xv, const YView& yv, float* dx,
                   int* status, int sm_count, cudaStream_t stream) {
    uint32_t nsplit = std::min<uint32_t>(8u, std::max<uint32_t>(1u, (C + 1023u) / 1024u));
    const uint32_t slab = ((C + nsplit - 1u) / nsplit + 3u) & ~3u;
    nsplit = (C + slab - 1u) / slab;
    {
        auto kern = hsdr_dx_kernel<MT, A, U>;
        const size_t smem = (static_cast<size_t>(MT) * slab + 8u * A * MT) * sizeof(float);
        noalloc_smem(kern, smem);
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(nsplit, (K + 8u * A - 1u) / (8u * A), 1);
        cfg.blockDim = dim3(256, 1, 1);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = nsplit;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        const cudaError_t e = cudaLaunchKernelEx(&cfg, kern, D, K, C, slab, xv, dx, static_cast<int>(nsplit));
        if (e != cudaSuccess) throw Error(CSDR_ERR_CUDA, std::string("hsdr_dx_kernel: ") + cudaGetErrorString(e));
    }
    {
        constexpr uint32_t RP = kGatherThreads / MT;
        uint32_t rows_per_cta = (R + 4u * sm_count - 1u) / (4u * sm_count);
        rows_per_cta = std::max(RP, (rows_per_cta + RP - 1u) / RP * RP);
        const uint32_t slots = S * k;
        const size_t cap16 = (static_cast<size_t>(rows_per_cta) * slots * 2u + 31u) >> 4;
        const size_t base = cap16 * 16u + ((S + 3u) & ~3u) * sizeof(float);
        const size_t dx_bytes = static_cast<size_t>(K) * MT * sizeof(float);
        const int dx_in_smem = base + dx_bytes <= 160u * 1024u;
        const size_t smem = base + (dx_in_smem ? dx_bytes : 0u);
        auto kern = hsdr_gather_kernel<MT>;
        noalloc_smem(kern, smem);
        kern<<<(R + rows_per_cta - 1u) / rows_per_cta, kGatherThreads, smem, stream>>>(
            codes, R, S, k, scales, dx, K, rows_per_cta, dx_in_smem, yv, status);
        noalloc_check("hsdr_gather_kernel");
    }
}

}  // namespace
}  // namespace csdr

extern "C" int csdr_matmul_rowtiles_noalloc(const float* dict_dev, const uint16_t* codes_dev,
                                            const float* scales_dev, uint32_t rows, uint32_t cols,
                                            uint32_t n_atoms, uint32_t n_stages, uint32_t k_per_stage,
                                            const void* x_dev, int x_dtype, int x_layout, size_t batch,
                                            float* y_dev, int y_layout, void* stream) {
    using namespace csdr;
    return guard([&] {
        if (!dict_dev || !codes_dev || !scales_dev || !x_dev || !y_dev)
            throw Error(CSDR_ERR_INVALID_ARG, "null argument");
        if (!rows || !cols || !n_atoms || !n_stages || !k_per_stage)
            throw Error(CSDR_ERR_INVALID_ARG, "zero-sized geometry field");
        if (n_atoms > kNoAllocMaxAtoms)
            throw Error(CSDR_ERR_LIMIT, "csdr_matmul_rowtiles_noalloc: n_atoms " + std::to_string(n_atoms) +
                                            " exceeds the fixed scratch of " + std::to_string(kNoAllocMaxAtoms) +
                                            " atoms; use csdr_matmul_device_async");
        if (n_atoms > 0x7FFFu || cols > 0xFFFFu || (cols & 3u))
            throw Error(CSDR_ERR_LIMIT, "csdr_matmul_rowtiles_noalloc: cols must be a multiple of 4 and at most 65535");
        if (batch > 0xFFFFFFFFull) throw Error(CSDR_ERR_LIMIT, "batch too large");
        if ((reinterpret_cast<uintptr_t>(dict_dev) | reinterpret_cast<uintptr_t>(codes_dev)) & 15u)
            throw Error(CSDR_ERR_INVALID_ARG, "dictionary and code stream must be 16-byte aligned");
        if ((x_dtype != CSDR_DTYPE_F32 && x_dtype != CSDR_DTYPE_BF16) ||
            (x_layout != CSDR_LAYOUT_FEATURE_MAJOR && x_layout != CSDR_LAYOUT_TOKEN_MAJOR) ||
            (y_layout != CSDR_LAYOUT_FEATURE_MAJOR && y_layout != CSDR_LAYOUT_TOKEN_MAJOR))
            throw Error(CSDR_ERR_INVALID_ARG, "unknown dtype or layout");
        if (batch == 0) return;
        int device = 0, sm_count = 0;
        CSDR_CUDA(cudaGetDevice(&device));
        CSDR_CUDA(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device));
        const NoAllocScratch sc = noalloc_scratch(device);  // first call on a device looks the addresses up
        cudaStream_t st = static_cast<cudaStream_t>(stream);
        // token tile: the widest power of two <= 16 whose x slab fits in 200 KiB of shared memory
        uint32_t nsplit = std::min<uint32_t>(8u, std::max<uint32_t>(1u, (cols + 1023u) / 1024u));
        const uint32_t slab = ((cols + nsplit - 1u) / nsplit + 3u) & ~3u;
        const int mt_cap = fit_mt(16, 0, (static_cast<size_t>(slab) + 32u) * sizeof(float), 200u * 1024u);
        if (mt_cap == 0) throw Error(CSDR_ERR_LIMIT, "csdr_matmul_rowtiles_noalloc: row too wide for shared memory");
        for (size_t b0 = 0; b0 < batch; b0 += mt_cap) {
            const uint32_t m = static_cast<uint32_t>(std::min<size_t>(mt_cap, batch - b0));
            XView xv{x_dev, x_dtype, x_layout, cols, static_cast<uint32_t>(batch), static_cast<uint32_t>(b0), m};
            YView yv{y_dev, y_layout, rows, static_cast<uint32_t>(batch), static_cast<uint32_t>(b0), m, nullptr};
            switch (pick_mt(m)) {
                case 1: noalloc_chunk<1, 1, 8>(dict_dev, codes_dev, scales_dev, rows, cols, n_atoms, n_stages, k_per_stage, xv, yv, sc.dx, sc.status, sm_count, st); break;
                case 2: noalloc_chunk<2, 1, 8>(dict_dev, codes_dev, scales_dev, rows, cols, n_atoms, n_stages, k_per_stage, xv, yv, sc.dx, sc.status, sm_count, st); break;
                case 4: noalloc_chunk<4, 2, 4>(dict_dev, codes_dev, scales_dev, rows, cols, n_atoms, n_stages, k_per_stage, xv, yv, sc.dx, sc.status, sm_count, st); break;
                case 8: noalloc_chunk<8, 4, 2>(dict_dev, codes_dev, scales_dev, rows, cols, n_atoms, n_stages, k_per_stage, xv, yv, sc.dx, sc.status, sm_count, st); break;
                default: noalloc_chunk<16, 4, 2>(dict_dev, codes_dev, scales_dev, rows, cols, n_atoms, n_stages, k_per_stage, xv, yv, sc.dx, sc.status, sm_count, st); break;
            }
        }
    });
}


extern "C" int csdr_matmul_rowtiles_noalloc_status(void* stream, int* bad_codes) {
    using namespace csdr;
    return guard([&] {
        if (!bad_codes) throw Error(CSDR_ERR_INVALID_ARG, "null argument");
        int device = 0;
        CSDR_CUDA(cudaGetDevice(&device));
        const NoAllocScratch sc = noalloc_scratch(device);
        cudaStream_t st = static_cast<cudaStream_t>(stream);
        int word = 0;
        CSDR_CUDA(cudaMemcpyAsync(&word, sc.status, sizeof(int), cudaMemcpyDeviceToHost, st));
        CSDR_CUDA(cudaMemsetAsync(sc.status, 0, sizeof(int), st));
        CSDR_CUDA(cudaStreamSynchronize(st));
        *bad_codes = word != 0;
        if (word != 0)
            throw Error(CSDR_ERR_CODE_RANGE, "csdr_matmul_rowtiles_noalloc: a packed code named an atom >= n_atoms "
                                             "(it contributed nothing to its row)");
    });
}
