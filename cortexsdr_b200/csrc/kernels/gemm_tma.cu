// TMA-fed tensor-core projection Dx = D * X^T for wide token tiles of 1-D row-tile HSDR segments
// on sm_100a. Same arithmetic as the register-fed kernel in gemm_tcgen05.cu (bf16 hi/lo split of
// the fp32 dictionary and activations, fp32 accumulation in tensor memory; reference loop:
// strategies/HierarchicalSDRStrategy.cpp:1304-1318), but the split happens once per dictionary
// instead of once per CTA, and nothing passes through registers on the way to the MMA:
//
//   * the dictionary is kept as two bf16 planes hi = bf16(d), lo = bf16(d - hi), built on the
//     first wide call and cached beside the fp32 atoms (shared by every segment and row shard
//     that uses the dictionary);
//   * activations that are already bf16, token-major and 16-byte aligned are read in place;
//     anything else is split into planes by a small kernel first;
//   * one CTA owns (128 atoms) x (N tokens) x (a range of 64-column blocks). Warp 0 issues
//     cp.async.bulk.tensor loads (128-byte swizzle, the layout the MMA descriptors name) into a
//     ring of stages and arms each stage's mbarrier with the expected byte count; warp 1 waits
//     for a stage, issues tcgen05.mma (hi*hi + lo*hi [+ hi*lo]) and commits the stage back to the
//     loader; warps 2-5 read the accumulators out of tensor memory at the end;
//   * the column ranges of one output tile form a thread-block cluster (co-scheduled by the
//     hardware): every CTA writes its accumulator tile to a partial buffer (L2-resident), the
//     cluster meets at its barrier, and each CTA sums its share of the rows over the ranks in
//     rank order (so the result does not depend on timing) and writes those rows of Dx. No
//     separate reduction kernel, no spin-waits between CTAs.
//
// Every mbarrier wait is a bounded try_wait loop; a wait that runs out sets the context's status
// word, the roles stop issuing work, and the CTA still meets its cluster barriers and frees its
// tensor memory.
#include <cooperative_groups.h>
#include <cuda.h>
#include <cuda_bf16.h>

#include <algorithm>

#include "../internal.hpp"
#include "gemm_tcgen05.hpp"
#include "views.cuh"

namespace cg = cooperative_groups;

namespace csdr {

namespace tma_detail {

constexpr uint32_t kThreads = 192;       // loader warp, MMA warp, four epilogue warps
constexpr uint32_t kBlockK = 64;         // bf16 per tile row = 128 bytes = one swizzle span
constexpr uint32_t kTileM = 128;         // atoms per CTA = MMA M
constexpr uint32_t kATile = kTileM * 128u;
constexpr uint32_t kMaxStages = 4;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// K-major operand, 128-byte swizzle: 8 rows x 128 B per swizzle atom, atoms 1024 B apart.
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>(1) << 16;
    d |= static_cast<uint64_t>(1024u >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}

// kind::f16: D fp32, A and B bf16, both K-major, M = 128, N = n.
__device__ __forceinline__ uint32_t make_idesc(uint32_t n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((kTileM >> 4) << 24);
}

__device__ __forceinline__ void mma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                         uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, uint32_t limit) {
    for (uint32_t i = 0; i < limit; ++i) {
        uint32_t done;
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
            "selp.u32 %0, 1, 0, p;\n"
            "}\n"
            : "=r"(done)
            : "r"(bar), "r"(parity)
            : "memory");
        if (done) return true;
    }
    return false;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t x, uint32_t y,
                                            uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
        : "memory");
}

constexpr uint32_t kMaxGroup = 4;       // dictionaries that may share one launch (q|k|v, gate|up)

// Tensor maps of the dictionaries' bf16 planes, one pair per group member.
struct GroupMaps {
    CUtensorMap hi[kMaxGroup], lo[kMaxGroup];
};

struct Params {
    uint32_t n_seg;
    uint32_t tile_begin[kMaxGroup + 1];   // first atom tile (blockIdx.x) of each member
    float* dx_of[kMaxGroup];              // each member's Dx, [K_s][dx_stride]
    uint32_t M;             // tokens
    uint32_t dx_stride;     // floats between Dx rows (>= M); transposed: between token rows (>= atoms)
    uint32_t transposed;    // Dx leaves token-major, [token][atom], instead of [atom][token]
    uint32_t n_tile;        // MMA N: 16, 32, 64 or 128
    uint32_t tmem_cols;     // power of two >= max(32, n_tile)
    uint32_t n_kb;          // C / 64
    uint32_t kb_per_cta;
    uint32_t stages;
    uint32_t x_has_lo;
    float* part;            // [tile][rank][128][N] accumulator tiles of the column ranges
    // Tensor-parallel exchange (xch_ranks > 1): the finished rows of this rank's partial
    // projection go straight into every rank's slot for this rank instead of dx_of[]; see
    // struct Exchange. xch_off[i]: member i's offset inside a block; xch_sums: this rank's
    // per-token sums of squares to push along (block offset 0), or null.
    uint32_t xch_ranks, xch_rank, xch_blk;
    uint32_t xch_off[kMaxGroup];
    float* xch_slots[kMaxExchangeRanks];
    uint32_t* xch_flags[kMaxExchangeRanks];
    uint32_t* xch_seq;
    uint32_t* xch_done;
    const float* xch_sums;
    // Shares of per-token sums of squares left by the gather before this launch (NextNorm): one
    // CTA adds them up for the gather behind this launch. Null: none.
    const float* norm_partial;
    uint32_t norm_ctas;
    float* norm_sumsq;
    int* status;
    uint32_t spin;               // mbarrier try_wait rounds before a wait gives up
    unsigned long long* trace;   // optional: 16 global-timer stamps per CTA (phase boundaries)
    uint32_t trace_ctas;
};

// One thread of a role records when that role passed a phase boundary.
__device__ __forceinline__ void stamp(const Params& p, int slot) {
    if (p.trace) {
        const uint32_t cta = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
        if (cta < p.trace_ctas) {
            unsigned long long t;
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
            p.trace[cta * 16u + slot] = t;
        }
    }
}

// grid (atom tiles of every member, token tiles, column ranges); cluster (1, 1, column ranges)
__global__ void __launch_bounds__(kThreads, 1)
hsdr_dx_tma_kernel(const __grid_constant__ GroupMaps maps, const __grid_constant__ CUtensorMap map_xhi,
                   const __grid_constant__ CUtensorMap map_xlo, const __grid_constant__ Params p) {
    extern __shared__ __align__(1024) unsigned char tma_smem_raw[];
    // the gather behind this kernel may start its prologue (code prefetch) right away; it waits
    // for this grid's completion before it touches Dx
    asm volatile("griddepcontrol.launch_dependents;");
    __shared__ __align__(8) unsigned long long full_bar[kMaxStages];
    __shared__ __align__(8) unsigned long long empty_bar[kMaxStages];
    __shared__ __align__(8) unsigned long long accum_bar;
    __shared__ uint32_t tmem_base_s;
    __shared__ volatile int failed_s;
    cg::cluster_group cluster = cg::this_cluster();
    const uint32_t n_ranks = cluster.num_blocks();
    const uint32_t rank = cluster.block_rank();
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    unsigned char* smem = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(tma_smem_raw) + 1023u) & ~static_cast<uintptr_t>(1023));
    const uint32_t N = p.n_tile;
    const uint32_t b_tile = N * 128u;
    const uint32_t stage_bytes = 2u * kATile + (p.x_has_lo ? 2u : 1u) * b_tile;
    uint32_t seg = 0;
#pragma unroll
    for (uint32_t i = 1; i < kMaxGroup; ++i)
        if (i < p.n_seg && blockIdx.x >= p.tile_begin[i]) seg = i;
    const uint32_t atom0 = (blockIdx.x - p.tile_begin[seg]) * kTileM;
    float* const dx = p.dx_of[seg];
    const CUtensorMap* map_ahi = &maps.hi[seg];
    const CUtensorMap* map_alo = &maps.lo[seg];
    const uint32_t tok0 = blockIdx.y * N;
    const uint32_t kb_begin = min(p.n_kb, rank * p.kb_per_cta);
    const uint32_t kb_end = min(p.n_kb, kb_begin + p.kb_per_cta);
    const uint32_t n_it = kb_end - kb_begin;

    if (tid == 0) {
        stamp(p, 0);
        for (uint32_t i = 0; i < kMaxStages; ++i) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&full_bar[i])));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&empty_bar[i])));
        }
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&accum_bar)));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        failed_s = 0;
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)),
                     "r"(p.tmem_cols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_s;
    if (tid == 0) stamp(p, 1);
    if (warp == 0) {
        // ---- loader ----
        // The dictionary planes do not depend on earlier work on the stream: the first round of
        // stages gets its weight tiles before the dependency wait, the activation tiles after.
        if (lane == 0) {
            const uint32_t pre = min(p.stages, n_it);
            for (uint32_t it = 0; it < pre; ++it) {
                const uint32_t bar = smem_u32(&full_bar[it]);
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(stage_bytes)
                             : "memory");
                const uint32_t dst = smem_u32(smem + it * stage_bytes);
                const uint32_t c0 = (kb_begin + it) * kBlockK;
                tma_load_2d(dst, map_ahi, c0, atom0, bar);
                tma_load_2d(dst + kATile, map_alo, c0, atom0, bar);
            }
            asm volatile("griddepcontrol.wait;" ::: "memory");
            for (uint32_t it = 0; it < pre; ++it) {
                const uint32_t bar = smem_u32(&full_bar[it]);
                const uint32_t dst = smem_u32(smem + it * stage_bytes);
                const uint32_t c0 = (kb_begin + it) * kBlockK;
                tma_load_2d(dst + 2u * kATile, &map_xhi, c0, tok0, bar);
                if (p.x_has_lo) tma_load_2d(dst + 2u * kATile + b_tile, &map_xlo, c0, tok0, bar);
            }
            for (uint32_t it = pre; it < n_it; ++it) {
                const uint32_t s = it % p.stages, use = it / p.stages;
                if (!mbar_wait(smem_u32(&empty_bar[s]), (use - 1u) & 1u, p.spin)) {
                    failed_s = 1;
                    break;
                }
                if (failed_s) break;
                const uint32_t bar = smem_u32(&full_bar[s]);
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(stage_bytes)
                             : "memory");
                const uint32_t dst = smem_u32(smem + s * stage_bytes);
                const uint32_t c0 = (kb_begin + it) * kBlockK;
                tma_load_2d(dst, map_ahi, c0, atom0, bar);
                tma_load_2d(dst + kATile, map_alo, c0, atom0, bar);
                tma_load_2d(dst + 2u * kATile, &map_xhi, c0, tok0, bar);
                if (p.x_has_lo) tma_load_2d(dst + 2u * kATile + b_tile, &map_xlo, c0, tok0, bar);
            }
        }
    } else if (warp == 1) {
        // ---- MMA issue ----
        if (lane == 0) {
            const uint32_t idesc = make_idesc(N);
            for (uint32_t it = 0; it < n_it; ++it) {
                const uint32_t s = it % p.stages, use = it / p.stages;
                if (!mbar_wait(smem_u32(&full_bar[s]), use & 1u, p.spin)) {
                    failed_s = 1;
                    break;
                }
                if (failed_s) break;
                if (it == 0) stamp(p, 2);
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t a_hi = smem_u32(smem + s * stage_bytes), a_lo = a_hi + kATile;
                const uint32_t b_hi = a_hi + 2u * kATile, b_lo = b_hi + b_tile;
#pragma unroll
                for (uint32_t k = 0; k < kBlockK / 16u; ++k) {     // four K = 16 steps, 32 bytes apart
                    const uint64_t ah = make_desc(a_hi + k * 32u), al = make_desc(a_lo + k * 32u);
                    const uint64_t bh = make_desc(b_hi + k * 32u);
                    mma_bf16(tmem_base, ah, bh, idesc, (it | k) != 0u);
                    mma_bf16(tmem_base, al, bh, idesc, 1u);
                    if (p.x_has_lo) mma_bf16(tmem_base, ah, make_desc(b_lo + k * 32u), idesc, 1u);
                }
                // the stage is free again once every MMA issued so far has read it
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                                 smem_u32(&empty_bar[s]))
                             : "memory");
            }
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                             smem_u32(&accum_bar))
                         : "memory");
            stamp(p, 3);
        }
    }
    // ---- column-range reduction through L2. Every CTA writes its accumulator tile to the
    // launch's partial buffer, the cluster meets at its barrier (release/acquire at cluster scope
    // covers those global writes), and each CTA then sums its share of the tile's rows over the
    // ranks, in rank order, into Dx. (Remote shared memory was measured at ~20 GB/s per SM on
    // this part, several times slower than the same exchange through L2.) ----
    const uint32_t tile = blockIdx.y * gridDim.x + blockIdx.x;
    float* part = p.part + static_cast<size_t>(tile) * n_ranks * kTileM * N;
    const uint32_t pstride = N + 4u;
    float* ptile = reinterpret_cast<float*>(smem);
    bool done = true;
    if (p.norm_partial && warp >= 2 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) {
        // the four epilogue warps of one CTA have nothing to do until the accumulator is
        // complete: they add up the shares, 32 partial sums of every token in a fixed order of
        // CTAs, then those in order
        __shared__ float share_s[32][16];
        asm volatile("griddepcontrol.wait;" ::: "memory");
        const uint32_t t = tid - 64u, q = t & 3u, j = t >> 2;
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
        for (uint32_t c = j; c < p.norm_ctas; c += 32u) {
            const float4 v = __ldcg(reinterpret_cast<const float4*>(p.norm_partial + static_cast<size_t>(c) * 16u) + q);
            a.x += v.x;
            a.y += v.y;
            a.z += v.z;
            a.w += v.w;
        }
        *reinterpret_cast<float4*>(&share_s[j][q * 4u]) = a;
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (t < 16u && t < p.M) {
            float s = 0.0f;
            for (uint32_t i = 0; i < 32u; ++i) s += share_s[i][t];
            p.norm_sumsq[t] = s;
        }
    }
    if (warp >= 2) {
        done = __all_sync(0xFFFFFFFFu, mbar_wait(smem_u32(&accum_bar), 0u, p.spin));   // warp-uniform
        if (!done) failed_s = 1;
        if (tid == 64) stamp(p, 4);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t quad = warp & 3u;                  // TMEM lanes 32*quad .. +31
        const uint32_t row = quad * 32u + lane;
        // rows of the accumulator tile go to shared memory first (stage memory is free: this
        // CTA's MMAs are done and nobody else touches it), padded so that 128-bit row writes do
        // not collide; the copy to global memory below is then fully coalesced
        float* prow = ptile + static_cast<size_t>(row) * pstride;
        for (uint32_t ch = 0; ch < N / 16u; ++ch) {
            uint32_t r[16];
            if (done && n_it > 0u) {
                const uint32_t taddr = tmem_base + ((quad * 32u) << 16) + ch * 16u;
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
                    : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                      "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
                      "=r"(r[15])
                    : "r"(taddr)
                    : "memory");
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) r[j] = 0u;   // an empty column range adds nothing
            }
#pragma unroll
            for (int j = 0; j < 4; ++j)
                *reinterpret_cast<uint4*>(prow + ch * 16u + j * 4) = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    // exchange: the sequence number this launch will publish. Read here, behind the accumulator
    // wait (so behind the loader's dependency wait: every earlier launch, the previous
    // exchange's included, has completed), and before this CTA is counted out below (the
    // launch's last CTA advances the counter only after every CTA has been counted)
    const uint32_t xseq = p.xch_ranks > 1u ? *reinterpret_cast<volatile uint32_t*>(p.xch_seq) + 1u : 0u;
    const size_t xslot = (static_cast<size_t>(xseq & 1u) * p.xch_ranks + p.xch_rank) * p.xch_blk;
    // a finished piece of Dx: four tokens of one atom, to the local buffer or to every rank
    auto emit = [&](uint32_t atom, uint32_t tok, const float4& v, bool vec) {
        if (p.transposed) {   // local only: four tokens of one atom go to four token rows
            float* dst = dx + static_cast<size_t>(tok) * p.dx_stride + atom;
            dst[0] = v.x;
            if (tok + 1u < p.M) dst[p.dx_stride] = v.y;
            if (tok + 2u < p.M) dst[2u * static_cast<size_t>(p.dx_stride)] = v.z;
            if (tok + 3u < p.M) dst[3u * static_cast<size_t>(p.dx_stride)] = v.w;
            return;
        }
        const size_t o = static_cast<size_t>(atom) * p.dx_stride + tok;
        if (p.xch_ranks > 1u) {
            const size_t xo = xslot + p.xch_off[seg] + o;
#pragma unroll
            for (uint32_t r = 0; r < kMaxExchangeRanks; ++r) {
                if (r < p.xch_ranks) {
                    float* dst = p.xch_slots[r] + xo;
                    if (vec) *reinterpret_cast<float4*>(dst) = v;
                    else {
                        dst[0] = v.x;
                        if (tok + 1u < p.M) dst[1] = v.y;
                        if (tok + 2u < p.M) dst[2] = v.z;
                        if (tok + 3u < p.M) dst[3] = v.w;
                    }
                }
            }
        } else {
            float* dst = dx + o;
            if (vec) *reinterpret_cast<float4*>(dst) = v;
            else {
                dst[0] = v.x;
                if (tok + 1u < p.M) dst[1] = v.y;
                if (tok + 2u < p.M) dst[2] = v.z;
                if (tok + 3u < p.M) dst[3] = v.w;
            }
        }
    };

    {
        // one rank and an aligned token count: the tile is Dx itself; otherwise this rank's slab
        const bool direct = n_ranks == 1u && ((p.M | p.dx_stride) & 3u) == 0;
        const uint32_t n4 = N / 4u;
        if (direct && p.transposed) {
            // token-major out: four consecutive atoms of one token per store, so that a warp writes
            // whole lines of a token's row
            constexpr uint32_t r4n = kTileM / 4u;
            for (uint32_t i = tid; i < N * r4n; i += kThreads) {
                const uint32_t tc = i / r4n, r4 = i - tc * r4n;
                if (tok0 + tc < p.M) {
                    const float* src = ptile + static_cast<size_t>(r4 * 4u) * pstride + tc;
                    const float4 v = make_float4(src[0], src[pstride], src[2u * pstride], src[3u * pstride]);
                    *reinterpret_cast<float4*>(dx + static_cast<size_t>(tok0 + tc) * p.dx_stride + atom0 + r4 * 4u) = v;
                }
            }
        } else
        for (uint32_t i = tid; i < kTileM * n4; i += kThreads) {
            const uint32_t row = i / n4, c4 = i - row * n4;
            const float4 v = *reinterpret_cast<const float4*>(ptile + static_cast<size_t>(row) * pstride + c4 * 4u);
            if (direct) {
                if (tok0 + c4 * 4u < p.M) emit(atom0 + row, tok0 + c4 * 4u, v, true);
            } else {
                *reinterpret_cast<float4*>(part + (static_cast<size_t>(rank) * kTileM + row) * N + c4 * 4u) = v;
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (tid == 0 && failed_s) atomicExch(p.status, 1);    // a bounded wait ran out: the host reports it
    if (tid == 0) stamp(p, 5);
    cluster.sync();                                       // every rank's tile is in the partial buffer
    if (tid == 0) stamp(p, 6);
    if (!(n_ranks == 1u && ((p.M | p.dx_stride) & 3u) == 0)) {
        const uint32_t rows_each = (kTileM + n_ranks - 1u) / n_ranks;
        const uint32_t row_begin = min(kTileM, rank * rows_each);
        const uint32_t rows_mine = min(kTileM, row_begin + rows_each) - row_begin;
        const uint32_t n4 = N / 4u;
        const bool vec = ((p.M | p.dx_stride) & 3u) == 0;
        const float* tile_part = p.part + static_cast<size_t>(tile) * n_ranks * kTileM * N;
        // two items per pass, every rank's piece of both requested before the first add: the
        // loads are L2 round trips and must overlap
        for (uint32_t i0 = tid; i0 < rows_mine * n4; i0 += 2u * kThreads) {
            float4 v[2][16];
#pragma unroll
            for (uint32_t h = 0; h < 2u; ++h) {
                const uint32_t i = i0 + h * kThreads;
                if (i < rows_mine * n4) {
                    const uint32_t row = row_begin + i / n4, c4 = i % n4;
                    const float* src = tile_part + static_cast<size_t>(row) * N + c4 * 4u;
#pragma unroll
                    for (uint32_t r = 0; r < 16u; ++r)
                        if (r < n_ranks)
                            v[h][r] = __ldcg(reinterpret_cast<const float4*>(src + static_cast<size_t>(r) * kTileM * N));
                }
            }
#pragma unroll
            for (uint32_t h = 0; h < 2u; ++h) {
                const uint32_t i = i0 + h * kThreads;
                if (i >= rows_mine * n4) break;
                const uint32_t row = row_begin + i / n4, c4 = i % n4;
                float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (uint32_t r = 0; r < 16u; ++r)
                    if (r < n_ranks) {
                        acc.x += v[h][r].x;
                        acc.y += v[h][r].y;
                        acc.z += v[h][r].z;
                        acc.w += v[h][r].w;
                    }
                const uint32_t atom = atom0 + row, tok = tok0 + c4 * 4u;
                if (tok < p.M) emit(atom, tok, acc, vec);   // vec: tok and M are multiples of four
            }
        }
    }
    if (tid == 0) stamp(p, 7);
    if (p.xch_ranks > 1u) {
        // this rank's sums of squares ride along (one CTA pushes them), then the launch is
        // counted out: the last CTA raises this rank's flag in every rank's region
        if (p.xch_sums && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && tid < p.M) {
            const float v = __ldcg(p.xch_sums + tid);
            for (uint32_t r = 0; r < p.xch_ranks; ++r) p.xch_slots[r][xslot + tid] = v;
        }
        // one system-scope fence per CTA: the barrier orders every thread's peer stores before
        // thread 0's fence (fences are cumulative), and the fence before the count
        __syncthreads();
        if (tid == 0) {
            __threadfence_system();
            const uint32_t total = gridDim.x * gridDim.y * gridDim.z;
            if (atomicAdd(p.xch_done, 1u) == total - 1u) {
                *p.xch_done = 0u;
                __threadfence_system();
                for (uint32_t r = 0; r < p.xch_ranks; ++r)
                    *reinterpret_cast<volatile uint32_t*>(p.xch_flags[r] + (xseq & 1u) * p.xch_ranks + p.xch_rank) = xseq;
                *reinterpret_cast<volatile uint32_t*>(p.xch_seq) = xseq;
            }
        }
    }
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(p.tmem_cols) : "memory");
    }
}

// fp32 -> bf16 hi / lo planes, element order unchanged (the dictionary: [K][C]).
__global__ void split_planes_kernel(const float4* __restrict__ src, uint2* __restrict__ hi, uint2* __restrict__ lo,
                                    size_t n4) {
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n4;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const float4 v = src[i];
        const __nv_bfloat162 h01 = __floats2bfloat162_rn(v.x, v.y), h23 = __floats2bfloat162_rn(v.z, v.w);
        const __nv_bfloat162 l01 = __floats2bfloat162_rn(v.x - __low2float(h01), v.y - __high2float(h01));
        const __nv_bfloat162 l23 = __floats2bfloat162_rn(v.z - __low2float(h23), v.w - __high2float(h23));
        hi[i] = make_uint2(*reinterpret_cast<const uint32_t*>(&h01), *reinterpret_cast<const uint32_t*>(&h23));
        lo[i] = make_uint2(*reinterpret_cast<const uint32_t*>(&l01), *reinterpret_cast<const uint32_t*>(&l23));
    }
}

// Activations of any supported dtype/layout -> token-major bf16 planes [M][C].
__global__ void x_planes_kernel(XView xv, __nv_bfloat16* __restrict__ hi, __nv_bfloat16* __restrict__ lo) {
    const size_t n = static_cast<size_t>(xv.M) * xv.C;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const uint32_t b = static_cast<uint32_t>(i / xv.C), c = static_cast<uint32_t>(i - static_cast<size_t>(b) * xv.C);
        const float v = load_x(xv, c, b);
        const __nv_bfloat16 h = __float2bfloat16_rn(v);
        hi[i] = h;
        if (lo) lo[i] = __float2bfloat16_rn(v - __bfloat162float(h));
    }
}

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
    static EncodeFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q{};
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeFn>(p);
    }();
    return fn;
}

// bf16 matrix [rows][cols] row-major; box = 64 columns x box_rows rows, 128-byte swizzle.
// Rows past the end read as zero.
CUtensorMap make_map(const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
    CUtensorMap m{};
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {cols * 2u};
    const cuuint32_t box[2] = {kBlockK, box_rows};
    const cuuint32_t estr[2] = {1u, 1u};
    EncodeFn fn = encode_fn();
    if (!fn) throw Error(CSDR_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    const CUresult rc = fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) throw Error(CSDR_ERR_CUDA, "cuTensorMapEncodeTiled failed (" + std::to_string(rc) + ")");
    return m;
}

// bf16 planes of one dictionary, cached on the fp32 atom buffer.
struct Planes {
    DevPtr buf;           // hi plane then lo plane
    CUtensorMap map_hi, map_lo;
};

std::shared_ptr<Planes> planes_for(csdr_context* ctx, const csdr_segment* seg) {
    DeviceBuffer* atoms = seg->atoms.get();
    if (atoms->aux) return std::static_pointer_cast<Planes>(atoms->aux);
    const Geometry& g = seg->g;
    const size_t n = static_cast<size_t>(g.n_atoms) * g.cols;
    auto pl = std::make_shared<Planes>();
    pl->buf = std::make_shared<DeviceBuffer>(n * 4u, ctx->device);
    __nv_bfloat16* hi = static_cast<__nv_bfloat16*>(pl->buf->ptr);
    __nv_bfloat16* lo = hi + n;
    {
        LaunchScope ls(ctx, KC_DECODER_OP);
        split_planes_kernel<<<static_cast<unsigned>(std::min<size_t>((n / 4u + 255u) / 256u, 4096u)), 256, 0, ctx->stream>>>(
            static_cast<const float4*>(atoms->ptr), reinterpret_cast<uint2*>(hi), reinterpret_cast<uint2*>(lo), n / 4u);
        ls.done("split_planes_kernel");
    }
    pl->map_hi = make_map(hi, g.n_atoms, g.cols, kTileM);
    pl->map_lo = make_map(lo, g.n_atoms, g.cols, kTileM);
    atoms->aux = pl;
    return pl;
}

}  // namespace tma_detail

bool dx_tma_supported(const csdr_context* ctx, const csdr_segment* seg, size_t batch) {
    using namespace tma_detail;
    const Geometry& g = seg->g;
    (void)batch;
    // rows of the bf16 planes must be 16-byte multiples for the tensor maps; a last 64-column
    // block that sticks out past the row end reads as zero on both operands
    return ctx->tma && g.row_tiles() && g.n_atoms % kTileM == 0 && g.cols % 8u == 0 && encode_fn() != nullptr;
}

XPlanesView make_x_planes(csdr_context* ctx, const void* x, int x_dtype, int x_layout, uint32_t M, uint32_t cols) {
    using namespace tma_detail;
    // in place when the activations already are what the loader wants
    if (x_dtype == CSDR_DTYPE_BF16 && x_layout == CSDR_LAYOUT_TOKEN_MAJOR && (reinterpret_cast<uintptr_t>(x) & 15u) == 0 &&
        (cols & 7u) == 0)
        return XPlanesView{static_cast<const __nv_bfloat16*>(x), nullptr};
    const bool has_lo = x_dtype == CSDR_DTYPE_F32;
    const size_t n = static_cast<size_t>(M) * cols;
    __nv_bfloat16* buf = static_cast<__nv_bfloat16*>(ctx->scratch_get(5, n * (has_lo ? 4u : 2u)));
    XView xv{x, x_dtype, x_layout, cols, M, 0u, M};
    LaunchScope ls(ctx, KC_DECODER_OP);
    x_planes_kernel<<<static_cast<unsigned>(std::min<size_t>((n + 255u) / 256u, 2048u)), 256, 0, ctx->stream>>>(
        xv, buf, has_lo ? buf + n : nullptr);
    ls.done("x_planes_kernel");
    return XPlanesView{buf, has_lo ? buf + n : nullptr};
}

void launch_dx_tma_group(csdr_context* ctx, const csdr_segment* const* segs, uint32_t n_seg, XPlanesView x, uint32_t M,
                         float* const* dx, uint32_t dx_stride, const Exchange* xch, const float* blk_base,
                         const float* sums, bool transposed, const NormShares* shares) {
    using namespace tma_detail;
    if (transposed && ((xch && xch->ranks > 1u) || n_seg != 1u))
        throw Error(CSDR_ERR_INVALID_ARG, "a token-major projection is local and has one dictionary");
    if (n_seg == 0 || n_seg > kMaxGroup) throw Error(CSDR_ERR_LIMIT, "projection group holds 1 to 4 dictionaries");
    const uint32_t cols = segs[0]->g.cols;
    const bool has_lo = x.lo != nullptr;
    uint32_t N = 16;
    while (N < 128u && N < M) N <<= 1;
    const CUtensorMap map_xhi = make_map(x.hi, M, cols, N);
    const CUtensorMap map_xlo = has_lo ? make_map(x.lo, M, cols, N) : map_xhi;

    GroupMaps maps{};
    Params p{};
    p.n_seg = n_seg;
    uint32_t atom_tiles = 0;
    for (uint32_t i = 0; i < n_seg; ++i) {
        if (segs[i]->g.cols != cols) throw Error(CSDR_ERR_GEOMETRY, "projection group: members differ in columns");
        auto planes = planes_for(ctx, segs[i]);
        maps.hi[i] = planes->map_hi;
        maps.lo[i] = planes->map_lo;
        p.tile_begin[i] = atom_tiles;
        p.dx_of[i] = dx[i];
        atom_tiles += segs[i]->g.n_atoms / kTileM;
    }
    for (uint32_t i = n_seg; i <= kMaxGroup; ++i) p.tile_begin[i] = atom_tiles;

    const uint32_t tok_tiles = (M + N - 1u) / N;
    const uint32_t n_kb = (cols + kBlockK - 1u) / kBlockK;
    const uint32_t stage_bytes = 2u * kATile + (has_lo ? 2u : 1u) * N * 128u;

    const size_t smem_max = ctx->smem_optin - 4096u;   // static barriers, the shares block and alignment slack
    if (!ctx->tma_attrs_set) {
        ctx->opt_in_smem(reinterpret_cast<const void*>(hsdr_dx_tma_kernel), smem_max);
        if (cudaFuncSetAttribute(hsdr_dx_tma_kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess)
            ctx->tma_max_cluster = 16;
        else
            (void)cudaGetLastError();
        ctx->tma_attrs_set = true;
    }
    const int max_cluster = ctx->tma_max_cluster;
    uint32_t stages = std::min<uint32_t>(kMaxStages, static_cast<uint32_t>((smem_max - 1024u) / stage_bytes));
    // no more stages than column blocks: a short reduction (2-D tile products: two blocks) leaves
    // room for a second CTA on the SM, whose set-up then overlaps this one's epilogue
    stages = std::max(1u, std::min(stages, n_kb));
    const size_t smem = std::max<size_t>(static_cast<size_t>(stages) * stage_bytes,
                                         static_cast<size_t>(kTileM) * (N + 4u) * 4u) + 1024u;

    cudaLaunchConfig_t cfg{};
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = ctx->pdl ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 2;

    // Column ranges per tile = cluster size: the largest one for which every cluster of the
    // launch is resident at once (the hardware places a cluster inside one GPC, so the answer
    // depends on the cluster size; asked once per (size, shared memory) and remembered).
    const uint32_t tiles = atom_tiles * tok_tiles;
    std::unordered_map<uint64_t, int>& fit = ctx->cluster_fit;   // (ranks, smem) -> clusters resident at once
    uint32_t ranks = 1;
    for (uint32_t r = std::min<uint32_t>({static_cast<uint32_t>(max_cluster), n_kb,
                                          std::max(1u, static_cast<uint32_t>(ctx->sm_count) / tiles)});
         r > 1u; --r) {
        const uint64_t key = (static_cast<uint64_t>(r) << 32) | static_cast<uint64_t>(smem);
        auto itf = fit.find(key);
        if (itf == fit.end()) {
            cfg.gridDim = dim3(atom_tiles, tok_tiles, r);
            attr[0].val.clusterDim.z = r;
            int n_clusters = 0;
            if (cudaOccupancyMaxActiveClusters(&n_clusters, hsdr_dx_tma_kernel, &cfg) != cudaSuccess) {
                (void)cudaGetLastError();
                n_clusters = 0;
            }
            itf = fit.emplace(key, n_clusters).first;
        }
        if (itf->second >= static_cast<int>(tiles)) {
            ranks = r;
            break;
        }
    }
    cfg.gridDim = dim3(atom_tiles, tok_tiles, ranks);
    attr[0].val.clusterDim.z = ranks;

    p.M = M;
    p.dx_stride = dx_stride;
    p.transposed = transposed ? 1u : 0u;
    p.n_tile = N;
    p.tmem_cols = std::max(32u, N);
    p.n_kb = n_kb;
    p.kb_per_cta = (n_kb + ranks - 1u) / ranks;
    p.stages = stages;
    p.x_has_lo = has_lo ? 1u : 0u;
    p.part = ranks > 1u || ((M | dx_stride) & 3u) ? static_cast<float*>(ctx->scratch_get(
                                                         1, static_cast<size_t>(tiles) * ranks * kTileM * N * 4u))
                                                   : nullptr;
    p.status = ctx->status_word;
    p.spin = ctx->spin_limit_barrier;
    p.trace = ctx->gemv_trace ? static_cast<unsigned long long*>(ctx->gemv_trace->ptr) : nullptr;
    p.trace_ctas = static_cast<uint32_t>(ctx->sm_count) * 2u;
    if (xch && xch->ranks > 1u) {
        if (M > 16u) throw Error(CSDR_ERR_LIMIT, "the peer-memory exchange carries single token tiles (at most 16 tokens)");
        p.xch_ranks = xch->ranks;
        p.xch_rank = xch->rank;
        p.xch_blk = xch->blk_floats;
        for (uint32_t i = 0; i < n_seg; ++i) {
            p.xch_off[i] = static_cast<uint32_t>(dx[i] - blk_base);
            if (p.xch_off[i] + static_cast<size_t>(segs[i]->g.n_atoms) * dx_stride > xch->blk_floats)
                throw Error(CSDR_ERR_LIMIT, "projection group does not fit an exchange slot");
        }
        for (uint32_t r = 0; r < xch->ranks; ++r) {
            p.xch_slots[r] = xch->slots[r];
            p.xch_flags[r] = xch->flags[r];
        }
        p.xch_seq = xch->seq;
        p.xch_done = xch->done;
        p.xch_sums = sums;
    }

    if (shares && shares->ctas) {
        if (M > 16u || shares->ctas > kNextNormCtas)
            throw Error(CSDR_ERR_INVALID_ARG, "shares of sums of squares come from a gather over a single token tile");
        p.norm_partial = shares->partial;
        p.norm_ctas = shares->ctas;
        p.norm_sumsq = shares->sumsq;
    }
    LaunchScope ls(ctx, KC_GEMM);
    CSDR_CUDA(cudaLaunchKernelEx(&cfg, hsdr_dx_tma_kernel, maps, map_xhi, map_xlo, p));
    ls.done("hsdr_dx_tma_kernel");
}

void dx_tma_prepare(csdr_context* ctx, const csdr_segment* seg) { (void)tma_detail::planes_for(ctx, seg); }

void launch_dx_tma(csdr_context* ctx, const csdr_segment* seg, const MatmulArgs& a, float* dx, uint32_t dx_stride) {
    const uint32_t M = static_cast<uint32_t>(a.batch);
    const XPlanesView x = make_x_planes(ctx, a.x, a.x_dtype, a.x_layout, M, seg->g.cols);
    launch_dx_tma_group(ctx, &seg, 1, x, M, &dx, dx_stride, nullptr, nullptr, nullptr, false);
}

}  // namespace csdr
