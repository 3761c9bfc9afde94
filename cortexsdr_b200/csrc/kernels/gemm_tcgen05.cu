// Tensor-core path for wide token tiles (batched decode at M >= 16, prefill) of 1-D row-tile
// HSDR segments on sm_100a: the dictionary projection Dx = D * X^T runs on the 5th-generation
// tensor cores (tcgen05.mma, accumulators in tensor memory), the signed gather over Dx stays
// on the CUDA cores.
//
// Reference arithmetic: the Dx loop and the gather loop of matmulRowMajor
// (strategies/HierarchicalSDRStrategy.cpp:1304-1336), which the reference runs in fp32.
//
// Precision. The dictionary is fp32 in the archive and the tolerance is 1e-3 relative with
// fp32 accumulation; one bf16 (or tf32) rounding of D would sit right at that limit. So the
// weights are rebuilt in shared memory as TWO bf16 tiles, hi = bf16(d) and lo = bf16(d - hi),
// and likewise fp32 activations; the product is hi*hi + hi*lo + lo*hi on the tensor cores with
// fp32 accumulation in TMEM (error ~2^-16 per term). bf16 activations need only hi*hi + lo*hi.
//
// One CTA = one (128-atom tile, token tile of N <= 256, column range). Per 64-column block:
// all eight warps pull the fp32 block with 128-bit loads, split it, and write the bf16 tiles
// in the K-major 128-byte-swizzle layout the MMA's shared-memory descriptors name; a
// generic->async proxy fence and a CTA barrier later, one thread issues the MMAs and commits
// them to the stage's mbarrier; two stages, so the next block's loads overlap the MMAs. The
// epilogue reads TMEM with tcgen05.ld (warp w owns lanes 32*(w%4)..+31 = atoms) and writes
// Dx, or one column-split partial of it. Every wait on an mbarrier is bounded.
#include <cuda_bf16.h>

#include <algorithm>
#include <cstdlib>

#include "../internal.hpp"
#include "gemm_tcgen05.hpp"
#include "views.cuh"

namespace csdr {

namespace {

constexpr int kTcThreads = 256;
constexpr uint32_t kBlockK = 64;          // bf16 elements per row of a tile = 128 bytes = one swizzle span
constexpr uint32_t kTileM = 128;          // atoms per CTA = MMA M
constexpr uint32_t kATileBytes = kTileM * 128u;   // 16 KB

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// Shared-memory matrix descriptor, K-major operand, 128-byte swizzle: rows of 128 bytes, eight
// rows (1024 bytes) per swizzle atom, atoms stacked along M/N with a 1024-byte stride.
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);          // start address, 16-byte units
    d |= static_cast<uint64_t>(1) << 16;                             // leading byte offset (unused for swizzled K-major)
    d |= static_cast<uint64_t>(1024u >> 4) << 32;                    // stride byte offset: 8 rows * 128 B
    d |= static_cast<uint64_t>(1) << 46;                             // descriptor version for sm_100
    d |= static_cast<uint64_t>(2) << 61;                             // layout: 128-byte swizzle
    return d;
}

// Instruction descriptor, kind::f16: D fp32, A and B bf16, both K-major, M = 128, N = n.
__device__ __forceinline__ uint32_t make_idesc(uint32_t n) {
    uint32_t d = 0;
    d |= 1u << 4;              // D format: f32
    d |= 1u << 7;              // A format: bf16
    d |= 1u << 10;             // B format: bf16
    d |= (n >> 3) << 17;       // N / 8
    d |= (kTileM >> 4) << 24;  // M / 16
    return d;
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

// Bounded wait on an mbarrier phase; false when it ran out.
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

// byte offset of (row, 16-byte chunk) inside a K-major 128-byte-swizzle tile
__device__ __forceinline__ uint32_t swz(uint32_t row, uint32_t chunk) {
    return (row >> 3) * 1024u + (row & 7u) * 128u + ((chunk ^ (row & 7u)) << 4);
}

__device__ __forceinline__ void split4(const float4 v, uint2& hi, uint2& lo) {
    const __nv_bfloat16 h0 = __float2bfloat16_rn(v.x), h1 = __float2bfloat16_rn(v.y);
    const __nv_bfloat16 h2 = __float2bfloat16_rn(v.z), h3 = __float2bfloat16_rn(v.w);
    const __nv_bfloat16 l0 = __float2bfloat16_rn(v.x - __bfloat162float(h0));
    const __nv_bfloat16 l1 = __float2bfloat16_rn(v.y - __bfloat162float(h1));
    const __nv_bfloat16 l2 = __float2bfloat16_rn(v.z - __bfloat162float(h2));
    const __nv_bfloat16 l3 = __float2bfloat16_rn(v.w - __bfloat162float(h3));
    hi.x = static_cast<uint32_t>(__bfloat16_as_ushort(h0)) | (static_cast<uint32_t>(__bfloat16_as_ushort(h1)) << 16);
    hi.y = static_cast<uint32_t>(__bfloat16_as_ushort(h2)) | (static_cast<uint32_t>(__bfloat16_as_ushort(h3)) << 16);
    lo.x = static_cast<uint32_t>(__bfloat16_as_ushort(l0)) | (static_cast<uint32_t>(__bfloat16_as_ushort(l1)) << 16);
    lo.y = static_cast<uint32_t>(__bfloat16_as_ushort(l2)) | (static_cast<uint32_t>(__bfloat16_as_ushort(l3)) << 16);
}

struct TcParams {
    const float* D;       // [K][C]
    uint32_t K, C;
    XView x;              // tokens b0..b0+M of the activation matrix
    uint32_t n_tile;      // MMA N: 16, 32, 64, 128 or 256
    uint32_t tmem_cols;   // power of two >= max(32, n_tile)
    uint32_t kb_per_split;
    uint32_t n_kb;        // C / 64
    uint32_t n_split;
    float* out;           // [n_split][K][M] (n_split == 1: Dx itself)
    int* status;
    uint32_t spin;        // mbarrier try_wait rounds before a wait gives up
    int x_has_lo;         // 0 when the activations are bf16 already
};

// grid (K/128, token tiles, column splits)
__global__ void __launch_bounds__(kTcThreads)
hsdr_dx_tcgen05_kernel(const __grid_constant__ TcParams p) {
    extern __shared__ __align__(1024) unsigned char tc_smem_raw[];
    __shared__ __align__(8) unsigned long long mbar[3];   // stage 0, stage 1, final
    __shared__ uint32_t tmem_base_s;
    __shared__ int failed_s;
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    unsigned char* smem = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(tc_smem_raw) + 1023u) & ~static_cast<uintptr_t>(1023));
    const uint32_t N = p.n_tile;
    const uint32_t b_tile_bytes = N * 128u;
    const uint32_t stage_bytes = 2u * kATileBytes + 2u * b_tile_bytes;   // A_hi, A_lo, B_hi, B_lo
    const uint32_t atom0 = blockIdx.x * kTileM;
    const uint32_t tok0 = blockIdx.y * N;
    const uint32_t kb_begin = blockIdx.z * p.kb_per_split;
    const uint32_t kb_end = min(p.n_kb, kb_begin + p.kb_per_split);
    const uint32_t kSpin = p.spin;   // a fraction of a second of polling by default, then give up

    if (tid == 0) {
        for (int i = 0; i < 3; ++i)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&mbar[i])));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        failed_s = 0;
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)),
                     "r"(p.tmem_cols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_s;
    const uint32_t idesc = make_idesc(N);
    // x fast paths (whole launch): token-major rows that can be read 128 / 64 bits at a time
    const bool tm_f32 = p.x.dtype == CSDR_DTYPE_F32 && p.x.layout == CSDR_LAYOUT_TOKEN_MAJOR &&
                        ((reinterpret_cast<uintptr_t>(p.x.x) | (static_cast<uintptr_t>(p.x.C) * 4u)) & 15u) == 0;
    const bool tm_bf16 = p.x.dtype == CSDR_DTYPE_BF16 && p.x.layout == CSDR_LAYOUT_TOKEN_MAJOR &&
                         ((reinterpret_cast<uintptr_t>(p.x.x) | (static_cast<uintptr_t>(p.x.C) * 2u)) & 7u) == 0;
    // This thread's share of a weight block: 8 units of (row, four columns); requested one
    // block ahead so the HBM latency hides behind the previous block's conversion and MMAs.
    constexpr uint32_t kAUnits = kTileM * 16u / kTcThreads;   // 8
    float4 dreg[kAUnits];
    auto request_weights = [&](uint32_t kb) {
        const uint32_t c0 = kb * kBlockK;
#pragma unroll
        for (uint32_t i = 0; i < kAUnits; ++i) {
            const uint32_t u = tid + i * kTcThreads, r = u >> 4, c4 = u & 15u;
            dreg[i] = atom0 + r < p.K
                          ? ldg_stream_f4(reinterpret_cast<const float4*>(p.D + static_cast<size_t>(atom0 + r) * p.C + c0) + c4)
                          : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    };
    if (kb_begin < kb_end) request_weights(kb_begin);

    uint32_t it = 0;
    for (uint32_t kb = kb_begin; kb < kb_end; ++kb, ++it) {
        const uint32_t s = it & 1u;
        unsigned char* st = smem + s * stage_bytes;
        unsigned char* a_hi = st;
        unsigned char* a_lo = st + kATileBytes;
        unsigned char* b_hi = st + 2u * kATileBytes;
        unsigned char* b_lo = b_hi + b_tile_bytes;
        // the MMAs that read this stage two blocks ago must be done before it is overwritten
        if (it >= 2u && !mbar_wait(smem_u32(&mbar[s]), ((it >> 1) - 1u) & 1u, kSpin)) failed_s = 1;
        const uint32_t c0 = kb * kBlockK;
        // ---- weights: 128 atoms x 64 columns fp32 -> bf16 hi / lo tiles ----
#pragma unroll
        for (uint32_t i = 0; i < kAUnits; ++i) {
            const uint32_t u = tid + i * kTcThreads, r = u >> 4, c4 = u & 15u;
            uint2 hi, lo;
            split4(dreg[i], hi, lo);
            const uint32_t off = swz(r, c4 >> 1) + (c4 & 1u) * 8u;
            *reinterpret_cast<uint2*>(a_hi + off) = hi;
            *reinterpret_cast<uint2*>(a_lo + off) = lo;
        }
        if (kb + 1u < kb_end) request_weights(kb + 1u);
        // ---- activations: N tokens x 64 columns -> bf16 hi / lo tiles ----
        for (uint32_t u = tid; u < N * 16u; u += kTcThreads) {
            const uint32_t r = u >> 4, c4 = u & 15u;
            const uint32_t tok = tok0 + r;
            uint2 hi = make_uint2(0u, 0u), lo = make_uint2(0u, 0u);
            if (tok < p.x.M) {
                if (tm_f32) {
                    const float4 v = *(reinterpret_cast<const float4*>(static_cast<const float*>(p.x.x) +
                                                                       static_cast<size_t>(p.x.b0 + tok) * p.x.C + c0) + c4);
                    split4(v, hi, lo);
                } else if (tm_bf16) {
                    hi = *(reinterpret_cast<const uint2*>(static_cast<const __nv_bfloat16*>(p.x.x) +
                                                          static_cast<size_t>(p.x.b0 + tok) * p.x.C + c0) + c4);
                } else {
                    const float4 v = make_float4(load_x(p.x, c0 + c4 * 4u, tok), load_x(p.x, c0 + c4 * 4u + 1u, tok),
                                                 load_x(p.x, c0 + c4 * 4u + 2u, tok), load_x(p.x, c0 + c4 * 4u + 3u, tok));
                    split4(v, hi, lo);
                }
            }
            const uint32_t off = swz(r, c4 >> 1) + (c4 & 1u) * 8u;
            *reinterpret_cast<uint2*>(b_hi + off) = hi;
            if (p.x_has_lo) *reinterpret_cast<uint2*>(b_lo + off) = lo;
        }
        // generic-proxy writes -> visible to the tensor core's async proxy, then everyone is done
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        if (failed_s) break;   // a wait ran out somewhere in the CTA: stop issuing work
        if (tid == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t a_hi_addr = smem_u32(a_hi), a_lo_addr = smem_u32(a_lo);
            const uint32_t b_hi_addr = smem_u32(b_hi), b_lo_addr = smem_u32(b_lo);
#pragma unroll
            for (uint32_t k = 0; k < kBlockK / 16u; ++k) {          // four K = 16 steps, 32 bytes apart
                const uint64_t ah = make_desc(a_hi_addr + k * 32u), al = make_desc(a_lo_addr + k * 32u);
                const uint64_t bh = make_desc(b_hi_addr + k * 32u), bl = make_desc(b_lo_addr + k * 32u);
                mma_bf16(tmem_base, ah, bh, idesc, (it | k) != 0u);
                mma_bf16(tmem_base, al, bh, idesc, 1u);
                if (p.x_has_lo) mma_bf16(tmem_base, ah, bl, idesc, 1u);
            }
            // arrive on this stage's barrier when every MMA issued so far has finished
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                             smem_u32(&mbar[s]))
                         : "memory");
        }
    }
    // ---- all MMAs done? ----
    if (tid == 0) {
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                         smem_u32(&mbar[2]))
                     : "memory");
    }
    if (!mbar_wait(smem_u32(&mbar[2]), 0u, kSpin)) failed_s = 1;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    __syncthreads();
    const bool good = failed_s == 0 && it > 0u;

    // ---- epilogue: TMEM -> registers -> global. Warp w reads lanes 32*(w%4)..+31; warps 4-7
    // take the upper half of the token columns. ----
    if (good) {
        const uint32_t lane_grp = warp & 3u;
        const uint32_t atom = atom0 + lane_grp * 32u + lane;
        const uint32_t half = warp >> 2;
        const uint32_t chunks = N / 16u;                       // 16-column chunks
        const uint32_t ch_begin = half * ((chunks + 1u) / 2u);
        const uint32_t ch_end = half ? chunks : (chunks + 1u) / 2u;
        float* orow = p.out + (static_cast<size_t>(blockIdx.z) * p.K + atom) * p.x.M;
        for (uint32_t ch = ch_begin; ch < ch_end; ++ch) {
            uint32_t r[16];
            const uint32_t taddr = tmem_base + ((lane_grp * 32u) << 16) + ch * 16u;
            asm volatile(
                "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
                : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                  "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                : "r"(taddr)
                : "memory");
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (atom < p.K) {
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const uint32_t tok = tok0 + ch * 16u + j;
                    if (tok < p.x.M) orow[tok] = __uint_as_float(r[j]);
                }
            }
        }
    } else if (tid == 0 && failed_s) {
        atomicExch(p.status, 1);   // a bounded wait ran out: the host reports it
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(p.tmem_cols) : "memory");
    }
}

// Dx[i] = sum over column splits, in split order.
__global__ void dx_reduce_kernel(const float* __restrict__ part, uint32_t n, uint32_t n_split,
                                 float* __restrict__ dx) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float v = 0.0f;
    for (uint32_t s0 = 0; s0 < n_split; s0 += 8u) {
        float a[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) a[j] = s0 + j < n_split ? __ldcg(part + static_cast<size_t>(s0 + j) * n + i) : 0.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j) v += a[j];
    }
    dx[i] = v;
}

// Gather for wide token tiles. CTA = (a run of rows, one 64-token slice); the Dx slice [K][64]
// sits in shared memory. A half-warp owns one output row at a time: each lane carries four
// tokens, so one 128-bit shared-memory read per code serves the whole row and the two halves of
// a warp read two different atoms without a bank conflict. Rows are taken in blocks of eight
// whose codes are prefetched into registers one block ahead and parked in shared memory; the
// eight results stay in registers so that either output layout leaves in 16/32-byte pieces.
// Sums run in the order of the stream (stage-major, slot-minor).
constexpr uint32_t kWideTokens = 64;
constexpr uint32_t kWideThreads = 512;
constexpr uint32_t kWideHalfWarps = kWideThreads / 16u;
constexpr uint32_t kWideRows = 8;        // rows per block of a half-warp
constexpr uint32_t kWideMaxSlots = 64;   // S*k the code parking area is sized for
constexpr uint32_t kWideCodeWords = ((kWideRows * kWideMaxSlots + 2u) / 2u + 1u) & ~1u;   // per half-warp, u32; even: 64-bit code reads
constexpr uint32_t kWideWordsPerLane = (kWideCodeWords + 15u) / 16u;

inline size_t gather_wide_smem(uint32_t K) {
    return (static_cast<size_t>(K) * kWideTokens + kWideMaxSlots) * 4u +
           static_cast<size_t>(kWideHalfWarps) * kWideCodeWords * 4u;
}

__global__ void __launch_bounds__(kWideThreads, 1)
hsdr_gather_wide_kernel(const uint16_t* __restrict__ codes, uint32_t R, uint32_t S, uint32_t k,
                        const float* __restrict__ scales, const float* __restrict__ dx, uint32_t K,
                        uint32_t M /* tokens in dx rows */, uint32_t rows_per_cta, YView yv,
                        const float* residual /* laid out like y, added on the way out; may be y itself */,
                        TokenScale ts, int* status, uint32_t spin) {
    extern __shared__ __align__(16) float wsm[];
    asm volatile("griddepcontrol.launch_dependents;");
    __shared__ __align__(8) unsigned long long dx_bar;
    if (threadIdx.x == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&dx_bar)));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    float* dxs = wsm;                                           // [K][64]
    float* gs = wsm + static_cast<size_t>(K) * kWideTokens;     // stage scales, [<= 64]
    uint32_t* csm = reinterpret_cast<uint32_t*>(gs + kWideMaxSlots);   // [half-warp][kWideCodeWords]
    const uint32_t tid = threadIdx.x;
    const uint32_t hw = tid >> 4, l16 = tid & 15u;
    const uint32_t t0 = blockIdx.y * kWideTokens;
    const uint32_t tw = min(kWideTokens, M - t0);
    const uint32_t slots = S * k;
    const uint32_t row_lo = blockIdx.x * rows_per_cta;          // multiple of kWideRows
    const uint32_t row_hi = min(R, row_lo + rows_per_cta);
    const uint32_t n_blocks = row_lo < row_hi ? (row_hi - row_lo + kWideRows - 1u) / kWideRows : 0u;
    const uint32_t iters = (n_blocks + kWideHalfWarps - 1u) / kWideHalfWarps;

    // Codes of a block start on an even u16 offset from the stream's base (eight rows), so the
    // parity of the base decides whether 32-bit loads must start one code early.
    uint32_t nx[kWideWordsPerLane];
    auto fetch = [&](uint32_t blk) {
#pragma unroll
        for (uint32_t i = 0; i < kWideWordsPerLane; ++i) nx[i] = 0u;
        if (blk >= n_blocks) return;
        const uint32_t r0 = row_lo + blk * kWideRows;
        const uint16_t* bp = codes + static_cast<size_t>(r0) * slots;
        const uint32_t off = static_cast<uint32_t>(reinterpret_cast<uintptr_t>(bp) >> 1) & 1u;
        const uint32_t* wp = reinterpret_cast<const uint32_t*>(bp - off);
        const uint32_t nwords = (min(kWideRows, row_hi - r0) * slots + off + 1u) / 2u;
#pragma unroll
        for (uint32_t i = 0; i < kWideWordsPerLane; ++i)
            if (i * 16u + l16 < nwords) nx[i] = __ldg(wp + i * 16u + l16);
    };
    fetch(hw);

    if (tid < kWideMaxSlots) gs[tid] = tid < S ? scales[tid] : 0.0f;
    // Dx is the output of the kernel before this one on the stream
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // stage the Dx slice (zero beyond the last token): asynchronous 16-byte copies, all of a
    // thread's requests in flight at once
    const bool bulk = (M & 3u) == 0 && (reinterpret_cast<uintptr_t>(dx) & 15u) == 0;
    if (bulk) {
        // bulk copies completing on the barrier: the whole slice at once when it is the whole of Dx
        // (64 tokens in all), else one copy per atom row; tokens past the end are zeroed by hand
        if (tid == 0)
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(&dx_bar)), "r"(K * tw * 4u)
                         : "memory");
        if (M == kWideTokens) {
            if (tid == 0)
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                                 smem_u32(dxs)),
                             "l"(dx), "r"(K * kWideTokens * 4u), "r"(smem_u32(&dx_bar))
                             : "memory");
        } else {
            for (uint32_t a = tid; a < K; a += kWideThreads) {
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                                 smem_u32(dxs + static_cast<size_t>(a) * kWideTokens)),
                             "l"(dx + static_cast<size_t>(a) * M + t0), "r"(tw * 4u), "r"(smem_u32(&dx_bar))
                             : "memory");
            }
            if (tw < kWideTokens)
                for (uint32_t i = tid; i < K * (kWideTokens - tw); i += kWideThreads) {
                    const uint32_t a = i / (kWideTokens - tw), t = tw + i - a * (kWideTokens - tw);
                    dxs[static_cast<size_t>(a) * kWideTokens + t] = 0.0f;
                }
        }
    } else {
        for (uint32_t i = tid; i < K * kWideTokens; i += kWideThreads) {
            const uint32_t a = i / kWideTokens, t = i - a * kWideTokens;
            dxs[i] = t < tw ? __ldcg(dx + static_cast<size_t>(a) * M + t0 + t) : 0.0f;
        }
    }
    __syncthreads();
    {
        // the whole CTA goes on or gives up together (a wait that ran out: the host reads the
        // status word, nothing is gathered)
        const bool landed = !bulk || mbar_wait(smem_u32(&dx_bar), 0u, spin);
        if (!__syncthreads_and(landed)) {
            if (tid == 0) atomicExch(status, 1);
            return;
        }
    }

    const float4* dxs4 = reinterpret_cast<const float4*>(dxs) + l16;
    uint32_t* my_csm = csm + hw * kWideCodeWords;
    const bool y_vec = (reinterpret_cast<uintptr_t>(yv.y) & 15u) == 0;
    for (uint32_t it = 0; it < iters; ++it) {
        const uint32_t blk = hw + it * kWideHalfWarps;
        __syncwarp();                       // the previous block's code reads are over
#pragma unroll
        for (uint32_t i = 0; i < kWideWordsPerLane; ++i)
            if (i * 16u + l16 < kWideCodeWords) my_csm[i * 16u + l16] = nx[i];
        __syncwarp();
        fetch(blk + kWideHalfWarps);
        if (blk >= n_blocks) continue;
        const uint32_t r0 = row_lo + blk * kWideRows;
        const uint32_t nrows = min(kWideRows, row_hi - r0);
        const uint32_t off =
            static_cast<uint32_t>(reinterpret_cast<uintptr_t>(codes + static_cast<size_t>(r0) * slots) >> 1) & 1u;
        const uint16_t* crow = reinterpret_cast<const uint16_t*>(my_csm) + off;
        // All eight rows of the block advance together: their lookups are independent, which
        // keeps enough shared-memory reads in flight per warp, and the accumulators are the
        // block's results. Rows past the end of the run read codes that are real (an earlier
        // block's) or zero, so their lookups stay inside the slice; their results are never
        // stored. Codes come four slots at a time (one 64-bit read per row) when the stream's
        // layout allows it.
        float out[kWideRows][4];
#pragma unroll
        for (uint32_t i = 0; i < kWideRows; ++i) out[i][0] = out[i][1] = out[i][2] = out[i][3] = 0.0f;
        auto step = [&](uint32_t i, uint32_t code, uint32_t gbits) {
            const float4 v = dxs4[(code & 0x7FFFu) * (kWideTokens / 4u)];
            const float scale = __uint_as_float(gbits ^ ((code & 0x8000u) << 16));
            out[i][0] = fmaf(scale, v.x, out[i][0]);
            out[i][1] = fmaf(scale, v.y, out[i][1]);
            out[i][2] = fmaf(scale, v.z, out[i][2]);
            out[i][3] = fmaf(scale, v.w, out[i][3]);
        };
        if (off == 0u && (k & 3u) == 0u) {
            for (uint32_t st = 0; st < S; ++st) {
                const uint32_t gbits = __float_as_uint(gs[st]);
                for (uint32_t j0 = 0; j0 < k; j0 += 4u) {
                    uint2 c4[kWideRows];     // rows are slots*2 bytes apart, slots a multiple of four here
#pragma unroll
                    for (uint32_t i = 0; i < kWideRows; ++i)
                        c4[i] = *reinterpret_cast<const uint2*>(crow + i * slots + st * k + j0);
#pragma unroll
                    for (uint32_t i = 0; i < kWideRows; ++i) step(i, c4[i].x & 0xFFFFu, gbits);
#pragma unroll
                    for (uint32_t i = 0; i < kWideRows; ++i) step(i, c4[i].x >> 16, gbits);
#pragma unroll
                    for (uint32_t i = 0; i < kWideRows; ++i) step(i, c4[i].y & 0xFFFFu, gbits);
#pragma unroll
                    for (uint32_t i = 0; i < kWideRows; ++i) step(i, c4[i].y >> 16, gbits);
                }
            }
        } else {
            for (uint32_t st = 0; st < S; ++st) {
                const uint32_t gbits = __float_as_uint(gs[st]);
                for (uint32_t j = 0; j < k; ++j) {
                    uint32_t code[kWideRows];
#pragma unroll
                    for (uint32_t i = 0; i < kWideRows; ++i) code[i] = crow[i * slots + st * k + j];
#pragma unroll
                    for (uint32_t i = 0; i < kWideRows; ++i) step(i, code[i], gbits);
                }
            }
        }
        const uint32_t tl = 4u * l16;               // first token of this lane inside the slice
        if (tl >= tw) continue;
        if (ts.sumsq) {
            // RMS normalisation folded behind the product: y = (W (w*h)) / rms(h), per token
#pragma unroll
            for (uint32_t j = 0; j < 4; ++j) {
                const float inv = tl + j < tw ? rsqrtf(ts.sumsq[t0 + tl + j] * ts.inv_width + ts.eps) : 0.0f;
#pragma unroll
                for (uint32_t rb = 0; rb < kWideRows; ++rb) out[rb][j] *= inv;
            }
        }
        if (yv.bias) {
#pragma unroll
            for (uint32_t rb = 0; rb < kWideRows; ++rb) {
                const float bias = rb < nrows ? yv.bias[r0 + rb] : 0.0f;
#pragma unroll
                for (uint32_t j = 0; j < 4; ++j) out[rb][j] += bias;
            }
        }
        if (yv.layout == CSDR_LAYOUT_FEATURE_MAJOR) {
            // y[r][token]: a row's 64 tokens are contiguous
            const size_t col = static_cast<size_t>(yv.b0) + t0 + tl;
            const bool vec = y_vec && (yv.Mtotal & 3u) == 0 && (col & 3u) == 0 && tl + 3u < tw;
#pragma unroll
            for (uint32_t rb = 0; rb < kWideRows; ++rb) {
                if (rb >= nrows) break;
                const size_t o = static_cast<size_t>(r0 + rb) * yv.Mtotal + col;
                float* dst = yv.y + o;
                if (residual) {
#pragma unroll
                    for (uint32_t j = 0; j < 4; ++j)
                        if (tl + j < tw) out[rb][j] += residual[o + j];
                }
                if (vec) *reinterpret_cast<float4*>(dst) = make_float4(out[rb][0], out[rb][1], out[rb][2], out[rb][3]);
                else {
#pragma unroll
                    for (uint32_t j = 0; j < 4; ++j)
                        if (tl + j < tw) dst[j] = out[rb][j];
                }
            }
        } else {
            // y[token][r]: eight consecutive rows of one token are contiguous
            const bool vec = y_vec && (yv.R & 3u) == 0 && nrows == kWideRows;
#pragma unroll
            for (uint32_t j = 0; j < 4; ++j) {
                if (tl + j >= tw) break;
                const size_t o = (static_cast<size_t>(yv.b0) + t0 + tl + j) * yv.R + r0;
                float* dst = yv.y + o;
                if (residual) {
#pragma unroll
                    for (uint32_t rb = 0; rb < kWideRows; ++rb)
                        if (rb < nrows) out[rb][j] += residual[o + rb];
                }
                if (vec) {
                    reinterpret_cast<float4*>(dst)[0] = make_float4(out[0][j], out[1][j], out[2][j], out[3][j]);
                    reinterpret_cast<float4*>(dst)[1] = make_float4(out[4][j], out[5][j], out[6][j], out[7][j]);
                } else {
#pragma unroll
                    for (uint32_t rb = 0; rb < kWideRows; ++rb)
                        if (rb < nrows) dst[rb] = out[rb][j];
                }
            }
        }
    }
}

// Compact gather for one token tile (M <= 16) over a group of segments that were projected
// together: CTA -> (member, run of rows). Same arithmetic as hsdr_gather_kernel (matmul.cu): the
// member's Dx [K][MT] and the CTA's code rows sit in shared memory, thread = (row, token), sums in
// stream order with one multiply and one add per code. Codes and scales are fetched before the
// dependency wait; Dx only after it.
constexpr uint32_t kGroupThreads = 256;
constexpr uint32_t kGatherGroupMax = 4;

struct GatherMember {
    const uint16_t* codes;
    const float* scales;
    const float* dx;        // [K][MT]
    float* y;
    const float* bias;
    const float* residual;
    uint32_t R, S, k, K;
    uint32_t cta_begin, rows_per_cta;
};

struct GatherGroupParams {
    GatherMember m[kGatherGroupMax];
    uint32_t n_seg, M, m_total, code_cap16;
    uint32_t region_bytes;    // shared memory of one member: codes | scales | Dx
    int y_layout;
    TokenScale ts;
    __nv_bfloat16* act_hi;    // SwiGLU pair: planes of silu(member 0) * member 1, laid out like y
    __nv_bfloat16* act_lo;
    NextNorm next;            // NORM instances only
    unsigned long long* trace;   // optional: global-timer stamps in slots 8..11 of a CTA's 16
    uint32_t trace_ctas;
    int* status;                 // context status word: a wait that ran out is recorded here
    uint32_t spin;               // mbarrier try_wait rounds before the wait for Dx gives up
};

__device__ __forceinline__ void gather_stamp(const GatherGroupParams& g, int slot) {
    if (g.trace && blockIdx.x < g.trace_ctas) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
        g.trace[blockIdx.x * 16u + slot] = t;
    }
}



__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Tensor-parallel exchange, receiving side: waits (bounded) until every rank's flag of the
// current parity shows the sequence number the projection kernel before this launch published,
// then adds the ranks' slots up in rank order into the local projection block. A launch of its
// own, so that the slots cross L2 once: summing them in every gather CTA's staging loop read
// ranks x 32 KB per CTA, 64 MB per exchange at 8 ranks.
struct ReduceParams {
    const float* slots;       // this rank's slot area, [2][ranks][blk_floats]
    const uint32_t* flags;    // this rank's flag words, [2][ranks]
    const uint32_t* seq;
    uint32_t ranks, blk_floats, off_floats, count4;
    float* dst;               // local block, at off_floats
    int* status;
    uint32_t spin;            // polls of a flag word before giving up (a few seconds by default)
};

__global__ void __launch_bounds__(256) exchange_reduce_kernel(const __grid_constant__ ReduceParams p) {
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    __shared__ int late_s;
    const uint32_t tid = threadIdx.x;
    const uint32_t seq = *reinterpret_cast<const volatile uint32_t*>(p.seq);   // set by the projection before this launch
    const uint32_t par = seq & 1u;
    if (tid == 0) late_s = 0;
    __syncthreads();
    if (tid < p.ranks) {
        const uint32_t* f = p.flags + par * p.ranks + tid;
        // once a wait has run out on this context nothing after it waits again: the step is lost
        // anyway, and the host must get its error quickly
        const bool already_failed = *reinterpret_cast<const volatile int*>(p.status) != 0;
        uint32_t spins = 0;
        while (ld_acquire_sys(f) != seq) {
            if (already_failed || ++spins > p.spin) {
                late_s = 1;
                break;
            }
        }
    }
    __syncthreads();
    if (tid == 0 && late_s && blockIdx.x == 0) atomicExch(p.status, 1);   // gave up: the host will see it
    const float* slot0 = p.slots + static_cast<size_t>(par) * p.ranks * p.blk_floats + p.off_floats;
    float4* dst = reinterpret_cast<float4*>(p.dst);
    for (uint32_t i = blockIdx.x * blockDim.x + tid; i < p.count4; i += gridDim.x * blockDim.x) {
        float4 v[kMaxExchangeRanks];               // all ranks' pieces in flight, then the adds
#pragma unroll
        for (uint32_t r = 0; r < kMaxExchangeRanks; ++r)
            if (r < p.ranks) v[r] = __ldcg(reinterpret_cast<const float4*>(slot0 + static_cast<size_t>(r) * p.blk_floats) + i);
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (uint32_t r = 0; r < kMaxExchangeRanks; ++r)   // rank order: every rank gets the same sum
            if (r < p.ranks) {
                acc.x += v[r].x;
                acc.y += v[r].y;
                acc.z += v[r].z;
                acc.w += v[r].w;
            }
        dst[i] = acc;
    }
}

// PAIR: the group is (gate, up) of a SwiGLU block with equal row counts; a CTA gathers the same
// rows of both and writes silu(gate) * up as bf16 planes (silu_mul, api/cortex_sdk.cpp:1245-1256,
// folded in), so the two fp32 intermediates never exist.
// NORM (one member, token-major y): the first half of the next RMS normalisation rides along,
// see NextNorm.
template <int MT, bool PAIR, bool NORM>
__global__ void __launch_bounds__(kGroupThreads)
hsdr_gather_group_kernel(const __grid_constant__ GatherGroupParams g) {
    static_assert(!(PAIR && NORM), "the SwiGLU pair has no next norm");
    extern __shared__ __align__(16) unsigned char ggsm[];
    asm volatile("griddepcontrol.launch_dependents;");
    __shared__ __align__(8) unsigned long long dx_bar;
    if (threadIdx.x == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&dx_bar)));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    constexpr uint32_t NM = PAIR ? 2u : 1u;      // members this CTA works on
    uint32_t mi0 = 0;
    if (!PAIR) {
#pragma unroll
        for (uint32_t i = 1; i < kGatherGroupMax; ++i)
            if (i < g.n_seg && blockIdx.x >= g.m[i].cta_begin) mi0 = i;
    }
    const GatherMember& m0 = g.m[mi0];
    const uint32_t tid = threadIdx.x;
    if (tid == 0) gather_stamp(g, 8);
    const uint32_t row0 = (blockIdx.x - m0.cta_begin) * m0.rows_per_cta;
    const bool active = row0 < m0.R;
    const uint32_t rows_here = active ? min(m0.rows_per_cta, m0.R - row0) : 0u;

    // per member: codes (16-byte units) | scales | Dx
    const uint32_t region = g.region_bytes;
    uint32_t skip[NM];
#pragma unroll
    for (uint32_t q = 0; q < NM; ++q) {
        const GatherMember& m = g.m[mi0 + q];
        const uint32_t slots = m.S * m.k;
        const size_t code_byte0 = static_cast<size_t>(row0) * slots * 2u;
        const size_t aligned0 = code_byte0 & ~static_cast<size_t>(15);
        skip[q] = static_cast<uint32_t>(code_byte0 - aligned0) >> 1;
        const uint32_t n16 = active ? (skip[q] * 2u + rows_here * slots * 2u + 15u) >> 4 : 0u;
        uint4* cs16 = reinterpret_cast<uint4*>(ggsm + q * region);
        float* sc = reinterpret_cast<float*>(ggsm + q * region + static_cast<size_t>(g.code_cap16) * 16u);
        const unsigned char* src = reinterpret_cast<const unsigned char*>(m.codes) + aligned0;
        for (uint32_t i = tid; i < n16; i += kGroupThreads)
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(
                             static_cast<uint32_t>(__cvta_generic_to_shared(cs16 + i))),
                         "l"(src + static_cast<size_t>(i) * 16u)
                         : "memory");
        for (uint32_t i = tid; i < m.S; i += kGroupThreads) sc[i] = m.scales[i];
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (tid == 0) gather_stamp(g, 9);
    __shared__ float inv_rms_s[16];
    // Dx of the member(s): one bulk copy each, completing on the barrier, where the block is whole
    // 16-byte units on a 16-byte boundary (always, for dictionaries of the tensor-core path);
    // 16-byte asynchronous copies by every thread otherwise
    bool bulk = active;
#pragma unroll
    for (uint32_t q = 0; q < NM; ++q) {
        const GatherMember& m = g.m[mi0 + q];
        bulk = bulk && ((m.K * MT) & 3u) == 0u && (reinterpret_cast<uintptr_t>(m.dx) & 15u) == 0u;
    }
    if (active && bulk) {
        if (tid == 0) {
            uint32_t total = 0;
#pragma unroll
            for (uint32_t q = 0; q < NM; ++q) total += g.m[mi0 + q].K * MT * 4u;
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(&dx_bar)), "r"(total) : "memory");
#pragma unroll
            for (uint32_t q = 0; q < NM; ++q) {
                const GatherMember& m = g.m[mi0 + q];
                float* dxs = reinterpret_cast<float*>(ggsm + q * region + static_cast<size_t>(g.code_cap16) * 16u) + 64;
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                                 smem_u32(dxs)),
                             "l"(m.dx), "r"(m.K * MT * 4u), "r"(smem_u32(&dx_bar))
                             : "memory");
            }
        }
    } else if (active) {
#pragma unroll
        for (uint32_t q = 0; q < NM; ++q) {
            const GatherMember& m = g.m[mi0 + q];
            float* dxs = reinterpret_cast<float*>(ggsm + q * region + static_cast<size_t>(g.code_cap16) * 16u) + 64;
            const uint32_t n4 = (m.K * MT) >> 2;
            for (uint32_t i = tid; i < n4; i += kGroupThreads)
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(
                                 static_cast<uint32_t>(__cvta_generic_to_shared(dxs + i * 4u))),
                             "l"(m.dx + static_cast<size_t>(i) * 4u)
                             : "memory");
            for (uint32_t i = (n4 << 2) + tid; i < m.K * MT; i += kGroupThreads) dxs[i] = m.dx[i];
        }
    }
    if (g.ts.sumsq && tid < MT) inv_rms_s[tid] = rsqrtf(g.ts.sumsq[tid < g.M ? tid : 0] * g.ts.inv_width + g.ts.eps);
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    {
        // the whole CTA goes on or gives up together (a wait that ran out: the host reads the
        // status word, nothing is gathered)
        const bool landed = !(active && bulk) || mbar_wait(smem_u32(&dx_bar), 0u, g.spin);
        if (!__syncthreads_and(landed)) {
            if (tid == 0) atomicExch(g.status, 1);
            return;
        }
    }
    if (tid == 0) gather_stamp(g, 10);
    if (!NORM && !active) return;
    // A thread gathers one row for TV tokens (four from a 4-token tile up: one 128-bit read of
    // Dx serves four sums, and a row's codes, read eight to a 128-bit word where the row starts
    // on a 16-byte boundary, are shared by fewer threads); TQ threads side by side cover a row.
    constexpr uint32_t TV = MT >= 4 ? 4u : static_cast<uint32_t>(MT);
    constexpr uint32_t TQ = MT / TV;
    constexpr uint32_t RP = kGroupThreads / TQ;
    const uint32_t b0 = (tid % TQ) * TV;
    float ss[TV];       // NORM: this thread's shares of its tokens' sums of squares
#pragma unroll
    for (uint32_t j = 0; j < TV; ++j) ss[j] = 0.0f;
    for (uint32_t rl = tid / TQ; rl < rows_here; rl += RP) {
        float res[NM][TV];
        // what the epilogue adds and multiplies comes from global memory and does not depend on
        // the sums: requested here, it arrives while the codes are walked
        float resid[TV], wnext = 0.0f;
        if (!PAIR) {
#pragma unroll
            for (uint32_t j = 0; j < TV; ++j) {
                const uint32_t b = b0 + j, r = row0 + rl;
                const size_t o = g.y_layout == CSDR_LAYOUT_FEATURE_MAJOR ? static_cast<size_t>(r) * g.m_total + b
                                                                          : static_cast<size_t>(b) * m0.R + r;
                resid[j] = (m0.residual && b < g.M) ? m0.residual[o] : 0.0f;
            }
            if (NORM) wnext = g.next.w[row0 + rl];
        }
#pragma unroll
        for (uint32_t q = 0; q < NM; ++q) {
            const GatherMember& m = g.m[mi0 + q];
            const unsigned char* base = ggsm + q * region;
            const uint16_t* cs = reinterpret_cast<const uint16_t*>(base) + skip[q];
            const float* sc = reinterpret_cast<const float*>(base + static_cast<size_t>(g.code_cap16) * 16u);
            const float* dxs = sc + 64;
            const uint16_t* rc = cs + rl * (m.S * m.k);
            float acc[TV];
#pragma unroll
            for (uint32_t j = 0; j < TV; ++j) acc[j] = 0.0f;
            auto add = [&](uint32_t code, float gamma) {
                const float scale = (code & 0x8000u) ? -gamma : gamma;
                const float* dp = dxs + (code & 0x7FFFu) * MT + b0;
                if constexpr (TV == 4u) {
                    const float4 d = *reinterpret_cast<const float4*>(dp);
                    acc[0] = __fadd_rn(acc[0], __fmul_rn(scale, d.x));
                    acc[1] = __fadd_rn(acc[1], __fmul_rn(scale, d.y));
                    acc[2] = __fadd_rn(acc[2], __fmul_rn(scale, d.z));
                    acc[3] = __fadd_rn(acc[3], __fmul_rn(scale, d.w));
                } else {
#pragma unroll
                    for (uint32_t j = 0; j < TV; ++j) acc[j] = __fadd_rn(acc[j], __fmul_rn(scale, dp[j]));
                }
            };
            if (((m.k & 7u) | skip[q]) == 0u) {      // rows of whole 16-byte words, the first one aligned
                for (uint32_t l = 0; l < m.S; ++l) {
                    const float gamma = sc[l];
                    for (uint32_t k8 = 0; k8 < m.k; k8 += 8u) {
                        const uint4 c = *reinterpret_cast<const uint4*>(rc + l * m.k + k8);
                        add(c.x & 0xFFFFu, gamma);
                        add(c.x >> 16, gamma);
                        add(c.y & 0xFFFFu, gamma);
                        add(c.y >> 16, gamma);
                        add(c.z & 0xFFFFu, gamma);
                        add(c.z >> 16, gamma);
                        add(c.w & 0xFFFFu, gamma);
                        add(c.w >> 16, gamma);
                    }
                }
            } else {
                for (uint32_t l = 0; l < m.S; ++l) {
                    const float gamma = sc[l];
#pragma unroll 4
                    for (uint32_t kk = 0; kk < m.k; ++kk) add(rc[l * m.k + kk], gamma);
                }
            }
#pragma unroll
            for (uint32_t j = 0; j < TV; ++j) {
                if (g.ts.sumsq) acc[j] *= inv_rms_s[b0 + j];
                if (m.bias) acc[j] += m.bias[row0 + rl];
                res[q][j] = acc[j];
            }
        }
        const uint32_t r = row0 + rl;
#pragma unroll
        for (uint32_t j = 0; j < TV; ++j) {
            const uint32_t b = b0 + j;
            if (b >= g.M) continue;
            const size_t o = g.y_layout == CSDR_LAYOUT_FEATURE_MAJOR ? static_cast<size_t>(r) * g.m_total + b
                                                                      : static_cast<size_t>(b) * m0.R + r;
            if (PAIR) {
                const float x = res[0][j];
                const float sig = 1.0f / (1.0f + expf(-x));
                const float v = (x * sig) * res[NM - 1][j];
                const __nv_bfloat16 h = __float2bfloat16_rn(v);
                g.act_hi[o] = h;
                g.act_lo[o] = __float2bfloat16_rn(v - __bfloat162float(h));
            } else {
                float acc = res[0][j];
                if (m0.residual) acc += resid[j];
                m0.y[o] = acc;
                if (NORM) {
                    ss[j] = fmaf(acc, acc, ss[j]);
                    const float p = acc * wnext;
                    const __nv_bfloat16 h = __float2bfloat16_rn(p);
                    g.next.hi[o] = h;
                    g.next.lo[o] = __float2bfloat16_rn(p - __bfloat162float(h));
                }
            }
        }
    }
    if (tid == 0) gather_stamp(g, 11);
    if (NORM) {
        __shared__ float red_s[RP * MT];       // index = row lane * MT + token
#pragma unroll
        for (uint32_t j = 0; j < TV; ++j) red_s[(tid / TQ) * MT + b0 + j] = ss[j];
        __syncthreads();
        if (tid < 16u) {
            float t = 0.0f;
            if (tid < MT)
                for (uint32_t j = 0; j < RP; ++j) t += red_s[j * MT + tid];
            g.next.partial[blockIdx.x * 16u + tid] = t;
        }
    }
}

template <int MT>
uint32_t launch_gather_group_t(csdr_context* ctx, GatherGroupParams& g, uint32_t total_rows, uint32_t max_k, uint32_t max_slots) {
    const bool pair = g.act_hi != nullptr, norm = g.next.w != nullptr;
    // CTAs over the whole group (a pair walks the rows of one member), two per SM: the rows of a
    // CTA still fit one pass of its threads at 16 tokens, and an SM takes
    // in two copies of Dx instead of three (1, 2 and 3 per SM measured within 1.5 % of each other on
    // the 7B-shaped decode, 2 ahead)
    uint32_t want = 2u * static_cast<uint32_t>(ctx->sm_count);
    if (norm) want = std::min(want, kNextNormCtas);
    const uint32_t rows_all = pair ? g.m[0].R : total_rows;
    const uint32_t rows_per_cta = std::max(kGroupThreads / MT, (rows_all + want - 1u) / want);
    uint32_t ctas = 0;
    for (uint32_t i = 0; i < g.n_seg; ++i) {
        g.m[i].cta_begin = pair ? 0u : ctas;
        g.m[i].rows_per_cta = rows_per_cta;
        if (!pair || i == 0) ctas += (g.m[i].R + rows_per_cta - 1u) / rows_per_cta;
    }
    g.code_cap16 = (rows_per_cta * max_slots * 2u + 15u + 16u) >> 4;
    g.region_bytes = static_cast<uint32_t>(static_cast<size_t>(g.code_cap16) * 16u + 64u * 4u + static_cast<size_t>(max_k) * MT * 4u);
    const size_t smem = static_cast<size_t>(g.region_bytes) * (pair ? 2u : 1u);
    auto kern = pair ? hsdr_gather_group_kernel<MT, true, false>
                     : norm ? hsdr_gather_group_kernel<MT, false, true> : hsdr_gather_group_kernel<MT, false, false>;
    ctx->opt_in_smem(reinterpret_cast<const void*>(kern), smem);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(ctas, 1, 1);
    cfg.blockDim = dim3(kGroupThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = ctx->pdl ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    LaunchScope ls(ctx, KC_GATHER);
    CSDR_CUDA(cudaLaunchKernelEx(&cfg, kern, g));
    ls.done("hsdr_gather_group_kernel");
    return ctas;
}

void launch_gather_wide(csdr_context* ctx, const csdr_segment* seg, const float* dx, uint32_t M, const YView& yv,
                        const float* residual, const TokenScale& ts) {
    const Geometry& g = seg->g;
    const size_t smem = gather_wide_smem(g.n_atoms);
    ctx->opt_in_smem(reinterpret_cast<const void*>(hsdr_gather_wide_kernel), smem);
    // one CTA per SM (the slice fills most of its shared memory): split the rows so that
    // slices x row runs covers the GPU once, in runs that are multiples of eight rows
    const uint32_t slices = (M + kWideTokens - 1u) / kWideTokens;
    const uint32_t want = std::max(1u, static_cast<uint32_t>(ctx->sm_count) / slices);
    uint32_t rows_per_cta = (g.rows + want - 1u) / want;
    rows_per_cta = (rows_per_cta + kWideRows - 1u) / kWideRows * kWideRows;
    const uint32_t runs = (g.rows + rows_per_cta - 1u) / rows_per_cta;
    LaunchScope ls(ctx, KC_GATHER);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(runs, slices, 1);
    cfg.blockDim = dim3(kWideThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = ctx->pdl ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    CSDR_CUDA(cudaLaunchKernelEx(&cfg, hsdr_gather_wide_kernel, seg->codes_ptr(), g.rows, g.n_stages, g.k,
                                 static_cast<const float*>(seg->scales->ptr), dx, g.n_atoms, M, rows_per_cta, yv,
                                 residual, ts, ctx->status_word, ctx->spin_limit_barrier));
    ls.done("hsdr_gather_wide_kernel");
}

}  // namespace

bool wide_group_supported(const csdr_context* ctx, const csdr_segment* const* segs, uint32_t n, size_t batch) {
    if (n == 0 || n > kGatherGroupMax) return false;
    for (uint32_t i = 0; i < n; ++i) {
        if (!tcgen05_supported(ctx, segs[i], batch) || !dx_tma_supported(ctx, segs[i], batch)) return false;
        if (segs[i]->g.cols != segs[0]->g.cols || segs[i]->g.n_stages > 64u) return false;
    }
    return true;
}

WideDx launch_wide_project(csdr_context* ctx, const csdr_segment* const* segs, uint32_t n, XPlanesView x, uint32_t M,
                           float* dx_base, const Exchange* xch, const float* blk_base, const float* sums,
                           const NormShares* shares) {
    if (n == 0 || n > kGatherGroupMax) throw Error(CSDR_ERR_LIMIT, "matmul group holds 1 to 4 segments");
    WideDx w{};
    if (M <= 16u) {
        w.tile_mt = 1;
        while (w.tile_mt < M) w.tile_mt <<= 1;
    }
    w.stride = w.tile_mt ? w.tile_mt : M;
    size_t total_atoms = 0;
    for (uint32_t i = 0; i < n; ++i) total_atoms += segs[i]->g.n_atoms;
    w.floats = total_atoms * w.stride;
    w.base = dx_base ? dx_base
                     : static_cast<float*>(ctx->scratch_get(0, total_atoms * std::max<size_t>(w.stride, 16u) * 4u));
    size_t off = 0;
    for (uint32_t i = 0; i < n; ++i) {
        w.dx[i] = w.base + off;
        off += static_cast<size_t>(segs[i]->g.n_atoms) * w.stride;
    }
    launch_dx_tma_group(ctx, segs, n, x, M, w.dx, w.stride, xch, blk_base, sums, false, shares);
    return w;
}

namespace {
uint32_t gather_tile_group(csdr_context* ctx, const csdr_segment* const* segs, uint32_t n, const WideDx& w, uint32_t M,
                       const WideOut* outs, int y_layout, const TokenScale& ts, __nv_bfloat16* act_hi = nullptr,
                       __nv_bfloat16* act_lo = nullptr, const NextNorm* next = nullptr) {
    GatherGroupParams g{};
    if (next) g.next = *next;
    g.trace = ctx->gemv_trace ? static_cast<unsigned long long*>(ctx->gemv_trace->ptr) : nullptr;
    g.trace_ctas = static_cast<uint32_t>(ctx->sm_count) * 2u;
    g.status = ctx->status_word;
    g.spin = ctx->spin_limit_barrier;
    if (act_hi) {
        if (n != 2 || segs[0]->g.rows != segs[1]->g.rows || !act_lo)
            throw Error(CSDR_ERR_INVALID_ARG, "a SwiGLU pair is two segments with the same number of rows");
        g.act_hi = act_hi;
        g.act_lo = act_lo;
    }
    g.n_seg = n;
    g.M = M;
    g.m_total = M;
    g.y_layout = y_layout;
    g.ts = ts;
    uint32_t total_rows = 0, max_k = 0, max_slots = 0;
    for (uint32_t i = 0; i < n; ++i) {
        const Geometry& sg = segs[i]->g;
        g.m[i] = GatherMember{segs[i]->codes_ptr(), static_cast<const float*>(segs[i]->scales->ptr), w.dx[i], outs[i].y,
                              outs[i].bias, outs[i].residual, sg.rows, sg.n_stages, sg.k, sg.n_atoms, 0u, 0u};
        total_rows += sg.rows;
        max_k = std::max(max_k, sg.n_atoms);
        max_slots = std::max(max_slots, sg.slots());
    }
    switch (w.tile_mt) {
        case 1: return launch_gather_group_t<1>(ctx, g, total_rows, max_k, max_slots);
        case 2: return launch_gather_group_t<2>(ctx, g, total_rows, max_k, max_slots);
        case 4: return launch_gather_group_t<4>(ctx, g, total_rows, max_k, max_slots);
        case 8: return launch_gather_group_t<8>(ctx, g, total_rows, max_k, max_slots);
        default: return launch_gather_group_t<16>(ctx, g, total_rows, max_k, max_slots);
    }
}
}  // namespace

uint32_t launch_wide_gather(csdr_context* ctx, const csdr_segment* const* segs, uint32_t n, const WideDx& w, uint32_t M,
                            const WideOut* outs, int y_layout, const TokenScale& ts, const NextNorm* next) {
    if (w.tile_mt) {
        const bool ride = next && next->w && n == 1u && y_layout == CSDR_LAYOUT_TOKEN_MAJOR;
        const uint32_t ctas = gather_tile_group(ctx, segs, n, w, M, outs, y_layout, ts, nullptr, nullptr, ride ? next : nullptr);
        return ride ? ctas : 0u;
    }
    for (uint32_t i = 0; i < n; ++i) {
        YView yv{outs[i].y, y_layout, segs[i]->g.rows, M, 0u, M, outs[i].bias};
        launch_gather_wide(ctx, segs[i], w.dx[i], M, yv, outs[i].residual, ts);
    }
    return 0u;
}

void launch_exchange_reduce(csdr_context* ctx, const Exchange& x, uint32_t off_floats, size_t floats, float* dst) {
    if (x.ranks < 2u) return;
    if ((off_floats & 3u) || (floats & 3u) || off_floats + floats > x.blk_floats)
        throw Error(CSDR_ERR_INVALID_ARG, "exchange: block range must be whole float4s inside a slot");
    ReduceParams p{};
    p.slots = x.slots[x.rank];
    p.flags = x.flags[x.rank];
    p.seq = x.seq;
    p.ranks = x.ranks;
    p.blk_floats = x.blk_floats;
    p.off_floats = off_floats;
    p.count4 = static_cast<uint32_t>(floats / 4u);
    p.dst = dst;
    p.status = x.status;
    p.spin = ctx->spin_limit_exchange;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(std::max(1u, std::min(64u, (p.count4 + 255u) / 256u)), 1, 1);
    cfg.blockDim = dim3(256, 1, 1);
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = ctx->pdl ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    LaunchScope ls(ctx, KC_DECODER_OP);
    CSDR_CUDA(cudaLaunchKernelEx(&cfg, exchange_reduce_kernel, p));
    ls.done("exchange_reduce_kernel");
}

void launch_wide_gather_swiglu(csdr_context* ctx, const csdr_segment* const* gate_up, const WideDx& w, uint32_t M,
                               const TokenScale& ts, __nv_bfloat16* act_hi, __nv_bfloat16* act_lo) {
    if (!w.tile_mt) throw Error(CSDR_ERR_LIMIT, "the fused SwiGLU gather takes single token tiles (at most 16 tokens)");
    const WideOut none[2] = {WideOut{nullptr, nullptr, nullptr}, WideOut{nullptr, nullptr, nullptr}};
    gather_tile_group(ctx, gate_up, 2, w, M, none, CSDR_LAYOUT_TOKEN_MAJOR, ts, act_hi, act_lo);
}

void launch_matmul_wide_group(csdr_context* ctx, const csdr_segment* const* segs, uint32_t n, XPlanesView x,
                              uint32_t M, const WideOut* outs, int y_layout) {
    const WideDx w = launch_wide_project(ctx, segs, n, x, M, nullptr);
    launch_wide_gather(ctx, segs, n, w, M, outs, y_layout, TokenScale{});
}

bool tcgen05_supported(const csdr_context* ctx, const csdr_segment* seg, size_t batch) {
    const Geometry& g = seg->g;
    if (!ctx->tensor_cores || batch < ctx->tc_min_batch) return false;
    if (!g.row_tiles() || g.n_atoms % kTileM) return false;
    // the TMA-fed projection takes any multiple of eight columns, the register-fed one whole
    // 64-column blocks
    if (g.cols % kBlockK && !dx_tma_supported(ctx, seg, batch)) return false;
    if (g.slots() > kWideMaxSlots) return false;
    return gather_wide_smem(g.n_atoms) <= ctx->smem_optin;
}

void launch_matmul_tcgen05(csdr_context* ctx, const csdr_segment* seg, const MatmulArgs& a) {
    const Geometry& g = seg->g;
    const uint32_t M = static_cast<uint32_t>(a.batch);
    // token tile: the smallest supported MMA N that covers the batch, capped at 128 so that two
    // stages of operands (2 x (32 KB + 2 x N x 128 B)) stay well inside shared memory
    uint32_t N = 16;
    while (N < 128u && N < M) N <<= 1;
    const uint32_t tok_tiles = (M + N - 1u) / N;
    const uint32_t atom_tiles = g.n_atoms / kTileM;
    const uint32_t n_kb = g.cols / kBlockK;
    // Enough CTAs to have every SM streaming (two per SM while the tiles are few).
    uint32_t n_split = std::max<uint32_t>(1u, 2u * static_cast<uint32_t>(ctx->sm_count) / std::max(1u, atom_tiles * tok_tiles));
    n_split = std::min(n_split, n_kb);
    const uint32_t kb_per_split = (n_kb + n_split - 1u) / n_split;
    n_split = (n_kb + kb_per_split - 1u) / kb_per_split;

    const size_t dx_floats = static_cast<size_t>(g.n_atoms) * M;
    float* dx = static_cast<float*>(ctx->scratch_get(0, std::max<size_t>(dx_floats * 4u, static_cast<size_t>(g.n_atoms) * 64u)));
    const bool use_tma = dx_tma_supported(ctx, seg, a.batch);
    // up to 16 tokens: Dx rows padded to the compact gather's tile width (the register-fed
    // kernel writes rows of exactly M, so there only M == 16 qualifies)
    uint32_t tile_mt = 0;
    if (M <= 16u && (use_tma || M == 16u)) {
        tile_mt = 1;
        while (tile_mt < M) tile_mt <<= 1;
    }
    if (use_tma) launch_dx_tma(ctx, seg, a, dx, tile_mt ? tile_mt : M);

    TcParams p{};
    p.D = static_cast<const float*>(seg->atoms->ptr);
    p.K = g.n_atoms;
    p.C = g.cols;
    p.x = XView{a.x, a.x_dtype, a.x_layout, g.cols, M, 0u, M};
    p.n_tile = N;
    p.tmem_cols = std::max(32u, N);
    p.kb_per_split = kb_per_split;
    p.n_kb = n_kb;
    p.n_split = n_split;
    p.status = ctx->status_word;
    p.spin = ctx->spin_limit_barrier;
    p.x_has_lo = a.x_dtype == CSDR_DTYPE_F32 ? 1 : 0;
    float* part = (n_split > 1 && !use_tma) ? static_cast<float*>(ctx->scratch_get(1, dx_floats * n_split * 4u)) : dx;
    p.out = part;
    if (!use_tma) {
        const size_t smem = 2u * (2u * kATileBytes + 2u * static_cast<size_t>(N) * 128u) + 1024u;
        ctx->opt_in_smem(reinterpret_cast<const void*>(hsdr_dx_tcgen05_kernel), smem);
        LaunchScope ls(ctx, KC_GEMM);
        hsdr_dx_tcgen05_kernel<<<dim3(atom_tiles, tok_tiles, n_split), kTcThreads, smem, ctx->stream>>>(p);
        ls.done("hsdr_dx_tcgen05_kernel");
    }
    if (n_split > 1 && !use_tma) {
        LaunchScope ls(ctx, KC_DECODER_OP);
        dx_reduce_kernel<<<static_cast<unsigned>((dx_floats + 255) / 256), 256, 0, ctx->stream>>>(
            part, static_cast<uint32_t>(dx_floats), n_split, dx);
        ls.done("dx_reduce_kernel");
    }
    if (tile_mt) {
        // one token tile: Dx is exactly the [n_atoms][mt] block the compact gathers expect; the
        // group gather (a row for four tokens per thread) as a group of one where its scale block fits
        if (g.n_stages <= 64u) {
            WideDx w{};
            w.base = dx;
            w.dx[0] = dx;
            w.floats = static_cast<size_t>(g.n_atoms) * tile_mt;
            w.stride = tile_mt;
            w.tile_mt = tile_mt;
            const WideOut out{a.y, a.bias, nullptr};
            gather_tile_group(ctx, &seg, 1, w, M, &out, a.y_layout, TokenScale{});
            return;
        }
        launch_gather_tile(ctx, seg, dx, static_cast<int>(tile_mt), a.y, a.y_layout, M, 0u, M, a.bias);
        return;
    }
    YView yv{a.y, a.y_layout, g.rows, M, 0u, M, a.bias};
    launch_gather_wide(ctx, seg, dx, M, yv, nullptr, TokenScale{});
}

}  // namespace csdr
