// One-launch decode GEMV for 1-D row-tile HSDR segments on sm_100a.
//
// The reference computes Y = W x in two loops (matmulRowMajor,
// strategies/HierarchicalSDRStrategy.cpp:1304-1336): Dx = D x, then a signed gather over
// Dx per output row. Here both loops live in one persistent kernel:
//
//   prologue   every CTA requests the dictionary slab of its first task (128-bit streaming
//              loads into registers) and its rows of the code stream (16-byte cp.async into
//              shared memory). Neither depends on the activations, so this runs BEFORE the
//              programmatic-dependent-launch wait: in a chain of matmuls the weight traffic
//              of launch n+1 overlaps the tail of launch n.
//   phase A    after the wait: x slab to shared memory, FMAs, warp-shuffle reduction. Each
//              column-split partial leaves as ONE 64-bit word {value, launch epoch}. The
//              epoch is read (a plain load) from a word in device memory that CTA 0 moves on
//              once every CTA has read it, so a captured CUDA graph tags every replay afresh.
//   hand-over  no barrier, no atomics, no fence (a device-wide fence behind an 8 MB read
//              burst was measured at up to 7 us): phase B polls the partial words
//              themselves, sixteen independent loads per thread per round, until every word
//              carries this launch's epoch. Words are written with st.relaxed.gpu.b64 and
//              polled with ld.relaxed.gpu.b64 (single-copy atomic by the memory model), so a
//              matching tag proves the value beside it. The poll is bounded: the first wait
//              that runs out records a status word and every later poll of the launch gives
//              up after one look, so a launch waits at most one limit in all.
//   phase B    Dx = sum of the partials in split order (results do not depend on
//              scheduling), signed gather in the reference's order, y out. With wide token
//              tiles a gather CTA owns a group of four tokens, so it polls only that slice.
//
// Up to four segments that consume the same x (q|k|v, gate|up) share one launch.
#include <algorithm>

#include "../internal.hpp"
#include "gemv_fused.hpp"
#include "views.cuh"

namespace csdr {

namespace {

constexpr int kThreads = 256;

struct FusedSeg {
    const float* D;
    const uint16_t* codes;
    const float* scales;
    uint32_t K, R, S, k;
    uint32_t task0;         // first phase-A task of this segment
    uint32_t part_off;      // word offset of its partial block: [nsplit][K][MT]
    uint32_t rows_per_cta;  // phase B
    YView y;
};

struct FusedParams {
    FusedSeg seg[kMaxFusedGroup];
    uint32_t n_seg, n_tasks, C, slab, nsplit;
    uint32_t gather_ctas;   // CTAs that take part in phase B = row chunks * token groups
    XView x;
    unsigned long long* part;  // {float bits (low half), epoch (high half)} per partial
    uint32_t* seq;          // device: launch tag words (read_launch_tag / retire_launch_tag)
    int* status;
    uint32_t spin_limit;
    unsigned long long* trace;  // optional: 16 global-timer stamps per CTA (phase boundaries)
    const float* norm_w;    // y = W rmsnorm(x; norm_w, norm_eps); needs the whole x per CTA
    float norm_eps;
    uint32_t swiglu;        // segment 1's rows leave as silu(segment 0's row) * row
};

__device__ __forceinline__ void stamp(const FusedParams& p, int slot) {
    if (p.trace && threadIdx.x == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        p.trace[blockIdx.x * 16u + slot] = t;
    }
}

__device__ __forceinline__ unsigned long long ld_poll(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.relaxed.gpu.global.b64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_tagged(unsigned long long* p, float value, uint32_t epoch) {
    const unsigned long long w = (static_cast<unsigned long long>(epoch) << 32) | __float_as_uint(value);
    asm volatile("st.relaxed.gpu.global.b64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst))),
                 "l"(gmem_src)
                 : "memory");
}
__device__ __forceinline__ void cp_async4(void* smem_dst, const void* gmem_src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst))),
                 "l"(gmem_src)
                 : "memory");
}

// x slab -> shared memory, 128-bit when the source rows are contiguous fp32.
template <int MT>
__device__ __forceinline__ void stage_x(const XView& xv, uint32_t c0, uint32_t cw, uint32_t cols, float* xs) {
    const bool rows_contig = xv.layout == CSDR_LAYOUT_TOKEN_MAJOR || xv.Mtotal == 1;
    if (xv.dtype == CSDR_DTYPE_F32 && rows_contig && (cw & 3u) == 0 &&
        ((reinterpret_cast<uintptr_t>(xv.x) | (static_cast<uintptr_t>(xv.C) * 4u) | (static_cast<uintptr_t>(c0) * 4u)) & 15u) == 0) {
        const uint32_t cols4 = cols >> 2, cw4 = cw >> 2;
        for (uint32_t i = threadIdx.x; i < MT * cols4; i += kThreads) {
            const uint32_t b = i / cols4, c4 = i - b * cols4;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (b < xv.M && c4 < cw4)
                v = *(reinterpret_cast<const float4*>(static_cast<const float*>(xv.x) +
                                                      static_cast<size_t>(xv.b0 + b) * xv.C + c0) + c4);
            reinterpret_cast<float4*>(xs)[i] = v;
        }
    } else {
        for (uint32_t i = threadIdx.x; i < MT * cols; i += kThreads) {
            const uint32_t b = i / cols, c = i - b * cols;
            xs[i] = (b < xv.M && c < cw) ? load_x(xv, c0 + c, b) : 0.0f;
        }
    }
}

// Shared-memory plan, fixed for the whole kernel so that the prologue can fill the
// phase-B part while phase A still uses its own:
//   xs      [MT][xcols]    activations (xcols = C when they fit, else one column slab)
//   codes   per segment: the CTA's rows of the code stream, 16-byte units
//   scales  per segment: S floats (padded to 4)
//   dxs     [max K][MTG]   Dx slice of the segment being gathered
struct SmemPlan {
    uint32_t xcols;                       // C (whole x resident) or slab
    uint32_t codes_off[kMaxFusedGroup];   // byte offsets
    uint32_t scales_off[kMaxFusedGroup];
    uint32_t dxs_off;
    uint32_t normw_off;                   // the norm weights of the folded normalisation, [C]
};

// Register budget: two launches must be able to sit on an SM together (two CTAs each), or the
// next launch's weight prefetch cannot start before this one retires.
template <int MT, int A, int U>
__global__ void __launch_bounds__(kThreads, (MT <= 4 ? 4 : 3))
hsdr_gemv_fused_kernel(const __grid_constant__ FusedParams p, const __grid_constant__ SmemPlan plan) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    asm volatile("griddepcontrol.launch_dependents;");
    stamp(p, 0);
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    constexpr uint32_t kAtomsPerCta = 8u * A;
    constexpr uint32_t MTG = MT < 4 ? MT : 4;   // tokens per gather CTA
    constexpr uint32_t kTokenGroups = MT / MTG;
    const bool whole_x = plan.xcols == p.C;
    const uint32_t xcols4 = plan.xcols >> 2;
    const bool gathers = blockIdx.x < p.gather_ctas;
    const uint32_t tg = blockIdx.x % kTokenGroups, rchunk = blockIdx.x / kTokenGroups;

    // One unit of phase-A work: 32*U float4 columns of 8*A atoms.
    struct Item {
        uint32_t task, base, s, ag, split, cw4;
    };
    auto locate = [&](Item& it) {
        uint32_t s = 0;
#pragma unroll
        for (uint32_t i = 1; i < kMaxFusedGroup; ++i)
            if (i < p.n_seg && it.task >= p.seg[i].task0) s = i;
        const uint32_t local = it.task - p.seg[s].task0;
        it.s = s;
        it.ag = local / p.nsplit;
        it.split = local - it.ag * p.nsplit;
        const uint32_t c0 = it.split * p.slab;
        it.cw4 = (c0 < p.C ? min(p.slab, p.C - c0) : 0u) >> 2;
    };
    auto advance = [&](Item& it) {
        it.base += 32u * U;
        if (it.base >= it.cw4) {
            it.task += gridDim.x;
            it.base = 0;
            if (it.task < p.n_tasks) locate(it);
        }
    };
    auto load_d = [&](const Item& it, float4 (&d)[U][A]) {
        const FusedSeg& sg = p.seg[it.s];
        const uint32_t c0 = it.split * p.slab;
        const uint32_t atom0 = it.ag * kAtomsPerCta + warp * A;
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const uint32_t c4 = it.base + u * 32u + lane;
#pragma unroll
            for (int a = 0; a < A; ++a) {
                const bool ok = c4 < it.cw4 && atom0 + a < sg.K;
                d[u][a] = ok ? ldg_stream_f4(reinterpret_cast<const float4*>(
                                                 sg.D + static_cast<size_t>(atom0 + a) * p.C + c0) + c4)
                             : make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
    };

    // ---- prologue: nothing here depends on the activations ----
    float4 d_cur[U][A];
    Item cur{blockIdx.x, 0, 0, 0, 0, 0};
    if (cur.task < p.n_tasks) {
        locate(cur);
        load_d(cur, d_cur);
    }
    if (gathers) {
        // this CTA's rows of every segment's code stream, and the stage scales (non-blocking)
        for (uint32_t si = 0; si < p.n_seg; ++si) {
            const FusedSeg& sg = p.seg[si];
            const uint32_t row0 = rchunk * sg.rows_per_cta;
            if (row0 < sg.R) {
                const uint32_t rows_here = min(sg.rows_per_cta, sg.R - row0);
                const uint32_t slots = sg.S * sg.k;
                const size_t code_byte0 = static_cast<size_t>(row0) * slots * 2u;
                const size_t aligned0 = code_byte0 & ~static_cast<size_t>(15);
                const uint32_t skip2 = static_cast<uint32_t>(code_byte0 - aligned0);
                const uint32_t n16 = (skip2 + rows_here * slots * 2u + 15u) >> 4;
                unsigned char* cs = smem_raw + plan.codes_off[si];
                const unsigned char* src = reinterpret_cast<const unsigned char*>(sg.codes) + aligned0;
                for (uint32_t i = tid; i < n16; i += kThreads) cp_async16(cs + i * 16u, src + i * 16u);
                float* sc = reinterpret_cast<float*>(smem_raw + plan.scales_off[si]);
                for (uint32_t i = tid; i < sg.S; i += kThreads) cp_async4(sc + i, sg.scales + i);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    if (p.norm_w) {
        // the norm weights are static too: into shared memory before the wait
        unsigned char* nw = smem_raw + plan.normw_off;
        for (uint32_t i = tid; i < (p.C >> 2); i += kThreads) cp_async16(nw + i * 16u, p.norm_w + i * 4u);
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    // x and the partial buffer belong to earlier work on the stream
    stamp(p, 1);
    asm volatile("griddepcontrol.wait;" ::: "memory");
    stamp(p, 2);
    __shared__ uint32_t epoch_s;
    // thread 0 reads the launch's tag (one L2 round trip) while the others already stage the activations
    if (tid == 0) epoch_s = read_launch_tag(p.seq);

    // ---- phase A ----
    float* xs = reinterpret_cast<float*>(smem_raw);
    const float4* xs4 = reinterpret_cast<const float4*>(xs);
    __shared__ float ssq_s[kThreads / 32][MT];
    __shared__ float inv_s[MT];
    const bool stage_whole = whole_x && (blockIdx.x < p.n_tasks || (p.norm_w && gathers));
    if (stage_whole) stage_x<MT>(p.x, 0, p.C, p.C, xs);
    __syncthreads();
    const uint32_t epoch = epoch_s;
    if (stage_whole) {
        if (p.norm_w) {
            // rms_norm (api/cortex_sdk.cpp:1208-1232) split in two: the weights go onto the staged row
            // here, 1 / rms onto the gathered rows; every CTA sums the squares of the whole row
            float4* xw = reinterpret_cast<float4*>(xs);
            const float4* w4 = reinterpret_cast<const float4*>(smem_raw + plan.normw_off);
            asm volatile("cp.async.wait_group 0;" ::: "memory");   // this thread's share of the weights is the share it reads
#pragma unroll
            for (int b = 0; b < MT; ++b) {
                float ss = 0.0f;
                for (uint32_t c4 = tid; c4 < xcols4; c4 += kThreads) {
                    const float4 v = xw[b * xcols4 + c4];
                    const float4 w = w4[c4];
                    ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
                    xw[b * xcols4 + c4] = make_float4(v.x * w.x, v.y * w.y, v.z * w.z, v.w * w.w);
                }
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, off);
                if (lane == 0) ssq_s[warp][b] = ss;
            }
            __syncthreads();
            if (tid < MT) {
                float ss = 0.0f;
#pragma unroll
                for (int w = 0; w < kThreads / 32; ++w) ss += ssq_s[w][tid];
                inv_s[tid] = 1.0f / sqrtf(ss / static_cast<float>(p.C) + p.norm_eps);
            }
            __syncthreads();
        }
    }
    stamp(p, 3);
    float acc[A][MT];
    bool have = true;  // d_cur already holds the first unit (prologue)
    while (cur.task < p.n_tasks) {
        if (!have) load_d(cur, d_cur);
        have = false;
        const uint32_t c0 = cur.split * p.slab;
        if (cur.base == 0) {
#pragma unroll
            for (int a = 0; a < A; ++a)
#pragma unroll
                for (int b = 0; b < MT; ++b) acc[a][b] = 0.0f;
            if (!whole_x) {
                __syncthreads();  // every warp is done with the previous slab
                stage_x<MT>(p.x, c0, cur.cw4 << 2, p.slab, xs);
                __syncthreads();
            }
        }
        const uint32_t xoff4 = whole_x ? (c0 >> 2) : 0u;
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const uint32_t c4 = cur.base + u * 32u + lane;
            if (c4 < cur.cw4) {
#pragma unroll
                for (int b = 0; b < MT; ++b) {
                    const float4 x4 = xs4[b * xcols4 + xoff4 + c4];
#pragma unroll
                    for (int a = 0; a < A; ++a) {
                        acc[a][b] = fmaf(d_cur[u][a].x, x4.x, acc[a][b]);
                        acc[a][b] = fmaf(d_cur[u][a].y, x4.y, acc[a][b]);
                        acc[a][b] = fmaf(d_cur[u][a].z, x4.z, acc[a][b]);
                        acc[a][b] = fmaf(d_cur[u][a].w, x4.w, acc[a][b]);
                    }
                }
            }
        }
        if (cur.base + 32u * U >= cur.cw4) {
            // last column chunk of the task: reduce over the warp; lanes 0..MT-1 publish
            // {value, epoch} words, no fence needed
            const FusedSeg& sg = p.seg[cur.s];
            const uint32_t atom0 = cur.ag * kAtomsPerCta + warp * A;
#pragma unroll
            for (int a = 0; a < A; ++a) {
                float mine = 0.0f;
#pragma unroll
                for (int b = 0; b < MT; ++b) {
                    float v = acc[a][b];
#pragma unroll
                    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, off);
                    if (lane == b) mine = v;
                }
                if (lane < MT && atom0 + a < sg.K)
                    st_tagged(p.part + sg.part_off + (static_cast<size_t>(cur.split) * sg.K + atom0 + a) * MT + lane,
                              mine, epoch);
            }
            stamp(p, 8);
        }
        advance(cur);
    }
    stamp(p, 4);
    if (!gathers) return;
    asm volatile("cp.async.wait_group 0;" ::: "memory");

    // ---- phase B ----
    float* dxs = reinterpret_cast<float*>(smem_raw + plan.dxs_off);
    bool late = false;
    // a wait that ran out earlier on this context (or in this launch) is not repeated
    uint32_t limit = *reinterpret_cast<const volatile int*>(p.status) != 0 ? 0u : p.spin_limit;
    const unsigned long long want_tag = static_cast<unsigned long long>(epoch) << 32;
    for (uint32_t si = 0; si < p.n_seg; ++si) {
        const FusedSeg& sg = p.seg[si];
        const uint32_t row0 = rchunk * sg.rows_per_cta;
        if (row0 < sg.R) {
            // -- hand-over: poll this token group's partial words, 16 loads in flight --
            const unsigned long long* part = p.part + sg.part_off;
            const uint32_t n_el = sg.K * MTG;                       // dxs elements
            const uint32_t mine_el = tid < n_el ? (n_el - tid + kThreads - 1u) / kThreads : 0u;
            const uint32_t n_w = mine_el * p.nsplit;               // words this thread owns
            uint32_t j0 = 0, sp0 = 0;                              // (element ordinal, split) of word w0
            for (uint32_t w0 = 0; w0 < n_w; w0 += 16u) {
                unsigned long long e[16];
                for (uint32_t spins = 0;; ++spins) {
                    uint32_t j = j0, sp = sp0;
                    bool ok = true;
#pragma unroll
                    for (int q = 0; q < 16; ++q) {
                        if (w0 + q < n_w) {
                            const uint32_t el = tid + j * kThreads;
                            const uint32_t a = el / MTG, b = el - a * MTG;
                            e[q] = ld_poll(part + (static_cast<size_t>(sp) * sg.K + a) * MT + tg * MTG + b);
                            if (++sp == p.nsplit) {
                                sp = 0;
                                ++j;
                            }
                        } else {
                            e[q] = want_tag;
                        }
                    }
#pragma unroll
                    for (int q = 0; q < 16; ++q) ok = ok && static_cast<uint32_t>(e[q] >> 32) == epoch;
                    if (ok) break;
                    if (spins >= limit) {  // gave up: the host will see it; nothing after this waits
                        late = true;
                        limit = 0u;
                        break;
                    }
                }
#pragma unroll
                for (int q = 0; q < 16; ++q) {
                    if (w0 + q < n_w) {
                        const uint32_t el = tid + j0 * kThreads;
                        const float prev = sp0 ? dxs[el] : 0.0f;  // split order, whatever the batch boundaries
                        dxs[el] = prev + __uint_as_float(static_cast<uint32_t>(e[q]));
                        if (++sp0 == p.nsplit) {
                            sp0 = 0;
                            ++j0;
                        }
                    }
                }
            }
        }
        __syncthreads();  // dxs complete; first pass: also the cp.async fills
        if (si == 0) stamp(p, 5);
        if (row0 < sg.R) {
            const uint32_t rows_here = min(sg.rows_per_cta, sg.R - row0);
            const uint32_t slots = sg.S * sg.k;
            const uint32_t skip = static_cast<uint32_t>((static_cast<size_t>(row0) * slots * 2u) & 15u) >> 1;
            const uint16_t* cs = reinterpret_cast<const uint16_t*>(smem_raw + plan.codes_off[si]) + skip;
            const float* sc = reinterpret_cast<const float*>(smem_raw + plan.scales_off[si]);
            const uint32_t b = tid % MTG;
            constexpr uint32_t RP = kThreads / MTG;
            for (uint32_t rl = tid / MTG; rl < rows_here; rl += RP) {
                const uint16_t* rc = cs + rl * slots;
                // what the epilogue adds comes from global memory and does not depend on the sum:
                // requested here, it arrives while the codes are walked
                const uint32_t tok = tg * MTG + b;
                const uint32_t r = row0 + rl;
                const bool live = tok < sg.y.M;
                const size_t yi = live ? y_index(sg.y, r, tok) : 0;
                const float bias_v = live && sg.y.bias ? sg.y.bias[r] : 0.0f;
                const float resid_v = live && sg.y.residual ? sg.y.residual[yi] : 0.0f;
                float accr = 0.0f;
                for (uint32_t l = 0; l < sg.S; ++l) {
                    const float gamma = sc[l];
                    const uint16_t* lc = rc + l * sg.k;
                    for (uint32_t k0 = 0; k0 < sg.k; k0 += 8u) {
                        // eight independent lookups in flight, then the adds in slot order
                        float t[8];
#pragma unroll
                        for (int q = 0; q < 8; ++q) {
                            const uint32_t code = k0 + q < sg.k ? lc[k0 + q] : 0u;
                            const float v = dxs[(code & 0x7FFFu) * MTG + b];
                            t[q] = __fmul_rn((code & 0x8000u) ? -gamma : gamma, v);
                        }
#pragma unroll
                        for (int q = 0; q < 8; ++q)
                            if (k0 + q < sg.k) accr = __fadd_rn(accr, t[q]);
                    }
                }
                if (live) {
                    if (p.norm_w) accr *= inv_s[tok];
                    if (sg.y.bias) accr += bias_v;
                    if (p.swiglu && si == 1u) {
                        // silu_mul (api/cortex_sdk.cpp:1245-1256); this thread wrote the gate row itself
                        const float gv = p.seg[0].y.y[yi];
                        accr = (gv * (1.0f / (1.0f + expf(-gv)))) * accr;
                    }
                    if (sg.y.residual) accr += resid_v;
                    sg.y.y[yi] = accr;
                }
            }
        }
        __syncthreads();  // dxs is rewritten for the next segment
    }
    if (late) atomicExch(p.status, 1);
    // CTA 0 (always a gather CTA) retires the launch's tag: every CTA has read it long ago
    if (blockIdx.x == 0 && warp == 0 && !retire_launch_tag(p.seq, epoch, lane, limit ? limit : 1u) && lane == 0)
        atomicExch(p.status, 1);
    stamp(p, 7);
}

template <int MT, int A, int U>
void launch_t(csdr_context* ctx, FusedParams& p, uint32_t max_k, bool pdl) {
    auto kern = hsdr_gemv_fused_kernel<MT, A, U>;
    // Activations stay whole in shared memory when they are small; otherwise one slab at a time.
    SmemPlan plan{};
    constexpr uint32_t token_groups = MT <= 4 ? 1u : MT / 4u;
    plan.xcols = static_cast<size_t>(MT) * p.C * 4u <= 64u * 1024u ? p.C : p.slab;
    // Phase B sizes depend on the grid, which depends on the shared memory: size for the
    // smallest grid this kernel can get (one CTA per SM), then launch with what fits.
    auto plan_for = [&](uint32_t gather_ctas) {
        size_t off = static_cast<size_t>(MT) * plan.xcols * 4u;
        for (uint32_t i = 0; i < p.n_seg; ++i) {
            const uint32_t chunks = std::max<uint32_t>(1u, gather_ctas / token_groups);
            const uint32_t rpc = ((p.seg[i].R + chunks - 1u) / chunks + 7u) & ~7u;
            p.seg[i].rows_per_cta = rpc;
            plan.codes_off[i] = static_cast<uint32_t>(off);
            off += ((static_cast<size_t>(rpc) * p.seg[i].S * p.seg[i].k * 2u + 31u) & ~static_cast<size_t>(15));
        }
        for (uint32_t i = 0; i < p.n_seg; ++i) {
            plan.scales_off[i] = static_cast<uint32_t>(off);
            off += ((p.seg[i].S + 3u) & ~3u) * 4u;
        }
        plan.dxs_off = static_cast<uint32_t>(off);
        off += static_cast<size_t>(max_k) * (MT < 4 ? MT : 4) * 4u;
        plan.normw_off = static_cast<uint32_t>(off);
        return off + (p.norm_w ? static_cast<size_t>(p.C) * 4u : 0u);
    };
    const uint32_t want_gather = p.gather_ctas;
    const size_t smem = plan_for(std::min<uint32_t>(want_gather, static_cast<uint32_t>(ctx->sm_count)));
    if (smem > ctx->smem_optin) throw Error(CSDR_ERR_LIMIT, "fused GEMV: shared memory need exceeds the device limit");
    ctx->opt_in_smem(reinterpret_cast<const void*>(kern), smem);
    std::pair<size_t, int>& occ = ctx->occupancy[reinterpret_cast<const void*>(kern)];
    if (occ.second == 0 || occ.first != smem) {
        CSDR_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ.second, kern, kThreads, smem));
        occ.first = smem;
    }
    const int occ_cached = occ.second;
    if (occ_cached < 1)
        throw Error(CSDR_ERR_LIMIT, "fused GEMV does not fit on an SM (token tile " + std::to_string(MT) + ", " +
                                        std::to_string(smem) + " bytes of shared memory, " + std::to_string(p.n_seg) + " segments)");
    // Every CTA must be resident for the barrier: at most what one otherwise idle GPU holds.
    const uint32_t grid = static_cast<uint32_t>(ctx->sm_count) * static_cast<uint32_t>(std::min(occ_cached, 2));
    p.gather_ctas = std::max(token_groups, std::min(want_gather, grid) / token_groups * token_groups);
    plan_for(p.gather_ctas);  // never larger than the size computed above
    // whole-x residency only pays when a CTA walks several column slabs (the folded normalisation
    // needs it regardless: every CTA sums the squares of the whole row)
    if (!p.norm_w && plan.xcols == p.C && p.n_tasks <= grid && p.slab < p.C) {
        plan.xcols = p.slab;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = pdl ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    LaunchScope ls(ctx, KC_GEMV_FUSED);
    CSDR_CUDA(cudaLaunchKernelEx(&cfg, kern, p, plan));
    ls.done("hsdr_gemv_fused_kernel");
}

}  // namespace

bool gemv_fused_supported(const csdr_context* ctx, const csdr_segment* const* segs, uint32_t n, uint32_t mt) {
    if (!ctx->fused_gemv || n == 0 || n > kMaxFusedGroup) return false;
    const Geometry& g0 = segs[0]->g;
    for (uint32_t i = 0; i < n; ++i) {
        const Geometry& g = segs[i]->g;
        if (!g.row_tiles() || g.cols != g0.cols || g.cols % 4u) return false;
        if (static_cast<size_t>(g.n_atoms) * mt * 4u > 64u * 1024u) return false;
    }
    return true;
}

bool gemv_fused_glue_supported(const csdr_context* ctx, const csdr_segment* const* segs, uint32_t n, uint32_t mt,
                               const FusedGlue& glue) {
    if (!gemv_fused_supported(ctx, segs, n, mt)) return false;
    if (glue.norm_w && static_cast<size_t>(mt) * segs[0]->g.cols * 4u > 64u * 1024u) return false;
    if (glue.swiglu && (n != 2u || segs[0]->g.rows != segs[1]->g.rows)) return false;
    return true;
}

void launch_gemv_fused(csdr_context* ctx, const csdr_segment* const* segs, uint32_t n, const void* x,
                       int x_dtype, int x_layout, uint32_t m_total, uint32_t b0, uint32_t m,
                       float* const* ys, int y_layout, const float* const* biases, int mt, const FusedGlue* glue) {
    FusedParams p{};
    if (glue) {
        if (!gemv_fused_glue_supported(ctx, segs, n, static_cast<uint32_t>(mt), *glue))
            throw Error(CSDR_ERR_UNSUPPORTED, "fused GEMV: the folded glue does not fit this launch");
        if ((glue->norm_w && reinterpret_cast<uintptr_t>(glue->norm_w) % 16u) || (glue->norm_w && x_dtype != CSDR_DTYPE_F32))
            throw Error(CSDR_ERR_INVALID_ARG, "fused GEMV: folded normalisation wants fp32 activations and 16-byte aligned weights");
        p.norm_w = glue->norm_w;
        p.norm_eps = glue->norm_eps;
        p.swiglu = glue->swiglu ? 1u : 0u;
    }
    const Geometry& g0 = segs[0]->g;
    const uint32_t C = g0.cols;
    // Column slabs of about 1024 floats, each a multiple of 4 (128-bit loads).
    uint32_t nsplit = std::max<uint32_t>(1u, (C + 1023u) / 1024u);
    const uint32_t slab = ((C + nsplit - 1u) / nsplit + 3u) & ~3u;
    nsplit = (C + slab - 1u) / slab;
    const int A = mt <= 2 ? 1 : 2;
    p.n_seg = n;
    p.C = C;
    p.slab = slab;
    p.nsplit = nsplit;
    p.x = XView{x, x_dtype, x_layout, C, m_total, b0, m};
    uint32_t task = 0, part_off = 0, max_rows = 0, max_k = 0;
    for (uint32_t i = 0; i < n; ++i) {
        const Geometry& g = segs[i]->g;
        FusedSeg& s = p.seg[i];
        s.D = static_cast<const float*>(segs[i]->atoms->ptr);
        s.codes = segs[i]->codes_ptr();
        s.scales = static_cast<const float*>(segs[i]->scales->ptr);
        s.K = g.n_atoms;
        s.R = g.rows;
        s.S = g.n_stages;
        s.k = g.k;
        s.task0 = task;
        s.part_off = part_off;
        s.y = YView{ys[i], y_layout, g.rows, m_total, b0, m, biases ? biases[i] : nullptr, glue ? glue->residual[i] : nullptr};
        task += ((g.n_atoms + 8u * A - 1u) / (8u * A)) * nsplit;
        part_off += nsplit * g.n_atoms * mt;
        max_rows = std::max(max_rows, g.rows);
        max_k = std::max(max_k, g.n_atoms);
    }
    p.n_tasks = task;
    p.part = static_cast<unsigned long long*>(
        ctx->scratch_get(4, std::max<size_t>(static_cast<size_t>(part_off) * 8u, 2u << 20)));
    p.seq = ctx->gemv_seq;
    p.status = ctx->status_word;
    p.trace = ctx->gemv_trace ? static_cast<unsigned long long*>(ctx->gemv_trace->ptr) : nullptr;
    p.spin_limit = ctx->spin_limit_gemv;  // each poll is an L2 round trip: about a second by default
    // Phase B: as many (row chunk, token group) jobs as there is work for; launch_t caps it at the grid.
    p.gather_ctas = std::max<uint32_t>(1u, static_cast<uint32_t>(static_cast<size_t>(max_rows) * mt / 32u));
    const bool pdl = ctx->pdl;
    switch (mt) {
        case 1: launch_t<1, 1, 8>(ctx, p, max_k, pdl); break;
        case 2: launch_t<2, 1, 8>(ctx, p, max_k, pdl); break;
        case 4: launch_t<4, 2, 4>(ctx, p, max_k, pdl); break;
        case 8: launch_t<8, 2, 2>(ctx, p, max_k, pdl); break;
        default: launch_t<16, 2, 1>(ctx, p, max_k, pdl); break;
    }
}

}  // namespace csdr
