// A list of decode GEMVs in ONE persistent launch, for 1-D row-tile HSDR segments on sm_100a.
//
// The reference issues every y = W x as its own call (matmulRowMajor,
// strategies/HierarchicalSDRStrategy.cpp:1257-1338: Dx = D x, then a signed gather over Dx per
// output row), and so does a chain of single launches: each pays the same latencies in a row -
// activations in, partial results across, gather, kernel boundary - while the 9 MB of weights
// need 1.4 us of HBM time. Here a list of products runs as one grid of one CTA per SM whose warps
// have three roles:
//
//   loader    (1 warp)  walks the flat list of work units (task, group of 8 atoms) this CTA owns
//                       and keeps a ring of shared-memory stages full: per stage 8 dictionary rows
//                       x 1024 columns - ONE cp.async.bulk copy, from a copy of the dictionary
//                       re-laid in exactly these blocks when the list kernel first meets it - and,
//                       for activations that were there before the launch, the matching slab of
//                       them, all signalling the stage's mbarrier. The dictionary is static, so
//                       the first ring-full of weight copies is issued BEFORE the
//                       programmatic-dependent-launch wait, and the weights of a task whose
//                       activations another task of the list is still producing are in flight
//                       while it waits.
//   products  (8 warps) one atom per warp: dot products of the staged row slab with the staged
//                       activations, accumulated over the row's slabs in registers, reduced with
//                       warp shuffles, and published as ONE 64-bit word {value, launch tag} per
//                       (atom, token): the finished Dx, no column-split partials. Activations that
//                       an earlier task of the list produces arrive as such tagged words too: the
//                       eight warps poll their slices of the slab until every word carries the
//                       launch's tag.
//   gather    (4 warps) each warp on its own, no barrier between them: prefetches its rows of its
//                       next task's code stream (cp.async), polls the task's Dx words until they
//                       carry the launch's tag, then the signed gather in the reference's order
//                       and the task's epilogue. Lists of plain, independent products give every
//                       fourth task to a warp; lists with dependencies split each task's rows
//                       over the four warps instead (shortest path through a chain).
//
// A matching tag proves the value beside it (64-bit relaxed gpu-scope accesses are single-copy
// atomic), so no hand-over needs a fence, a counter or an atomic, and the data itself is what is
// polled. The tag is one more than the tag of the launch before, read from device memory with a
// plain load (CTA 0's loader moves the word on once every CTA has left the tag it read in a slot
// of its own), so a captured CUDA graph tags every replay afresh.
//
// The decoder glue of api/cortex_sdk.cpp:1569-1679 is folded in so that a block of the decoder
// is one list: bias, residual add (add_vectors, :1234-1243) and SwiGLU against the task before
// (silu_mul, :1245-1256) are epilogues of the gather; RMS normalisation (rms_norm, :1208-1232)
// of activations that come from an earlier task is split in two: the product warps multiply
// the slab by the norm weights as they stage it and sum the squares of what they staged (every
// unit sees the whole activation row), the task's first unit publishes that sum as one more
// tagged word per token, and the gather scales its rows by 1 / sqrt(mean + eps).
//
// Every wait is bounded (mbarrier phases, polls): one that runs out sets the status word, all
// roles of the CTA stop waiting, and the kernel returns. All CTAs must be resident (grid = SM
// count, one per SM).
#include <algorithm>
#include <cstdlib>

#include "../internal.hpp"
#include "gemv_queue.hpp"
#include "views.cuh"

namespace csdr {

namespace {

constexpr uint32_t kLoaderWarps = 1, kProductWarps = 8, kGatherWarps = 4;
constexpr uint32_t kThreads = 32u * (kLoaderWarps + kProductWarps + kGatherWarps);
constexpr uint32_t kProductThreads = 32u * kProductWarps;
constexpr uint32_t kAtomsPerUnit = 8;          // one per product warp
constexpr uint32_t kSlab = 1024;               // columns per stage (a multiple of 1024)
constexpr uint32_t kMaxStages = 8;
constexpr uint32_t kMaxTokens = 4;

enum : uint32_t { EPI_PLAIN = 0, EPI_SWIGLU = 1 };
enum : uint32_t { X_PLAIN = 0, X_TAGGED = 1 };

typedef unsigned long long u64;

struct QTask {
    const float* D;           // the dictionary in stage blocks (stage_blocks_kernel), not row-major
    const uint16_t* codes;
    const float* scales;
    const void* x;            // X_PLAIN: activations (dtype, layout); X_TAGGED: u64 words [M][C]
    float* y;                 // fp32 result, or null when only the tagged copy is wanted
    u64* y_tag;               // tagged copy [M][R] for a later task of the list, or null
    const float* bias;
    const float* residual;    // [M][R] token-major, may alias y
    const float* gate;        // EPI_SWIGLU: the gate projection's rows, [M][R]
    const float* norm_w;      // X_TAGGED only: y = W rmsnorm(x; norm_w, norm_eps)
    uint32_t K, R, C, S, k;
    uint32_t unit0;           // first flat unit of this task
    uint32_t n_units;
    uint32_t dx_off;          // word offset of its Dx slot: [K][MT]
    uint32_t rows_per_cta;
    uint32_t x_kind, x_dtype, x_layout, y_layout;
    uint32_t M;
    float norm_eps;
    uint32_t epilogue;
};

struct QParams {
    QTask task[kMaxQueueTasks];
    uint32_t n_tasks, n_units;
    uint32_t n_stages;          // ring depth
    uint32_t stage_bytes;       // D slab + x slab
    uint32_t gw_bytes;          // shared memory of one gather warp: Dx copy + two code buffers + scales
    uint32_t dxs_bytes;         // the Dx copy inside it
    uint32_t codes_bytes;       // one code buffer inside it
    uint32_t split_rows;        // 1: a task's rows are split over the gather warps; 0: tasks are dealt out to them
    u64* dx;                    // tagged Dx words
    u64* sumsq;                 // tagged sums of squares of a task's activations: [task][kMaxTokens]
    uint32_t* seq;              // launch tag words (read_launch_tag / retire_launch_tag)
    int* status;
    uint32_t spin_poll, spin_barrier;
    uint32_t poll_sleep_ns;     // pause between two looks at words another CTA has yet to write
    unsigned long long* trace;  // optional: global-timer stamps, [cta][8 tasks][8 slots] (tuning)
};

// slots: 0 first activations staged, 1 Dx of the CTA's first unit of the task published,
// 2 gather warp 0 saw the watch words, 3 swept Dx, 4 rows written; 5 kernel entry, 6 tag taken;
// slot 7 of tasks 1, 3, 4: the loader starts, has issued its first copies, is past the dependency wait
__device__ __forceinline__ void stamp(const QParams& p, uint32_t task, uint32_t slot) {
    if (p.trace && task < 8u) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        p.trace[(static_cast<size_t>(blockIdx.x) * 8u + task) * 8u + slot] = t;
    }
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// Bounded wait on an mbarrier phase; gives up at once when another role already has.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, uint32_t limit, const volatile int* failed) {
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
        if (*failed) return false;
    }
    return false;
}

__device__ __forceinline__ u64 ld_tagged(const u64* p) {
    u64 v;
    asm volatile("ld.relaxed.gpu.global.b64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_tagged(u64* p, float value, uint32_t tag) {
    const u64 w = (static_cast<u64>(tag) << 32) | __float_as_uint(value);
    asm volatile("st.relaxed.gpu.global.b64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}

__device__ __forceinline__ XView x_view(const QTask& t) {
    return XView{t.x, static_cast<int>(t.x_dtype), static_cast<int>(t.x_layout), t.C, t.M, 0u, t.M};
}

// Polls `n` tagged words (word i of this lane at src[i * stride]) in batches of B loads in
// flight until every one carries `tag`; stores the values through `put(i, value)`. Bounded:
// returns false when a batch did not complete within `limit` rounds (or another role gave up).
template <int B, typename Put>
__device__ __forceinline__ bool poll_words(const u64* src, uint32_t n, uint32_t stride, uint32_t tag, uint32_t& limit,
                                           const volatile int* failed, bool backoff, Put&& put) {
    bool ok = true;
    for (uint32_t i0 = 0; i0 < n; i0 += B) {
        u64 e[B];
        for (uint32_t spins = 0;; ++spins) {
            bool all = true;
#pragma unroll
            for (int q = 0; q < B; ++q) e[q] = i0 + q < n ? ld_tagged(src + static_cast<size_t>(i0 + q) * stride) : (static_cast<u64>(tag) << 32);
#pragma unroll
            for (int q = 0; q < B; ++q) all = all && static_cast<uint32_t>(e[q] >> 32) == tag;
            if (all) break;
            if (spins >= limit || *failed) {
                ok = false;
                limit = 0u;   // nothing after a wait that ran out waits again
                break;
            }
            if (backoff) __nanosleep(128);   // a warp that trails the products on purpose polls gently
        }
#pragma unroll
        for (int q = 0; q < B; ++q)
            if (i0 + q < n) put(i0 + q, __uint_as_float(static_cast<uint32_t>(e[q])));
    }
    return ok;
}

// Shared memory: [n_stages][stage_bytes] | per gather warp: Dx copy, codes [2][codes_bytes], scales [2][16]
template <int MT>
__global__ void __launch_bounds__(kThreads, 1) hsdr_gemv_queue_kernel(const __grid_constant__ QParams p) {
    extern __shared__ __align__(128) unsigned char qsm[];
    __shared__ __align__(8) u64 full_bar[kMaxStages], empty_bar[kMaxStages];
    __shared__ int failed_s;
    __shared__ uint32_t tag_s;
    __shared__ float ssq_s[kProductWarps][kMaxTokens];
    __shared__ float inv_s[kMaxTokens];
    asm volatile("griddepcontrol.launch_dependents;");
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const uint32_t NS = p.n_stages;
    if (tid == 0) {
        stamp(p, 0, 5);
        for (uint32_t s = 0; s < NS; ++s) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&full_bar[s])));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(&empty_bar[s])), "r"(kProductWarps));
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        failed_s = 0;
    }
    __syncthreads();
    const volatile int* failed = &failed_s;

    // Unit u of the flat list -> (task, atom group); `ti` only ever moves forward.
    auto task_of = [&](uint32_t u, uint32_t& ti) {
        while (ti + 1u < p.n_tasks && u >= p.task[ti + 1u].unit0) ++ti;
    };
    auto stages_of = [&](const QTask& t) { return (t.C + kSlab - 1u) / kSlab; };

    if (warp == 0) {
        // ================= loader =================
        uint32_t it_issue = 0, it_fill = 0;                 // stage counters over this CTA's whole walk
        uint32_t ui = blockIdx.x, us = 0, uti = 0;           // weight cursor: unit, slab within it, task
        uint32_t fi = blockIdx.x, fs = 0, fti = 0;           // activation cursor
        bool ok = true;
        auto issue = [&]() {   // dictionary rows of (ui, us) into slot it_issue % NS
            task_of(ui, uti);
            const QTask& t = p.task[uti];
            const uint32_t slot = it_issue % NS;
            const uint32_t atom0 = (ui - t.unit0) * kAtomsPerUnit;
            const uint32_t c0 = us * kSlab;
            const uint32_t cw = min(kSlab, t.C - c0);
            const uint32_t n_atoms = min(kAtomsPerUnit, t.K - atom0);
            const uint32_t bar = smem_u32(&full_bar[slot]);
            if (lane == 0)
                asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(n_atoms * cw * 4u)
                             : "memory");
            __syncwarp();
            if (lane == 0) {
                // the stage's rows are ONE block of the re-laid dictionary (stage_blocks_kernel): one copy
                // (eight copies of one row slab each kept the loader busy issuing: 10 % of the pass)
                const float* src = t.D + static_cast<size_t>(atom0) * t.C + static_cast<size_t>(n_atoms) * c0;
                const uint32_t dst = smem_u32(qsm + static_cast<size_t>(slot) * p.stage_bytes);
                asm volatile(
                    "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                    "l"(src), "r"(n_atoms * cw * 4u), "r"(bar)
                    : "memory");
            }
            ++it_issue;
            if (++us == stages_of(t)) {
                us = 0;
                ui += gridDim.x;
            }
        };
        auto fill = [&]() {   // activations of (fi, fs) into slot it_fill % NS; then the stage is armed
            task_of(fi, fti);
            const QTask& t = p.task[fti];
            const uint32_t slot = it_fill % NS;
            const uint32_t c0 = fs * kSlab;
            const uint32_t cw = min(kSlab, t.C - c0);
            float* xs = reinterpret_cast<float*>(qsm + static_cast<size_t>(slot) * p.stage_bytes + kAtomsPerUnit * kSlab * 4u);
            const uint32_t bar = smem_u32(&full_bar[slot]);
            if (t.x_kind == X_PLAIN) {
                const XView xv = x_view(t);
                const bool rows_contig = xv.layout == CSDR_LAYOUT_TOKEN_MAJOR || xv.Mtotal == 1;
                if (xv.dtype == CSDR_DTYPE_F32 && rows_contig &&
                    ((reinterpret_cast<uintptr_t>(xv.x) | (static_cast<uintptr_t>(xv.C) * 4u)) & 15u) == 0) {
                    // one bulk copy per token, completing on the stage's barrier like the weights
                    if (lane == 0)
                        asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(xv.M * cw * 4u)
                                     : "memory");
                    __syncwarp();
                    if (lane < xv.M) {
                        const float* src = static_cast<const float*>(xv.x) + static_cast<size_t>(lane) * xv.C + c0;
                        asm volatile(
                            "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                                smem_u32(xs + lane * kSlab)),
                            "l"(src), "r"(cw * 4u), "r"(bar)
                            : "memory");
                    }
                } else {
                    for (uint32_t i = lane; i < MT * kSlab; i += 32u) {
                        const uint32_t b = i / kSlab, c = i - b * kSlab;
                        if (c < cw && b < xv.M) xs[i] = load_x(xv, c0 + c, b);
                    }
                }
            }   // X_TAGGED: the product warps fetch the slab themselves when they reach the stage
            __syncwarp();
            if (lane == 0) {
                u64 st;
                asm volatile("mbarrier.arrive.release.cta.shared::cta.b64 %0, [%1];" : "=l"(st) : "r"(bar) : "memory");
                (void)st;
            }
            ++it_fill;
            if (++fs == stages_of(t)) {
                fs = 0;
                fi += gridDim.x;
            }
        };
        // The first weight copies do not depend on anything before this launch: two stages go out
        // ahead of the dependency wait. Not the whole ring: the launch tag and the first activation
        // slabs are small loads that would queue up behind 160 KB of weight traffic per SM (the tag
        // came back 2 us late with five stages ahead of it); the loop below fills the rest of the
        // ring, activations first.
        if (lane == 0) stamp(p, 1, 7);
        while (ui < p.n_units && it_issue < min(NS, 2u)) issue();
        if (lane == 0) stamp(p, 3, 7);
        asm volatile("griddepcontrol.wait;" ::: "memory");
        if (lane == 0) stamp(p, 4, 7);
        if (lane == 0) {
            tag_s = read_launch_tag(p.seq);
            stamp(p, 0, 6);
        }
        asm volatile("bar.sync 3, %0;" ::"n"(kThreads) : "memory");
        while (ok && (it_fill < it_issue || ui < p.n_units)) {
            while (it_fill < it_issue) fill();
            if (ui < p.n_units) {
                // slot of the next stage: free once the products have drained its previous use
                const uint32_t slot = it_issue % NS, use = it_issue / NS;
                if (!mbar_wait(smem_u32(&empty_bar[slot]), (use - 1u) & 1u, p.spin_barrier, failed)) {
                    ok = false;
                    break;
                }
                issue();
            }
        }
        // CTA 0's loader has nothing left to do: it retires the launch's tag for the next launch
        if (blockIdx.x == 0 && !retire_launch_tag(p.seq, tag_s, lane, p.spin_poll)) ok = false;
        if (!ok) {
            if (lane == 0) {
                failed_s = 1;
                atomicExch(p.status, 1);
            }
            // weight copies still in flight land in this CTA's shared memory: complete the phases that
            // were armed with bytes but never received their arrival, then wait for the bytes
            for (uint32_t itx = it_fill; itx < it_issue; ++itx) {
                if (lane == 0) {
                    u64 st;
                    asm volatile("mbarrier.arrive.release.cta.shared::cta.b64 %0, [%1];"
                                 : "=l"(st)
                                 : "r"(smem_u32(&full_bar[itx % NS]))
                                 : "memory");
                    (void)st;
                }
            }
            __syncwarp();
            volatile int never = 0;
            for (uint32_t back = 0; back < NS && back < it_issue; ++back) {
                const uint32_t itx = it_issue - 1u - back;
                mbar_wait(smem_u32(&full_bar[itx % NS]), (itx / NS) & 1u, p.spin_barrier, &never);
            }
        }
    } else if (warp <= kProductWarps) {
        // ================= products =================
        asm volatile("griddepcontrol.wait;" ::: "memory");
        asm volatile("bar.sync 3, %0;" ::"n"(kThreads) : "memory");
        const uint32_t tag = tag_s;
        const uint32_t w = warp - 1u;                         // atom within the unit
        uint32_t limit = *reinterpret_cast<const volatile int*>(p.status) != 0 ? 0u : p.spin_poll;
        uint32_t it = 0, ti = 0;
        bool ok = true;
        for (uint32_t u = blockIdx.x; u < p.n_units; u += gridDim.x) {
            task_of(u, ti);
            const QTask& t = p.task[ti];
            const uint32_t atom = (u - t.unit0) * kAtomsPerUnit + w;
            const uint32_t n_st = stages_of(t);
            float acc[MT], ssq[MT];
#pragma unroll
            for (int b = 0; b < MT; ++b) acc[b] = ssq[b] = 0.0f;
            for (uint32_t s = 0; s < n_st; ++s, ++it) {
                const uint32_t slot = it % NS;
                unsigned char* st = qsm + static_cast<size_t>(slot) * p.stage_bytes;
                const uint32_t cw = min(kSlab, t.C - s * kSlab);
                if (t.x_kind == X_TAGGED) {
                    // this warp's eighth of the slab, token by token, 128 columns (four per lane) at a time
                    float* xs = reinterpret_cast<float*>(st + kAtomsPerUnit * kSlab * 4u);
#pragma unroll 1
                    for (uint32_t part = 0; part < kSlab / 1024u; ++part) {
                    const uint32_t c_lane = w * (kSlab / 8u) + part * 128u + lane * 4u;
                    if (c_lane < cw) {
                        const u64* src = static_cast<const u64*>(t.x) + s * kSlab + c_lane;
                        // word i of this lane: token i / 4, column c_lane + i % 4
                        u64 e[4 * MT];
                        for (uint32_t spins = 0;; ++spins) {
                            bool all = true;
#pragma unroll
                            for (int q = 0; q < 4 * MT; ++q) {
                                const uint32_t b = q >> 2;
                                e[q] = b < t.M ? ld_tagged(src + static_cast<size_t>(b) * t.C + (q & 3)) : (static_cast<u64>(tag) << 32);
                            }
#pragma unroll
                            for (int q = 0; q < 4 * MT; ++q) all = all && static_cast<uint32_t>(e[q] >> 32) == tag;
                            if (all) break;
                            if (spins >= limit || *failed) {   // gave up: every role of the CTA stops waiting
                                ok = false;
                                limit = 0u;
                                failed_s = 1;
                                break;
                            }
                            // every product warp of every CTA that owns a unit of this task is waiting here:
                            // polling flat out, they fill the L2 queues the producers' stores have to pass
                            __nanosleep(p.poll_sleep_ns);
                        }
                        float4 wv = make_float4(1.f, 1.f, 1.f, 1.f);
                        if (t.norm_w) wv = __ldg(reinterpret_cast<const float4*>(t.norm_w + s * kSlab + c_lane));
#pragma unroll
                        for (int b = 0; b < MT; ++b) {
                            const float4 h = make_float4(__uint_as_float(static_cast<uint32_t>(e[4 * b])), __uint_as_float(static_cast<uint32_t>(e[4 * b + 1])),
                                                         __uint_as_float(static_cast<uint32_t>(e[4 * b + 2])), __uint_as_float(static_cast<uint32_t>(e[4 * b + 3])));
                            // the squares of the raw values, for the 1 / rms the gather applies behind the product
                            ssq[b] = fmaf(h.x, h.x, fmaf(h.y, h.y, fmaf(h.z, h.z, fmaf(h.w, h.w, ssq[b]))));
                            *reinterpret_cast<float4*>(xs + b * kSlab + c_lane) = make_float4(h.x * wv.x, h.y * wv.y, h.z * wv.z, h.w * wv.w);
                        }
                    }
                    }
                    asm volatile("bar.sync 1, %0;" ::"n"(kProductThreads) : "memory");   // the whole slab is staged
                    if (s == 0 && tid == 32u) stamp(p, ti, 0);
                }
                // after a wait has run out the warp keeps walking its stages (the named barrier above
                // needs all eight warps) but no longer waits or computes
                if (!mbar_wait(smem_u32(&full_bar[slot]), (it / NS) & 1u, ok ? p.spin_barrier : 1u, failed)) {
                    ok = false;
                    failed_s = 1;
                }
                if (ok && atom < t.K) {
                    const float4* d4 = reinterpret_cast<const float4*>(st + static_cast<size_t>(w) * cw * 4u);   // rows packed at the slab's width
                    const float4* x4 = reinterpret_cast<const float4*>(st + kAtomsPerUnit * kSlab * 4u);
                    const uint32_t cw4 = cw >> 2;
#pragma unroll
                    for (uint32_t j = 0; j < kSlab / 128u; ++j) {
                        const uint32_t c4 = j * 32u + lane;
                        if (c4 < cw4) {
                            const float4 d = d4[c4];
#pragma unroll
                            for (int b = 0; b < MT; ++b) {
                                if (static_cast<uint32_t>(b) < t.M) {   // rows past the batch hold nothing
                                    const float4 xv = x4[b * (kSlab / 4u) + c4];
                                    acc[b] = fmaf(d.x, xv.x, acc[b]);
                                    acc[b] = fmaf(d.y, xv.y, acc[b]);
                                    acc[b] = fmaf(d.z, xv.z, acc[b]);
                                    acc[b] = fmaf(d.w, xv.w, acc[b]);
                                }
                            }
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) {
                    u64 stt;
                    asm volatile("mbarrier.arrive.release.cta.shared::cta.b64 %0, [%1];" : "=l"(stt) : "r"(smem_u32(&empty_bar[slot])) : "memory");
                    (void)stt;
                }
            }
            float mine = 0.0f;
#pragma unroll
            for (int b = 0; b < MT; ++b) {
                float v = acc[b];
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, off);
                if (lane == static_cast<uint32_t>(b)) mine = v;
            }
            if (ok && lane < MT && atom < t.K) st_tagged(p.dx + t.dx_off + static_cast<size_t>(atom) * MT + lane, mine, tag);
            if (tid == 32u) stamp(p, ti, 1);
            if (t.norm_w) {
                // every unit has staged the whole activation row; the task's first unit publishes the sum
                // of squares per token: lanes, then warps, in order
#pragma unroll
                for (int b = 0; b < MT; ++b) {
                    float v = ssq[b];
#pragma unroll
                    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, off);
                    if (lane == 0) ssq_s[w][b] = v;
                }
                asm volatile("bar.sync 1, %0;" ::"n"(kProductThreads) : "memory");
                if (u == t.unit0 && w == 0 && lane < t.M && ok) {
                    float v = 0.0f;
                    for (uint32_t q = 0; q < kProductWarps; ++q) v += ssq_s[q][lane];
                    st_tagged(p.sumsq + static_cast<size_t>(ti) * kMaxTokens + lane, v, tag);
                }
                asm volatile("bar.sync 1, %0;" ::"n"(kProductThreads) : "memory");
            }
        }
        if (!ok && lane == 0) atomicExch(p.status, 1);
    } else {
        // ================= gather: four warps =================
        const uint32_t g = warp - (kLoaderWarps + kProductWarps);
        unsigned char* mine = qsm + static_cast<size_t>(NS) * p.stage_bytes + static_cast<size_t>(g) * p.gw_bytes;
        float* dxs = reinterpret_cast<float*>(mine);
        float* dxs0 = reinterpret_cast<float*>(qsm + static_cast<size_t>(NS) * p.stage_bytes);   // warp 0's copy, shared when rows are split
        unsigned char* codes_buf = mine + p.dxs_bytes;
        float* scales_buf = reinterpret_cast<float*>(codes_buf + 2u * static_cast<size_t>(p.codes_bytes));
        const uint32_t t_first = p.split_rows ? 0u : g, t_step = p.split_rows ? 1u : kGatherWarps;
        // rows of task t this warp gathers
        auto my_rows = [&](const QTask& t, uint32_t& row0, uint32_t& rows_here) {
            uint32_t r0 = blockIdx.x * t.rows_per_cta, n = r0 < t.R ? min(t.rows_per_cta, t.R - r0) : 0u;
            if (p.split_rows) {
                const uint32_t per = t.rows_per_cta / kGatherWarps;   // rows_per_cta is a multiple of 8
                const uint32_t lo = min(n, g * per), hi = min(n, (g + 1u) * per);
                r0 += lo;
                n = hi - lo;
            }
            row0 = r0;
            rows_here = n;
        };
        auto fetch_codes = [&](uint32_t ti, uint32_t buf) {   // non-blocking; one commit group per call
            if (ti < p.n_tasks) {
                const QTask& t = p.task[ti];
                uint32_t row0, rows_here;
                my_rows(t, row0, rows_here);
                if (rows_here) {
                    const uint32_t slots = t.S * t.k;
                    const size_t byte0 = static_cast<size_t>(row0) * slots * 2u;
                    const size_t aligned0 = byte0 & ~static_cast<size_t>(15);
                    const uint32_t n16 = (static_cast<uint32_t>(byte0 - aligned0) + rows_here * slots * 2u + 15u) >> 4;
                    unsigned char* dst = codes_buf + buf * static_cast<size_t>(p.codes_bytes);
                    const unsigned char* src = reinterpret_cast<const unsigned char*>(t.codes) + aligned0;
                    for (uint32_t i = lane; i < n16; i += 32u)
                        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst + i * 16u)), "l"(src + i * 16u)
                                     : "memory");
                    float* sc = scales_buf + buf * 16u;
                    if (lane < t.S && lane < 16u)
                        asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(sc + lane)), "l"(t.scales + lane) : "memory");
                }
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        };
        fetch_codes(t_first, 0);                             // static weights: before the dependency wait
        asm volatile("griddepcontrol.wait;" ::: "memory");
        asm volatile("bar.sync 3, %0;" ::"n"(kThreads) : "memory");
        const uint32_t tag = tag_s;
        uint32_t limit = *reinterpret_cast<const volatile int*>(p.status) != 0 ? 0u : p.spin_poll;
        bool late = false;
        uint32_t buf = 0;
        for (uint32_t ti = t_first; ti < p.n_tasks; ti += t_step, buf ^= 1u) {
            const QTask& t = p.task[ti];
            fetch_codes(ti + t_step, buf ^ 1u);
            uint32_t row0, rows_here;
            my_rows(t, row0, rows_here);
            // hand-over. First a light watch on one word per unit (its last atom, first token), so that
            // nobody sweeps the whole slot again and again while the products are still at work; then
            // this task's Dx words, sixteen loads in flight per lane (stragglers are polled where they
            // are). With a task's rows split over the warps, the four warps share ONE copy of Dx: warp 0
            // watches, all 128 threads sweep - every poller less is load off the few L2 lines all CTAs
            // are asking for.
            const bool coop = p.split_rows != 0u;
            const bool cta_rows = blockIdx.x * t.rows_per_cta < t.R;
            float* dx_use = coop ? dxs0 : dxs;
            float inv = 1.0f;
            if (coop ? cta_rows : rows_here != 0u) {
                if (!coop || g == 0) {
                    const uint32_t n_u = t.n_units;
                    const uint32_t n_watch = lane < n_u ? (n_u - lane + 31u) / 32u : 0u;
                    for (uint32_t spins = 0;; ++spins) {
                        bool all = true;
                        for (uint32_t q = 0; q < n_watch; ++q) {
                            const uint32_t unit = lane + q * 32u;
                            const uint32_t atom = min(unit * kAtomsPerUnit + kAtomsPerUnit - 1u, t.K - 1u);
                            all = all && static_cast<uint32_t>(ld_tagged(p.dx + t.dx_off + static_cast<size_t>(atom) * MT) >> 32) == tag;
                        }
                        if (__all_sync(0xFFFFFFFFu, all)) break;
                        if (__any_sync(0xFFFFFFFFu, spins >= limit || *failed)) break;   // the sweep below records the failure
                        __nanosleep(coop ? p.poll_sleep_ns : 256u);
                    }
                    if (g == 0 && lane == 0) stamp(p, ti, 2);
                }
                if (coop) asm volatile("bar.sync 2, %0;" ::"n"(32u * kGatherWarps) : "memory");
                const uint32_t n_w = t.K * MT;
                const uint32_t me = coop ? g * 32u + lane : lane, step = coop ? 32u * kGatherWarps : 32u;
                const uint32_t n_mine = me < n_w ? (n_w - me + step - 1u) / step : 0u;
                if (!poll_words<16>(p.dx + t.dx_off + me, n_mine, step, tag, limit, failed, !coop,
                                    [&](uint32_t i, float v) { dx_use[me + i * step] = v; }))
                    late = true;
                if (t.norm_w) {
                    // 1 / rms of this task's activations: the sum of squares its first unit published
                    float ss = 0.0f;
                    const bool owns = coop ? (g == 0 && lane < t.M) : lane < t.M;
                    if (owns && !poll_words<1>(p.sumsq + static_cast<size_t>(ti) * kMaxTokens + lane, 1u, 1u, tag, limit, failed, false,
                                               [&](uint32_t, float v) { ss = v; }))
                        late = true;
                    const float mine_inv = 1.0f / sqrtf(ss / static_cast<float>(t.C) + t.norm_eps);
                    if (coop) {
                        if (owns) inv_s[lane] = mine_inv;
                    } else {
                        inv = __shfl_sync(0xFFFFFFFFu, mine_inv, lane % MT);
                    }
                }
                if (coop) {
                    asm volatile("bar.sync 2, %0;" ::"n"(32u * kGatherWarps) : "memory");
                    if (t.norm_w) inv = inv_s[lane % MT];
                }
            }
            if (g == 0 && lane == 0) stamp(p, ti, 3);
            asm volatile("cp.async.wait_group 1;" ::: "memory");      // this task's codes (the next task's may still fly)
            __syncwarp();
            const uint32_t b = lane % MT;
            if (rows_here) {
                const uint32_t slots = t.S * t.k;
                const uint32_t skip = static_cast<uint32_t>((static_cast<size_t>(row0) * slots * 2u) & 15u) >> 1;
                const uint16_t* cs = reinterpret_cast<const uint16_t*>(codes_buf + buf * static_cast<size_t>(p.codes_bytes)) + skip;
                const float* sc = scales_buf + buf * 16u;
                constexpr uint32_t RP = 32u / MT;
                for (uint32_t rl = lane / MT; rl < rows_here; rl += RP) {
                    const uint16_t* rc = cs + rl * slots;
                    float accr = 0.0f;
                    for (uint32_t l = 0; l < t.S; ++l) {
                        const float gamma = sc[l];
                        const uint16_t* lc = rc + l * t.k;
                        for (uint32_t k0 = 0; k0 < t.k; k0 += 8u) {
                            float v[8];
#pragma unroll
                            for (int q = 0; q < 8; ++q) {
                                const uint32_t code = k0 + q < t.k ? lc[k0 + q] : 0u;
                                const uint32_t a = code & 0x7FFFu;
                                const float dv = a < t.K ? dx_use[a * MT + b] : 0.0f;
                                v[q] = __fmul_rn((code & 0x8000u) ? -gamma : gamma, dv);
                            }
#pragma unroll
                            for (int q = 0; q < 8; ++q)
                                if (k0 + q < t.k) accr = __fadd_rn(accr, v[q]);
                        }
                    }
                    if (b < t.M) {
                        const uint32_t r = row0 + rl;
                        if (t.norm_w) accr *= inv;
                        if (t.bias) accr += t.bias[r];
                        const size_t tm = static_cast<size_t>(b) * t.R + r;
                        if (t.epilogue == EPI_SWIGLU) {
                            const float gv = t.gate[tm];
                            accr = (gv * (1.0f / (1.0f + expf(-gv)))) * accr;
                        }
                        if (t.residual) accr += t.residual[tm];
                        if (t.y) t.y[t.y_layout == CSDR_LAYOUT_FEATURE_MAJOR ? static_cast<size_t>(r) * t.M + b : tm] = accr;
                        if (t.y_tag) st_tagged(t.y_tag + tm, accr, tag);
                    }
                }
            }
            __syncwarp();   // the warp's code buffer is free for its next task
            if (coop && cta_rows) asm volatile("bar.sync 2, %0;" ::"n"(32u * kGatherWarps) : "memory");   // so is the shared Dx copy
            if (g == 0 && lane == 0) stamp(p, ti, 4);
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        if (late && lane == 0) {
            failed_s = 1;
            atomicExch(p.status, 1);
        }
    }
}

uint32_t stage_bytes_for(int mt) { return kAtomsPerUnit * kSlab * 4u + static_cast<uint32_t>(mt) * kSlab * 4u; }
uint32_t codes_bytes_for(uint32_t max_code_bytes) { return (max_code_bytes + 31u + 127u) & ~127u; }
uint32_t dxs_bytes_for(uint32_t max_k, int mt) { return (max_k * static_cast<uint32_t>(mt) * 4u + 127u) & ~127u; }
size_t tail_bytes_for(uint32_t max_k, int mt, uint32_t max_code_bytes) {
    return static_cast<size_t>(kGatherWarps) * (dxs_bytes_for(max_k, mt) + 2u * codes_bytes_for(max_code_bytes) + 128u);
}
// All the shared memory a CTA can opt into, less the kernel's static part and the per-CTA reserve:
// one CTA per SM anyway, and every stage more is 32 KB more of weights in flight.
size_t smem_budget(const csdr_context* ctx) { return ctx->smem_optin > 4096u ? ctx->smem_optin - 4096u : ctx->smem_optin; }
uint32_t rows_per_cta_for(const csdr_context* ctx, uint32_t rows) {
    const uint32_t G = static_cast<uint32_t>(ctx->sm_count);
    return ((rows + G - 1u) / G + 7u) & ~7u;
}
bool needs_split(const QueueItem* items, uint32_t n) {
    for (uint32_t i = 0; i < n; ++i)
        if (items[i].dep >= 0 || items[i].swiglu_gate || items[i].norm_weight || items[i].residual)
            return true;
    // independent products: a warp per task, the tasks' gathers side by side (with the rows split,
    // one task's hand-over and gather follow the other's: 2.8 us each, measured); a single
    // product has nothing to run beside
    return n < 2u;
}
// bytes of code stream one gather warp stages per task
uint32_t code_bytes_per_warp(const csdr_context* ctx, const Geometry& g, bool split) {
    const uint32_t rpc = rows_per_cta_for(ctx, g.rows);
    return (split ? rpc / kGatherWarps : rpc) * g.slots() * 2u;
}

// The dictionary re-laid for the loader: atoms in groups of eight (a unit), a unit's columns in
// slabs of kSlab, and the rows of one (unit, slab) one behind the other - the bytes of one stage,
// contiguous. Block (u, s) starts at float u * 8 * C + n_u * s * kSlab (n_u = atoms of unit u:
// 8, fewer in the last unit) and holds n_u rows of cw_s = min(kSlab, C - s * kSlab) floats.
__global__ void __launch_bounds__(256)
stage_blocks_kernel(const float* __restrict__ D, uint32_t K, uint32_t C, float* __restrict__ out) {
    const size_t n = static_cast<size_t>(K) * C;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const uint32_t a = static_cast<uint32_t>(i / C), c = static_cast<uint32_t>(i - static_cast<size_t>(a) * C);
        const uint32_t u = a / kAtomsPerUnit, r = a - u * kAtomsPerUnit;
        const uint32_t s = c / kSlab, cc = c - s * kSlab;
        const uint32_t n_u = min(kAtomsPerUnit, K - u * kAtomsPerUnit), cw = min(kSlab, C - s * kSlab);
        out[static_cast<size_t>(u) * kAtomsPerUnit * C + static_cast<size_t>(n_u) * s * kSlab + static_cast<size_t>(r) * cw + cc] = D[i];
    }
}

// Built on a dictionary's first use by the list kernel and kept with it (as many bytes again as the
// atoms): not inside a stream capture, like every first use that allocates.
const DeviceBuffer* stage_blocks_of(csdr_context* ctx, const csdr_segment* seg) {
    DeviceBuffer* atoms = seg->atoms.get();
    if (!atoms->stage_blocks) {
        const Geometry& g = seg->g;
        auto blocks = std::make_shared<DeviceBuffer>(static_cast<size_t>(g.n_atoms) * g.cols * sizeof(float), ctx->device);
        const size_t n = static_cast<size_t>(g.n_atoms) * g.cols;
        LaunchScope ls(ctx, KC_GEMV_QUEUE);
        stage_blocks_kernel<<<static_cast<unsigned>(std::min<size_t>((n + 255) / 256, static_cast<size_t>(ctx->sm_count) * 16)), 256, 0, ctx->stream>>>(
            static_cast<const float*>(atoms->ptr), g.n_atoms, g.cols, static_cast<float*>(blocks->ptr));
        ls.done("stage_blocks_kernel");
        atoms->stage_blocks = blocks;
    }
    return atoms->stage_blocks.get();
}

template <int MT>
void launch_t(csdr_context* ctx, QParams& p, uint32_t max_k, uint32_t max_code_bytes) {
    auto kern = hsdr_gemv_queue_kernel<MT>;
    p.stage_bytes = stage_bytes_for(MT);
    p.codes_bytes = codes_bytes_for(max_code_bytes);
    p.dxs_bytes = dxs_bytes_for(max_k, MT);
    p.gw_bytes = p.dxs_bytes + 2u * p.codes_bytes + 128u;
    const size_t tail = tail_bytes_for(max_k, MT, max_code_bytes);
    const size_t budget = smem_budget(ctx);
    if (tail + 3u * p.stage_bytes > budget) throw Error(CSDR_ERR_LIMIT, "GEMV queue: shared memory need exceeds the device limit");
    p.n_stages = static_cast<uint32_t>(std::min<size_t>(kMaxStages, (budget - tail) / p.stage_bytes));
    const size_t smem = tail + static_cast<size_t>(p.n_stages) * p.stage_bytes;
    ctx->opt_in_smem(reinterpret_cast<const void*>(kern), smem);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(static_cast<unsigned>(ctx->sm_count), 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = ctx->pdl ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    LaunchScope ls(ctx, KC_GEMV_QUEUE);
    CSDR_CUDA(cudaLaunchKernelEx(&cfg, kern, p));
    ls.done("hsdr_gemv_queue_kernel");
}

}  // namespace

bool gemv_queue_supported(const csdr_context* ctx, const QueueItem* items, uint32_t n) {
    if (!ctx->gemv_queue || n == 0) return false;
    const size_t batch = items[0].batch;
    if (batch == 0 || batch > kMaxTokens) return false;
    const int mt = batch <= 1 ? 1 : batch <= 2 ? 2 : 4;
    for (uint32_t i0 = 0; i0 < n; i0 += kMaxQueueTasks) {
        const uint32_t cnt = std::min(kMaxQueueTasks, n - i0);
        const bool split = needs_split(items + i0, cnt);
        uint32_t max_k = 0, max_code_bytes = 0;
        for (uint32_t i = i0; i < i0 + cnt; ++i) {
            const QueueItem& it = items[i];
            const Geometry& g = it.seg->g;
            if (!g.row_tiles() || g.cols % 4u || it.batch != batch) return false;
            if (g.n_atoms > 4096u || g.n_stages > 16u) return false;
            const bool glue = it.residual || it.swiglu_gate || it.norm_weight || it.dep >= 0;
            if (glue && it.y_layout != CSDR_LAYOUT_TOKEN_MAJOR && batch > 1) return false;
            // dependencies point backwards, inside one launch's worth of tasks, at the very buffer read
            if (it.dep >= static_cast<int>(i)) return false;
            if (it.dep >= 0 && it.dep < static_cast<int>(i0)) return false;
            if (it.dep >= 0) {
                const QueueItem& src = items[it.dep];
                if (it.x_dtype != CSDR_DTYPE_F32 || it.seg->g.cols != src.seg->g.rows || it.x != src.y) return false;
                if (src.y_layout != CSDR_LAYOUT_TOKEN_MAJOR && batch > 1) return false;
            }
            if (it.norm_weight && it.dep < 0) return false;   // the norm rides on activations staged by the product warps
            // the SwiGLU epilogue reads the gate rows this warp's own lanes wrote: the task before, same rows
            if (it.swiglu_gate && (i == i0 || items[i - 1].seg->g.rows != g.rows || items[i - 1].y != it.swiglu_gate)) return false;
            max_k = std::max(max_k, g.n_atoms);
            max_code_bytes = std::max(max_code_bytes, code_bytes_per_warp(ctx, g, split));
        }
        // the ring needs three stages beside the gather warps' buffers
        if (tail_bytes_for(max_k, mt, max_code_bytes) + 3u * stage_bytes_for(mt) > smem_budget(ctx)) return false;
    }
    return true;
}

void launch_gemv_queue(csdr_context* ctx, const QueueItem* items, uint32_t n) {
    const uint32_t batch = static_cast<uint32_t>(items[0].batch);
    const int mt = batch <= 1 ? 1 : batch <= 2 ? 2 : 4;
    if (!ctx->queue_sync) {
        CSDR_CUDA(cudaMalloc(&ctx->queue_sync, (2u + kMaxTagCtas) * sizeof(uint32_t)));   // the launch tag words
        CSDR_CUDA(cudaMemsetAsync(ctx->queue_sync, 0, (2u + kMaxTagCtas) * sizeof(uint32_t), ctx->stream));
    }
    for (uint32_t i0 = 0; i0 < n; i0 += kMaxQueueTasks) {
        const uint32_t cnt = std::min(kMaxQueueTasks, n - i0);
        const bool split = needs_split(items + i0, cnt);
        QParams p{};
        // scratch words: sums of squares, Dx slots, then a tagged copy of every output a later task reads
        const size_t sumsq_words = static_cast<size_t>(kMaxQueueTasks) * kMaxTokens;
        size_t words = sumsq_words;
        uint32_t unit = 0, max_k = 0, max_code_bytes = 0;
        size_t tag_off[kMaxQueueTasks] = {};      // 0 = no tagged copy of this task's y
        for (uint32_t i = 0; i < cnt; ++i) {
            const QueueItem& it = items[i0 + i];
            const Geometry& g = it.seg->g;
            QTask& t = p.task[i];
            t.dx_off = static_cast<uint32_t>(words - sumsq_words);
            words += (static_cast<size_t>(g.n_atoms) * mt + 3u) & ~static_cast<size_t>(3);
            if (it.dep >= 0) {
                const uint32_t d = static_cast<uint32_t>(it.dep) - i0;
                if (!tag_off[d]) {
                    tag_off[d] = words;
                    words += static_cast<size_t>(batch) * items[it.dep].seg->g.rows;
                }
            }
        }
        u64* scratch = static_cast<u64*>(ctx->scratch_get(6, std::max<size_t>(words * 8u, 4u << 20)));
        p.sumsq = scratch;
        p.dx = scratch + sumsq_words;
        for (uint32_t i = 0; i < cnt; ++i) {
            const QueueItem& it = items[i0 + i];
            const Geometry& g = it.seg->g;
            QTask& t = p.task[i];
            t.D = static_cast<const float*>(stage_blocks_of(ctx, it.seg)->ptr);
            t.codes = it.seg->codes_ptr();
            t.scales = static_cast<const float*>(it.seg->scales->ptr);
            t.x = it.x;
            t.x_kind = X_PLAIN;
            if (it.dep >= 0) {
                const uint32_t d = static_cast<uint32_t>(it.dep) - i0;
                t.x = scratch + tag_off[d];
                t.x_kind = X_TAGGED;
            }
            t.y = it.y;
            t.y_tag = tag_off[i] ? scratch + tag_off[i] : nullptr;
            t.bias = it.bias;
            t.residual = it.residual;
            t.gate = it.swiglu_gate;
            t.norm_w = it.norm_weight;
            t.norm_eps = it.norm_eps;
            t.K = g.n_atoms;
            t.R = g.rows;
            t.C = g.cols;
            t.S = g.n_stages;
            t.k = g.k;
            t.unit0 = unit;
            t.n_units = (g.n_atoms + kAtomsPerUnit - 1u) / kAtomsPerUnit;
            t.rows_per_cta = rows_per_cta_for(ctx, g.rows);
            t.x_dtype = static_cast<uint32_t>(it.x_dtype);
            t.x_layout = static_cast<uint32_t>(it.x_layout);
            t.y_layout = static_cast<uint32_t>(it.y_layout);
            t.M = batch;
            t.epilogue = it.swiglu_gate ? EPI_SWIGLU : EPI_PLAIN;
            unit += t.n_units;
            max_k = std::max(max_k, g.n_atoms);
            max_code_bytes = std::max(max_code_bytes, code_bytes_per_warp(ctx, g, split));
        }
        p.n_tasks = cnt;
        p.n_units = unit;
        p.split_rows = split ? 1u : 0u;
        p.seq = ctx->queue_sync;
        p.poll_sleep_ns = ctx->queue_poll_sleep_ns;
        p.status = ctx->status_word;
        p.spin_poll = ctx->spin_limit_gemv;
        p.spin_barrier = ctx->spin_limit_barrier;
        p.trace = ctx->gemv_trace ? static_cast<unsigned long long*>(ctx->gemv_trace->ptr) : nullptr;
        switch (mt) {
            case 1: launch_t<1>(ctx, p, max_k, max_code_bytes); break;
            case 2: launch_t<2>(ctx, p, max_k, max_code_bytes); break;
            default: launch_t<4>(ctx, p, max_k, max_code_bytes); break;
        }
    }
}

}  // namespace csdr
