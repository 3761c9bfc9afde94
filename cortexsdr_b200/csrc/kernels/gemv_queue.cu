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
//                       x 1024 columns and the matching slab of the activations, all as
//                       cp.async.bulk copies that signal the stage's mbarrier (activations that
//                       are not fp32 token-major are converted by the warp itself). The dictionary
//                       is static, so the first ring-full of weight copies is issued BEFORE the
//                       programmatic-dependent-launch wait, and across a dependency between two
//                       tasks of the list the weights of the later task are already in flight
//                       while its activations are still being produced.
//   products  (8 warps) one atom per warp: dot products of the staged row slab with the staged
//                       activations, accumulated over the row's slabs in registers, reduced with
//                       warp shuffles, stored as the finished Dx (no column-split partials); the
//                       warp then checks in on the task's counter (release).
//   gather    (4 warps) trails behind, task by task: prefetches its rows of the next task's code
//                       stream (cp.async), waits for the current task's counter (acquire), copies
//                       Dx to shared memory, then the signed gather in the reference's order and
//                       the task's epilogue, and checks in on the task's row counter.
//
// Epilogues fold the decoder glue of api/cortex_sdk.cpp:1569-1679 into the gather so that a block
// of the decoder is one list: bias; residual add (add_vectors, :1234-1243); SwiGLU against an
// earlier task's rows (silu_mul, :1245-1256); and the two halves of RMS normalisation (rms_norm,
// :1208-1232): a task may leave y * w beside y together with per-CTA sums of squares of y, and a
// later task that consumes y * w multiplies its own product by 1 / sqrt(mean + eps).
// A task may name an earlier task of the list whose rows must all be written before its
// activations are read.
//
// Every wait is bounded (mbarrier phases, counters): one that runs out sets the status word, all
// roles of the CTA stop waiting, and the kernel returns. Counters live in two sets used by
// alternate launches; a launch clears the set of the launch after it. All CTAs must be resident
// (grid = SM count, one per SM).
#include <algorithm>

#include "../internal.hpp"
#include "gemv_queue.hpp"
#include "views.cuh"

namespace csdr {

namespace {

constexpr uint32_t kLoaderWarps = 1, kProductWarps = 8, kGatherWarps = 4;
constexpr uint32_t kThreads = 32u * (kLoaderWarps + kProductWarps + kGatherWarps);
constexpr uint32_t kGatherThreads = 32u * kGatherWarps;
constexpr uint32_t kAtomsPerUnit = 8;          // one per product warp
constexpr uint32_t kSlab = 1024;               // columns per stage
constexpr uint32_t kMaxStages = 8;
constexpr uint32_t kMaxTokens = 4;

enum : uint32_t { EPI_PLAIN = 0, EPI_SWIGLU = 1 };

struct QTask {
    const float* D;
    const uint16_t* codes;
    const float* scales;
    const void* x;
    float* y;
    const float* bias;
    const float* residual;    // [M][R] token-major, may alias y
    const float* gate;        // EPI_SWIGLU: the gate projection's rows, [M][R]
    const float* prep_w;      // leave y * w in prep_out and this CTA's sums of squares of y in the task's slot
    float* prep_out;
    uint32_t K, R, C, S, k;
    uint32_t unit0;           // first flat unit of this task
    uint32_t n_units;
    uint32_t dx_off;          // float offset of its Dx slot: [K][MT]
    uint32_t rows_per_cta;
    uint32_t x_dtype, x_layout, y_layout;
    uint32_t M;
    int32_t dep;              // earlier task whose rows must be complete before x is read, or -1
    int32_t scale_from;       // earlier task whose sums of squares normalise this product, or -1
    float scale_eps, scale_inv_width;
    uint32_t epilogue;
};

struct QParams {
    QTask task[kMaxQueueTasks];
    uint32_t n_tasks, n_units;
    uint32_t n_stages;          // ring depth
    uint32_t stage_bytes;       // D slab + x slab
    uint32_t codes_bytes;       // one code buffer of the gather role
    float* dx;                  // Dx slots
    float* sumsq;               // [task][grid][kMaxTokens] per-CTA sums of squares
    uint32_t* seq;              // [0] queue launches completed, [1] CTAs that have read [0]
    uint32_t* counters;         // [2 sets][kMaxQueueTasks][2]: products checked in, CTAs whose rows are written
    int* status;
    uint32_t spin_poll, spin_barrier;
};

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

// Bounded wait until a counter reaches its target (acquire): one look, then at most `limit` more.
__device__ __forceinline__ bool count_wait(const uint32_t* c, uint32_t target, uint32_t limit, const volatile int* failed) {
    for (uint32_t i = 0;; ++i) {
        uint32_t v;
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(c) : "memory");
        if (v >= target) return true;
        if (i >= limit || *failed) return false;
    }
}

__device__ __forceinline__ void count_arrive(uint32_t* c) {
    asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(c) : "memory");
}

// Queue launches completed so far; its parity names this launch's counter set. The thread that
// calls this checks in (acq_rel) after reading; the CTA that checks in last knows every CTA has
// read the count and advances it for the next launch.
__device__ __forceinline__ uint32_t take_launch_index(uint32_t* seq) {
    uint32_t done, prev;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(done) : "l"(seq) : "memory");
    asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(prev) : "l"(seq + 1) : "memory");
    if (prev == gridDim.x - 1u) {
        seq[1] = 0u;
        asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(seq), "r"(done + 1u) : "memory");
    }
    return done;
}

__device__ __forceinline__ XView x_view(const QTask& t) {
    return XView{t.x, static_cast<int>(t.x_dtype), static_cast<int>(t.x_layout), t.C, t.M, 0u, t.M};
}

// Shared memory: [n_stages][stage_bytes] | dxs [max K][MT] | codes [2][codes_bytes] | scales [2][16]
template <int MT>
__global__ void __launch_bounds__(kThreads, 1) hsdr_gemv_queue_kernel(const __grid_constant__ QParams p) {
    extern __shared__ __align__(128) unsigned char qsm[];
    __shared__ __align__(8) unsigned long long full_bar[kMaxStages], empty_bar[kMaxStages];
    __shared__ int failed_s;
    __shared__ uint32_t set_s;
    __shared__ float red_s[kGatherThreads];
    __shared__ float inv_s[kMaxTokens];
    asm volatile("griddepcontrol.launch_dependents;");
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const uint32_t NS = p.n_stages;
    if (tid == 0) {
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
        uint32_t dep_seen = 0xFFFFFFFFu;                     // task whose dependency has been awaited
        const uint32_t* cnt = nullptr;                       // this launch's counter set (known after the wait)
        uint32_t limit = p.spin_poll;
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
            if (lane < n_atoms) {
                const float* src = t.D + static_cast<size_t>(atom0 + lane) * t.C + c0;
                const uint32_t dst = smem_u32(qsm + static_cast<size_t>(slot) * p.stage_bytes + lane * (kSlab * 4u));
                asm volatile(
                    "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                    "l"(src), "r"(cw * 4u), "r"(bar)
                    : "memory");
            }
            ++it_issue;
            if (++us == stages_of(t)) {
                us = 0;
                ui += gridDim.x;
            }
        };
        auto fill = [&]() -> bool {   // activations of (fi, fs) into slot it_fill % NS; then the stage is armed
            task_of(fi, fti);
            const QTask& t = p.task[fti];
            if (t.dep >= 0 && dep_seen != fti) {
                // the rows this task reads are written by another task of the list
                int seen = 1;
                if (lane == 0) seen = count_wait(cnt + 2 * t.dep + 1, gridDim.x, limit, failed) ? 1 : 0;
                seen = __shfl_sync(0xFFFFFFFFu, seen, 0);
                if (!seen) return false;
                asm volatile("fence.proxy.async;" ::: "memory");   // the bulk copies below read those rows
                dep_seen = fti;
            }
            const uint32_t slot = it_fill % NS;
            const uint32_t c0 = fs * kSlab;
            const uint32_t cw = min(kSlab, t.C - c0);
            float* xs = reinterpret_cast<float*>(qsm + static_cast<size_t>(slot) * p.stage_bytes + kAtomsPerUnit * kSlab * 4u);
            const uint32_t bar = smem_u32(&full_bar[slot]);
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
            __syncwarp();
            if (lane == 0) {
                unsigned long long st;
                asm volatile("mbarrier.arrive.release.cta.shared::cta.b64 %0, [%1];" : "=l"(st) : "r"(bar) : "memory");
                (void)st;
            }
            ++it_fill;
            if (++fs == stages_of(t)) {
                fs = 0;
                fi += gridDim.x;
            }
            return true;
        };
        // the first ring-full of weight copies does not depend on anything before this launch
        while (ui < p.n_units && it_issue < NS) issue();
        asm volatile("griddepcontrol.wait;" ::: "memory");
        if (lane == 0) {
            const uint32_t done = take_launch_index(p.seq);
            set_s = done & 1u;
            // the other set belongs to the launch after this one: clear it (its last user has finished)
            if (blockIdx.x == 0) {
                uint32_t* other = p.counters + ((done + 1u) & 1u) * (2u * kMaxQueueTasks);
                for (uint32_t i = 0; i < 2u * kMaxQueueTasks; ++i) other[i] = 0u;
            }
        }
        asm volatile("bar.sync 3, %0;" ::"n"(kThreads) : "memory");
        cnt = p.counters + set_s * (2u * kMaxQueueTasks);
        if (*reinterpret_cast<const volatile int*>(p.status) != 0) limit = 0u;
        while (ok && (it_fill < it_issue || ui < p.n_units)) {
            while (ok && it_fill < it_issue) ok = fill();
            if (ok && ui < p.n_units) {
                // slot of the next stage: free once the products have drained its previous use
                const uint32_t slot = it_issue % NS, use = it_issue / NS;
                if (!mbar_wait(smem_u32(&empty_bar[slot]), (use - 1u) & 1u, p.spin_barrier, failed)) {
                    ok = false;
                    break;
                }
                issue();
            }
        }
        if (!ok) {
            if (lane == 0) {
                failed_s = 1;
                atomicExch(p.status, 1);
            }
            // weight copies still in flight land in this CTA's shared memory: complete the phases that
            // were armed with bytes but never received their arrival, then wait for the bytes
            for (uint32_t itx = it_fill; itx < it_issue; ++itx) {
                if (lane == 0) {
                    unsigned long long st;
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
        uint32_t* cnt = p.counters + set_s * (2u * kMaxQueueTasks);
        const uint32_t w = warp - 1u;                         // atom within the unit
        uint32_t it = 0, ti = 0;
        bool ok = true;
        for (uint32_t u = blockIdx.x; ok && u < p.n_units; u += gridDim.x) {
            task_of(u, ti);
            const QTask& t = p.task[ti];
            const uint32_t atom = (u - t.unit0) * kAtomsPerUnit + w;
            const uint32_t n_st = stages_of(t);
            float acc[MT];
#pragma unroll
            for (int b = 0; b < MT; ++b) acc[b] = 0.0f;
            for (uint32_t s = 0; s < n_st; ++s, ++it) {
                const uint32_t slot = it % NS;
                if (!mbar_wait(smem_u32(&full_bar[slot]), (it / NS) & 1u, p.spin_barrier, failed)) {
                    ok = false;
                    break;
                }
                if (atom < t.K) {
                    const unsigned char* st = qsm + static_cast<size_t>(slot) * p.stage_bytes;
                    const float4* d4 = reinterpret_cast<const float4*>(st + w * (kSlab * 4u));
                    const float4* x4 = reinterpret_cast<const float4*>(st + kAtomsPerUnit * kSlab * 4u);
                    const uint32_t cw4 = min(kSlab, t.C - s * kSlab) >> 2;
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
                    unsigned long long stt;
                    asm volatile("mbarrier.arrive.release.cta.shared::cta.b64 %0, [%1];" : "=l"(stt) : "r"(smem_u32(&empty_bar[slot])) : "memory");
                    (void)stt;
                }
            }
            if (!ok) break;
            float mine = 0.0f;
#pragma unroll
            for (int b = 0; b < MT; ++b) {
                float v = acc[b];
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, off);
                if (lane == static_cast<uint32_t>(b)) mine = v;
            }
            if (lane < MT && atom < t.K) p.dx[t.dx_off + static_cast<size_t>(atom) * MT + lane] = mine;
            __syncwarp();
            if (lane == 0) count_arrive(cnt + 2 * ti);          // this warp's share of the task's Dx is written
        }
        if (!ok && lane == 0) {
            failed_s = 1;
            atomicExch(p.status, 1);
        }
    } else {
        // ================= gather =================
        const uint32_t gt = tid - 32u * (kLoaderWarps + kProductWarps);
        unsigned char* tail = qsm + static_cast<size_t>(NS) * p.stage_bytes;
        uint32_t max_k = 0;
        for (uint32_t i = 0; i < p.n_tasks; ++i) max_k = max(max_k, p.task[i].K);
        float* dxs = reinterpret_cast<float*>(tail);
        unsigned char* codes_buf = tail + ((static_cast<size_t>(max_k) * MT * 4u + 127u) & ~static_cast<size_t>(127));
        float* scales_buf = reinterpret_cast<float*>(codes_buf + 2u * static_cast<size_t>(p.codes_bytes));
        auto fetch_codes = [&](uint32_t ti) {   // this CTA's rows of task ti's code stream, non-blocking
            const QTask& t = p.task[ti];
            const uint32_t row0 = blockIdx.x * t.rows_per_cta;
            if (row0 < t.R) {
                const uint32_t rows_here = min(t.rows_per_cta, t.R - row0);
                const uint32_t slots = t.S * t.k;
                const size_t byte0 = static_cast<size_t>(row0) * slots * 2u;
                const size_t aligned0 = byte0 & ~static_cast<size_t>(15);
                const uint32_t n16 = (static_cast<uint32_t>(byte0 - aligned0) + rows_here * slots * 2u + 15u) >> 4;
                unsigned char* dst = codes_buf + (ti & 1u) * static_cast<size_t>(p.codes_bytes);
                const unsigned char* src = reinterpret_cast<const unsigned char*>(t.codes) + aligned0;
                for (uint32_t i = gt; i < n16; i += kGatherThreads)
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst + i * 16u)), "l"(src + i * 16u)
                                 : "memory");
                float* sc = scales_buf + (ti & 1u) * 16u;
                for (uint32_t i = gt; i < t.S && i < 16u; i += kGatherThreads)
                    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(sc + i)), "l"(t.scales + i) : "memory");
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        };
        fetch_codes(0);                                      // static weights: before the dependency wait
        asm volatile("griddepcontrol.wait;" ::: "memory");
        asm volatile("bar.sync 3, %0;" ::"n"(kThreads) : "memory");
        uint32_t* cnt = p.counters + set_s * (2u * kMaxQueueTasks);
        uint32_t limit = *reinterpret_cast<const volatile int*>(p.status) != 0 ? 0u : p.spin_poll;
        bool late = false;
        for (uint32_t ti = 0; ti < p.n_tasks; ++ti) {
            const QTask& t = p.task[ti];
            if (ti + 1u < p.n_tasks) fetch_codes(ti + 1u);
            else asm volatile("cp.async.commit_group;" ::: "memory");
            const uint32_t row0 = blockIdx.x * t.rows_per_cta;
            const bool active = row0 < t.R;
            // hand-over: every product warp of every unit of this task has checked in
            if (gt == 0) {
                bool seen = count_wait(cnt + 2 * ti, t.n_units * kProductWarps, limit, failed);
                if (seen && t.scale_from >= 0) seen = count_wait(cnt + 2 * t.scale_from + 1, gridDim.x, limit, failed);
                if (!seen) {
                    late = true;
                    failed_s = 1;
                }
            }
            asm volatile("bar.sync 2, %0;" ::"n"(kGatherThreads) : "memory");
            if (*failed) limit = 0u;
            if (active) {
                const float* src = p.dx + t.dx_off;
                const uint32_t n4 = (t.K * MT) >> 2;
                for (uint32_t i = gt; i < n4; i += kGatherThreads)
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dxs + i * 4u)), "l"(src + i * 4u) : "memory");
                for (uint32_t i = (n4 << 2) + gt; i < t.K * MT; i += kGatherThreads) dxs[i] = __ldcg(src + i);
            }
            if (t.scale_from >= 0 && gt < t.M) {
                // 1 / rms of the rows this task's activations came from: the per-CTA sums in CTA order
                const float* ps = p.sumsq + static_cast<size_t>(t.scale_from) * gridDim.x * kMaxTokens + gt;
                float ss = 0.0f;
                for (uint32_t c = 0; c < gridDim.x; ++c) ss += __ldcg(ps + static_cast<size_t>(c) * kMaxTokens);
                inv_s[gt] = 1.0f / sqrtf(ss * t.scale_inv_width + t.scale_eps);
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
            asm volatile("cp.async.wait_group 0;" ::: "memory");      // this task's codes and Dx (the next task's codes flew during the wait above)
            asm volatile("bar.sync 2, %0;" ::"n"(kGatherThreads) : "memory");
            float ss_mine = 0.0f;
            const uint32_t b = gt % MT;
            if (active) {
                const uint32_t rows_here = min(t.rows_per_cta, t.R - row0);
                const uint32_t slots = t.S * t.k;
                const uint32_t skip = static_cast<uint32_t>((static_cast<size_t>(row0) * slots * 2u) & 15u) >> 1;
                const uint16_t* cs = reinterpret_cast<const uint16_t*>(codes_buf + (ti & 1u) * static_cast<size_t>(p.codes_bytes)) + skip;
                const float* sc = scales_buf + (ti & 1u) * 16u;
                constexpr uint32_t RP = kGatherThreads / MT;
                const float inv = t.scale_from >= 0 && b < t.M ? inv_s[b] : 1.0f;
                for (uint32_t rl = gt / MT; rl < rows_here; rl += RP) {
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
                                const float dv = a < t.K ? dxs[a * MT + b] : 0.0f;
                                v[q] = __fmul_rn((code & 0x8000u) ? -gamma : gamma, dv);
                            }
#pragma unroll
                            for (int q = 0; q < 8; ++q)
                                if (k0 + q < t.k) accr = __fadd_rn(accr, v[q]);
                        }
                    }
                    if (b < t.M) {
                        const uint32_t r = row0 + rl;
                        if (t.scale_from >= 0) accr *= inv;
                        if (t.bias) accr += t.bias[r];
                        const size_t tm = static_cast<size_t>(b) * t.R + r;
                        if (t.epilogue == EPI_SWIGLU) {
                            const float g = t.gate[tm];
                            accr = (g * (1.0f / (1.0f + expf(-g)))) * accr;
                        }
                        if (t.residual) accr += t.residual[tm];
                        const size_t yi = t.y_layout == CSDR_LAYOUT_FEATURE_MAJOR ? static_cast<size_t>(r) * t.M + b : tm;
                        t.y[yi] = accr;
                        if (t.prep_w) {
                            t.prep_out[tm] = accr * t.prep_w[r];
                            ss_mine = fmaf(accr, accr, ss_mine);
                        }
                    }
                }
            }
            if (t.prep_w) {
                // this CTA's sums of squares per token, added up in thread order
                red_s[gt] = ss_mine;
                asm volatile("bar.sync 2, %0;" ::"n"(kGatherThreads) : "memory");
                if (gt < kMaxTokens) {
                    float ss = 0.0f;
                    if (gt < MT)
                        for (uint32_t j = gt; j < kGatherThreads; j += MT) ss += red_s[j];
                    p.sumsq[(static_cast<size_t>(ti) * gridDim.x + blockIdx.x) * kMaxTokens + gt] = ss;
                }
            }
            asm volatile("bar.sync 2, %0;" ::"n"(kGatherThreads) : "memory");   // rows written; dxs and the code buffer are free
            if (gt == 0) count_arrive(cnt + 2 * ti + 1);
        }
        if (late && gt == 0) atomicExch(p.status, 1);
    }
}

uint32_t stage_bytes_for(int mt) { return kAtomsPerUnit * kSlab * 4u + static_cast<uint32_t>(mt) * kSlab * 4u; }
uint32_t codes_bytes_for(uint32_t max_code_bytes) { return (max_code_bytes + 31u + 127u) & ~127u; }
size_t tail_bytes_for(uint32_t max_k, int mt, uint32_t max_code_bytes) {
    return ((static_cast<size_t>(max_k) * mt * 4u + 127u) & ~static_cast<size_t>(127)) + 2u * codes_bytes_for(max_code_bytes) + 128u;
}
size_t smem_budget(const csdr_context* ctx) { return std::min<size_t>(ctx->smem_optin, 216u * 1024u); }
uint32_t rows_per_cta_for(const csdr_context* ctx, uint32_t rows) {
    const uint32_t G = static_cast<uint32_t>(ctx->sm_count);
    return ((rows + G - 1u) / G + 7u) & ~7u;
}

template <int MT>
void launch_t(csdr_context* ctx, QParams& p, uint32_t max_k, uint32_t max_code_bytes) {
    auto kern = hsdr_gemv_queue_kernel<MT>;
    p.stage_bytes = stage_bytes_for(MT);
    p.codes_bytes = codes_bytes_for(max_code_bytes);
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
    uint32_t max_k = 0, max_code_bytes = 0;
    for (uint32_t i = 0; i < n; ++i) {
        const QueueItem& it = items[i];
        const Geometry& g = it.seg->g;
        if (!g.row_tiles() || g.cols % 4u || it.batch != batch) return false;
        if (g.n_atoms > 4096u || g.n_stages > 16u) return false;
        const bool glue = it.residual || it.swiglu_gate || it.prep_weight || it.scale_from >= 0;
        if (glue && it.y_layout != CSDR_LAYOUT_TOKEN_MAJOR && batch > 1) return false;
        // dependencies point backwards, inside one launch's worth of tasks
        const int first = static_cast<int>(i / kMaxQueueTasks * kMaxQueueTasks);
        if (it.dep >= static_cast<int>(i) || it.scale_from >= static_cast<int>(i)) return false;
        if ((it.dep >= 0 && it.dep < first) || (it.scale_from >= 0 && it.scale_from < first)) return false;
        if (it.prep_weight && !it.prep_out) return false;
        // the SwiGLU epilogue reads the gate rows this CTA's own threads wrote: same row count, earlier task
        if (it.swiglu_gate && (i == static_cast<uint32_t>(first) || items[i - 1].seg->g.rows != g.rows || items[i - 1].y != it.swiglu_gate))
            return false;
        max_k = std::max(max_k, g.n_atoms);
        max_code_bytes = std::max(max_code_bytes, rows_per_cta_for(ctx, g.rows) * g.slots() * 2u);
    }
    // the ring needs three stages beside the gather role's buffers
    return tail_bytes_for(max_k, mt, max_code_bytes) + 3u * stage_bytes_for(mt) <= smem_budget(ctx);
}

void launch_gemv_queue(csdr_context* ctx, const QueueItem* items, uint32_t n) {
    const uint32_t batch = static_cast<uint32_t>(items[0].batch);
    const int mt = batch <= 1 ? 1 : batch <= 2 ? 2 : 4;
    const uint32_t G = static_cast<uint32_t>(ctx->sm_count);
    if (!ctx->queue_sync) {
        // [0..1] launch counter pair, then two counter sets; zeroed once, the launches keep them so
        const size_t words = 2u + 2u * 2u * kMaxQueueTasks;
        CSDR_CUDA(cudaMalloc(&ctx->queue_sync, words * sizeof(uint32_t)));
        CSDR_CUDA(cudaMemsetAsync(ctx->queue_sync, 0, words * sizeof(uint32_t), ctx->stream));
    }
    for (uint32_t i0 = 0; i0 < n; i0 += kMaxQueueTasks) {
        const uint32_t cnt = std::min(kMaxQueueTasks, n - i0);
        QParams p{};
        uint32_t unit = 0, dx_off = 0, max_k = 0, max_code_bytes = 0;
        for (uint32_t i = 0; i < cnt; ++i) {
            const QueueItem& it = items[i0 + i];
            const Geometry& g = it.seg->g;
            QTask& t = p.task[i];
            t.D = static_cast<const float*>(it.seg->atoms->ptr);
            t.codes = it.seg->codes_ptr();
            t.scales = static_cast<const float*>(it.seg->scales->ptr);
            t.x = it.x;
            t.y = it.y;
            t.bias = it.bias;
            t.residual = it.residual;
            t.gate = it.swiglu_gate;
            t.prep_w = it.prep_weight;
            t.prep_out = it.prep_out;
            t.K = g.n_atoms;
            t.R = g.rows;
            t.C = g.cols;
            t.S = g.n_stages;
            t.k = g.k;
            t.unit0 = unit;
            t.n_units = (g.n_atoms + kAtomsPerUnit - 1u) / kAtomsPerUnit;
            t.dx_off = dx_off;
            t.rows_per_cta = rows_per_cta_for(ctx, g.rows);
            t.x_dtype = static_cast<uint32_t>(it.x_dtype);
            t.x_layout = static_cast<uint32_t>(it.x_layout);
            t.y_layout = static_cast<uint32_t>(it.y_layout);
            t.M = batch;
            t.dep = it.dep >= 0 ? it.dep - static_cast<int>(i0) : -1;
            t.scale_from = it.scale_from >= 0 ? it.scale_from - static_cast<int>(i0) : -1;
            t.scale_eps = it.scale_eps;
            t.scale_inv_width = it.scale_width ? 1.0f / static_cast<float>(it.scale_width) : 0.0f;
            t.epilogue = it.swiglu_gate ? EPI_SWIGLU : EPI_PLAIN;
            unit += t.n_units;
            dx_off += (g.n_atoms * static_cast<uint32_t>(mt) + 3u) & ~3u;
            max_k = std::max(max_k, g.n_atoms);
            max_code_bytes = std::max(max_code_bytes, t.rows_per_cta * g.slots() * 2u);
        }
        p.n_tasks = cnt;
        p.n_units = unit;
        const size_t sumsq_floats = static_cast<size_t>(kMaxQueueTasks) * G * kMaxTokens;
        float* scratch = static_cast<float*>(
            ctx->scratch_get(6, std::max<size_t>((static_cast<size_t>(dx_off) + sumsq_floats) * 4u, 2u << 20)));
        p.sumsq = scratch;
        p.dx = scratch + sumsq_floats;
        p.seq = ctx->queue_sync;
        p.counters = ctx->queue_sync + 2;
        p.status = ctx->status_word;
        p.spin_poll = ctx->spin_limit_gemv;
        p.spin_barrier = ctx->spin_limit_barrier;
        switch (mt) {
            case 1: launch_t<1>(ctx, p, max_k, max_code_bytes); break;
            case 2: launch_t<2>(ctx, p, max_k, max_code_bytes); break;
            default: launch_t<4>(ctx, p, max_k, max_code_bytes); break;
        }
    }
}

}  // namespace csdr
