// A queue of decode GEMVs in ONE persistent launch, for 1-D row-tile HSDR segments on sm_100a.
//
// The reference issues every y = W x as its own call (matmulRowMajor,
// strategies/HierarchicalSDRStrategy.cpp:1257-1338: Dx = D x, then a signed gather over Dx per
// output row), and so does a chain of single launches: each pays the same latencies in a row -
// activations in, partial results across, gather, kernel boundary - while the 9 MB of weights
// need 1.4 us of HBM time. Here a list of independent products (q|k|v, gate|up, the
// heads of a batch of requests, a benchmark's weight copies) runs as one grid of one CTA per SM
// whose warps have three roles that never wait for each other inside a task:
//
//   loader    (1 warp)  walks the flat list of work units (task, group of 8 atoms) this CTA owns
//                       and keeps a ring of shared-memory stages full: per stage 8 dictionary
//                       rows x 1024 columns as eight cp.async.bulk copies that signal the stage's
//                       mbarrier, plus the matching slab of the activations. The dictionary is
//                       static, so the first ring-full of copies is issued BEFORE the
//                       programmatic-dependent-launch wait. The weight stream never stops at a
//                       task boundary.
//   products  (8 warps) one atom per warp: dot products of the staged row slab with the staged
//                       activations, accumulated over the row's slabs in registers, reduced with
//                       warp shuffles, and published as ONE 64-bit word {value, launch epoch} per
//                       (atom, token) - the finished Dx, no column-split partials.
//   gather    (4 warps) trails behind, task by task: prefetches its rows of the next task's code
//                       stream (cp.async), polls the current task's Dx words until they carry this
//                       launch's epoch (bounded; a wait that runs out sets the status word and
//                       nothing after it waits again), then the signed gather in the reference's
//                       order, bias, y out.
//
// Every task has its own Dx slot in the scratch buffer, so the products never overwrite what a
// slower gather still needs; the epoch comes from a device counter that the last CTA to have
// read it advances (graph replays tag afresh). All CTAs must be resident (grid = SM count, one per SM).
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

struct QTask {
    const float* D;
    const uint16_t* codes;
    const float* scales;
    const void* x;
    float* y;
    const float* bias;
    uint32_t K, R, C, S, k;
    uint32_t unit0;          // first flat unit of this task
    uint32_t dx_off;         // word offset of its Dx slot: [K][MT]
    uint32_t rows_per_cta;
    uint32_t x_dtype, x_layout, y_layout;
    uint32_t M_total, b0, M;
};

struct QParams {
    QTask task[kMaxQueueTasks];
    uint32_t n_tasks, n_units;
    uint32_t n_stages;          // ring depth
    uint32_t stage_bytes;       // D slab + x slab
    uint32_t codes_bytes;       // one code buffer of the gather role
    unsigned long long* dx;     // tagged words
    uint32_t* seq;              // [0] launches completed, [1] CTAs that have read [0]
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

__device__ __forceinline__ unsigned long long ld_poll(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.relaxed.gpu.global.b64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

// The launch's tag: launches completed + 1. The thread that calls this checks in with an acq_rel
// atomic after reading the counter; the CTA that checks in last knows every CTA has read it and
// advances it for the next launch (never to the value whose successor would be the tag 0).
__device__ __forceinline__ uint32_t take_epoch(uint32_t* seq) {
    uint32_t done, prev;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(done) : "l"(seq) : "memory");
    asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(prev) : "l"(seq + 1) : "memory");
    if (prev == gridDim.x - 1u) {
        seq[1] = 0u;
        const uint32_t next = done + 1u;
        asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(seq), "r"(next == 0xFFFFFFFFu ? 0u : next) : "memory");
    }
    return done + 1u;
}

__device__ __forceinline__ XView x_view(const QTask& t) {
    return XView{t.x, static_cast<int>(t.x_dtype), static_cast<int>(t.x_layout), t.C, t.M_total, t.b0, t.M};
}

// Shared memory: [n_stages][stage_bytes] | dxs [max K][MT] | codes [2][codes_bytes] | scales [2][16]
template <int MT>
__global__ void __launch_bounds__(kThreads, 1) hsdr_gemv_queue_kernel(const __grid_constant__ QParams p) {
    extern __shared__ __align__(128) unsigned char qsm[];
    __shared__ __align__(8) unsigned long long full_bar[kMaxStages], empty_bar[kMaxStages];
    __shared__ int failed_s;
    __shared__ uint32_t epoch_s;
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
        uint32_t ui = blockIdx.x, us = 0, uti = 0;           // issue cursor: unit, slab within it, task
        uint32_t fi = blockIdx.x, fs = 0, fti = 0;           // fill cursor
        bool waited = false;
        bool ok = true;
        auto issue = [&]() {   // D rows of (ui, us) into slot it_issue % NS
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
        auto fill = [&]() {    // activations of (fi, fs) into slot it_fill % NS, then the stage is armed
            task_of(fi, fti);
            const QTask& t = p.task[fti];
            const uint32_t slot = it_fill % NS;
            const uint32_t c0 = fs * kSlab;
            const uint32_t cw = min(kSlab, t.C - c0);
            float* xs = reinterpret_cast<float*>(qsm + static_cast<size_t>(slot) * p.stage_bytes + kAtomsPerUnit * kSlab * 4u);
            const XView xv = x_view(t);
            const bool rows_contig = xv.layout == CSDR_LAYOUT_TOKEN_MAJOR || xv.Mtotal == 1;
            if (xv.dtype == CSDR_DTYPE_F32 && rows_contig &&
                ((reinterpret_cast<uintptr_t>(xv.x) | (static_cast<uintptr_t>(xv.C) * 4u)) & 15u) == 0) {
                const uint32_t cw4 = cw >> 2;
#pragma unroll
                for (int b = 0; b < MT; ++b) {
                    const float4* src = reinterpret_cast<const float4*>(static_cast<const float*>(xv.x) +
                                                                        static_cast<size_t>(xv.b0 + min(static_cast<uint32_t>(b), xv.M - 1u)) * xv.C + c0);
                    float4* dst = reinterpret_cast<float4*>(xs + b * kSlab);
                    const bool live = static_cast<uint32_t>(b) < xv.M;
#pragma unroll
                    for (uint32_t j = 0; j < kSlab / 128u; ++j) {
                        const uint32_t c4 = j * 32u + lane;
                        if (c4 < cw4) dst[c4] = live ? __ldcg(src + c4) : make_float4(0.f, 0.f, 0.f, 0.f);
                    }
                }
            } else {
                for (uint32_t i = lane; i < MT * kSlab; i += 32u) {
                    const uint32_t b = i / kSlab, c = i - b * kSlab;
                    if (c < cw) xs[i] = b < xv.M ? load_x(xv, c0 + c, b) : 0.0f;
                }
            }
            __syncwarp();
            if (lane == 0) {
                unsigned long long st;
                asm volatile("mbarrier.arrive.release.cta.shared::cta.b64 %0, [%1];" : "=l"(st) : "r"(smem_u32(&full_bar[slot])) : "memory");
                (void)st;
            }
            ++it_fill;
            if (++fs == stages_of(t)) {
                fs = 0;
                fi += gridDim.x;
            }
        };
        // the first ring-full of weight copies does not depend on the activations
        while (ui < p.n_units && it_issue < NS) issue();
        asm volatile("griddepcontrol.wait;" ::: "memory");
        waited = true;
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
        if (!ok) {
            if (lane == 0) {
                failed_s = 1;
                atomicExch(p.status, 1);
            }
            // copies still in flight land in this CTA's shared memory: wait for them before leaving
            for (uint32_t back = 0; back < NS && back < it_issue; ++back) {
                const uint32_t itx = it_issue - 1u - back;
                if (itx >= it_fill) {   // armed with bytes, never completed by the arrival: complete it now
                    if (lane == 0) {
                        unsigned long long st;
                        asm volatile("mbarrier.arrive.release.cta.shared::cta.b64 %0, [%1];"
                                     : "=l"(st)
                                     : "r"(smem_u32(&full_bar[itx % NS]))
                                     : "memory");
                        (void)st;
                    }
                }
            }
            __syncwarp();
            volatile int never = 0;
            for (uint32_t back = 0; back < NS && back < it_issue; ++back) {
                const uint32_t itx = it_issue - 1u - back;
                mbar_wait(smem_u32(&full_bar[itx % NS]), (itx / NS) & 1u, p.spin_barrier, &never);
            }
        }
        (void)waited;
    } else if (warp <= kProductWarps) {
        // ================= products =================
        asm volatile("griddepcontrol.wait;" ::: "memory");
        if (tid == 32u) epoch_s = take_epoch(p.seq);
        asm volatile("bar.sync 3, %0;" ::"n"(32u * (kProductWarps + kGatherWarps)) : "memory");
        const uint32_t epoch = epoch_s;
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
                                const float4 xv = x4[b * (kSlab / 4u) + c4];
                                acc[b] = fmaf(d.x, xv.x, acc[b]);
                                acc[b] = fmaf(d.y, xv.y, acc[b]);
                                acc[b] = fmaf(d.z, xv.z, acc[b]);
                                acc[b] = fmaf(d.w, xv.w, acc[b]);
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
            if (lane < MT && atom < t.K) {
                const unsigned long long word = (static_cast<unsigned long long>(epoch) << 32) | __float_as_uint(mine);
                asm volatile("st.relaxed.gpu.global.b64 [%0], %1;" ::"l"(p.dx + t.dx_off + static_cast<size_t>(atom) * MT + lane),
                             "l"(word)
                             : "memory");
            }
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
        asm volatile("bar.sync 3, %0;" ::"n"(32u * (kProductWarps + kGatherWarps)) : "memory");
        const uint32_t epoch = epoch_s;
        uint32_t limit = *reinterpret_cast<const volatile int*>(p.status) != 0 ? 0u : p.spin_poll;
        bool late = false;
        for (uint32_t ti = 0; ti < p.n_tasks; ++ti) {
            const QTask& t = p.task[ti];
            if (ti + 1u < p.n_tasks) fetch_codes(ti + 1u);
            else asm volatile("cp.async.commit_group;" ::: "memory");
            const uint32_t row0 = blockIdx.x * t.rows_per_cta;
            const bool active = row0 < t.R;
            if (active) {
                // hand-over: this task's Dx words, up to eight loads in flight per thread
                const unsigned long long* src = p.dx + t.dx_off;
                const uint32_t n_w = t.K * MT;
                for (uint32_t w0 = gt; w0 < n_w; w0 += 8u * kGatherThreads) {
                    unsigned long long e[8];
                    for (uint32_t spins = 0;; ++spins) {
                        bool all = true;
#pragma unroll
                        for (int q = 0; q < 8; ++q) {
                            const uint32_t wi = w0 + q * kGatherThreads;
                            e[q] = wi < n_w ? ld_poll(src + wi) : (static_cast<unsigned long long>(epoch) << 32);
                        }
#pragma unroll
                        for (int q = 0; q < 8; ++q) all = all && static_cast<uint32_t>(e[q] >> 32) == epoch;
                        if (all) break;
                        if (spins >= limit || *failed) {
                            late = true;
                            limit = 0u;
                            break;
                        }
                    }
#pragma unroll
                    for (int q = 0; q < 8; ++q) {
                        const uint32_t wi = w0 + q * kGatherThreads;
                        if (wi < n_w) dxs[wi] = __uint_as_float(static_cast<uint32_t>(e[q]));
                    }
                }
            }
            asm volatile("cp.async.wait_group 1;" ::: "memory");      // this task's codes (the next task's may still fly)
            asm volatile("bar.sync 2, %0;" ::"n"(kGatherThreads) : "memory");
            if (active) {
                const uint32_t rows_here = min(t.rows_per_cta, t.R - row0);
                const uint32_t slots = t.S * t.k;
                const uint32_t skip = static_cast<uint32_t>((static_cast<size_t>(row0) * slots * 2u) & 15u) >> 1;
                const uint16_t* cs = reinterpret_cast<const uint16_t*>(codes_buf + (ti & 1u) * static_cast<size_t>(p.codes_bytes)) + skip;
                const float* sc = scales_buf + (ti & 1u) * 16u;
                const uint32_t b = gt % MT;
                constexpr uint32_t RP = kGatherThreads / MT;
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
                        if (t.bias) accr += t.bias[r];
                        const size_t yi = t.y_layout == CSDR_LAYOUT_FEATURE_MAJOR
                                              ? static_cast<size_t>(r) * t.M_total + (t.b0 + b)
                                              : static_cast<size_t>(t.b0 + b) * t.R + r;
                        t.y[yi] = accr;
                    }
                }
            }
            asm volatile("bar.sync 2, %0;" ::"n"(kGatherThreads) : "memory");   // dxs and the code buffer are reused
        }
        if (late) atomicExch(p.status, 1);
    }
}

uint32_t stage_bytes_for(int mt) { return kAtomsPerUnit * kSlab * 4u + static_cast<uint32_t>(mt) * kSlab * 4u; }
uint32_t codes_bytes_for(uint32_t max_code_bytes) { return (max_code_bytes + 31u + 127u) & ~127u; }
size_t tail_bytes_for(uint32_t max_k, int mt, uint32_t max_code_bytes) {
    return ((static_cast<size_t>(max_k) * mt * 4u + 127u) & ~static_cast<size_t>(127)) + 2u * codes_bytes_for(max_code_bytes) + 128u;
}
size_t smem_budget(const csdr_context* ctx) { return std::min<size_t>(ctx->smem_optin, 220u * 1024u); }
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
    if (batch == 0 || batch > 4) return false;
    const int mt = batch <= 1 ? 1 : batch <= 2 ? 2 : 4;
    uint32_t max_k = 0, max_code_bytes = 0;
    for (uint32_t i = 0; i < n; ++i) {
        const Geometry& g = items[i].seg->g;
        if (!g.row_tiles() || g.cols % 4u || items[i].batch != batch) return false;
        if (g.n_atoms > 4096u || g.n_stages > 16u) return false;
        max_k = std::max(max_k, g.n_atoms);
        max_code_bytes = std::max(max_code_bytes, rows_per_cta_for(ctx, g.rows) * g.slots() * 2u);
    }
    // the ring needs three stages beside the gather role's buffers
    return tail_bytes_for(max_k, mt, max_code_bytes) + 3u * stage_bytes_for(mt) <= smem_budget(ctx);
}

void launch_gemv_queue(csdr_context* ctx, const QueueItem* items, uint32_t n) {
    const uint32_t batch = static_cast<uint32_t>(items[0].batch);
    const int mt = batch <= 1 ? 1 : batch <= 2 ? 2 : 4;
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
            t.K = g.n_atoms;
            t.R = g.rows;
            t.C = g.cols;
            t.S = g.n_stages;
            t.k = g.k;
            t.unit0 = unit;
            t.dx_off = dx_off;
            t.rows_per_cta = rows_per_cta_for(ctx, g.rows);
            t.x_dtype = static_cast<uint32_t>(it.x_dtype);
            t.x_layout = static_cast<uint32_t>(it.x_layout);
            t.y_layout = static_cast<uint32_t>(it.y_layout);
            t.M_total = batch;
            t.b0 = 0;
            t.M = batch;
            unit += (g.n_atoms + kAtomsPerUnit - 1u) / kAtomsPerUnit;
            dx_off += g.n_atoms * static_cast<uint32_t>(mt);
            max_k = std::max(max_k, g.n_atoms);
            max_code_bytes = std::max(max_code_bytes, t.rows_per_cta * g.slots() * 2u);
        }
        p.n_tasks = cnt;
        p.n_units = unit;
        p.dx = static_cast<unsigned long long*>(ctx->scratch_get(4, std::max<size_t>(static_cast<size_t>(dx_off) * 8u, 2u << 20)));
        p.seq = ctx->gemv_seq;
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
