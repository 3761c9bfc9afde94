// Activation / output views and small device helpers shared by the matmul kernels.
#pragma once

#include <cuda_bf16.h>

#include <cstdint>

#include "../../../include/cortexsdr_b200.h"

namespace csdr {

// Streaming 128-bit load: the dictionary is read once per launch, keep it out of L1.
__device__ __forceinline__ float4 ldg_stream_f4(const float4* p) {
    float4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                 : "l"(p));
    return v;
}

struct XView {
    const void* x;
    int dtype;       // CSDR_DTYPE_*
    int layout;      // CSDR_LAYOUT_*
    uint32_t C;      // features
    uint32_t Mtotal; // tokens in the whole activation matrix
    uint32_t b0;     // first token of this launch's chunk
    uint32_t M;      // tokens in this chunk (<= MT)
};

__device__ __forceinline__ float load_x(const XView& v, uint32_t c, uint32_t b) {
    const size_t i = v.layout == CSDR_LAYOUT_FEATURE_MAJOR
                         ? static_cast<size_t>(c) * v.Mtotal + (v.b0 + b)
                         : static_cast<size_t>(v.b0 + b) * v.C + c;
    if (v.dtype == CSDR_DTYPE_BF16)
        return __bfloat162float(static_cast<const __nv_bfloat16*>(v.x)[i]);
    return static_cast<const float*>(v.x)[i];
}

struct YView {
    float* y;
    int layout;
    uint32_t R;
    uint32_t Mtotal;
    uint32_t b0;
    uint32_t M;
    const float* bias;
    const float* residual = nullptr;   // added behind the product, indexed like y (may be y itself)
};

__device__ __forceinline__ size_t y_index(const YView& v, uint32_t r, uint32_t b) {
    return v.layout == CSDR_LAYOUT_FEATURE_MAJOR
               ? static_cast<size_t>(r) * v.Mtotal + (v.b0 + b)
               : static_cast<size_t>(v.b0 + b) * v.R + r;
}

// The tag of a launch: one more than the tag of the launch before it on the context (never 0, the
// value fresh scratch holds), kept in DEVICE memory so that a captured CUDA graph tags every replay
// afresh. seq[0] is the last tag handed out; seq[2 + cta] is where a CTA leaves the tag it took.
//   * Every CTA reads seq[0] with a plain load behind its dependency wait (the launch before has
//     completed by then, its write of seq[0] is visible) and leaves tag = seq[0] + 1 in its own
//     slot: no atomic, nothing to wait for.
//   * One warp of CTA 0 that has nothing else to do retires the tag: it waits (bounded) until
//     every CTA's slot holds the tag - every CTA has read seq[0] - and only then writes
//     seq[0] = tag for the next launch.
constexpr uint32_t kMaxTagCtas = 1022;   // seq holds 2 + kMaxTagCtas words
__device__ __forceinline__ uint32_t read_launch_tag(uint32_t* seq) {
    uint32_t last;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(last) : "l"(seq) : "memory");
    const uint32_t tag = last + 1u == 0u ? 1u : last + 1u;
    asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(seq + 2u + blockIdx.x), "r"(tag) : "memory");
    return tag;
}
// Called by all 32 lanes of one warp of CTA 0. False when the wait ran out (the tag is retired all
// the same, so that the context does not reuse it; the caller records the failure).
__device__ __forceinline__ bool retire_launch_tag(uint32_t* seq, uint32_t tag, uint32_t lane, uint32_t limit) {
    bool done = false;
    for (uint32_t spins = 0; spins <= limit && !done; ++spins) {
        bool ok = true;
        for (uint32_t i = lane; i < gridDim.x; i += 32u) {
            uint32_t v;
            asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(seq + 2u + i) : "memory");
            ok = ok && v == tag;
        }
        done = __all_sync(0xFFFFFFFFu, ok);
        if (!done) __nanosleep(200);
    }
    if (lane == 0) asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(seq), "r"(tag) : "memory");
    return done;
}

}  // namespace csdr
