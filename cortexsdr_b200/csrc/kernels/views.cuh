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

// The tag of a launch: (launches completed) mod (2^32 - 1), plus one - never 0, the value fresh
// scratch holds. One 64-bit word in device memory keeps {launches completed (high half), CTAs of
// the running launch that have checked in (low half)}; a CTA checks in with ONE atomic add, whose
// return value also carries the count it needs, and the CTA that checks in last adds the rest of
// 2^32 so that the high half moves on and the low half returns to zero. Every CTA of a launch
// reads the same high half (it only moves after the last check-in), and the next launch checks
// in behind its dependency wait, when this launch's stores are visible. Because the word lives
// on the device, a captured CUDA graph tags every replay afresh.
__device__ __forceinline__ uint32_t take_launch_tag(unsigned long long* seq) {
    unsigned long long old;
    asm volatile("atom.relaxed.gpu.global.add.u64 %0, [%1], 1;" : "=l"(old) : "l"(seq) : "memory");
    if (static_cast<uint32_t>(old) == gridDim.x - 1u) {
        const unsigned long long rest = (1ull << 32) - gridDim.x;
        asm volatile("red.relaxed.gpu.global.add.u64 [%0], %1;" ::"l"(seq), "l"(rest) : "memory");
    }
    return static_cast<uint32_t>((old >> 32) % 0xFFFFFFFFull) + 1u;
}

}  // namespace csdr
