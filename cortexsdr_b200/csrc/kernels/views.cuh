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

}  // namespace csdr
