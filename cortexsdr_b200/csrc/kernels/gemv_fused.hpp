// One-launch decode GEMV over up to kMaxFusedGroup row-tile segments sharing one activation.
#pragma once

#include <cstdint>

struct csdr_context;
struct csdr_segment;

namespace csdr {

constexpr uint32_t kMaxFusedGroup = 4;

// True when every segment is a 1-D row-tile image with the same column count (a multiple
// of 4) and a dictionary small enough for the gather phase's shared memory.
bool gemv_fused_supported(const csdr_context* ctx, const csdr_segment* const* segs, uint32_t n, uint32_t mt);

// Decoder glue folded into the launch (api/cortex_sdk.cpp:1208-1256): RMS normalisation of the
// activations (the slab is multiplied by the norm weights as it is staged, every CTA sums the
// squares of the row it staged, the gather scales its rows by 1 / sqrt(mean + eps)); a residual
// per member, added behind the product (may be the member's own output); SwiGLU for a
// (gate, up) pair: member 1's rows leave as silu(member 0's row) * row.
struct FusedGlue {
    const float* norm_w = nullptr;
    float norm_eps = 0.0f;
    const float* residual[kMaxFusedGroup] = {};
    bool swiglu = false;
};
// Whether the glue can ride on a launch of these segments at token tile mt: the normalisation
// needs the whole activation row in every CTA's shared memory; SwiGLU two members of equal rows.
bool gemv_fused_glue_supported(const csdr_context* ctx, const csdr_segment* const* segs, uint32_t n, uint32_t mt,
                               const FusedGlue& glue);

// Tokens [b0, b0+m) of an activation matrix of m_total tokens; mt = token tile (1,2,4,8,16) >= m.
void launch_gemv_fused(csdr_context* ctx, const csdr_segment* const* segs, uint32_t n, const void* x,
                       int x_dtype, int x_layout, uint32_t m_total, uint32_t b0, uint32_t m,
                       float* const* ys, int y_layout, const float* const* biases, int mt,
                       const FusedGlue* glue = nullptr);

}  // namespace csdr
