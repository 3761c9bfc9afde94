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

// Tokens [b0, b0+m) of an activation matrix of m_total tokens; mt = token tile (1,2,4,8,16) >= m.
void launch_gemv_fused(csdr_context* ctx, const csdr_segment* const* segs, uint32_t n, const void* x,
                       int x_dtype, int x_layout, uint32_t m_total, uint32_t b0, uint32_t m,
                       float* const* ys, int y_layout, const float* const* biases, int mt);

}  // namespace csdr
