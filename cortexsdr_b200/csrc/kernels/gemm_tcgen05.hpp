// Tensor-core (tcgen05 / TMEM) path for wide token tiles of 1-D row-tile HSDR segments.
#pragma once

#include <cstddef>

struct csdr_context;
struct csdr_segment;

namespace csdr {

struct MatmulArgs;

// 1-D row tiles, n_atoms a multiple of 128, cols a multiple of 64, batch at least the
// context's tensor-core threshold.
bool tcgen05_supported(const csdr_context* ctx, const csdr_segment* seg, size_t batch);

// The whole batch in one pass: projection on the tensor cores, column-split reduction, gather.
void launch_matmul_tcgen05(csdr_context* ctx, const csdr_segment* seg, const MatmulArgs& a);

// TMA-fed projection (gemm_tma.cu): Dx [n_atoms][dx_stride >= batch] for the whole batch in one
// launch, from bf16 dictionary planes that are built on the first call and cached with the
// dictionary.
bool dx_tma_supported(const csdr_context* ctx, const csdr_segment* seg, size_t batch);
void launch_dx_tma(csdr_context* ctx, const csdr_segment* seg, const MatmulArgs& a, float* dx, uint32_t dx_stride);

}  // namespace csdr
