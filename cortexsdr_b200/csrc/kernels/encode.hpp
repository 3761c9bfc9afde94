// Device side of the HSDR encoder's fast mode: see encode.cu.
#pragma once

#include <cstdint>

#include "../internal.hpp"

namespace csdr {

// W (row-major, C columns) -> tiles [n_rt * n_ct][tr * tc] of its aligned top-left block.
void launch_extract_tiles(csdr_context* ctx, const float* W, uint32_t C, uint32_t tr, uint32_t tc, uint32_t n_rt,
                          uint32_t n_ct, float* tiles);
// norms[t] = Euclidean norm of tile t, as a double.
void launch_tile_norms(csdr_context* ctx, const float* tiles, uint32_t n_tiles, uint32_t T, double* norms);
// D[j] = tiles[picks[j]] / |tiles[picks[j]]| * init_scale.
void launch_init_atoms(csdr_context* ctx, const float* tiles, const uint32_t* picks_dev, uint32_t K, uint32_t T, float init_scale,
                       float* D);
// The coding pass: packed codes [n_tiles][S][k] of the tiles against dictionary D (K x T).
void launch_code_tiles(csdr_context* ctx, const float* tiles, uint32_t n_tiles, uint32_t T, const DevPtr& D, uint32_t K,
                       uint32_t S, uint32_t k, const float* gammas_dev, uint16_t* codes_dev);

// One dictionary-update round (atomUpdateStep, strategies/HierarchicalSDRStrategy.cpp:281-489): every
// atom moves half a least-squares step toward the residuals of the tiles that use it. `target` is
// the mean tile norm over sqrt(S * k); the pick arrays name, per atom, the tile that replaces it
// when nothing uses it / when its candidate is not finite (drawn on the host as the reference
// draws them).
void launch_atom_update(csdr_context* ctx, const float* tiles, uint32_t n_tiles, uint32_t T, float* D, uint32_t K,
                        uint32_t S, uint32_t k, const float* gammas_dev, const uint16_t* codes_dev, double target,
                        const uint32_t* pick_unused_dev, const uint32_t* pick_nonfinite_dev);
// Non-finite dictionary values become 0 (:598-604).
void launch_finite_sweep(csdr_context* ctx, float* D, size_t n);

}  // namespace csdr
