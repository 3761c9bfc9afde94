// extern "C" face of the HSDR encoder and of its coding pass alone.
//
// HierarchicalSDRStrategy::compress (strategies/HierarchicalSDRStrategy.cpp:1068-1236) around
// fitHierarchicalKSVD (:494-607): tiles of the aligned top-left block, a dictionary of K tiles
// picked by std::mt19937(0xC0DE), normalised and scaled by the mean tile norm over sqrt(S * k),
// one coding pass, then ksvd_iters rounds of (atomUpdateStep :281-489, coding pass), the sweep of
// non-finite values, and the payload "HSDR" v2 with the raw edge strips behind it. The random
// draws and the byte layout are host work; everything that touches the tensor runs on the device
// (kernels/encode.cu). As in compress, the fit runs on all tiles (max_tiles_for_fit only bounds
// the reference's streaming and grouped encoders).
#include <algorithm>
#include <cmath>
#include <cstring>
#include <vector>

#include "internal.hpp"
#include "kernels/encode.hpp"

using namespace csdr;

namespace {

// std::mt19937 as the standard defines it (Matsumoto and Nishimura 1998; seeding by Knuth's
// 1812433253 recurrence).
struct Mt19937 {
    uint32_t mt[624];
    int i = 624;
    explicit Mt19937(uint32_t seed) {
        mt[0] = seed;
        for (int j = 1; j < 624; ++j) mt[j] = 1812433253u * (mt[j - 1] ^ (mt[j - 1] >> 30)) + static_cast<uint32_t>(j);
    }
    uint32_t next() {
        if (i >= 624) {
            for (int j = 0; j < 624; ++j) {
                const uint32_t y = (mt[j] & 0x80000000u) | (mt[(j + 1) % 624] & 0x7FFFFFFFu);
                mt[j] = mt[(j + 397) % 624] ^ (y >> 1) ^ ((y & 1u) ? 0x9908B0DFu : 0u);
            }
            i = 0;
        }
        uint32_t y = mt[i++];
        y ^= y >> 11;
        y ^= (y << 7) & 0x9D2C5680u;
        y ^= (y << 15) & 0xEFC60000u;
        y ^= y >> 18;
        return y;
    }
    // uniform in [0, range): the multiply-shift draw with rejection (Lemire 2019) that GCC's
    // uniform_int_distribution performs for a 32-bit generator, which the reference was built with
    uint32_t below(uint32_t range) {
        uint64_t prod = static_cast<uint64_t>(next()) * range;
        uint32_t low = static_cast<uint32_t>(prod);
        if (low < range) {
            const uint32_t threshold = (0u - range) % range;
            while (low < threshold) {
                prod = static_cast<uint64_t>(next()) * range;
                low = static_cast<uint32_t>(prod);
            }
        }
        return static_cast<uint32_t>(prod >> 32);
    }
};

void put32(uint8_t* p, uint32_t v) { std::memcpy(p, &v, 4); }
void put16(uint8_t* p, uint16_t v) { std::memcpy(p, &v, 2); }

// fitHierarchicalKSVD (:494-607) on a pool of tiles resident on the device (one tensor's, or the
// pooled tiles of several tensors as fitSharedDictionary :1446-1469 hands them in): dictionary
// init, a coding pass, ksvd_iters rounds of (atom update, coding pass), the non-finite sweep.
void fit_tiles(csdr_context* ctx, const DevPtr& tiles, uint32_t n_tiles, size_t T, uint16_t n_atoms, uint8_t n_stages,
               uint8_t k_per_stage, float stage_decay, uint8_t ksvd_iters, DevPtr* D_out, std::vector<float>* gam_out,
               DevPtr* codes_out) {
    const size_t n_codes = static_cast<size_t>(n_tiles) * n_stages * k_per_stage;
    // mean tile norm, summed in tile order on the host from per-tile doubles (:527-533)
    DevPtr norms = std::make_shared<DeviceBuffer>(static_cast<size_t>(n_tiles) * 8, ctx->device);
    launch_tile_norms(ctx, static_cast<const float*>(tiles->ptr), n_tiles, static_cast<uint32_t>(T), static_cast<double*>(norms->ptr));
    std::vector<double> nh(n_tiles);
    CSDR_CUDA(cudaMemcpyAsync(nh.data(), norms->ptr, nh.size() * 8, cudaMemcpyDeviceToHost, ctx->stream));
    CSDR_CUDA(cudaStreamSynchronize(ctx->stream));
    double norm_sum = 0.0;
    for (double v : nh) norm_sum += v;
    const double mean_d = norm_sum / static_cast<double>(n_tiles);
    const float mean = static_cast<float>(mean_d);
    const float root = std::sqrt(static_cast<float>(static_cast<uint32_t>(n_stages) * k_per_stage));
    const float init_scale = mean / (root > 1.0f ? root : 1.0f);
    // tile picks (:513-517)
    Mt19937 gen(0xC0DEu);
    std::vector<uint32_t> picks(n_atoms);
    for (uint32_t j = 0; j < n_atoms; ++j) picks[j] = gen.below(n_tiles);
    DevPtr picks_d = upload(ctx, picks.data(), picks.size() * 4);
    DevPtr D = std::make_shared<DeviceBuffer>(static_cast<size_t>(n_atoms) * T * 4, ctx->device);
    launch_init_atoms(ctx, static_cast<const float*>(tiles->ptr), static_cast<const uint32_t*>(picks_d->ptr), n_atoms,
                      static_cast<uint32_t>(T), init_scale, static_cast<float*>(D->ptr));
    std::vector<float> gam(n_stages);
    for (uint8_t l = 0; l < n_stages; ++l) gam[l] = std::pow(stage_decay, static_cast<float>(l));   // :507-509
    DevPtr gam_d = upload(ctx, gam.data(), gam.size() * 4);
    DevPtr codes = std::make_shared<DeviceBuffer>(n_codes * 2, ctx->device);
    launch_code_tiles(ctx, static_cast<const float*>(tiles->ptr), n_tiles, static_cast<uint32_t>(T), D, n_atoms, n_stages,
                      k_per_stage, static_cast<const float*>(gam_d->ptr), static_cast<uint16_t*>(codes->ptr));
    if (ksvd_iters) {
        // the update's target norm (:306-318) from the same tile norms, in double
        const double target = std::max(mean_d / std::sqrt(static_cast<double>(static_cast<uint32_t>(n_stages) * k_per_stage)), 1e-6);
        std::vector<uint32_t> pick_a(n_atoms), pick_b(n_atoms);
        DevPtr pick_a_d = std::make_shared<DeviceBuffer>(static_cast<size_t>(n_atoms) * 4, ctx->device);
        DevPtr pick_b_d = std::make_shared<DeviceBuffer>(static_cast<size_t>(n_atoms) * 4, ctx->device);
        for (uint8_t it = 0; it < ksvd_iters; ++it) {
            // one draw of the fit's generator per round seeds the replacements (:320); an atom's
            // own generator is seeded with it and the atom's number times a salt (:395-400, :430-436)
            const uint64_t base_seed = static_cast<uint64_t>(gen.next()) ^ 0xA0B1C2D3ull;
            for (uint32_t j = 0; j < n_atoms; ++j) {
                Mt19937 unused(static_cast<uint32_t>(base_seed ^ static_cast<uint64_t>(static_cast<uint32_t>(j * 0x9E3779B1u))));
                pick_a[j] = unused.below(n_tiles);
                Mt19937 nonfinite(static_cast<uint32_t>(base_seed ^ static_cast<uint64_t>(static_cast<uint32_t>(j * 0xB7E15163u))));
                pick_b[j] = nonfinite.below(n_tiles);
            }
            CSDR_CUDA(cudaMemcpyAsync(pick_a_d->ptr, pick_a.data(), pick_a.size() * 4, cudaMemcpyHostToDevice, ctx->stream));
            CSDR_CUDA(cudaMemcpyAsync(pick_b_d->ptr, pick_b.data(), pick_b.size() * 4, cudaMemcpyHostToDevice, ctx->stream));
            launch_atom_update(ctx, static_cast<const float*>(tiles->ptr), n_tiles, static_cast<uint32_t>(T),
                               static_cast<float*>(D->ptr), n_atoms, n_stages, k_per_stage, static_cast<const float*>(gam_d->ptr),
                               static_cast<const uint16_t*>(codes->ptr), target, static_cast<const uint32_t*>(pick_a_d->ptr),
                               static_cast<const uint32_t*>(pick_b_d->ptr));
            launch_code_tiles(ctx, static_cast<const float*>(tiles->ptr), n_tiles, static_cast<uint32_t>(T), D, n_atoms, n_stages,
                              k_per_stage, static_cast<const float*>(gam_d->ptr), static_cast<uint16_t*>(codes->ptr));
        }
    }
    launch_finite_sweep(ctx, static_cast<float*>(D->ptr), static_cast<size_t>(n_atoms) * T);
    *D_out = D;
    *gam_out = gam;
    *codes_out = codes;
}

}  // namespace

extern "C" {

int csdr_encode_codes(csdr_context* ctx, const float* tiles, size_t n_tiles, size_t tile_dim, const float* atoms,
                      uint16_t n_atoms, uint8_t n_stages, uint8_t k_per_stage, const float* stage_scales,
                      uint16_t* codes_out, size_t capacity) {
    return guard([&] {
        require_ctx(ctx);
        if (!tiles || !atoms || !stage_scales || !codes_out) throw Error(CSDR_ERR_INVALID_ARG, "null argument");
        if (!n_tiles || !tile_dim || !n_atoms || !n_stages || !k_per_stage || n_atoms > 0x7FFF)
            throw Error(CSDR_ERR_INVALID_ARG, "zero or out-of-range size");
        if (n_tiles > 0xFFFFFFFFull || tile_dim > 0xFFFFFFFFull) throw Error(CSDR_ERR_LIMIT, "too many tiles");
        const size_t n_codes = n_tiles * n_stages * k_per_stage;
        if (capacity < n_codes) throw Error(CSDR_ERR_BUFFER, "code buffer too small");
        DevPtr t = upload(ctx, tiles, n_tiles * tile_dim * 4);
        DevPtr d = upload(ctx, atoms, static_cast<size_t>(n_atoms) * tile_dim * 4);
        DevPtr g = upload(ctx, stage_scales, 4u * n_stages);
        DevPtr c = std::make_shared<DeviceBuffer>(n_codes * 2, ctx->device);
        launch_code_tiles(ctx, static_cast<const float*>(t->ptr), static_cast<uint32_t>(n_tiles), static_cast<uint32_t>(tile_dim), d,
                          n_atoms, n_stages, k_per_stage, static_cast<const float*>(g->ptr), static_cast<uint16_t*>(c->ptr));
        CSDR_CUDA(cudaMemcpyAsync(codes_out, c->ptr, n_codes * 2, cudaMemcpyDeviceToHost, ctx->stream));
        CSDR_CUDA(cudaStreamSynchronize(ctx->stream));
    });
}

int csdr_hsdr_encode(csdr_context* ctx, const float* W, uint32_t rows, uint32_t cols, uint16_t tile_rows,
                     uint16_t tile_cols, uint16_t n_atoms, uint8_t n_stages, uint8_t k_per_stage, float stage_decay,
                     uint8_t ksvd_iters, void* payload_out, size_t capacity, size_t* n_out) {
    return guard([&] {
        require_ctx(ctx);
        if (!W || !n_out) throw Error(CSDR_ERR_INVALID_ARG, "null argument");
        if (!rows || !cols || !tile_rows || !tile_cols || !n_atoms || !n_stages || !k_per_stage || n_atoms > 0x7FFF)
            throw Error(CSDR_ERR_INVALID_ARG, "HSDR: zero or out-of-range config field");
        const uint32_t R_full = rows / tile_rows * tile_rows, C_full = cols / tile_cols * tile_cols;
        if (!R_full || !C_full) throw Error(CSDR_ERR_GEOMETRY, "HSDR: tensor smaller than one tile");
        const uint32_t n_rt = R_full / tile_rows, n_ct = C_full / tile_cols;
        const uint64_t n_tiles64 = static_cast<uint64_t>(n_rt) * n_ct;
        if (n_tiles64 < n_atoms) throw Error(CSDR_ERR_GEOMETRY, "HSDR: not enough tiles to fit dictionary");   // :1143-1145
        const uint32_t n_tiles = static_cast<uint32_t>(n_tiles64);
        const size_t T = static_cast<size_t>(tile_rows) * tile_cols;
        const size_t n_codes = static_cast<size_t>(n_tiles) * n_stages * k_per_stage;
        const size_t edge_floats = static_cast<size_t>(R_full) * (cols - C_full) + static_cast<size_t>(rows - R_full) * cols;
        const size_t hdr = 36, total = hdr + 4u * n_stages + 4u * static_cast<size_t>(n_atoms) * T + 2u * n_codes + 4u * edge_floats;
        *n_out = total;
        if (!payload_out || capacity < total) throw Error(CSDR_ERR_BUFFER, "payload buffer too small");
        uint8_t* out = static_cast<uint8_t*>(payload_out);

        DevPtr Wd = upload(ctx, W, static_cast<size_t>(rows) * cols * 4);
        DevPtr tiles = std::make_shared<DeviceBuffer>(static_cast<size_t>(n_tiles) * T * 4, ctx->device);
        launch_extract_tiles(ctx, static_cast<const float*>(Wd->ptr), cols, tile_rows, tile_cols, n_rt, n_ct,
                             static_cast<float*>(tiles->ptr));
        std::vector<float> gam;
        DevPtr D, codes;
        fit_tiles(ctx, tiles, n_tiles, T, n_atoms, n_stages, k_per_stage, stage_decay, ksvd_iters, &D, &gam, &codes);

        // the payload (serialize, :1198-1235): header | stage scales | dictionary | codes | edge strips
        std::memset(out, 0, hdr);
        std::memcpy(out, "HSDR", 4);
        put32(out + 4, 2u);
        put32(out + 8, rows);
        put32(out + 12, cols);
        put32(out + 16, n_tiles);
        put16(out + 20, tile_rows);
        put16(out + 22, tile_cols);
        put16(out + 24, n_atoms);
        out[26] = n_stages;
        out[27] = k_per_stage;
        std::memcpy(out + 28, &stage_decay, 4);
        put32(out + 32, static_cast<uint32_t>(4u * edge_floats));
        std::memcpy(out + hdr, gam.data(), 4u * n_stages);
        uint8_t* dict_at = out + hdr + 4u * n_stages;
        uint8_t* codes_at = dict_at + 4u * static_cast<size_t>(n_atoms) * T;
        CSDR_CUDA(cudaMemcpyAsync(dict_at, D->ptr, 4u * static_cast<size_t>(n_atoms) * T, cudaMemcpyDeviceToHost, ctx->stream));
        CSDR_CUDA(cudaMemcpyAsync(codes_at, codes->ptr, n_codes * 2, cudaMemcpyDeviceToHost, ctx->stream));
        CSDR_CUDA(cudaStreamSynchronize(ctx->stream));
        // raw strips: top-right, then bottom (:1185-1197)
        uint8_t* e = codes_at + 2u * n_codes;
        const size_t wr = static_cast<size_t>(cols - C_full) * 4;
        for (uint32_t r = 0; r < R_full && wr; ++r, e += wr) std::memcpy(e, W + static_cast<size_t>(r) * cols + C_full, wr);
        for (uint32_t r = R_full; r < rows; ++r, e += static_cast<size_t>(cols) * 4)
            std::memcpy(e, W + static_cast<size_t>(r) * cols, static_cast<size_t>(cols) * 4);
    });
}

int csdr_hsdr_encode_shared(csdr_context* ctx, const float* const* tensors, const uint32_t* rows, const uint32_t* cols,
                            size_t n_tensors, uint16_t tile_rows, uint16_t tile_cols, uint16_t n_atoms, uint8_t n_stages,
                            uint8_t k_per_stage, float stage_decay, uint8_t ksvd_iters, void* dict_out, size_t dict_capacity,
                            size_t* dict_bytes, void* const* codes_out, const size_t* codes_capacity, size_t* codes_bytes) {
    return guard([&] {
        require_ctx(ctx);
        if (!tensors || !rows || !cols || !n_tensors || !dict_bytes || !codes_bytes) throw Error(CSDR_ERR_INVALID_ARG, "null argument");
        if (!tile_rows || !tile_cols || !n_atoms || !n_stages || !k_per_stage || n_atoms > 0x7FFF)
            throw Error(CSDR_ERR_INVALID_ARG, "HSDR: zero or out-of-range config field");
        const size_t T = static_cast<size_t>(tile_rows) * tile_cols;
        uint64_t pooled = 0;
        for (size_t i = 0; i < n_tensors; ++i) {
            if (!tensors[i] || !rows[i] || !cols[i]) throw Error(CSDR_ERR_INVALID_ARG, "null or empty tensor");
            if (rows[i] % tile_rows || cols[i] % tile_cols)          // compressFP32WithExternalDictionary, :1698-1701
                throw Error(CSDR_ERR_GEOMETRY, "HSDR shared: shape not divisible by tile size");
            pooled += static_cast<uint64_t>(rows[i] / tile_rows) * (cols[i] / tile_cols);
        }
        if (pooled > 0xFFFFFFFFull) throw Error(CSDR_ERR_LIMIT, "too many tiles");
        if (pooled < n_atoms) throw Error(CSDR_ERR_GEOMETRY, "fitSharedDictionary: pooled tile count below n_atoms");   // :1455-1457
        const uint32_t n_pool = static_cast<uint32_t>(pooled);
        const size_t slots = static_cast<size_t>(n_stages) * k_per_stage;
        // sizes first: the dictionary record of a .hsda (20-byte config, counted scales, counted
        // atoms) and one codes-only "HSDC" stream per tensor (32-byte header + codes)
        const size_t dict_need = 20u + 4u + 4u * n_stages + 4u + 4u * static_cast<size_t>(n_atoms) * T;
        *dict_bytes = dict_need;
        bool fits = dict_out && dict_capacity >= dict_need && codes_out && codes_capacity;
        for (size_t i = 0; i < n_tensors; ++i) {
            const size_t tiles_i = static_cast<size_t>(rows[i] / tile_rows) * (cols[i] / tile_cols);
            codes_bytes[i] = 32u + 2u * tiles_i * slots;
            fits = fits && codes_out && codes_out[i] && codes_capacity[i] >= codes_bytes[i];
        }
        if (!fits) throw Error(CSDR_ERR_BUFFER, "output buffers too small");

        // the tensors' tiles pooled in order (the uncapped pool of compressGroupedSegments, :2383-2390)
        DevPtr pool = std::make_shared<DeviceBuffer>(static_cast<size_t>(n_pool) * T * 4, ctx->device);
        std::vector<size_t> first(n_tensors);
        size_t at = 0;
        for (size_t i = 0; i < n_tensors; ++i) {
            first[i] = at;
            const uint32_t n_rt = rows[i] / tile_rows, n_ct = cols[i] / tile_cols;
            DevPtr Wd = upload(ctx, tensors[i], static_cast<size_t>(rows[i]) * cols[i] * 4);
            launch_extract_tiles(ctx, static_cast<const float*>(Wd->ptr), cols[i], tile_rows, tile_cols, n_rt, n_ct,
                                 static_cast<float*>(pool->ptr) + at * T);
            CSDR_CUDA(cudaStreamSynchronize(ctx->stream));   // Wd goes away with this iteration
            at += static_cast<size_t>(n_rt) * n_ct;
        }
        std::vector<float> gam;
        DevPtr D, pool_codes;
        fit_tiles(ctx, pool, n_pool, T, n_atoms, n_stages, k_per_stage, stage_decay, ksvd_iters, &D, &gam, &pool_codes);
        // The fit's last step coded the whole pool against the dictionary as it stands before the
        // sweep of non-finite values; the reference codes every tensor again behind the sweep
        // (compressFP32WithExternalDictionary, :2466-2470). One more pass over the pool is that.
        DevPtr gam_d = upload(ctx, gam.data(), gam.size() * 4);
        launch_code_tiles(ctx, static_cast<const float*>(pool->ptr), n_pool, static_cast<uint32_t>(T), D, n_atoms, n_stages, k_per_stage,
                          static_cast<const float*>(gam_d->ptr), static_cast<uint16_t*>(pool_codes->ptr));

        uint8_t* d = static_cast<uint8_t*>(dict_out);
        std::memset(d, 0, 20);                       // HierarchicalSDRConfig as the reference's build lays it out
        put16(d + 0, tile_rows);
        put16(d + 2, tile_cols);
        put16(d + 4, n_atoms);
        d[6] = n_stages;
        d[7] = k_per_stage;
        d[8] = ksvd_iters;
        std::memcpy(d + 12, &stage_decay, 4);
        put32(d + 16, 0u);                           // max_tiles_for_fit: the fit ran on every tile
        put32(d + 20, n_stages);
        std::memcpy(d + 24, gam.data(), 4u * n_stages);
        put32(d + 24 + 4u * n_stages, static_cast<uint32_t>(static_cast<size_t>(n_atoms) * T));
        CSDR_CUDA(cudaMemcpyAsync(d + 28 + 4u * n_stages, D->ptr, 4u * static_cast<size_t>(n_atoms) * T, cudaMemcpyDeviceToHost,
                                  ctx->stream));
        for (size_t i = 0; i < n_tensors; ++i) {
            uint8_t* c = static_cast<uint8_t*>(codes_out[i]);
            const uint32_t tiles_i = (rows[i] / tile_rows) * (cols[i] / tile_cols);
            std::memset(c, 0, 32);                   // HSDRCodesHeader, :675-692
            std::memcpy(c, "HSDC", 4);
            put32(c + 4, 1u);
            put32(c + 8, rows[i]);
            put32(c + 12, cols[i]);
            put32(c + 16, tiles_i);
            put16(c + 20, tile_rows);
            put16(c + 22, tile_cols);
            put16(c + 24, n_atoms);
            c[26] = n_stages;
            c[27] = k_per_stage;
            std::memcpy(c + 28, &stage_decay, 4);
            CSDR_CUDA(cudaMemcpyAsync(c + 32, static_cast<const uint16_t*>(pool_codes->ptr) + first[i] * slots, 2u * tiles_i * slots,
                                      cudaMemcpyDeviceToHost, ctx->stream));
        }
        CSDR_CUDA(cudaStreamSynchronize(ctx->stream));
    });
}

}  // extern "C"
