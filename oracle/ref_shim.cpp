// TEST INFRASTRUCTURE ONLY — never linked into, loaded by, or shipped with the
// product library.
//
// A thin extern "C" face over the UNMODIFIED reference sources (compiled where
// they lie, outside this repository; see oracle/Makefile) so that Python tests
// and the bench's CPU-baseline leg can (a) produce archives with the reference's
// own encoder, and (b) run the reference's own CPU decode / fused matmul /
// dequantisation as the ground truth.
//
// Reference entry points wrapped here (paths relative to the reference tree):
//   HierarchicalSDRStrategy::compress            strategies/HierarchicalSDRStrategy.cpp:1068
//   HierarchicalSDRStrategy::decompress          strategies/HierarchicalSDRStrategy.cpp:1340
//   HierarchicalSDRStrategy::matmulRowMajor      strategies/HierarchicalSDRStrategy.cpp:1257
//   HierarchicalSDRStrategy::dequantizeToFP32    strategies/HierarchicalSDRStrategy.cpp:1017
//   compressGroupedSegments / SharedDictArchive  strategies/HierarchicalSDRStrategy.cpp:2211, :1972
//   HSDAReader::{decompress,matmul}              strategies/HierarchicalSDRStrategy.cpp:2523, :2536
//   AICompressor::compressModel (.sdr writer)    core/AICompressor.cpp:125
//   AIDecompressor::{readArchiveIndex,decompressSegment,readCompressedBytes}
//                                                core/AIDecompressor.cpp:78, :359, :418
#include "ai_compression/strategies/HierarchicalSDRStrategy.hpp"
#include "ai_compression/core/AICompressor.hpp"
#include "ai_compression/core/AIDecompressor.hpp"
#include "ai_compression/core/AIModelParser.hpp"
#include "ai_compression/core/ModelSegment.hpp"
#include "ai_compression/kernels/attention_kernels.hpp"
#include "ai_compression/kernels/blas_kernels.hpp"

#include <algorithm>
#include <chrono>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <memory>
#include <random>
#include <string>
#include <vector>

using namespace CortexAICompression;

namespace {

thread_local std::string g_err;

struct RefCfg {
    uint16_t tile_rows, tile_cols, n_atoms;
    uint8_t n_stages, k, ksvd_iters, pad;
    float decay;
    uint32_t max_tiles_for_fit;
};

HierarchicalSDRConfig toCfg(const RefCfg* c) {
    HierarchicalSDRConfig cfg;
    if (!c) return cfg;
    cfg.tile_rows = c->tile_rows;
    cfg.tile_cols = c->tile_cols;
    cfg.n_atoms = c->n_atoms;
    cfg.n_stages = c->n_stages;
    cfg.active_bits_per_stage = c->k;
    cfg.ksvd_iters = c->ksvd_iters;
    cfg.stage_decay = c->decay;
    cfg.max_tiles_for_fit = c->max_tiles_for_fit;
    return cfg;
}

struct SegDesc {
    const void* data;
    uint64_t nbytes;
    const char* name;
    const char* data_format;
    int32_t seg_type;
    uint32_t layer_index;
    uint32_t ndims;
    uint32_t dims[4];
    int32_t has_scale;
    float scale;
    float zero_point;
};

ModelSegment toSegment(const SegDesc& d) {
    ModelSegment seg;
    seg.type = static_cast<SegmentType>(d.seg_type);
    seg.name = d.name ? d.name : "";
    seg.layer_name = seg.name;
    seg.layer_index = d.layer_index;
    seg.data.resize(d.nbytes);
    if (d.nbytes) std::memcpy(seg.data.data(), d.data, d.nbytes);
    seg.original_size = seg.data.size();
    seg.data_format = d.data_format ? d.data_format : "";
    if (d.ndims > 0) {
        TensorMetadata meta;
        for (uint32_t i = 0; i < d.ndims; ++i) meta.dimensions.push_back(d.dims[i]);
        meta.sparsity_ratio = 0.0f;
        meta.is_sorted = false;
        if (d.has_scale) { meta.scale = d.scale; meta.zero_point = d.zero_point; }
        seg.tensor_metadata = meta;
        if (d.ndims == 2) {
            // Same convention as the reference's archive tests: dims = {R_out, C_in}.
            seg.input_shape = {1, d.dims[1]};
            seg.output_shape = {1, d.dims[0]};
            seg.layer_type = "LINEAR";
        }
    }
    return seg;
}

class ListParser : public IAIModelParser {
public:
    explicit ListParser(std::vector<ModelSegment> s) : segs_(std::move(s)) {}
    std::vector<ModelSegment> parse(const std::string&) const override { return segs_; }
private:
    std::vector<ModelSegment> segs_;
};

template <typename F>
long guarded(F&& f) {
    try {
        return f();
    } catch (const std::exception& e) {
        g_err = e.what();
        return -1;
    } catch (...) {
        g_err = "unknown exception";
        return -1;
    }
}

}  // namespace

extern "C" {

const char* ref_last_error() { return g_err.c_str(); }

// The reference's tests draw weights and activations from ONE std::mt19937 through
// fresh std::normal_distribution<float> objects (e.g. src/test_hsdr_roundtrip.cpp:205-227).
// This reproduces such a sequence: n_arrays consecutive arrays from one engine, each
// through its own distribution object, concatenated into out.
void ref_mt19937_normal(uint32_t seed, uint32_t n_arrays, const uint64_t* counts,
                        const float* means, const float* stddevs, float* out) {
    std::mt19937 rng(seed);
    for (uint32_t a = 0; a < n_arrays; ++a) {
        std::normal_distribution<float> dist(means[a], stddevs[a]);
        for (uint64_t i = 0; i < counts[a]; ++i) *out++ = dist(rng);
    }
}

void ref_free(void* p) { std::free(p); }

// The attention kernel the reference's decoder driver calls (kernels/attention_kernels.cpp:
// multi_head_attention, softmax from kernels/simd_kernels.cpp). q, k, v, out are
// (batch, seq, hidden) with hidden = heads * head_dim; kv heads already repeated by the caller
// as the driver does before the call.
long ref_multi_head_attention(const float* q, const float* k, const float* v, float* out, uint64_t batch,
                              uint64_t seq, uint64_t hidden, uint64_t heads, int causal) {
    return guarded([&]() -> long {
        CortexAICompression::Kernels::multi_head_attention(q, k, v, out, batch, seq, hidden, heads, causal != 0);
        return 0;
    });
}

// compress(): returns payload size, *out malloc'ed (free with ref_free). attn/mlp
// configs seed the strategy exactly as `HierarchicalSDRStrategy(attn, mlp)` does.
long ref_hsdr_compress(const SegDesc* seg, const RefCfg* attn_cfg, const RefCfg* mlp_cfg,
                       void** out) {
    return guarded([&]() -> long {
        HierarchicalSDRStrategy strat(toCfg(attn_cfg), mlp_cfg ? toCfg(mlp_cfg)
                                                              : HierarchicalSDRConfig::forMLP());
        auto bytes = strat.compress(toSegment(*seg));
        void* p = std::malloc(bytes.size() ? bytes.size() : 1);
        std::memcpy(p, bytes.data(), bytes.size());
        *out = p;
        return static_cast<long>(bytes.size());
    });
}

// decompress(): writes original_size bytes to out. Returns bytes written.
long ref_hsdr_decompress(const void* payload, uint64_t n, uint64_t original_size, void* out) {
    return guarded([&]() -> long {
        std::vector<std::byte> in(n);
        std::memcpy(in.data(), payload, n);
        HierarchicalSDRStrategy strat;
        auto bytes = strat.decompress(in, SegmentType::WEIGHTS_FP32, original_size);
        std::memcpy(out, bytes.data(), bytes.size());
        return static_cast<long>(bytes.size());
    });
}

// matmulRowMajor(): x is (C x batch) row-major, y is (R x batch) row-major.
// `payload_vec` lets a caller keep the std::vector alive across timed calls.
long ref_hsdr_matmul(const void* payload, uint64_t n, const float* x, uint64_t batch,
                     float* y, uint64_t y_cap) {
    return guarded([&]() -> long {
        std::vector<std::byte> in(n);
        std::memcpy(in.data(), payload, n);
        HierarchicalSDRStrategy strat;
        auto Y = strat.matmulRowMajor(in, x, batch);
        if (Y.size() > y_cap) throw std::runtime_error("ref_hsdr_matmul: output buffer too small");
        std::memcpy(y, Y.data(), Y.size() * sizeof(float));
        return static_cast<long>(Y.size());
    });
}

// Timed variant for the CPU baseline: the payload is copied into the byte vector
// ONCE (payload bytes already in memory, as the reference's own tests time it),
// then 2 warm-ups and `iters` timed calls of matmulRowMajor; *sec_median gets the
// median seconds per call. matmulRowMajor is single-threaded by construction.
long ref_hsdr_matmul_timed(const void* payload, uint64_t n, const float* x, uint64_t batch,
                           int iters, double* sec_median, float* y, uint64_t y_cap) {
    return guarded([&]() -> long {
        std::vector<std::byte> in(n);
        std::memcpy(in.data(), payload, n);
        HierarchicalSDRStrategy strat;
        std::vector<double> t;
        std::vector<float> Y;
        for (int i = 0; i < iters + 2; ++i) {
            auto t0 = std::chrono::steady_clock::now();
            Y = strat.matmulRowMajor(in, x, batch);
            auto t1 = std::chrono::steady_clock::now();
            if (i >= 2) t.push_back(std::chrono::duration<double>(t1 - t0).count());
        }
        std::sort(t.begin(), t.end());
        *sec_median = t[t.size() / 2];
        if (y) {
            if (Y.size() > y_cap) throw std::runtime_error("ref_hsdr_matmul_timed: buffer too small");
            std::memcpy(y, Y.data(), Y.size() * sizeof(float));
        }
        return static_cast<long>(Y.size());
    });
}

// The reference's non-fused route: decompress() then Kernels::linear_forward
// (kernels/blas_kernels.cpp:264; no BLAS here, so std::thread row chunks at batch 1
// and the plain gemm otherwise). x_tm is TOKEN-major (batch x C), y_tm (batch x R).
// Both halves are timed together; median of `iters` after 1 warm-up.
long ref_hsdr_decompress_dense_timed(const void* payload, uint64_t n, uint64_t R, uint64_t C,
                                     const float* x_tm, uint64_t batch, int iters,
                                     double* sec_median, float* y_tm) {
    return guarded([&]() -> long {
        std::vector<std::byte> in(n);
        std::memcpy(in.data(), payload, n);
        HierarchicalSDRStrategy strat;
        std::vector<double> t;
        std::vector<float> Y(R * batch);
        for (int i = 0; i < iters + 1; ++i) {
            auto t0 = std::chrono::steady_clock::now();
            auto W = strat.decompress(in, SegmentType::WEIGHTS_FP32, R * C * sizeof(float));
            Kernels::linear_forward(x_tm, reinterpret_cast<const float*>(W.data()), nullptr,
                                    Y.data(), batch, C, R);
            auto t1 = std::chrono::steady_clock::now();
            if (i >= 1) t.push_back(std::chrono::duration<double>(t1 - t0).count());
        }
        std::sort(t.begin(), t.end());
        *sec_median = t[t.size() / 2];
        if (y_tm) std::memcpy(y_tm, Y.data(), Y.size() * sizeof(float));
        return static_cast<long>(Y.size());
    });
}

long ref_dequantize(const SegDesc* seg, float* out, uint64_t out_cap) {
    return guarded([&]() -> long {
        auto v = HierarchicalSDRStrategy::dequantizeToFP32(toSegment(*seg));
        if (v.size() > out_cap) throw std::runtime_error("ref_dequantize: output buffer too small");
        std::memcpy(out, v.data(), v.size() * sizeof(float));
        return static_cast<long>(v.size());
    });
}

// compressGroupedSegments -> .hsda file. Returns number of dictionaries.
long ref_hsda_write(const SegDesc* segs, uint32_t n_segs, const RefCfg* attn_cfg,
                    const RefCfg* mlp_cfg, const char* path) {
    return guarded([&]() -> long {
        HierarchicalSDRStrategy strat(toCfg(attn_cfg), mlp_cfg ? toCfg(mlp_cfg)
                                                              : HierarchicalSDRConfig::forMLP());
        std::vector<ModelSegment> v;
        for (uint32_t i = 0; i < n_segs; ++i) v.push_back(toSegment(segs[i]));
        std::vector<std::string> skipped;
        auto archive = strat.compressGroupedSegments(v, &skipped);
        if (!skipped.empty()) throw std::runtime_error("ref_hsda_write: segment skipped: " + skipped[0]);
        archive.writeToFile(path);
        return static_cast<long>(archive.dictionaries.size());
    });
}

long ref_hsda_matmul(const char* path, const char* name, const float* x, uint64_t batch,
                     float* y, uint64_t y_cap) {
    return guarded([&]() -> long {
        HSDAReader rd = HSDAReader::fromFile(path);
        auto Y = rd.matmul(name, x, batch);
        if (Y.size() > y_cap) throw std::runtime_error("ref_hsda_matmul: output buffer too small");
        std::memcpy(y, Y.data(), Y.size() * sizeof(float));
        return static_cast<long>(Y.size());
    });
}

long ref_hsda_decompress(const char* path, const char* name, void* out, uint64_t out_cap) {
    return guarded([&]() -> long {
        HSDAReader rd = HSDAReader::fromFile(path);
        auto b = rd.decompress(name);
        if (b.size() > out_cap) throw std::runtime_error("ref_hsda_decompress: output buffer too small");
        std::memcpy(out, b.data(), b.size());
        return static_cast<long>(b.size());
    });
}

// AICompressor -> .sdr. HSDR (id 5) is the only registered strategy, on the four
// weight segment types the reference CLI registers it for; everything else lands
// as strategy id 0 (stored raw), as the reference writer does when nothing fits.
long ref_sdr_write(const SegDesc* segs, uint32_t n_segs, const RefCfg* attn_cfg,
                   const RefCfg* mlp_cfg, const char* path) {
    return guarded([&]() -> long {
        std::vector<ModelSegment> v;
        for (uint32_t i = 0; i < n_segs; ++i) v.push_back(toSegment(segs[i]));
        AICompressor compressor(std::make_unique<ListParser>(std::move(v)));
        auto strat = std::make_shared<HierarchicalSDRStrategy>(
            toCfg(attn_cfg), mlp_cfg ? toCfg(mlp_cfg) : HierarchicalSDRConfig::forMLP());
        constexpr uint8_t HSDR_ID = 5;
        compressor.registerStrategy(SegmentType::WEIGHTS_FP32, 1, HSDR_ID, strat);
        compressor.registerStrategy(SegmentType::ATTENTION_WEIGHTS, 1, HSDR_ID, strat);
        compressor.registerStrategy(SegmentType::FEED_FORWARD_WEIGHTS, 1, HSDR_ID, strat);
        compressor.registerStrategy(SegmentType::EMBEDDING_WEIGHTS, 1, HSDR_ID, strat);
        std::ofstream out(path, std::ios::binary | std::ios::trunc);
        if (!out) throw std::runtime_error(std::string("ref_sdr_write: cannot open ") + path);
        compressor.compressModel("", out);
        return static_cast<long>(n_segs);
    });
}

// Reference reader: decompress a named segment of a .sdr to fp32 bytes.
long ref_sdr_decompress(const char* path, const char* name, void* out, uint64_t out_cap) {
    return guarded([&]() -> long {
        AIDecompressor dec;
        dec.registerStrategy(5, std::make_shared<HierarchicalSDRStrategy>());
        std::ifstream in(path, std::ios::binary);
        if (!in) throw std::runtime_error(std::string("ref_sdr_decompress: cannot open ") + path);
        auto headers = dec.readArchiveHeaders(in);
        for (const auto& h : headers) {
            if (h.name != name) continue;
            ModelSegment s = dec.decompressSegment(path, h, h.data_offset);
            if (s.data.size() > out_cap) throw std::runtime_error("ref_sdr_decompress: buffer too small");
            std::memcpy(out, s.data.data(), s.data.size());
            return static_cast<long>(s.data.size());
        }
        throw std::runtime_error(std::string("Segment not found: ") + name);
    });
}

// Reference path of SDRModelLoader::matmulHSDR (SparseInferenceEngine.cpp:1074)
// restated over the reference's own reader + strategy: header lookup, strategy-id
// check, per-call file read, matmulRowMajor.
long ref_sdr_matmul(const char* path, const char* name, const float* x, uint64_t batch,
                    float* y, uint64_t y_cap) {
    return guarded([&]() -> long {
        AIDecompressor dec;
        std::ifstream in(path, std::ios::binary);
        if (!in) throw std::runtime_error(std::string("ref_sdr_matmul: cannot open ") + path);
        auto headers = dec.readArchiveHeaders(in);
        for (const auto& h : headers) {
            if (h.name != name) continue;
            if (h.compression_strategy_id != 5)
                throw std::runtime_error("matmulHSDR: segment '" + h.name +
                                         "' is not HSDR-encoded (strategy_id=" +
                                         std::to_string(h.compression_strategy_id) + ")");
            auto raw = dec.readCompressedBytes(path, h, h.data_offset);
            HierarchicalSDRStrategy strat;
            auto Y = strat.matmulRowMajor(raw, x, batch);
            if (Y.size() > y_cap) throw std::runtime_error("ref_sdr_matmul: buffer too small");
            std::memcpy(y, Y.data(), Y.size() * sizeof(float));
            return static_cast<long>(Y.size());
        }
        throw std::runtime_error(std::string("matmulHSDR: segment not found: ") + name);
    });
}

}  // extern "C"
