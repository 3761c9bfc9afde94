// C++17 host side of the routing entry points: the .sdr loader
// (SDRModelLoader, SparseInferenceEngine.cpp:725-751, :994, :1044-1091), the matmul
// routing of SDRInferenceEngine (matmulForLayer :1271-1311, applyLinearLayer HSDR
// branches :1487-1521), and the .hsda reader (HSDAReader,
// strategies/HierarchicalSDRStrategy.cpp:2506-2550). Everything numeric goes through
// the thin extern "C" CUDA layer; what the reference redoes on every call (file open,
// payload read, dictionary copy) happens here once per segment, on first use.
#include <cstring>
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

#include "../internal.hpp"

using namespace csdr;

struct csdr_archive {
    csdr_context* ctx = nullptr;
    ArchiveIndex index;
    std::unordered_map<std::string, csdr_segment*> images;  // HSDR device images
    std::unordered_map<std::string, DevPtr> raw;            // stored-raw fp32 matrices
    std::unordered_map<std::string, csdr_dictionary*> dicts;  // shared-dictionary resource segments, by name
    ~csdr_archive() {
        for (auto& kv : images) csdr_segment_destroy(kv.second);
        for (auto& kv : dicts) csdr_dictionary_destroy(kv.second);
    }
};

struct csdr_hsda {
    csdr_context* ctx = nullptr;
    HsdaFile file;
    std::vector<csdr_dictionary*> dicts;
    std::unordered_map<std::string, csdr_segment*> images;
    ~csdr_hsda() {
        for (auto& kv : images) csdr_segment_destroy(kv.second);
        for (auto* d : dicts) csdr_dictionary_destroy(d);
    }
};

namespace {

void rethrow_last(int rc) {
    if (rc != CSDR_OK) throw Error(rc, csdr_last_error());
}

void need_device(csdr_context* ctx) {
    if (!ctx) throw Error(CSDR_ERR_CUDA, "opened without a device context: no compute available (this library has no CPU path)");
    require_ctx(ctx);
}

const SegmentHeader& need_header(const csdr_archive* ar, const char* name, const char* who) {
    if (!ar || !name) throw Error(CSDR_ERR_INVALID_ARG, "null argument");
    const SegmentHeader* h = ar->index.find(name);
    if (!h) throw Error(CSDR_ERR_NOT_FOUND, std::string(who) + name);
    return *h;
}

// Device image of a shared-dictionary resource segment (kSharedDictFormat), uploaded once and
// shared by every tensor coded against it.
const csdr_dictionary* dictionary_of(csdr_archive* ar, const std::string& name, const std::string& user) {
    auto it = ar->dicts.find(name);
    if (it != ar->dicts.end()) return it->second;
    const SegmentHeader* dh = ar->index.find(name);
    if (!dh) throw Error(CSDR_ERR_NOT_FOUND, "shared dictionary '" + name + "' named by segment '" + user + "' is not in the archive");
    if (dh->strategy_id != 0 || dh->data_format != kSharedDictFormat)
        throw Error(CSDR_ERR_FORMAT, "segment '" + name + "' is not a shared-dictionary resource (stored raw, data_format hsdr_dict)");
    const std::vector<uint8_t> bytes = ar->index.read_payload(*dh);
    const HsdaDictionary d = parse_dictionary_record(bytes.data(), bytes.size(), "shared dictionary");
    csdr_dictionary* dict = nullptr;
    rethrow_last(csdr_dictionary_create(ar->ctx, d.tile_rows, d.tile_cols, d.n_atoms, d.n_stages, d.k_per_stage, d.atoms.data(),
                                        d.scales.data(), &dict));
    ar->dicts.emplace(name, dict);
    return dict;
}

const csdr_segment* image_of(csdr_archive* ar, const SegmentHeader& h) {
    auto it = ar->images.find(h.name);
    if (it != ar->images.end()) return it->second;
    const std::vector<uint8_t> bytes = ar->index.read_payload(h);
    csdr_segment* seg = nullptr;
    if (bytes.size() >= 4 && std::memcmp(bytes.data(), "HSDC", 4) == 0) {
        // codes only: the dictionary is a resource segment of this archive, named behind "hsdc@"
        const size_t plen = std::strlen(kSharedCodesPrefix);
        if (h.data_format.compare(0, plen, kSharedCodesPrefix) != 0 || h.data_format.size() == plen)
            throw Error(CSDR_ERR_FORMAT, "segment '" + h.name + "' holds codes only but names no shared dictionary (data_format hsdc@<segment>)");
        const csdr_dictionary* dict = dictionary_of(ar, h.data_format.substr(plen), h.name);
        rethrow_last(csdr_segment_create_shared(ar->ctx, bytes.data(), bytes.size(), dict, &seg));
    } else {
        rethrow_last(csdr_segment_create(ar->ctx, bytes.data(), bytes.size(), &seg));
    }
    ar->images.emplace(h.name, seg);
    return seg;
}

void fill_header(const SegmentHeader& s, csdr_segment_header* h) {
    std::memset(h, 0, sizeof(*h));
    h->name = s.name.c_str();
    h->data_format = s.data_format.c_str();
    h->layer_type = s.layer_type.c_str();
    h->original_type = s.original_type;
    h->strategy_id = s.strategy_id;
    h->original_size = s.original_size;
    h->compressed_size = s.compressed_size;
    h->data_offset = s.data_offset;
    h->layer_index = s.layer_index;
    h->n_dims = static_cast<uint32_t>(std::min<size_t>(8, s.dims.size()));
    for (uint32_t i = 0; i < h->n_dims; ++i) h->dims[i] = s.dims[i];
}

// Host-buffer product through a device image; x/y in the reference layout unless
// token_major.
void matmul_host(csdr_context* ctx, const csdr_segment* seg, const float* x, size_t batch,
                 float* y, bool token_major, const float* bias_host) {
    const Geometry& g = seg->g;
    const size_t xb = static_cast<size_t>(g.cols) * batch * 4, yb = static_cast<size_t>(g.rows) * batch * 4;
    const size_t xoff = (xb + 255) & ~static_cast<size_t>(255);
    const size_t yoff = (yb + 255) & ~static_cast<size_t>(255);
    unsigned char* buf = static_cast<unsigned char*>(
        ctx->scratch_get(3, xoff + yoff + static_cast<size_t>(g.rows) * 4));
    float* xd = reinterpret_cast<float*>(buf);
    float* yd = reinterpret_cast<float*>(buf + xoff);
    float* bd = reinterpret_cast<float*>(buf + xoff + yoff);
    CSDR_CUDA(cudaMemcpyAsync(xd, x, xb, cudaMemcpyHostToDevice, ctx->stream));
    if (bias_host)
        CSDR_CUDA(cudaMemcpyAsync(bd, bias_host, static_cast<size_t>(g.rows) * 4,
                                  cudaMemcpyHostToDevice, ctx->stream));
    const int layout = token_major ? CSDR_LAYOUT_TOKEN_MAJOR : CSDR_LAYOUT_FEATURE_MAJOR;
    rethrow_last(csdr_matmul_device_async(ctx, seg, xd, CSDR_DTYPE_F32, layout, batch, yd, layout,
                                          bias_host ? bd : nullptr));
    CSDR_CUDA(cudaMemcpyAsync(y, yd, yb, cudaMemcpyDeviceToHost, ctx->stream));
    CSDR_CUDA(cudaStreamSynchronize(ctx->stream));
}

void require_row_tiles(const csdr_segment* seg, const char* who) {
    const Geometry& g = seg->g;
    if (g.tile_rows != 1)
        throw Error(CSDR_ERR_GEOMETRY, std::string(who) +
                                           ": fused matmul requires tile_rows == 1; use decompress() + "
                                           "dense matmul for 2D tile encodings");
    if (g.tile_cols != g.cols)
        throw Error(CSDR_ERR_GEOMETRY, std::string(who) + ": 1D row-tile encoding must have tile_cols == original_cols");
}

}  // namespace

extern "C" {

int csdr_archive_open(csdr_context* ctx, const char* path, csdr_archive** out) {
    return guard([&] {
        // ctx may be NULL: index, headers and raw payload reads work without a device;
        // every compute entry point then fails with CSDR_ERR_CUDA.
        if (ctx) require_ctx(ctx);
        if (!path || !out) throw Error(CSDR_ERR_INVALID_ARG, "null argument");
        auto ar = std::make_unique<csdr_archive>();
        ar->ctx = ctx;
        ar->index = ArchiveIndex::open(path);
        *out = ar.release();
    });
}

int csdr_archive_close(csdr_archive* ar) {
    return guard([&] { delete ar; });
}

int csdr_archive_num_segments(const csdr_archive* ar, size_t* n) {
    return guard([&] {
        if (!ar || !n) throw Error(CSDR_ERR_INVALID_ARG, "null argument");
        *n = ar->index.segments.size();
    });
}

int csdr_archive_header_at(const csdr_archive* ar, size_t i, csdr_segment_header* h) {
    return guard([&] {
        if (!ar || !h) throw Error(CSDR_ERR_INVALID_ARG, "null argument");
        if (i >= ar->index.segments.size()) throw Error(CSDR_ERR_NOT_FOUND, "segment index out of range");
        fill_header(ar->index.segments[i], h);
    });
}

int csdr_archive_find(const csdr_archive* ar, const char* name, csdr_segment_header* h) {
    return guard([&] {
        const SegmentHeader& s = need_header(ar, name, "Segment not found: ");
        if (h) fill_header(s, h);
    });
}

int csdr_archive_read_payload(const csdr_archive* ar, const char* name, void* buf, size_t capacity,
                              size_t* n) {
    return guard([&] {
        const SegmentHeader& s = need_header(ar, name, "Segment not found: ");
        if (n) *n = s.compressed_size;
        if (!buf || capacity < s.compressed_size) throw Error(CSDR_ERR_BUFFER, "payload buffer too small");
        const auto bytes = ar->index.read_payload(s);
        std::memcpy(buf, bytes.data(), bytes.size());
    });
}

int csdr_archive_segment(csdr_archive* ar, const char* name, const csdr_segment** seg) {
    return guard([&] {
        const SegmentHeader& s = need_header(ar, name, "Segment not found: ");
        if (!seg) throw Error(CSDR_ERR_INVALID_ARG, "null argument");
        if (s.strategy_id != kHSDRStrategyId)
            throw Error(CSDR_ERR_STRATEGY, "segment '" + s.name + "' is not HSDR-encoded (strategy_id=" +
                                               std::to_string(s.strategy_id) + ")");
        need_device(ar->ctx);
        *seg = image_of(ar, s);
    });
}

int csdr_archive_release(csdr_archive* ar, const char* name) {
    return guard([&] {
        if (!ar) throw Error(CSDR_ERR_INVALID_ARG, "null argument");
        if (!name) {
            for (auto& kv : ar->images) csdr_segment_destroy(kv.second);
            ar->images.clear();
            for (auto& kv : ar->dicts) csdr_dictionary_destroy(kv.second);
            ar->dicts.clear();
            ar->raw.clear();
            return;
        }
        auto it = ar->images.find(name);
        if (it != ar->images.end()) {
            csdr_segment_destroy(it->second);
            ar->images.erase(it);
        }
        ar->raw.erase(name);
    });
}

int csdr_archive_resident_bytes(const csdr_archive* ar, size_t* bytes) {
    return guard([&] {
        if (!ar || !bytes) throw Error(CSDR_ERR_INVALID_ARG, "null argument");
        size_t n = 0;
        std::unordered_map<const void*, size_t> dictionaries;   // a shared dictionary counts once
        for (const auto& kv : ar->images) {
            const csdr_segment* sg = kv.second;
            dictionaries[sg->atoms->ptr] = sg->atoms->bytes;
            n += sg->codes->bytes + sg->scales->bytes + (sg->edges ? sg->edges->bytes : 0);
        }
        for (const auto& kv : ar->dicts) dictionaries[kv.second->atoms->ptr] = kv.second->atoms->bytes;
        for (const auto& kv : dictionaries) n += kv.second;
        for (const auto& kv : ar->raw) n += kv.second->bytes;
        *bytes = n;
    });
}

int csdr_archive_load_segment(csdr_archive* ar, const char* name, void* buf, size_t capacity,
                              size_t* n) {
    return guard([&] {
        const SegmentHeader& s = need_header(ar, name, "Segment not found: ");
        if (s.strategy_id == 0) {
            if (n) *n = s.compressed_size;
            if (!buf || capacity < s.compressed_size) throw Error(CSDR_ERR_BUFFER, "segment buffer too small");
            const auto bytes = ar->index.read_payload(s);
            std::memcpy(buf, bytes.data(), bytes.size());
            return;
        }
        if (s.strategy_id != kHSDRStrategyId)
            throw Error(CSDR_ERR_UNSUPPORTED, "Unknown or unregistered compression strategy ID: " +
                                                  std::to_string(s.strategy_id));
        need_device(ar->ctx);
        const csdr_segment* seg = image_of(ar, s);
        const size_t bytes = static_cast<size_t>(seg->g.rows) * seg->g.cols * 4;
        if (n) *n = bytes;
        if (!buf || capacity < bytes) throw Error(CSDR_ERR_BUFFER, "segment buffer too small");
        rethrow_last(csdr_decompress(ar->ctx, seg, static_cast<float*>(buf), bytes / 4));
    });
}

int csdr_archive_matmul_hsdr(csdr_archive* ar, const char* name, const float* x, size_t batch,
                             float* y, size_t y_capacity, size_t* n_out) {
    return guard([&] {
        const SegmentHeader& s = need_header(ar, name, "matmulHSDR: segment not found: ");
        if (s.strategy_id != kHSDRStrategyId)
            throw Error(CSDR_ERR_STRATEGY, "matmulHSDR: segment '" + s.name +
                                               "' is not HSDR-encoded (strategy_id=" +
                                               std::to_string(s.strategy_id) + ")");
        if (!x || !y) throw Error(CSDR_ERR_INVALID_ARG, "null argument");
        need_device(ar->ctx);
        const csdr_segment* seg = image_of(ar, s);
        require_row_tiles(seg, "HSDR matmul");
        const size_t need = static_cast<size_t>(seg->g.rows) * batch;
        if (n_out) *n_out = need;
        if (y_capacity < need) throw Error(CSDR_ERR_BUFFER, "matmulHSDR: output buffer too small");
        if (batch) matmul_host(ar->ctx, seg, x, batch, y, false, nullptr);
    });
}

int csdr_archive_matmul_for_layer(csdr_archive* ar, const char* name, const float* x, size_t batch,
                                  float* y, size_t y_capacity, size_t* n_out) {
    return guard([&] {
        const SegmentHeader& s = need_header(ar, name, "Segment not found: ");
        if (!x || !y) throw Error(CSDR_ERR_INVALID_ARG, "null argument");
        need_device(ar->ctx);
        if (s.strategy_id == kHSDRStrategyId) {
            const csdr_segment* seg = image_of(ar, s);
            const size_t need = static_cast<size_t>(seg->g.rows) * batch;
            if (n_out) *n_out = need;
            if (y_capacity < need) throw Error(CSDR_ERR_BUFFER, "matmulForLayer: output buffer too small");
            if (batch) matmul_host(ar->ctx, seg, x, batch, y, false, nullptr);
            return;
        }
        // Dense fallback, SparseInferenceEngine.cpp:1284-1310.
        if (s.strategy_id != 0)
            throw Error(CSDR_ERR_UNSUPPORTED, "matmulForLayer: segment '" + s.name +
                                                  "' uses a strategy this library does not decode");
        if (!s.has_meta || s.dims.size() != 2)
            throw Error(CSDR_ERR_GEOMETRY, "matmulForLayer: segment '" + s.name +
                                               "' has no 2-D tensor_metadata; cannot fall back to dense matmul");
        if (s.compressed_size % 4 || s.compressed_size < static_cast<uint64_t>(s.dims[0]) * s.dims[1] * 4)
            throw Error(CSDR_ERR_GEOMETRY, "matmulForLayer: segment '" + s.name + "' is not FP32");
        const uint32_t R = s.dims[0], C = s.dims[1];
        const size_t need = static_cast<size_t>(R) * batch;
        if (n_out) *n_out = need;
        if (y_capacity < need) throw Error(CSDR_ERR_BUFFER, "matmulForLayer: output buffer too small");
        if (!batch) return;
        auto it = ar->raw.find(s.name);
        if (it == ar->raw.end()) {
            const auto bytes = ar->index.read_payload(s);
            DevPtr w = upload(ar->ctx, bytes.data(), bytes.size());
            CSDR_CUDA(cudaStreamSynchronize(ar->ctx->stream));
            it = ar->raw.emplace(s.name, std::move(w)).first;
        }
        csdr_context* ctx = ar->ctx;
        const size_t xb = static_cast<size_t>(C) * batch * 4, yb = need * 4;
        const size_t xoff = (xb + 255) & ~static_cast<size_t>(255);
        unsigned char* buf = static_cast<unsigned char*>(ctx->scratch_get(3, xoff + yb));
        CSDR_CUDA(cudaMemcpyAsync(buf, x, xb, cudaMemcpyHostToDevice, ctx->stream));
        MatmulArgs a;
        a.x = buf;
        a.batch = batch;
        a.y = reinterpret_cast<float*>(buf + xoff);
        launch_dense_matmul(ctx, static_cast<const float*>(it->second->ptr), R, C, a);
        CSDR_CUDA(cudaMemcpyAsync(y, buf + xoff, yb, cudaMemcpyDeviceToHost, ctx->stream));
        CSDR_CUDA(cudaStreamSynchronize(ctx->stream));
    });
}

int csdr_archive_apply_linear(csdr_archive* ar, const char* layer, const float* input,
                              size_t input_size, const float* bias, float* output, size_t capacity,
                              size_t* n_out) {
    return guard([&] {
        if (!ar || !layer || !input || !output) throw Error(CSDR_ERR_INVALID_ARG, "null argument");
        // applyLinearLayer tries the layer name, then name + ".weight" (:1489-1494).
        const SegmentHeader* s = ar->index.find(layer);
        if (!s) s = ar->index.find(std::string(layer) + ".weight");
        if (!s) throw Error(CSDR_ERR_NOT_FOUND, std::string("Segment not found: ") + layer);
        if (s->strategy_id != kHSDRStrategyId)
            throw Error(CSDR_ERR_STRATEGY, "segment '" + s->name + "' is not HSDR-encoded (strategy_id=" +
                                               std::to_string(s->strategy_id) + ")");
        need_device(ar->ctx);
        const csdr_segment* seg = image_of(ar, *s);
        const size_t C = seg->g.cols, R = seg->g.rows;
        if (input_size == 0 || input_size % C)
            throw Error(CSDR_ERR_INVALID_ARG, "input size is not a multiple of the layer's input width");
        const size_t batch = input_size / C;
        if (n_out) *n_out = batch * R;
        if (capacity < batch * R) throw Error(CSDR_ERR_BUFFER, "output buffer too small");
        matmul_host(ar->ctx, seg, input, batch, output, true, bias);
    });
}

int csdr_hsda_open(csdr_context* ctx, const char* path, csdr_hsda** out) {
    return guard([&] {
        if (ctx) require_ctx(ctx);  // NULL: container structure only, as for archives
        if (!path || !out) throw Error(CSDR_ERR_INVALID_ARG, "null argument");
        auto h = std::make_unique<csdr_hsda>();
        h->ctx = ctx;
        h->file = HsdaFile::open(path);
        h->dicts.assign(h->file.dicts.size(), nullptr);
        *out = h.release();
    });
}

int csdr_hsda_close(csdr_hsda* h) {
    return guard([&] { delete h; });
}

int csdr_hsda_counts(const csdr_hsda* h, size_t* n_dicts, size_t* n_segments) {
    return guard([&] {
        if (!h) throw Error(CSDR_ERR_INVALID_ARG, "null argument");
        if (n_dicts) *n_dicts = h->file.dicts.size();
        if (n_segments) *n_segments = h->file.segments.size();
    });
}

int csdr_hsda_has_segment(const csdr_hsda* h, const char* name) {
    return (h && name && h->file.by_name.count(name)) ? 1 : 0;
}

int csdr_hsda_segment(csdr_hsda* h, const char* name, const csdr_segment** seg) {
    return guard([&] {
        if (!h || !name || !seg) throw Error(CSDR_ERR_INVALID_ARG, "null argument");
        auto it = h->file.by_name.find(name);
        if (it == h->file.by_name.end())
            throw Error(CSDR_ERR_NOT_FOUND, std::string("HSDAReader: segment not found: ") + name);
        need_device(h->ctx);
        auto im = h->images.find(name);
        if (im == h->images.end()) {
            const HsdaSegment& s = h->file.segments[it->second];
            if (!h->dicts[s.dict_index]) {
                // Dictionaries go to the device once, on first use by any of their segments.
                HsdaDictionary& d = h->file.dicts[s.dict_index];
                rethrow_last(csdr_dictionary_create(h->ctx, d.tile_rows, d.tile_cols, d.n_atoms,
                                                    d.n_stages, d.k_per_stage, d.atoms.data(),
                                                    d.scales.data(), &h->dicts[s.dict_index]));
                std::vector<float>().swap(d.atoms);
            }
            csdr_segment* sg = nullptr;
            rethrow_last(csdr_segment_create_shared(h->ctx, s.codes.data(), s.codes.size(),
                                                    h->dicts[s.dict_index], &sg));
            im = h->images.emplace(name, sg).first;
        }
        *seg = im->second;
    });
}

int csdr_hsda_matmul(csdr_hsda* h, const char* name, const float* x, size_t batch, float* y,
                     size_t y_capacity, size_t* n_out, int allow_2d) {
    return guard([&] {
        const csdr_segment* seg = nullptr;
        rethrow_last(csdr_hsda_segment(h, name, &seg));
        if (!x || !y) throw Error(CSDR_ERR_INVALID_ARG, "null argument");
        if (!allow_2d) require_row_tiles(seg, "matmulWithExternalDictionary");
        const size_t need = static_cast<size_t>(seg->g.rows) * batch;
        if (n_out) *n_out = need;
        if (y_capacity < need) throw Error(CSDR_ERR_BUFFER, "HSDAReader::matmul: output buffer too small");
        if (batch) matmul_host(h->ctx, seg, x, batch, y, false, nullptr);
    });
}

int csdr_hsda_decompress(csdr_hsda* h, const char* name, float* out, size_t capacity_floats,
                         size_t* n_out) {
    return guard([&] {
        const csdr_segment* seg = nullptr;
        rethrow_last(csdr_hsda_segment(h, name, &seg));
        const HsdaSegment& s = h->file.segments[h->file.by_name.at(name)];
        const size_t n = static_cast<size_t>(seg->g.rows) * seg->g.cols;
        // decompressWithExternalDictionary insists on the recorded size (:1812-1814).
        if (s.original_size != n * 4)
            throw Error(CSDR_ERR_FORMAT, "decompressWithExternalDictionary: originalSize mismatch");
        if (n_out) *n_out = n;
        if (!out || capacity_floats < n) throw Error(CSDR_ERR_BUFFER, "HSDAReader::decompress: buffer too small");
        rethrow_last(csdr_decompress(h->ctx, seg, out, capacity_floats));
    });
}

}  // extern "C"
