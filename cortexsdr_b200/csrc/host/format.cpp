#include "format.hpp"

#include <cstring>
#include <fstream>

namespace csdr {

namespace {

constexpr size_t kHSDRHeaderBytes = 36;
constexpr size_t kHSDCHeaderBytes = 32;

template <typename T>
T rd(const uint8_t* p) {
    T v;
    std::memcpy(&v, p, sizeof(T));
    return v;
}

// Bounded cursor over a little-endian byte stream.
struct Cursor {
    std::istream& in;
    const char* what;
    template <typename T>
    T pod() {
        T v{};
        in.read(reinterpret_cast<char*>(&v), sizeof(T));
        if (in.gcount() != static_cast<std::streamsize>(sizeof(T)))
            throw Error(CSDR_ERR_FORMAT, std::string(what) + ": truncated stream");
        return v;
    }
    std::string str(uint64_t max_len) {
        const uint32_t len = pod<uint32_t>();
        if (len > max_len) throw Error(CSDR_ERR_FORMAT, std::string(what) + ": string length out of range");
        std::string s(len, '\0');
        if (len) {
            in.read(s.data(), len);
            if (in.gcount() != static_cast<std::streamsize>(len))
                throw Error(CSDR_ERR_FORMAT, std::string(what) + ": truncated string");
        }
        return s;
    }
    template <typename T>
    void array(T* dst, size_t count) {
        if (!count) return;
        in.read(reinterpret_cast<char*>(dst), static_cast<std::streamsize>(sizeof(T) * count));
        if (in.gcount() != static_cast<std::streamsize>(sizeof(T) * count))
            throw Error(CSDR_ERR_FORMAT, std::string(what) + ": truncated array");
    }
};

std::vector<uint32_t> read_shape(Cursor& c) {
    std::vector<uint32_t> shape;
    if (c.pod<uint8_t>()) {
        const uint8_t n = c.pod<uint8_t>();
        shape.resize(n);
        for (auto& d : shape) d = c.pod<uint32_t>();
    }
    return shape;
}

}  // namespace

csdr_payload_info inspect_payload(const uint8_t* p, size_t n, bool check_codes) {
    if (!p) throw Error(CSDR_ERR_INVALID_ARG, "payload is null");
    if (n < kHSDCHeaderBytes) throw Error(CSDR_ERR_FORMAT, "HSDR: unexpected end-of-stream");
    csdr_payload_info v{};
    if (std::memcmp(p, "HSDR", 4) == 0) v.kind = CSDR_KIND_HSDR;
    else if (std::memcmp(p, "HSDC", 4) == 0) v.kind = CSDR_KIND_HSDC;
    else throw Error(CSDR_ERR_FORMAT, "HSDR: bad magic - not an HSDR/HSDC stream");
    const uint32_t version = rd<uint32_t>(p + 4);
    if (v.kind == CSDR_KIND_HSDR) {
        if (n < kHSDRHeaderBytes) throw Error(CSDR_ERR_FORMAT, "HSDR: unexpected end-of-stream");
        if (version != 2) throw Error(CSDR_ERR_FORMAT, "HSDR: unsupported version");
    } else if (version != 1) {
        throw Error(CSDR_ERR_FORMAT, "HSDR shared: unsupported codes-stream version");
    }
    v.rows = rd<uint32_t>(p + 8);
    v.cols = rd<uint32_t>(p + 12);
    v.n_tiles = rd<uint32_t>(p + 16);
    v.tile_rows = rd<uint16_t>(p + 20);
    v.tile_cols = rd<uint16_t>(p + 22);
    v.n_atoms = rd<uint16_t>(p + 24);
    v.n_stages = p[26];
    v.k_per_stage = p[27];
    v.stage_decay = rd<float>(p + 28);
    if (v.tile_rows == 0 || v.tile_cols == 0 || v.n_atoms == 0 || v.n_stages == 0 ||
        v.k_per_stage == 0 || v.rows == 0 || v.cols == 0)
        throw Error(CSDR_ERR_FORMAT, "HSDR: zero-sized geometry field");
    if (v.n_atoms > 0x7FFFu) throw Error(CSDR_ERR_FORMAT, "HSDR: n_atoms exceeds the 15-bit index range");
    const uint64_t tile_dim = static_cast<uint64_t>(v.tile_rows) * v.tile_cols;
    const uint64_t n_codes = static_cast<uint64_t>(v.n_tiles) * v.n_stages * v.k_per_stage;
    const uint64_t full_tiles =
        static_cast<uint64_t>(v.rows / v.tile_rows) * (v.cols / v.tile_cols);
    if (full_tiles != v.n_tiles)
        throw Error(CSDR_ERR_FORMAT, "HSDR: tile count does not match shape and tile size");
    if (v.kind == CSDR_KIND_HSDR) {
        v.edge_bytes = rd<uint32_t>(p + 32);
        v.off_scales = kHSDRHeaderBytes;
        v.off_dict = v.off_scales + 4ull * v.n_stages;
        v.off_codes = v.off_dict + 4ull * v.n_atoms * tile_dim;
        v.off_edges = v.off_codes + 2ull * n_codes;
        v.payload_bytes = v.off_edges + v.edge_bytes;
        const uint64_t r_full = static_cast<uint64_t>(v.rows / v.tile_rows) * v.tile_rows;
        const uint64_t c_full = static_cast<uint64_t>(v.cols / v.tile_cols) * v.tile_cols;
        const uint64_t need = 4ull * (r_full * (v.cols - c_full) + (v.rows - r_full) * v.cols);
        if (need != v.edge_bytes)
            throw Error(CSDR_ERR_FORMAT, "HSDR: edge strip size does not match shape");
    } else {
        if (v.rows % v.tile_rows || v.cols % v.tile_cols)
            throw Error(CSDR_ERR_FORMAT, "HSDR shared: shape not divisible by tile size");
        v.off_codes = kHSDCHeaderBytes;
        v.payload_bytes = v.off_codes + 2ull * n_codes;
    }
    if (v.payload_bytes > n) throw Error(CSDR_ERR_FORMAT, "HSDR: truncated stream");
    if (check_codes) {
        const uint8_t* c = p + v.off_codes;
        for (uint64_t i = 0; i < n_codes; ++i) {
            if ((rd<uint16_t>(c + 2 * i) & 0x7FFFu) >= v.n_atoms)
                throw Error(CSDR_ERR_CODE_RANGE, "HSDR: packed code names an atom index >= n_atoms");
        }
    }
    return v;
}

ArchiveIndex ArchiveIndex::open(const std::string& path) {
    std::ifstream in(path, std::ios::binary);
    if (!in) throw Error(CSDR_ERR_IO, "Failed to open archive: " + path);
    in.seekg(0, std::ios::end);
    const uint64_t file_size = static_cast<uint64_t>(in.tellg());
    in.seekg(0, std::ios::beg);
    Cursor c{in, "archive index"};
    char magic[8] = {};
    in.read(magic, 8);
    if (in.gcount() != 8 || std::memcmp(magic, "CORTEXSR", 8) != 0)
        throw Error(CSDR_ERR_FORMAT, "Invalid or missing archive magic number.");
    ArchiveIndex ar;
    ar.path = path;
    ar.file_size = file_size;
    ar.version = c.pod<uint32_t>();
    if (ar.version == 0 || ar.version > 2) throw Error(CSDR_ERR_FORMAT, "Unsupported archive version.");
    const uint64_t n_segments = c.pod<uint64_t>();
    const uint64_t index_offset = c.pod<uint64_t>();
    if (index_offset > file_size || n_segments > file_size)
        throw Error(CSDR_ERR_FORMAT, "archive index offset or segment count out of range");
    in.seekg(static_cast<std::streamoff>(index_offset), std::ios::beg);
    ar.segments.reserve(n_segments);
    for (uint64_t i = 0; i < n_segments; ++i) {
        SegmentHeader h;
        h.name = c.str(file_size);
        if (ar.version >= 2) h.data_format = c.str(file_size);
        h.layer_type = c.str(file_size);
        h.original_type = c.pod<uint8_t>();
        h.strategy_id = c.pod<uint8_t>();
        h.original_size = c.pod<uint64_t>();
        h.compressed_size = c.pod<uint64_t>();
        h.data_offset = c.pod<uint64_t>();
        h.layer_name = c.str(file_size);
        h.layer_index = c.pod<uint32_t>();
        h.has_meta = c.pod<uint8_t>() != 0;
        if (h.has_meta) {
            const uint8_t nd = c.pod<uint8_t>();
            h.dims.resize(nd);
            for (auto& d : h.dims) d = c.pod<uint32_t>();
            h.sparsity = c.pod<float>();
            h.is_sorted = c.pod<uint8_t>() != 0;
            h.has_scale = c.pod<uint8_t>() != 0;
            if (h.has_scale) h.scale = c.pod<float>();
            h.has_zero_point = c.pod<uint8_t>() != 0;
            if (h.has_zero_point) h.zero_point = c.pod<float>();
        }
        h.input_shape = read_shape(c);
        h.output_shape = read_shape(c);
        if (h.data_offset > file_size || h.compressed_size > file_size - h.data_offset)
            throw Error(CSDR_ERR_FORMAT, "segment payload lies outside the archive: " + h.name);
        ar.by_name.emplace(h.name, ar.segments.size());
        ar.segments.push_back(std::move(h));
    }
    return ar;
}

const SegmentHeader* ArchiveIndex::find(const std::string& name) const {
    auto it = by_name.find(name);
    return it == by_name.end() ? nullptr : &segments[it->second];
}

std::vector<uint8_t> ArchiveIndex::read_payload(const SegmentHeader& h) const {
    std::ifstream in(path, std::ios::binary);
    if (!in) throw Error(CSDR_ERR_IO, "Failed to open archive for raw segment read: " + path);
    in.seekg(static_cast<std::streamoff>(h.data_offset));
    std::vector<uint8_t> bytes(h.compressed_size);
    in.read(reinterpret_cast<char*>(bytes.data()), static_cast<std::streamsize>(bytes.size()));
    if (static_cast<uint64_t>(in.gcount()) != h.compressed_size)
        throw Error(CSDR_ERR_IO, "Failed to read compressed data for segment: " + h.name);
    return bytes;
}

HsdaDictionary parse_dictionary_record(const uint8_t* p, size_t n, const char* what) {
    const std::string w(what);
    size_t off = 0;
    auto need = [&](size_t bytes) {
        if (bytes > n - off) throw Error(CSDR_ERR_FORMAT, w + ": unexpected end of dictionary record");
    };
    HsdaDictionary d;
    need(20);
    d.tile_rows = rd<uint16_t>(p + 0);
    d.tile_cols = rd<uint16_t>(p + 2);
    d.n_atoms = rd<uint16_t>(p + 4);
    d.n_stages = p[6];
    d.k_per_stage = p[7];
    d.ksvd_iters = p[8];
    d.stage_decay = rd<float>(p + 12);
    d.max_tiles_for_fit = rd<uint32_t>(p + 16);
    off = 20;
    need(4);
    const uint32_t n_scales = rd<uint32_t>(p + off);
    off += 4;
    if (n_scales != d.n_stages) throw Error(CSDR_ERR_FORMAT, w + ": dictionary arrays do not match its config");
    need(4ull * n_scales);
    d.scales.resize(n_scales);
    std::memcpy(d.scales.data(), p + off, 4ull * n_scales);
    off += 4ull * n_scales;
    need(4);
    const uint32_t n_atom_floats = rd<uint32_t>(p + off);
    off += 4;
    if (static_cast<uint64_t>(n_atom_floats) != static_cast<uint64_t>(d.n_atoms) * d.tile_rows * d.tile_cols)
        throw Error(CSDR_ERR_FORMAT, w + ": dictionary arrays do not match its config");
    need(4ull * n_atom_floats);
    d.atoms.resize(n_atom_floats);
    std::memcpy(d.atoms.data(), p + off, 4ull * n_atom_floats);
    return d;
}

HsdaFile HsdaFile::open(const std::string& path) {
    std::ifstream in(path, std::ios::binary);
    if (!in) throw Error(CSDR_ERR_IO, "HSDA readFromFile: cannot open " + path);
    in.seekg(0, std::ios::end);
    const uint64_t file_size = static_cast<uint64_t>(in.tellg());
    in.seekg(0, std::ios::beg);
    Cursor c{in, "HSDA read"};
    char magic[4] = {};
    in.read(magic, 4);
    if (in.gcount() != 4 || std::memcmp(magic, "HSDA", 4) != 0)
        throw Error(CSDR_ERR_FORMAT, "HSDA read: bad magic - not an HSDA stream");
    if (c.pod<uint32_t>() != 1) throw Error(CSDR_ERR_FORMAT, "HSDA read: unsupported version");
    const uint32_t n_dicts = c.pod<uint32_t>();
    const uint32_t n_segs = c.pod<uint32_t>();
    if (n_dicts > file_size || n_segs > file_size)
        throw Error(CSDR_ERR_FORMAT, "HSDA read: counts out of range");
    HsdaFile f;
    f.dicts.resize(n_dicts);
    for (auto& d : f.dicts) {
        uint8_t raw[20];
        c.array(raw, 20);
        d.tile_rows = rd<uint16_t>(raw + 0);
        d.tile_cols = rd<uint16_t>(raw + 2);
        d.n_atoms = rd<uint16_t>(raw + 4);
        d.n_stages = raw[6];
        d.k_per_stage = raw[7];
        d.ksvd_iters = raw[8];
        d.stage_decay = rd<float>(raw + 12);
        d.max_tiles_for_fit = rd<uint32_t>(raw + 16);
        const uint32_t n_scales = c.pod<uint32_t>();
        if (n_scales > file_size / 4) throw Error(CSDR_ERR_FORMAT, "HSDA read: scale count out of range");
        d.scales.resize(n_scales);
        c.array(d.scales.data(), n_scales);
        const uint32_t n_atom_floats = c.pod<uint32_t>();
        if (n_atom_floats > file_size / 4) throw Error(CSDR_ERR_FORMAT, "HSDA read: atom count out of range");
        d.atoms.resize(n_atom_floats);
        c.array(d.atoms.data(), n_atom_floats);
        if (n_scales != d.n_stages ||
            static_cast<uint64_t>(n_atom_floats) !=
                static_cast<uint64_t>(d.n_atoms) * d.tile_rows * d.tile_cols)
            throw Error(CSDR_ERR_FORMAT, "HSDA read: dictionary arrays do not match its config");
    }
    f.segments.resize(n_segs);
    for (size_t i = 0; i < n_segs; ++i) {
        auto& s = f.segments[i];
        s.name = c.str(file_size);
        s.dict_index = c.pod<uint32_t>();
        if (s.dict_index >= f.dicts.size()) throw Error(CSDR_ERR_FORMAT, "HSDA read: dict_index out of range");
        s.original_size = c.pod<uint64_t>();
        s.original_type = c.pod<uint8_t>();
        const uint32_t codes_len = c.pod<uint32_t>();
        if (codes_len > file_size) throw Error(CSDR_ERR_FORMAT, "HSDA read: codes length out of range");
        s.codes.resize(codes_len);
        c.array(s.codes.data(), codes_len);
        f.by_name[s.name] = i;
    }
    return f;
}

}  // namespace csdr
