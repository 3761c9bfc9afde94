// Host-side readers for the three byte formats on the path: HSDR/HSDC segment
// payloads, the .sdr archive index, and the .hsda shared-dictionary container.
// Pure C++17, no CUDA. Byte layouts follow the reference writer
// (strategies/HierarchicalSDRStrategy.cpp:49-66, :675-692, :1198-1235, :1972-2002;
// core/AICompressor.cpp:233-312) so archives it produced open unchanged.
#pragma once

#include <cstddef>
#include <cstdint>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../../include/cortexsdr_b200.h"

namespace csdr {

// Error carrying one of the CSDR_ERR_* codes; never crosses the C boundary.
struct Error : std::runtime_error {
    int code;
    Error(int c, const std::string& m) : std::runtime_error(m), code(c) {}
};

constexpr uint8_t kHSDRStrategyId = 5;  // SparseInferenceEngine.cpp:734, :1082

// Parses and validates one payload. `check_codes` also walks the code stream and
// rejects any atom index >= n_atoms.
csdr_payload_info inspect_payload(const uint8_t* p, size_t n, bool check_codes = true);

struct SegmentHeader {
    std::string name, data_format, layer_type, layer_name;
    uint8_t original_type = 0;
    uint8_t strategy_id = 0;
    uint64_t original_size = 0, compressed_size = 0, data_offset = 0;
    uint32_t layer_index = 0;
    bool has_meta = false;
    std::vector<uint32_t> dims;
    float sparsity = 0.f;
    bool is_sorted = false;
    bool has_scale = false, has_zero_point = false;
    float scale = 0.f, zero_point = 0.f;
    std::vector<uint32_t> input_shape, output_shape;
};

// AIDecompressor::readArchiveIndex, core/AIDecompressor.cpp:78-262.
struct ArchiveIndex {
    std::string path;
    uint32_t version = 0;
    uint64_t file_size = 0;
    std::vector<SegmentHeader> segments;
    std::unordered_map<std::string, size_t> by_name;  // first occurrence wins, as a linear scan would

    static ArchiveIndex open(const std::string& path);
    const SegmentHeader* find(const std::string& name) const;
    // AIDecompressor::readCompressedBytes, core/AIDecompressor.cpp:418-435.
    std::vector<uint8_t> read_payload(const SegmentHeader& h) const;
};

// HierarchicalSDRConfig as written raw into a .hsda (20 bytes as compiled by the
// reference: 3 x u16, 4 x u8, 2 pad bytes, f32, u32; HierarchicalSDRStrategy.hpp:43-58).
struct HsdaDictionary {
    uint16_t tile_rows = 0, tile_cols = 0, n_atoms = 0;
    uint8_t n_stages = 0, k_per_stage = 0, ksvd_iters = 0;
    float stage_decay = 0.f;
    uint32_t max_tiles_for_fit = 0;
    std::vector<float> scales, atoms;
};
// One dictionary record as a .hsda holds it (raw config, u32 count + stage scales, u32 count +
// atoms), from memory; `what` prefixes the error text. Also the payload of a shared-dictionary
// resource segment inside a .sdr (see kSharedDictFormat).
HsdaDictionary parse_dictionary_record(const uint8_t* p, size_t n, const char* what);

// Shared dictionaries inside a .sdr. The reference keeps them in a container of their own
// (.hsda) because its archive has no "shared resources" section
// (ai_compression_cli.cpp:727-733, strategies/HierarchicalSDRStrategy.hpp:303-308). The
// convention read here needs no new section, only index fields the archive already has:
//   * a dictionary is an ordinary segment stored raw (strategy 0) whose data_format is
//     "hsdr_dict" and whose payload is one .hsda dictionary record;
//   * a tensor coded against it is an HSDR segment (strategy 5) whose payload is a codes-only
//     "HSDC" stream and whose data_format is "hsdc@" + the dictionary segment's name.
// The reference's index reader opens such an archive unchanged (it cannot run those tensors).
constexpr const char* kSharedDictFormat = "hsdr_dict";
constexpr const char* kSharedCodesPrefix = "hsdc@";

struct HsdaSegment {
    std::string name;
    uint32_t dict_index = 0;
    uint64_t original_size = 0;
    uint8_t original_type = 0;
    std::vector<uint8_t> codes;  // an "HSDC" payload
};
// SharedDictArchive::readFromStream, strategies/HierarchicalSDRStrategy.cpp:2004-2064.
struct HsdaFile {
    std::vector<HsdaDictionary> dicts;
    std::vector<HsdaSegment> segments;
    std::unordered_map<std::string, size_t> by_name;  // last occurrence wins (HSDAReader ctor, :2506-2513)
    static HsdaFile open(const std::string& path);
};

}  // namespace csdr
