// Internal types shared by the CUDA layer and the C++ host classes.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <memory>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/cortexsdr_b200.h"
#include "host/format.hpp"

namespace csdr {

void set_last_error(const std::string& msg);

// Runs f, turning any exception into a status code + thread-local message: nothing
// throws across the C boundary.
template <typename F>
int guard(F&& f) {
    try {
        f();
        return CSDR_OK;
    } catch (const Error& e) {
        set_last_error(e.what());
        return e.code;
    } catch (const std::bad_alloc&) {
        set_last_error("out of host memory");
        return CSDR_ERR_INVALID_ARG;
    } catch (const std::exception& e) {
        set_last_error(e.what());
        return CSDR_ERR_INVALID_ARG;
    } catch (...) {
        set_last_error("unknown error");
        return CSDR_ERR_INVALID_ARG;
    }
}

#define CSDR_CUDA(expr)                                                                   \
    do {                                                                                  \
        cudaError_t _e = (expr);                                                          \
        if (_e != cudaSuccess)                                                            \
            throw ::csdr::Error(CSDR_ERR_CUDA, std::string(#expr) + ": " +                \
                                                   cudaGetErrorString(_e));               \
    } while (0)

// Device buffer with shared ownership (dictionaries are shared between a segment,
// its row shards and, in a .hsda, every segment of a role).
struct DeviceBuffer {
    void* ptr = nullptr;
    size_t bytes = 0;
    int device = 0;
    // Derived data cached beside the buffer and freed with it (a dictionary's bf16 planes).
    std::shared_ptr<void> aux;
    // A dictionary's atoms re-laid in the blocks the list kernel's loader fetches (gemv_queue.cu).
    std::shared_ptr<DeviceBuffer> stage_blocks;
    DeviceBuffer(size_t n, int dev);
    ~DeviceBuffer();
    void release_data();   // frees the memory now; what hangs on `aux` stays
    DeviceBuffer(const DeviceBuffer&) = delete;
    DeviceBuffer& operator=(const DeviceBuffer&) = delete;
};
using DevPtr = std::shared_ptr<DeviceBuffer>;

struct Geometry {
    uint32_t rows = 0, cols = 0;       // logical shape of this image (a shard has fewer rows)
    uint32_t n_tiles = 0;
    uint32_t tile_rows = 0, tile_cols = 0;
    uint32_t n_atoms = 0, n_stages = 0, k = 0;
    uint32_t rows_full = 0, cols_full = 0;  // tiled region
    uint32_t n_col_tiles = 0;
    bool row_tiles() const { return tile_rows == 1 && tile_cols == cols; }
    uint32_t slots() const { return n_stages * k; }
    uint64_t tile_dim() const { return static_cast<uint64_t>(tile_rows) * tile_cols; }
};

}  // namespace csdr

namespace csdr {
// Kernel classes for launch counting and optional per-class device timing.
enum KernelClass {
    KC_UNPACK = 0, KC_DX, KC_GATHER, KC_TILE_PROJECT, KC_TILE_GATHER, KC_EDGE, KC_DENSE,
    KC_DECODE_ROWS, KC_DEQUANT, KC_GEMM, KC_DECODER_OP, KC_GEMV_FUSED, KC_ATTENTION, KC_GEMV_QUEUE, KC_ENCODE, KC_COUNT
};
const char* kernel_class_name(int cls);
struct TimedLaunch {
    int cls;
    cudaEvent_t start, stop;
};
}  // namespace csdr

struct csdr_context {
    int device = 0;
    cudaStream_t stream = nullptr;
    bool owns_stream = false;
    int sm_count = 0;
    size_t smem_optin = 0;
    uint64_t launches = 0;
    // Grow-only scratch (Dx partials, factored 2-D products, host staging).
    csdr::DevPtr scratch[8];  // 0 Dx, 1 tile products, 2 materialised W, 3 host staging, 4 fused-GEMV partials, 5 activation planes / wait self-test, 6 GEMV queue, 7 dense product before re-tiling
    void* scratch_get(int slot, size_t bytes);
    int* status_word = nullptr;  // device int: kernels record bounded-wait timeouts here
    // Page-locked, device-mapped host staging for the host-buffer entry points (grow-only).
    void* pinned = nullptr;
    size_t pinned_bytes = 0;
    void* pinned_get(size_t bytes);
    uint32_t notify_seq = 0;     // value of the last completion word written into `pinned`
    // Fused GEMV: every launch tags its partial results with a fresh non-zero epoch, taken from a
    // device counter ([0] launches completed, [1] finished CTAs) that the launch itself advances.
    uint32_t* gemv_seq = nullptr;
    uint32_t* queue_sync = nullptr;   // GEMV queue: launch counter pair, then two sets of task counters
    // Iteration limits of the bounded device-side waits (csdr_context_set_wait_limits).
    uint32_t spin_limit_gemv = 1000000u;      // fused GEMV hand-over polls (an L2 round trip each)
    uint32_t spin_limit_barrier = 4000000u;   // mbarrier try_wait rounds of the tensor-core kernels
    uint32_t spin_limit_exchange = 2000000u;  // polls of a peer's flag in the tensor-parallel exchange
    csdr::DevPtr gemv_trace;  // when set: 8 global-timer stamps per CTA of the last fused GEMV
    bool fused_gemv = true;  // CSDR_FUSED_GEMV=0 selects the two-kernel path
    bool gemv_queue = true;  // CSDR_GEMV_QUEUE=0 keeps lists of products on single and grouped launches
    bool cache_2d = true;            // CSDR_CACHE_2D=0: wide batches on 2-D tiles stay on the factored CUDA-core kernels
    uint32_t queue_poll_sleep_ns = 400;  // CSDR_QUEUE_POLL_SLEEP: pause between polls of the list kernel's dependent hand-overs
    uint32_t queue_min_group = 4;    // CSDR_QUEUE_MIN_GROUP: smallest same-x group the list kernel takes over grouped fused launches
    bool host_zero_copy = true;      // CSDR_HOST_ZERO_COPY=0: results of a host list go back by a copy even when the caller's memory is device-addressable
    bool tile_tc = true;             // CSDR_TILE_TC=0: 2-D tile products of a few tokens stay on the CUDA-core projection
    bool attention_rope_fold = true; // CSDR_ATTENTION_ROPE_FOLD=0: rotary embedding and cache write of a decode step as a kernel of their own
    bool decoder_fold = true;        // CSDR_DECODER_FOLD=0: norms, residuals and SwiGLU of a short decoder step as kernels of their own
    bool decoder_queue = false;      // CSDR_DECODER_QUEUE=1: decoder steps of up to four tokens run a block as three launches
    bool gemv_queue_single = false;  // CSDR_GEMV_QUEUE_SINGLE=1 sends single products of at most 4 tokens there too
    bool pdl = true;         // CSDR_PDL=0 launches without programmatic dependent launch
    bool tensor_cores = true;   // CSDR_TENSOR_CORES=0 keeps wide batches on the CUDA-core kernels
    bool tma = true;            // CSDR_TMA=0 keeps the register-fed tensor-core kernel
    size_t tc_min_batch = 8;    // CSDR_TC_MIN_BATCH: smallest batch sent to the tcgen05 path
    // Per-device launch facts, remembered per context (function attributes and occupancy belong
    // to a device; a process may hold contexts on several).
    void opt_in_smem(const void* kernel, size_t bytes);               // raises the opt-in when bytes needs it
    std::unordered_map<const void*, std::pair<size_t, int>> occupancy; // kernel -> (smem asked, CTAs per SM)
    bool tma_attrs_set = false;
    int tma_max_cluster = 8;
    std::unordered_map<uint64_t, int> cluster_fit;                    // (cluster size, smem) -> clusters resident
    uint64_t launches_by_class[csdr::KC_COUNT] = {};
    // When on, every launch is bracketed by two events on the stream (profile_read resolves them).
    bool profiling = false;
    std::vector<csdr::TimedLaunch> timed;
};

struct csdr_dictionary {
    csdr_context* ctx = nullptr;
    uint32_t tile_rows = 0, tile_cols = 0, n_atoms = 0, n_stages = 0, k = 0;
    csdr::DevPtr atoms;    // fp32 [n_atoms][tile_rows*tile_cols]
    csdr::DevPtr scales;   // fp32 [n_stages]
    std::vector<float> scales_host;
};

struct csdr_segment {
    csdr_context* ctx = nullptr;
    csdr_payload_info info{};   // header of the payload this image came from
    csdr::Geometry g;
    csdr::DevPtr atoms, scales; // shared with the dictionary / parent
    csdr::DevPtr codes;         // u16, 16-byte aligned, padded to a multiple of 16 bytes
    size_t codes_offset = 0;    // element offset of this image's first code within `codes`
    csdr::DevPtr edges;         // fp32: top-right strip then bottom strip; may be null
    std::vector<float> scales_host;
    // 2-D tile images only: the weight rebuilt once as a dense row-tile "dictionary" (one atom per
    // output row) whose cached bf16 planes feed the tensor-core kernel at wide batches - what the
    // reference's layer cache holds as fp32 after decompress(). Built on the first wide product.
    mutable std::shared_ptr<csdr_segment> dense;
    // 2-D tile images only: the dictionary seen as n_atoms * tile_rows rows of tile_cols columns,
    // the shape in which the tensor-core projection computes all tile products of a few tokens.
    mutable std::shared_ptr<csdr_segment> tile_view;
    const uint16_t* codes_ptr() const {
        return static_cast<const uint16_t*>(codes->ptr) + codes_offset;
    }
};

namespace csdr {

// Brackets one kernel launch: counts it, checks the launch error, and when the context
// is profiling records an event on either side.
struct LaunchScope {
    csdr_context* ctx;
    int cls;
    cudaEvent_t start = nullptr;
    LaunchScope(csdr_context* c, int k);
    void done(const char* what);
};

Geometry make_geometry(const csdr_payload_info& v);
DevPtr upload(csdr_context* ctx, const void* src, size_t bytes);
void require_ctx(csdr_context* ctx);

// ---- kernel launchers (kernels/*.cu). All asynchronous on ctx->stream. ----
void launch_unpack(csdr_context* ctx, const uint16_t* codes, size_t n, int32_t* idx, int8_t* sign);

struct MatmulArgs {
    const void* x = nullptr;   // device
    int x_dtype = CSDR_DTYPE_F32;
    int x_layout = CSDR_LAYOUT_FEATURE_MAJOR;
    size_t batch = 0;
    float* y = nullptr;        // device
    int y_layout = CSDR_LAYOUT_FEATURE_MAJOR;
    const float* bias = nullptr;
};
void launch_matmul(csdr_context* ctx, const csdr_segment* seg, const MatmulArgs& a);

// rows == nullptr: every row (decompress); else only the listed rows (embedding lookup).
void launch_decode_rows(csdr_context* ctx, const csdr_segment* seg, const int32_t* rows_dev,
                        size_t n_rows, float* out_dev);

void launch_dequantize(csdr_context* ctx, int fmt_id, const uint8_t* data_dev, size_t nbytes,
                       size_t n_out, float scale, float zero_point, float* out_dev);
// The same source dtypes as the reference's inference side widens a stored-raw tensor
// (SparseInferenceEngine.cpp:276-469): ggml's element order for q4_k / q5_k / q6_k.
void launch_dequantize_inference(csdr_context* ctx, int fmt_id, const uint8_t* data_dev, size_t nbytes, size_t n_out,
                                 float* out_dev);
int dequant_format_id(const char* fmt);               // -1 when unknown
size_t dequant_output_count(int fmt_id, size_t nbytes);  // throws on bad size

// Gather phase alone for one token tile: dx is [n_atoms][mt] fp32 (two-kernel layout),
// mt one of 1, 2, 4, 8, 16 and at least m.
void launch_gather_tile(csdr_context* ctx, const csdr_segment* seg, const float* dx, int mt, float* y, int y_layout,
                        uint32_t m_total, uint32_t b0, uint32_t m, const float* bias);

void launch_dense_matmul(csdr_context* ctx, const float* W_dev, uint32_t R, uint32_t C,
                         const MatmulArgs& a);

}  // namespace csdr
