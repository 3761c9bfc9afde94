// extern "C" face of the CUDA layer: contexts, device images of compressed segments,
// and the payload-level operations (unpack, fused matmul, decompress, dequantise).
// Archive-level and decoder entry points live in host/archive.cpp and decoder.cu.
#include <algorithm>
#include <cstdlib>
#include <chrono>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "internal.hpp"
#include "kernels/gemm_tcgen05.hpp"
#include "kernels/gemv_fused.hpp"
#include "kernels/gemv_queue.hpp"

namespace csdr {

namespace {
thread_local std::string g_last_error;
}

void set_last_error(const std::string& msg) { g_last_error = msg; }

DeviceBuffer::DeviceBuffer(size_t n, int dev) : bytes(n), device(dev) {
    CSDR_CUDA(cudaMalloc(&ptr, n ? n : 16));
}
DeviceBuffer::~DeviceBuffer() {
    if (ptr) cudaFree(ptr);
}
void DeviceBuffer::release_data() {
    if (ptr) cudaFree(ptr);
    ptr = nullptr;
    bytes = 0;
}

Geometry make_geometry(const csdr_payload_info& v) {
    Geometry g;
    g.rows = v.rows;
    g.cols = v.cols;
    g.n_tiles = v.n_tiles;
    g.tile_rows = v.tile_rows;
    g.tile_cols = v.tile_cols;
    g.n_atoms = v.n_atoms;
    g.n_stages = v.n_stages;
    g.k = v.k_per_stage;
    g.rows_full = (v.rows / v.tile_rows) * v.tile_rows;
    g.cols_full = (v.cols / v.tile_cols) * v.tile_cols;
    g.n_col_tiles = g.cols_full / v.tile_cols;
    return g;
}

// Code stream -> its own 16-byte-aligned device buffer, padded so that kernels may
// finish a 128-bit load past the last code. (Inside a payload the stream starts at
// 36 + 4*S + 4*K*T, 16-byte aligned only when S = 3 mod 4.)
DevPtr upload_codes(csdr_context* ctx, const uint8_t* codes, size_t n_codes) {
    const size_t bytes = ((n_codes * 2 + 15) & ~static_cast<size_t>(15)) + 16;
    auto buf = std::make_shared<DeviceBuffer>(bytes, ctx->device);
    CSDR_CUDA(cudaMemsetAsync(buf->ptr, 0, bytes, ctx->stream));
    CSDR_CUDA(cudaMemcpyAsync(buf->ptr, codes, n_codes * 2, cudaMemcpyHostToDevice, ctx->stream));
    return buf;
}

DevPtr upload(csdr_context* ctx, const void* src, size_t bytes) {
    auto buf = std::make_shared<DeviceBuffer>(bytes, ctx->device);
    if (bytes) CSDR_CUDA(cudaMemcpyAsync(buf->ptr, src, bytes, cudaMemcpyHostToDevice, ctx->stream));
    return buf;
}

const char* kernel_class_name(int cls) {
    static const char* names[KC_COUNT] = {"hsdr_unpack", "hsdr_dx", "hsdr_gather", "hsdr_tile_project",
                                          "hsdr_tile_gather", "hsdr_edge", "dense_rows", "hsdr_decode_rows",
                                          "dequant", "hsdr_gemm_tcgen05", "decoder_op", "hsdr_gemv_fused", "attention",
                                          "hsdr_gemv_queue", "hsdr_encode"};
    return (cls >= 0 && cls < KC_COUNT) ? names[cls] : "?";
}

LaunchScope::LaunchScope(csdr_context* c, int k) : ctx(c), cls(k) {
    if (ctx->profiling) {
        CSDR_CUDA(cudaEventCreate(&start));
        CSDR_CUDA(cudaEventRecord(start, ctx->stream));
    }
}

void LaunchScope::done(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) throw Error(CSDR_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e));
    ++ctx->launches;
    ++ctx->launches_by_class[cls];
    if (start) {
        cudaEvent_t stop;
        CSDR_CUDA(cudaEventCreate(&stop));
        CSDR_CUDA(cudaEventRecord(stop, ctx->stream));
        ctx->timed.push_back({cls, start, stop});
    }
}

void require_ctx(csdr_context* ctx) {
    if (!ctx) throw Error(CSDR_ERR_INVALID_ARG, "context is null");
    CSDR_CUDA(cudaSetDevice(ctx->device));
}

}  // namespace csdr

using namespace csdr;

namespace {
void rethrow(int rc) {
    if (rc != CSDR_OK) throw Error(rc, csdr_last_error());
}
}  // namespace

void* csdr_context::scratch_get(int slot, size_t bytes) {
    if (!scratch[slot] || scratch[slot]->bytes < bytes) {
        // Work queued on the stream may still use the old buffer.
        CSDR_CUDA(cudaStreamSynchronize(stream));
        scratch[slot].reset();
        scratch[slot] = std::make_shared<DeviceBuffer>(bytes, device);
        // Fresh scratch starts at zero: the fused GEMV reads epoch tags from it, and 0 is never a tag.
        CSDR_CUDA(cudaMemsetAsync(scratch[slot]->ptr, 0, bytes, stream));
    }
    return scratch[slot]->ptr;
}

namespace csdr_hostio {

// Host-buffer calls on small operands avoid the copy engines and the driver's stream wait:
// one CTA pulls x out of mapped page-locked memory (every element crosses the bus once), the
// product writes y straight into mapped memory, and a one-thread kernel behind it (launched
// early, released when the product's grid has completed and flushed) stores a sequence number
// that the host polls.
__global__ void __launch_bounds__(1024) host_x_pull_kernel(const float4* __restrict__ src, float4* __restrict__ dst,
                                                           uint32_t n4) {
    asm volatile("griddepcontrol.launch_dependents;");
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += gridDim.x * blockDim.x) dst[i] = src[i];
}

__global__ void host_notify_kernel(volatile uint32_t* word, uint32_t seq) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    *word = seq;
    __threadfence_system();
}

// Polls the completion word for a bounded time; false means "not seen, use the stream wait".
bool wait_host_word(const volatile uint32_t* word, uint32_t seq) {
    const auto t0 = std::chrono::steady_clock::now();
    for (uint32_t spin = 0;; ++spin) {
        if (*word == seq) return true;
        if ((spin & 255u) == 255u &&
            std::chrono::steady_clock::now() - t0 > std::chrono::microseconds(500))
            return false;
    }
}

}  // namespace csdr_hostio
using namespace csdr_hostio;

// The attribute belongs to the function on the device, not to a context: the record of what has
// been opted into is shared by all contexts of the process (a context that set a smaller value
// behind another's back would otherwise lower it).
void csdr_context::opt_in_smem(const void* kernel, size_t bytes) {
    if (bytes <= 40u * 1024u) return;   // static shared memory counts toward the 48 KB a kernel has without opting in
    static std::mutex mu;
    static std::map<std::pair<int, const void*>, size_t> optins;
    std::lock_guard<std::mutex> lock(mu);
    size_t& have = optins[{device, kernel}];
    if (bytes > have) {
        CSDR_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes)));
        have = bytes;
    }
}

void* csdr_context::pinned_get(size_t bytes) {
    if (pinned_bytes < bytes) {
        CSDR_CUDA(cudaStreamSynchronize(stream));
        if (pinned) cudaFreeHost(pinned);
        pinned = nullptr;
        pinned_bytes = 0;
        const size_t want = std::max<size_t>(bytes, 1u << 20);
        CSDR_CUDA(cudaHostAlloc(&pinned, want, cudaHostAllocMapped));
        pinned_bytes = want;
        // the completion word at the head must not hold a sequence number left by an earlier
        // owner of these pages (page-locked memory is recycled between contexts)
        std::memset(pinned, 0, 256);
    }
    return pinned;
}

extern "C" {

const char* csdr_last_error(void) { return g_last_error.c_str(); }
const char* csdr_version(void) { return "cortexsdr_b200 0.1 (sm_100a)"; }

int csdr_context_create(int device, void* stream, csdr_context** out) {
    return guard([&] {
        if (!out) throw Error(CSDR_ERR_INVALID_ARG, "out is null");
        int n = 0;
        if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0)
            throw Error(CSDR_ERR_CUDA, "no CUDA device: this library has no CPU path");
        if (device < 0) CSDR_CUDA(cudaGetDevice(&device));
        if (device >= n) throw Error(CSDR_ERR_INVALID_ARG, "device index out of range");
        CSDR_CUDA(cudaSetDevice(device));
        cudaDeviceProp prop{};
        CSDR_CUDA(cudaGetDeviceProperties(&prop, device));
        if (prop.major != 10)
            throw Error(CSDR_ERR_CUDA, std::string("built for sm_100a only; device is sm_") +
                                           std::to_string(prop.major) + std::to_string(prop.minor));
        auto ctx = std::make_unique<csdr_context>();
        ctx->device = device;
        ctx->sm_count = prop.multiProcessorCount;
        ctx->smem_optin = prop.sharedMemPerBlockOptin;
        if (stream) {
            ctx->stream = static_cast<cudaStream_t>(stream);
        } else {
            CSDR_CUDA(cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking));
            ctx->owns_stream = true;
        }
        CSDR_CUDA(cudaMalloc(&ctx->status_word, sizeof(int)));
        CSDR_CUDA(cudaMemsetAsync(ctx->status_word, 0, sizeof(int), ctx->stream));
        CSDR_CUDA(cudaMalloc(&ctx->gemv_seq, 1024 * sizeof(uint32_t)));   // launch tag words: last tag, pad, one slot per CTA
        CSDR_CUDA(cudaMemsetAsync(ctx->gemv_seq, 0, 1024 * sizeof(uint32_t), ctx->stream));
        if (const char* e = std::getenv("CSDR_FUSED_GEMV")) ctx->fused_gemv = e[0] != '0';
        if (const char* e = std::getenv("CSDR_GEMV_QUEUE")) ctx->gemv_queue = e[0] != '0';
        if (const char* e = std::getenv("CSDR_CACHE_2D")) ctx->cache_2d = e[0] != '0';
        if (const char* e = std::getenv("CSDR_DECODER_QUEUE")) ctx->decoder_queue = e[0] != '0';
        if (const char* e = std::getenv("CSDR_TILE_TC")) ctx->tile_tc = e[0] != '0';
        if (const char* e = std::getenv("CSDR_HOST_ZERO_COPY")) ctx->host_zero_copy = e[0] != '0';
        if (const char* e = std::getenv("CSDR_DECODER_FOLD")) ctx->decoder_fold = e[0] != '0';
        if (const char* e = std::getenv("CSDR_ATTENTION_ROPE_FOLD")) ctx->attention_rope_fold = e[0] != '0';
        if (const char* e = std::getenv("CSDR_QUEUE_POLL_SLEEP")) ctx->queue_poll_sleep_ns = static_cast<uint32_t>(std::max(0, std::atoi(e)));
        if (const char* e = std::getenv("CSDR_QUEUE_MIN_GROUP")) ctx->queue_min_group = static_cast<uint32_t>(std::max(1, std::atoi(e)));
        if (const char* e = std::getenv("CSDR_GEMV_QUEUE_SINGLE")) ctx->gemv_queue_single = e[0] != '0';
        if (const char* e = std::getenv("CSDR_PDL")) ctx->pdl = e[0] != '0';
        if (const char* e = std::getenv("CSDR_TENSOR_CORES")) ctx->tensor_cores = e[0] != '0';
        if (const char* e = std::getenv("CSDR_TMA")) ctx->tma = e[0] != '0';
        if (const char* e = std::getenv("CSDR_TC_MIN_BATCH")) ctx->tc_min_batch = static_cast<size_t>(std::max(1, std::atoi(e)));
        CSDR_CUDA(cudaStreamSynchronize(ctx->stream));
        *out = ctx.release();
    });
}

int csdr_context_destroy(csdr_context* ctx) {
    return guard([&] {
        if (!ctx) return;
        cudaSetDevice(ctx->device);
        cudaStreamSynchronize(ctx->stream);
        for (auto& s : ctx->scratch) s.reset();
        if (ctx->status_word) cudaFree(ctx->status_word);
        if (ctx->gemv_seq) cudaFree(ctx->gemv_seq);
        if (ctx->queue_sync) cudaFree(ctx->queue_sync);
        if (ctx->pinned) cudaFreeHost(ctx->pinned);
        if (ctx->owns_stream) cudaStreamDestroy(ctx->stream);
        delete ctx;
    });
}

int csdr_context_synchronize(csdr_context* ctx) {
    return guard([&] {
        require_ctx(ctx);
        int status = 0;
        CSDR_CUDA(cudaMemcpyAsync(&status, ctx->status_word, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
        CSDR_CUDA(cudaStreamSynchronize(ctx->stream));
        if (status != 0) {
            CSDR_CUDA(cudaMemsetAsync(ctx->status_word, 0, sizeof(int), ctx->stream));
            CSDR_CUDA(cudaStreamSynchronize(ctx->stream));
            if (status == 2)
                throw Error(CSDR_ERR_CODE_RANGE, "a gather met a packed code naming an atom >= n_atoms (it contributed "
                                                 "nothing to its row): results since the last synchronize are invalid");
            throw Error(CSDR_ERR_TIMEOUT,
                        "a device-side wait ran out (fused GEMV hand-over, a tensor-core kernel's barrier, or a "
                        "tensor-parallel peer that never raised its flag): results of the calls since the last "
                        "synchronize are invalid; set CSDR_FUSED_GEMV=0 if the GPU is shared with long-running "
                        "kernels");
        }
    });
}

int csdr_context_set_wait_limits(csdr_context* ctx, uint32_t gemv_polls, uint32_t barrier_rounds,
                                 uint32_t exchange_polls) {
    return guard([&] {
        require_ctx(ctx);
        const csdr_context fresh{};
        ctx->spin_limit_gemv = gemv_polls ? gemv_polls : fresh.spin_limit_gemv;
        ctx->spin_limit_barrier = barrier_rounds ? barrier_rounds : fresh.spin_limit_barrier;
        ctx->spin_limit_exchange = exchange_polls ? exchange_polls : fresh.spin_limit_exchange;
    });
}

int csdr_context_wait_selftest(csdr_context* ctx) {
    return guard([&] {
        require_ctx(ctx);
        // A two-rank exchange laid out in local scratch: [2][2] slots of 64 floats, then the flag
        // words, then the sequence counter. Rank 0's flag of parity 1 is raised, rank 1's never is.
        constexpr uint32_t blk = 64;
        float* region = static_cast<float*>(ctx->scratch_get(5, 4096));
        CSDR_CUDA(cudaMemsetAsync(region, 0, 4096, ctx->stream));
        uint32_t* flags = reinterpret_cast<uint32_t*>(region + 4 * blk);
        uint32_t* seq = flags + 16;
        const uint32_t one = 1;
        CSDR_CUDA(cudaMemcpyAsync(seq, &one, 4, cudaMemcpyHostToDevice, ctx->stream));
        CSDR_CUDA(cudaMemcpyAsync(flags + 2, &one, 4, cudaMemcpyHostToDevice, ctx->stream));
        Exchange x{};
        x.ranks = 2;
        x.rank = 0;
        x.blk_floats = blk;
        x.slots[0] = x.slots[1] = region;
        x.flags[0] = x.flags[1] = flags;
        x.seq = seq;
        x.status = ctx->status_word;
        launch_exchange_reduce(ctx, x, 0, blk, region + 8 * blk);
        rethrow(csdr_context_synchronize(ctx));
    });
}

int csdr_context_profile(csdr_context* ctx, int enable) {
    return guard([&] {
        require_ctx(ctx);
        CSDR_CUDA(cudaStreamSynchronize(ctx->stream));
        for (auto& t : ctx->timed) {
            cudaEventDestroy(t.start);
            cudaEventDestroy(t.stop);
        }
        ctx->timed.clear();
        ctx->profiling = enable != 0;
    });
}

int csdr_context_profile_read(csdr_context* ctx, int cls, uint64_t* launches, double* total_ms) {
    return guard([&] {
        require_ctx(ctx);
        if (cls < 0 || cls >= KC_COUNT) throw Error(CSDR_ERR_INVALID_ARG, "kernel class out of range");
        CSDR_CUDA(cudaStreamSynchronize(ctx->stream));
        uint64_t n = 0;
        double ms = 0.0;
        for (auto& t : ctx->timed) {
            if (t.cls != cls) continue;
            float e = 0.f;
            CSDR_CUDA(cudaEventElapsedTime(&e, t.start, t.stop));
            ms += e;
            ++n;
        }
        if (launches) *launches = ctx->profiling ? n : ctx->launches_by_class[cls];
        if (total_ms) *total_ms = ms;
    });
}

const char* csdr_kernel_class_name(int cls) { return kernel_class_name(cls); }

int csdr_context_gemv_trace(csdr_context* ctx, int enable, uint64_t* out, size_t capacity, size_t* n_out) {
    return guard([&] {
        require_ctx(ctx);
        CSDR_CUDA(cudaStreamSynchronize(ctx->stream));
        const size_t words = static_cast<size_t>(ctx->sm_count) * 64u;   // fused GEMV: 2 CTAs x 16 per SM; queue: 8 tasks x 8
        if (out && ctx->gemv_trace) {
            const size_t n = std::min(capacity, words);
            CSDR_CUDA(cudaMemcpy(out, ctx->gemv_trace->ptr, n * 8u, cudaMemcpyDeviceToHost));
            if (n_out) *n_out = n;
        } else if (n_out) {
            *n_out = 0;
        }
        if (enable && !ctx->gemv_trace) {
            ctx->gemv_trace = std::make_shared<DeviceBuffer>(words * 8u, ctx->device);
            CSDR_CUDA(cudaMemset(ctx->gemv_trace->ptr, 0, words * 8u));
        } else if (!enable) {
            ctx->gemv_trace.reset();
        }
    });
}

void* csdr_context_stream(csdr_context* ctx) { return ctx ? ctx->stream : nullptr; }
uint64_t csdr_context_launch_count(const csdr_context* ctx) { return ctx ? ctx->launches : 0; }

int csdr_payload_inspect(const void* payload, size_t nbytes, csdr_payload_info* info) {
    return guard([&] {
        if (!info) throw Error(CSDR_ERR_INVALID_ARG, "info is null");
        *info = inspect_payload(static_cast<const uint8_t*>(payload), nbytes, true);
    });
}

int csdr_segment_create(csdr_context* ctx, const void* payload, size_t nbytes, csdr_segment** out) {
    return guard([&] {
        require_ctx(ctx);
        if (!out) throw Error(CSDR_ERR_INVALID_ARG, "out is null");
        const uint8_t* p = static_cast<const uint8_t*>(payload);
        const csdr_payload_info v = inspect_payload(p, nbytes, true);
        if (v.kind != CSDR_KIND_HSDR)
            throw Error(CSDR_ERR_FORMAT, "HSDR: bad magic - a codes-only stream needs its dictionary");
        auto seg = std::make_unique<csdr_segment>();
        seg->ctx = ctx;
        seg->info = v;
        seg->g = make_geometry(v);
        seg->scales_host.resize(v.n_stages);
        std::memcpy(seg->scales_host.data(), p + v.off_scales, 4u * v.n_stages);
        seg->scales = upload(ctx, p + v.off_scales, 4u * v.n_stages);
        seg->atoms = upload(ctx, p + v.off_dict, v.off_codes - v.off_dict);
        seg->codes = upload_codes(ctx, p + v.off_codes, static_cast<size_t>(v.n_tiles) * v.n_stages * v.k_per_stage);
        if (v.edge_bytes) seg->edges = upload(ctx, p + v.off_edges, v.edge_bytes);
        CSDR_CUDA(cudaStreamSynchronize(ctx->stream));  // payload memory may go away on return
        *out = seg.release();
    });
}

int csdr_dictionary_create(csdr_context* ctx, uint16_t tile_rows, uint16_t tile_cols,
                           uint16_t n_atoms, uint8_t n_stages, uint8_t k_per_stage,
                           const float* atoms, const float* scales, csdr_dictionary** out) {
    return guard([&] {
        require_ctx(ctx);
        if (!out || !atoms || !scales) throw Error(CSDR_ERR_INVALID_ARG, "null argument");
        if (!tile_rows || !tile_cols || !n_atoms || !n_stages || !k_per_stage || n_atoms > 0x7FFF)
            throw Error(CSDR_ERR_INVALID_ARG, "dictionary config has a zero or out-of-range field");
        auto d = std::make_unique<csdr_dictionary>();
        d->ctx = ctx;
        d->tile_rows = tile_rows;
        d->tile_cols = tile_cols;
        d->n_atoms = n_atoms;
        d->n_stages = n_stages;
        d->k = k_per_stage;
        d->scales_host.assign(scales, scales + n_stages);
        d->scales = upload(ctx, scales, 4u * n_stages);
        d->atoms = upload(ctx, atoms, 4ull * n_atoms * tile_rows * tile_cols);
        CSDR_CUDA(cudaStreamSynchronize(ctx->stream));
        *out = d.release();
    });
}

int csdr_segment_create_shared(csdr_context* ctx, const void* codes, size_t nbytes,
                               const csdr_dictionary* dict, csdr_segment** out) {
    return guard([&] {
        require_ctx(ctx);
        if (!out || !dict) throw Error(CSDR_ERR_INVALID_ARG, "null argument");
        const uint8_t* p = static_cast<const uint8_t*>(codes);
        const csdr_payload_info v = inspect_payload(p, nbytes, true);
        if (v.kind != CSDR_KIND_HSDC) throw Error(CSDR_ERR_FORMAT, "HSDR shared: bad codes-stream magic");
        if (v.tile_rows != dict->tile_rows || v.tile_cols != dict->tile_cols ||
            v.n_atoms != dict->n_atoms || v.n_stages != dict->n_stages || v.k_per_stage != dict->k)
            throw Error(CSDR_ERR_GEOMETRY, "HSDR shared: stream geometry doesn't match dictionary config");
        auto seg = std::make_unique<csdr_segment>();
        seg->ctx = ctx;
        seg->info = v;
        seg->g = make_geometry(v);
        seg->scales_host = dict->scales_host;
        seg->scales = dict->scales;
        seg->atoms = dict->atoms;
        seg->codes = upload_codes(ctx, p + v.off_codes, static_cast<size_t>(v.n_tiles) * v.n_stages * v.k_per_stage);
        CSDR_CUDA(cudaStreamSynchronize(ctx->stream));
        *out = seg.release();
    });
}

int csdr_segment_destroy(csdr_segment* seg) {
    return guard([&] {
        if (!seg) return;
        cudaSetDevice(seg->ctx->device);
        cudaStreamSynchronize(seg->ctx->stream);
        delete seg;
    });
}

int csdr_dictionary_destroy(csdr_dictionary* dict) {
    return guard([&] {
        if (!dict) return;
        cudaSetDevice(dict->ctx->device);
        cudaStreamSynchronize(dict->ctx->stream);
        delete dict;
    });
}

int csdr_segment_info(const csdr_segment* seg, csdr_payload_info* info) {
    return guard([&] {
        if (!seg || !info) throw Error(CSDR_ERR_INVALID_ARG, "null argument");
        *info = seg->info;
        info->rows = seg->g.rows;
        info->cols = seg->g.cols;
        info->tile_cols = static_cast<uint16_t>(seg->g.tile_cols);
        info->n_tiles = seg->g.n_tiles;
    });
}

int csdr_segment_shard_cols(csdr_context* ctx, const csdr_segment* seg, uint32_t col_begin,
                            uint32_t col_end, csdr_segment** out) {
    return guard([&] {
        require_ctx(ctx);
        if (!seg || !out) throw Error(CSDR_ERR_INVALID_ARG, "null argument");
        const Geometry& g = seg->g;
        if (!g.row_tiles()) throw Error(CSDR_ERR_GEOMETRY, "column shards exist for 1-D row tiles only");
        if (col_begin >= col_end || col_end > g.cols)
            throw Error(CSDR_ERR_INVALID_ARG, "column range outside the matrix");
        if ((col_begin | col_end) & 3u)
            throw Error(CSDR_ERR_GEOMETRY, "column range must fall on multiples of four");
        if (col_end - col_begin > 0xFFFFu) throw Error(CSDR_ERR_LIMIT, "column shard wider than 65535");
        auto sh = std::make_unique<csdr_segment>();
        sh->ctx = ctx;
        sh->info = seg->info;
        sh->g = g;
        const uint32_t w = col_end - col_begin;
        sh->g.cols = sh->g.cols_full = sh->g.tile_cols = w;
        sh->scales_host = seg->scales_host;
        sh->scales = seg->scales;
        sh->codes = seg->codes;
        sh->codes_offset = seg->codes_offset;
        // the shard's own dictionary: columns [col_begin, col_end) of every atom, contiguous
        sh->atoms = std::make_shared<DeviceBuffer>(static_cast<size_t>(g.n_atoms) * w * 4, ctx->device);
        CSDR_CUDA(cudaMemcpy2DAsync(sh->atoms->ptr, static_cast<size_t>(w) * 4,
                                    static_cast<const float*>(seg->atoms->ptr) + col_begin,
                                    static_cast<size_t>(g.cols) * 4, static_cast<size_t>(w) * 4, g.n_atoms,
                                    cudaMemcpyDeviceToDevice, ctx->stream));
        CSDR_CUDA(cudaStreamSynchronize(ctx->stream));
        *out = sh.release();
    });
}

int csdr_segment_shard_rows(csdr_context* ctx, const csdr_segment* seg, uint32_t row_begin,
                            uint32_t row_end, csdr_segment** out) {
    return guard([&] {
        require_ctx(ctx);
        if (!seg || !out) throw Error(CSDR_ERR_INVALID_ARG, "null argument");
        const Geometry& g = seg->g;
        if (row_begin >= row_end || row_end > g.rows_full)
            throw Error(CSDR_ERR_INVALID_ARG, "row range outside the tiled region");
        if (row_begin % g.tile_rows || row_end % g.tile_rows)
            throw Error(CSDR_ERR_GEOMETRY, "row range must fall on tile-row boundaries");
        auto sh = std::make_unique<csdr_segment>();
        sh->ctx = ctx;
        sh->info = seg->info;
        sh->g = g;
        sh->g.rows = row_end - row_begin;
        sh->g.rows_full = sh->g.rows;
        sh->g.n_tiles = (sh->g.rows / g.tile_rows) * g.n_col_tiles;
        sh->scales_host = seg->scales_host;
        sh->scales = seg->scales;
        sh->atoms = seg->atoms;
        const size_t slots = g.slots();
        const size_t first = static_cast<size_t>(row_begin / g.tile_rows) * g.n_col_tiles * slots;
        const size_t n_codes = static_cast<size_t>(sh->g.n_tiles) * slots;
        const size_t bytes = ((n_codes * 2 + 15) & ~static_cast<size_t>(15)) + 16;
        sh->codes = std::make_shared<DeviceBuffer>(bytes, ctx->device);
        CSDR_CUDA(cudaMemsetAsync(sh->codes->ptr, 0, bytes, ctx->stream));
        CSDR_CUDA(cudaMemcpyAsync(sh->codes->ptr, seg->codes_ptr() + first, n_codes * 2,
                                  cudaMemcpyDeviceToDevice, ctx->stream));
        if (seg->edges && g.cols != g.cols_full) {
            // top-right strip rows of the shard
            const size_t w = g.cols - g.cols_full;
            sh->edges = std::make_shared<DeviceBuffer>(static_cast<size_t>(sh->g.rows) * w * 4, ctx->device);
            CSDR_CUDA(cudaMemcpyAsync(sh->edges->ptr,
                                      static_cast<const float*>(seg->edges->ptr) + static_cast<size_t>(row_begin) * w,
                                      static_cast<size_t>(sh->g.rows) * w * 4, cudaMemcpyDeviceToDevice,
                                      ctx->stream));
        }
        CSDR_CUDA(cudaStreamSynchronize(ctx->stream));
        *out = sh.release();
    });
}

int csdr_unpack_codes(csdr_context* ctx, const csdr_segment* seg, int32_t* idx_out,
                      int8_t* sign_out, size_t capacity) {
    return guard([&] {
        require_ctx(ctx);
        if (!seg || !idx_out || !sign_out) throw Error(CSDR_ERR_INVALID_ARG, "null argument");
        const size_t n = static_cast<size_t>(seg->g.n_tiles) * seg->g.slots();
        if (capacity < n) throw Error(CSDR_ERR_BUFFER, "unpack output buffers too small");
        const size_t idx_bytes = (n * 4 + 31) & ~static_cast<size_t>(31);
        unsigned char* buf = static_cast<unsigned char*>(ctx->scratch_get(3, idx_bytes + n + 32));
        int32_t* idx_dev = reinterpret_cast<int32_t*>(buf);
        int8_t* sign_dev = reinterpret_cast<int8_t*>(buf + idx_bytes);
        launch_unpack(ctx, seg->codes_ptr(), n, idx_dev, sign_dev);
        CSDR_CUDA(cudaMemcpyAsync(idx_out, idx_dev, n * 4, cudaMemcpyDeviceToHost, ctx->stream));
        CSDR_CUDA(cudaMemcpyAsync(sign_out, sign_dev, n, cudaMemcpyDeviceToHost, ctx->stream));
        CSDR_CUDA(cudaStreamSynchronize(ctx->stream));
    });
}

int csdr_matmul_device_async(csdr_context* ctx, const csdr_segment* seg, const void* x_dev,
                             int x_dtype, int x_layout, size_t batch, float* y_dev, int y_layout,
                             const float* bias_dev) {
    return guard([&] {
        require_ctx(ctx);
        if (!seg || !x_dev || !y_dev) throw Error(CSDR_ERR_INVALID_ARG, "null argument");
        if ((x_dtype != CSDR_DTYPE_F32 && x_dtype != CSDR_DTYPE_BF16) ||
            (x_layout != CSDR_LAYOUT_FEATURE_MAJOR && x_layout != CSDR_LAYOUT_TOKEN_MAJOR) ||
            (y_layout != CSDR_LAYOUT_FEATURE_MAJOR && y_layout != CSDR_LAYOUT_TOKEN_MAJOR))
            throw Error(CSDR_ERR_INVALID_ARG, "unknown dtype or layout");
        MatmulArgs a;
        a.x = x_dev;
        a.x_dtype = x_dtype;
        a.x_layout = x_layout;
        a.batch = batch;
        a.y = y_dev;
        a.y_layout = y_layout;
        a.bias = bias_dev;
        launch_matmul(ctx, seg, a);
    });
}

int csdr_matmul_group_device_async(csdr_context* ctx, const csdr_segment* const* segs, size_t n_segs,
                                   const void* x_dev, int x_dtype, int x_layout, size_t batch,
                                   float* const* ys_dev, int y_layout) {
    return guard([&] {
        require_ctx(ctx);
        if (!segs || !ys_dev || !x_dev || n_segs == 0) throw Error(CSDR_ERR_INVALID_ARG, "null argument");
        if (batch > 0xFFFFFFFFull) throw Error(CSDR_ERR_LIMIT, "batch too large");
        for (size_t i = 0; i < n_segs; ++i) {
            if (!segs[i] || !ys_dev[i]) throw Error(CSDR_ERR_INVALID_ARG, "null argument");
            if (segs[i]->g.cols != segs[0]->g.cols)
                throw Error(CSDR_ERR_GEOMETRY, "grouped matmul: every segment must consume the same activation width");
        }
        bool all_tc = true;
        for (size_t i = 0; i < n_segs; ++i) all_tc = all_tc && tcgen05_supported(ctx, segs[i], batch);
        if (all_tc) {
            // wide batch: the activations become bf16 planes once; groups of up to four
            // segments share one projection launch (and, up to 16 tokens, one gather launch)
            bool grouped = true;
            for (size_t i0 = 0; i0 < n_segs && grouped; i0 += 4)
                grouped = wide_group_supported(ctx, segs + i0, static_cast<uint32_t>(std::min<size_t>(4, n_segs - i0)), batch);
            if (grouped) {
                const XPlanesView xp = make_x_planes(ctx, x_dev, x_dtype, x_layout, static_cast<uint32_t>(batch), segs[0]->g.cols);
                for (size_t i0 = 0; i0 < n_segs; i0 += 4) {
                    const uint32_t n = static_cast<uint32_t>(std::min<size_t>(4, n_segs - i0));
                    WideOut outs[4];
                    for (uint32_t i = 0; i < n; ++i) outs[i] = WideOut{ys_dev[i0 + i], nullptr, nullptr};
                    launch_matmul_wide_group(ctx, segs + i0, n, xp, static_cast<uint32_t>(batch), outs, y_layout);
                }
                return;
            }
            for (size_t i = 0; i < n_segs; ++i) {
                MatmulArgs a;
                a.x = x_dev;
                a.x_dtype = x_dtype;
                a.x_layout = x_layout;
                a.batch = batch;
                a.y = ys_dev[i];
                a.y_layout = y_layout;
                launch_matmul_tcgen05(ctx, segs[i], a);
            }
            return;
        }
        if (n_segs >= ctx->queue_min_group && batch <= 4) {
            // long lists: any number of members in one persistent launch (short ones are quicker as
            // grouped launches of up to four)
            std::vector<QueueItem> items(n_segs);
            for (size_t i = 0; i < n_segs; ++i)
                items[i] = QueueItem{segs[i], x_dev, x_dtype, x_layout, batch, ys_dev[i], y_layout, nullptr};
            if (gemv_queue_supported(ctx, items.data(), static_cast<uint32_t>(n_segs))) {
                launch_gemv_queue(ctx, items.data(), static_cast<uint32_t>(n_segs));
                return;
            }
        }
        size_t done = 0;
        while (done < n_segs) {
            const uint32_t n = static_cast<uint32_t>(std::min<size_t>(kMaxFusedGroup, n_segs - done));
            bool fused = true;
            for (size_t b0 = 0; b0 < batch && fused; b0 += 16) {
                const uint32_t m = static_cast<uint32_t>(std::min<size_t>(16, batch - b0));
                const int mt = m <= 1 ? 1 : m <= 2 ? 2 : m <= 4 ? 4 : m <= 8 ? 8 : 16;
                fused = gemv_fused_supported(ctx, segs + done, n, mt);
            }
            if (fused) {
                for (size_t b0 = 0; b0 < batch; b0 += 16) {
                    const uint32_t m = static_cast<uint32_t>(std::min<size_t>(16, batch - b0));
                    const int mt = m <= 1 ? 1 : m <= 2 ? 2 : m <= 4 ? 4 : m <= 8 ? 8 : 16;
                    launch_gemv_fused(ctx, segs + done, n, x_dev, x_dtype, x_layout, static_cast<uint32_t>(batch),
                                      static_cast<uint32_t>(b0), m, ys_dev + done, y_layout, nullptr, mt);
                }
            } else {
                for (uint32_t i = 0; i < n; ++i) {
                    MatmulArgs a;
                    a.x = x_dev;
                    a.x_dtype = x_dtype;
                    a.x_layout = x_layout;
                    a.batch = batch;
                    a.y = ys_dev[done + i];
                    a.y_layout = y_layout;
                    launch_matmul(ctx, segs[done + i], a);
                }
            }
            done += n;
        }
    });
}

int csdr_matmul_queue_device_async(csdr_context* ctx, const csdr_matmul_task* tasks, size_t n_tasks) {
    return guard([&] {
        require_ctx(ctx);
        if (!tasks || n_tasks == 0) throw Error(CSDR_ERR_INVALID_ARG, "null argument");
        if (n_tasks > 0xFFFFu) throw Error(CSDR_ERR_LIMIT, "more than 65535 tasks in one list");
        std::vector<QueueItem> items(n_tasks);
        for (size_t i = 0; i < n_tasks; ++i) {
            const csdr_matmul_task& t = tasks[i];
            if (!t.seg || !t.x_dev || !t.y_dev) throw Error(CSDR_ERR_INVALID_ARG, "null argument");
            if ((t.x_dtype != CSDR_DTYPE_F32 && t.x_dtype != CSDR_DTYPE_BF16) ||
                (t.x_layout != CSDR_LAYOUT_FEATURE_MAJOR && t.x_layout != CSDR_LAYOUT_TOKEN_MAJOR) ||
                (t.y_layout != CSDR_LAYOUT_FEATURE_MAJOR && t.y_layout != CSDR_LAYOUT_TOKEN_MAJOR))
                throw Error(CSDR_ERR_INVALID_ARG, "unknown dtype or layout");
            if (t.batch > 0xFFFFFFFFull) throw Error(CSDR_ERR_LIMIT, "batch too large");
            if (t.after_task >= static_cast<int>(i) || t.after_task < -1)
                throw Error(CSDR_ERR_INVALID_ARG, "after_task must name an earlier task of the list, or be -1");
            items[i] = QueueItem{t.seg, t.x_dev, t.x_dtype, t.x_layout, t.batch, t.y_dev, t.y_layout, t.bias_dev};
            items[i].dep = t.after_task;
        }
        if (gemv_queue_supported(ctx, items.data(), static_cast<uint32_t>(n_tasks))) {
            launch_gemv_queue(ctx, items.data(), static_cast<uint32_t>(n_tasks));
            return;
        }
        for (const QueueItem& it : items) {   // anything else: one product at a time
            MatmulArgs a;
            a.x = it.x;
            a.x_dtype = it.x_dtype;
            a.x_layout = it.x_layout;
            a.batch = it.batch;
            a.y = it.y;
            a.y_layout = it.y_layout;
            a.bias = it.bias;
            launch_matmul(ctx, it.seg, a);
        }
    });
}

int csdr_matmul_queue(csdr_context* ctx, const csdr_matmul_host_task* tasks, size_t n_tasks) {
    return guard([&] {
        require_ctx(ctx);
        if (!tasks || n_tasks == 0) throw Error(CSDR_ERR_INVALID_ARG, "null argument");
        if (n_tasks > 0xFFFFu) throw Error(CSDR_ERR_LIMIT, "more than 65535 tasks in one list");
        // one staging block: every task's activations, then every task's result, 256-byte slots
        size_t x_bytes = 0, y_bytes = 0;
        for (size_t i = 0; i < n_tasks; ++i) {
            const csdr_matmul_host_task& t = tasks[i];
            if (!t.seg || !t.x || !t.y) throw Error(CSDR_ERR_INVALID_ARG, "null argument");
            if (t.batch == 0 || t.batch > 0xFFFFu) throw Error(CSDR_ERR_INVALID_ARG, "batch must be 1 to 65535");
            const Geometry& g = t.seg->g;
            if (!g.row_tiles())
                throw Error(CSDR_ERR_GEOMETRY, "HSDR matmul: fused matmul requires tile_rows == 1; use decompress() + "
                                               "dense matmul for 2D tile encodings");
            x_bytes += (static_cast<size_t>(g.cols) * t.batch * 4 + 255) & ~static_cast<size_t>(255);
            y_bytes += (static_cast<size_t>(g.rows) * t.batch * 4 + 255) & ~static_cast<size_t>(255);
        }
        // A caller whose activations (and results) sit one behind the other in PAGE-LOCKED memory, in
        // task order and in 256-byte multiples, has laid them out as the staging block is: the
        // copy engines then move them straight from (to) the caller's memory, one transfer each
        // way, and the two passes through a staging buffer fall away.
        unsigned char* y_mapped = nullptr;   // device view of the caller's page-locked results, when they have one
        auto page_locked_run = [&](bool outputs) {
            const unsigned char* expect = nullptr;
            for (size_t i = 0; i < n_tasks; ++i) {
                const csdr_matmul_host_task& t = tasks[i];
                const size_t nb = static_cast<size_t>(outputs ? t.seg->g.rows : t.seg->g.cols) * t.batch * 4;
                const unsigned char* p = reinterpret_cast<const unsigned char*>(outputs ? static_cast<const void*>(t.y) : t.x);
                if ((nb & 255u) || (i && p != expect)) return false;
                expect = p + nb;
            }
            const unsigned char* first = reinterpret_cast<const unsigned char*>(outputs ? static_cast<const void*>(tasks[0].y) : tasks[0].x);
            for (const unsigned char* q : {first, expect - 1}) {
                cudaPointerAttributes at{};
                if (cudaPointerGetAttributes(&at, q) != cudaSuccess) {
                    (void)cudaGetLastError();
                    return false;
                }
                if (at.type != cudaMemoryTypeHost) return false;
                if (outputs && q == first) y_mapped = static_cast<unsigned char*>(at.devicePointer);
            }
            return true;
        };
        const bool x_direct = page_locked_run(false), y_direct = page_locked_run(true);
        const bool y_zero_copy = y_direct && y_mapped != nullptr && ctx->host_zero_copy;
        unsigned char* hbuf = (x_direct && y_direct) ? nullptr
                                                     : static_cast<unsigned char*>(ctx->pinned_get(256 + x_bytes + y_bytes)) + 256;
        unsigned char* dbuf = static_cast<unsigned char*>(ctx->scratch_get(3, x_bytes + y_bytes));
        std::vector<QueueItem> items(n_tasks);
        size_t xo = 0, yo = x_bytes;
        for (size_t i = 0; i < n_tasks; ++i) {
            const csdr_matmul_host_task& t = tasks[i];
            const Geometry& g = t.seg->g;
            const size_t xb = static_cast<size_t>(g.cols) * t.batch * 4, yb = static_cast<size_t>(g.rows) * t.batch * 4;
            // tasks that share one host x share one staged copy
            size_t x_at = xo;
            bool shared = false;
            if (!x_direct)
                for (size_t j = i; j-- > 0 && i - j <= 4;)
                    if (tasks[j].x == t.x && tasks[j].batch == t.batch && tasks[j].seg->g.cols == g.cols) {
                        x_at = static_cast<const unsigned char*>(items[j].x) - dbuf;
                        shared = true;
                        break;
                    }
            if (!shared) {
                if (!x_direct) std::memcpy(hbuf + xo, t.x, xb);
                xo += (xb + 255) & ~static_cast<size_t>(255);
            }
            // results of a page-locked run that the device can address go straight to the caller's
            // memory, row by row as the gather finishes them: no copy behind the launch at all
            float* y_at = y_zero_copy ? reinterpret_cast<float*>(y_mapped + (yo - x_bytes)) : reinterpret_cast<float*>(dbuf + yo);
            items[i] = QueueItem{t.seg, dbuf + x_at, CSDR_DTYPE_F32, CSDR_LAYOUT_FEATURE_MAJOR, t.batch, y_at,
                                 CSDR_LAYOUT_FEATURE_MAJOR, nullptr};
            yo += (yb + 255) & ~static_cast<size_t>(255);
        }
        CSDR_CUDA(cudaMemcpyAsync(dbuf, x_direct ? tasks[0].x : static_cast<const void*>(hbuf), xo, cudaMemcpyHostToDevice, ctx->stream));
        if (gemv_queue_supported(ctx, items.data(), static_cast<uint32_t>(n_tasks))) {
            launch_gemv_queue(ctx, items.data(), static_cast<uint32_t>(n_tasks));
        } else {
            for (const QueueItem& it : items) {
                MatmulArgs a;
                a.x = it.x;
                a.batch = it.batch;
                a.y = it.y;
                launch_matmul(ctx, it.seg, a);
            }
        }
        if (!y_zero_copy)
            CSDR_CUDA(cudaMemcpyAsync(y_direct ? static_cast<void*>(tasks[0].y) : static_cast<void*>(hbuf + x_bytes), dbuf + x_bytes,
                                      yo - x_bytes, cudaMemcpyDeviceToHost, ctx->stream));
        CSDR_CUDA(cudaStreamSynchronize(ctx->stream));
        if (!y_direct) {
            yo = x_bytes;
            for (size_t i = 0; i < n_tasks; ++i) {
                const size_t yb = static_cast<size_t>(tasks[i].seg->g.rows) * tasks[i].batch * 4;
                std::memcpy(tasks[i].y, hbuf + yo, yb);
                yo += (yb + 255) & ~static_cast<size_t>(255);
            }
        }
    });
}

int csdr_matmul(csdr_context* ctx, const csdr_segment* seg, const float* x, size_t batch, float* y,
                int allow_2d) {
    return guard([&] {
        require_ctx(ctx);
        if (!seg || !x || !y) throw Error(CSDR_ERR_INVALID_ARG, "null argument");
        const Geometry& g = seg->g;
        if (!allow_2d) {
            // matmulRowMajor's own refusals, strategies/HierarchicalSDRStrategy.cpp:1273-1289.
            if (g.tile_rows != 1)
                throw Error(CSDR_ERR_GEOMETRY,
                            "HSDR matmul: fused matmul requires tile_rows == 1; use decompress() + "
                            "dense matmul for 2D tile encodings");
            if (g.tile_cols != g.cols)
                throw Error(CSDR_ERR_GEOMETRY,
                            "HSDR matmul: 1D row-tile encoding must have tile_cols == original_cols "
                            "(each tile is exactly one row of W)");
        }
        if (batch == 0) return;
        const size_t xb = static_cast<size_t>(g.cols) * batch * 4, yb = static_cast<size_t>(g.rows) * batch * 4;
        const size_t head = 256;                                   // completion word lives here
        const size_t xoff = (xb + 255) & ~static_cast<size_t>(255);
        // Small operands: x pulled by a kernel, y written by the product into mapped memory,
        // completion through a polled word. Large ones: plain DMAs from/to page-locked staging.
        const bool small = xb <= (256u << 10) && yb <= (256u << 10) && (xb & 15u) == 0;
        unsigned char* hbuf = static_cast<unsigned char*>(ctx->pinned_get(head + xoff + yb));
        unsigned char* dbuf = static_cast<unsigned char*>(ctx->scratch_get(3, xoff + (small ? 0 : yb)));
        volatile uint32_t* word = reinterpret_cast<volatile uint32_t*>(hbuf);
        unsigned char* xh = hbuf + head;
        float* yh = reinterpret_cast<float*>(hbuf + head + xoff);
        std::memcpy(xh, x, xb);
        float* xd = reinterpret_cast<float*>(dbuf);
        float* yd = reinterpret_cast<float*>(dbuf + xoff);
        MatmulArgs a;
        a.x = xd;
        a.batch = batch;
        if (small) {
            void* mapped = nullptr;
            CSDR_CUDA(cudaHostGetDevicePointer(&mapped, hbuf, 0));
            unsigned char* mb = static_cast<unsigned char*>(mapped);
            const uint32_t n4 = static_cast<uint32_t>(xb / 16u);
            {
                LaunchScope ls(ctx, KC_DECODER_OP);
                host_x_pull_kernel<<<std::min<uint32_t>(8u, (n4 + 1023u) / 1024u), 1024, 0, ctx->stream>>>(
                    reinterpret_cast<const float4*>(mb + head), reinterpret_cast<float4*>(xd), n4);
                ls.done("host_x_pull_kernel");
            }
            a.y = reinterpret_cast<float*>(mb + head + xoff);
            launch_matmul(ctx, seg, a);
            if (++ctx->notify_seq == 0) ++ctx->notify_seq;
            cudaLaunchConfig_t cfg{};
            cfg.gridDim = dim3(1, 1, 1);
            cfg.blockDim = dim3(1, 1, 1);
            cfg.stream = ctx->stream;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attr[0].val.programmaticStreamSerializationAllowed = ctx->pdl ? 1 : 0;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            {
                LaunchScope ls(ctx, KC_DECODER_OP);
                CSDR_CUDA(cudaLaunchKernelEx(&cfg, host_notify_kernel,
                                             reinterpret_cast<volatile uint32_t*>(mb), ctx->notify_seq));
                ls.done("host_notify_kernel");
            }
            if (!wait_host_word(word, ctx->notify_seq)) CSDR_CUDA(cudaStreamSynchronize(ctx->stream));
        } else {
            CSDR_CUDA(cudaMemcpyAsync(xd, xh, xb, cudaMemcpyHostToDevice, ctx->stream));
            a.y = yd;
            launch_matmul(ctx, seg, a);
            CSDR_CUDA(cudaMemcpyAsync(yh, yd, yb, cudaMemcpyDeviceToHost, ctx->stream));
            CSDR_CUDA(cudaStreamSynchronize(ctx->stream));
        }
        std::memcpy(y, yh, yb);
    });
}

int csdr_decompress_device_async(csdr_context* ctx, const csdr_segment* seg, float* out_dev) {
    return guard([&] {
        require_ctx(ctx);
        if (!seg || !out_dev) throw Error(CSDR_ERR_INVALID_ARG, "null argument");
        launch_decode_rows(ctx, seg, nullptr, seg->g.rows, out_dev);
    });
}

int csdr_decompress(csdr_context* ctx, const csdr_segment* seg, float* out_host,
                    size_t capacity_floats) {
    return guard([&] {
        require_ctx(ctx);
        if (!seg || !out_host) throw Error(CSDR_ERR_INVALID_ARG, "null argument");
        const size_t n = static_cast<size_t>(seg->g.rows) * seg->g.cols;
        if (capacity_floats < n) throw Error(CSDR_ERR_BUFFER, "decompress output buffer too small");
        float* dev = static_cast<float*>(ctx->scratch_get(2, n * 4));
        launch_decode_rows(ctx, seg, nullptr, seg->g.rows, dev);
        CSDR_CUDA(cudaMemcpyAsync(out_host, dev, n * 4, cudaMemcpyDeviceToHost, ctx->stream));
        CSDR_CUDA(cudaStreamSynchronize(ctx->stream));
    });
}

int csdr_dequantize(csdr_context* ctx, const char* fmt, const void* data, size_t nbytes,
                    float scale, float zero_point, float* out_host, size_t capacity_floats,
                    size_t* n_out) {
    return guard([&] {
        require_ctx(ctx);
        if (!data || !out_host) throw Error(CSDR_ERR_INVALID_ARG, "null argument");
        const int id = dequant_format_id(fmt);
        if (id < 0)
            throw Error(CSDR_ERR_UNSUPPORTED,
                        std::string("HSDR dequant: unsupported input dtype '") + (fmt ? fmt : "") +
                            "'; supported: f32, f16, bf16, i8, q4_0, q8_0, q4_k, q5_k, q6_k");
        const size_t n = dequant_output_count(id, nbytes);
        if (n_out) *n_out = n;
        if (capacity_floats < n) throw Error(CSDR_ERR_BUFFER, "dequantize output buffer too small");
        const size_t in_off = (n * 4 + 255) & ~static_cast<size_t>(255);
        unsigned char* buf = static_cast<unsigned char*>(ctx->scratch_get(2, in_off + nbytes + 16));
        CSDR_CUDA(cudaMemcpyAsync(buf + in_off, data, nbytes, cudaMemcpyHostToDevice, ctx->stream));
        launch_dequantize(ctx, id, buf + in_off, nbytes, n, scale, zero_point, reinterpret_cast<float*>(buf));
        CSDR_CUDA(cudaMemcpyAsync(out_host, buf, n * 4, cudaMemcpyDeviceToHost, ctx->stream));
        CSDR_CUDA(cudaStreamSynchronize(ctx->stream));
    });
}

int csdr_dequantize_inference(csdr_context* ctx, const char* fmt, const void* data, size_t nbytes,
                              size_t n_elements, float* out_host, size_t capacity_floats, size_t* n_out) {
    return guard([&] {
        require_ctx(ctx);
        if (!data || !out_host) throw Error(CSDR_ERR_INVALID_ARG, "null argument");
        const int id = dequant_format_id(fmt);
        if (id < 4)   // q4_0, q8_0, q4_k, q5_k, q6_k
            throw Error(CSDR_ERR_UNSUPPORTED, std::string("unsupported block format '") + (fmt ? fmt : "") +
                                                  "'; supported: q4_0, q8_0, q4_k, q5_k, q6_k");
        static const size_t unit[] = {18, 34, 144, 176, 210};
        const size_t bb = unit[id - 4], be = id < 6 ? 32 : 256;
        if (nbytes < bb) throw Error(CSDR_ERR_FORMAT, "fewer bytes than one block");
        // whole blocks only, trailing bytes ignored, count clipped to n_elements (:297-306)
        const size_t whole = nbytes / bb * bb;
        const size_t n = std::min(n_elements, whole / bb * be);
        if (n_out) *n_out = n;
        if (capacity_floats < n) throw Error(CSDR_ERR_BUFFER, "dequantize output buffer too small");
        const size_t in_off = (whole / bb * be * 4 + 255) & ~static_cast<size_t>(255);
        unsigned char* buf = static_cast<unsigned char*>(ctx->scratch_get(2, in_off + whole + 16));
        CSDR_CUDA(cudaMemcpyAsync(buf + in_off, data, whole, cudaMemcpyHostToDevice, ctx->stream));
        launch_dequantize_inference(ctx, id, buf + in_off, whole, n, reinterpret_cast<float*>(buf));
        CSDR_CUDA(cudaMemcpyAsync(out_host, buf, n * 4, cudaMemcpyDeviceToHost, ctx->stream));
        CSDR_CUDA(cudaStreamSynchronize(ctx->stream));
    });
}

}  // extern "C"
