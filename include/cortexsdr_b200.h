/*
 * cortexsdr_b200 — thin extern "C" CUDA layer for the HSDR on-demand inference
 * matmul on NVIDIA B200 (sm_100a).
 *
 * Plain pointers and sizes only; every function returns an int status (0 = ok,
 * negative = error, see CSDR_ERR_*); nothing throws across this boundary; there is
 * no CPU fallback — without a CUDA device every compute entry point fails with
 * CSDR_ERR_CUDA. A thread-local message for the last failure is available from
 * csdr_last_error().
 *
 * Each entry point names the reference interface it stands in for
 * (file:line inside the reference tree, under src/ai_compression/).
 *
 * Conventions
 *   - "payload" = the bytes of one compressed segment exactly as they sit in a .sdr
 *     archive ("HSDR" v2: header, stage scales, dictionary, packed codes, edge
 *     strips) or in a .hsda container ("HSDC" v1: header, packed codes).
 *   - Reference activation layout ("feature-major"): x is (C x batch) row-major,
 *     y is (R x batch) row-major — strategies/HierarchicalSDRStrategy.hpp:164-181.
 *   - "token-major": x is (batch x C), y is (batch x R) — the layout of
 *     SDRInferenceEngine::applyLinearLayer (SparseInferenceEngine.cpp:1481).
 *   - One context = one device + one stream; calls on a context are synchronous on
 *     return unless the name ends in _async. One thread per context.
 */
#ifndef CORTEXSDR_B200_H
#define CORTEXSDR_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define CSDR_API __attribute__((visibility("default")))
#else
#define CSDR_API
#endif

enum {
    CSDR_OK = 0,
    CSDR_ERR_INVALID_ARG = -1,
    CSDR_ERR_FORMAT = -2,       /* bad magic / version / truncated stream */
    CSDR_ERR_GEOMETRY = -3,     /* tile geometry not accepted by this entry point */
    CSDR_ERR_NOT_FOUND = -4,    /* segment name not in the archive */
    CSDR_ERR_STRATEGY = -5,     /* segment is not HSDR-encoded */
    CSDR_ERR_CUDA = -6,         /* CUDA runtime error, or no device */
    CSDR_ERR_TIMEOUT = -7,      /* a bounded device-side wait ran out */
    CSDR_ERR_IO = -8,
    CSDR_ERR_UNSUPPORTED = -9,
    CSDR_ERR_BUFFER = -10,      /* caller's output buffer too small */
    CSDR_ERR_CODE_RANGE = -11,  /* a packed code names an atom index >= n_atoms */
    CSDR_ERR_LIMIT = -12        /* size beyond a documented fixed maximum */
};

enum { CSDR_DTYPE_F32 = 0, CSDR_DTYPE_BF16 = 1,
       CSDR_DTYPE_F16 = 2 /* KV-cache element type only; activations are fp32 or bf16 */ };
enum { CSDR_LAYOUT_FEATURE_MAJOR = 0, CSDR_LAYOUT_TOKEN_MAJOR = 1 };
enum { CSDR_KIND_HSDR = 0, CSDR_KIND_HSDC = 1 };

typedef struct csdr_context csdr_context;
typedef struct csdr_segment csdr_segment;       /* device image of one compressed weight */
typedef struct csdr_dictionary csdr_dictionary; /* device image of a shared dictionary */
typedef struct csdr_archive csdr_archive;       /* an opened .sdr */
typedef struct csdr_hsda csdr_hsda;             /* an opened .hsda */
typedef struct csdr_decoder csdr_decoder;       /* device-resident decoder-layer driver */

/* Fields of the payload header (HSDRHeader, strategies/HierarchicalSDRStrategy.cpp:49-66;
 * HSDRCodesHeader, :675-692) plus the byte offsets of the streams behind it. */
typedef struct {
    int32_t kind;               /* CSDR_KIND_* */
    uint32_t rows, cols, n_tiles;
    uint16_t tile_rows, tile_cols, n_atoms;
    uint8_t n_stages, k_per_stage;
    float stage_decay;
    uint32_t edge_bytes;
    uint64_t off_scales, off_dict, off_codes, off_edges;
    uint64_t payload_bytes;     /* header + all streams */
} csdr_payload_info;

CSDR_API const char* csdr_last_error(void);
CSDR_API const char* csdr_version(void);

/* ---- context ---- */
/* device < 0 selects the current device. stream may be NULL (the context makes its
 * own non-blocking stream) or a cudaStream_t the caller owns. */
CSDR_API int csdr_context_create(int device, void* stream, csdr_context** out);
CSDR_API int csdr_context_destroy(csdr_context* ctx);
CSDR_API int csdr_context_synchronize(csdr_context* ctx);
CSDR_API void* csdr_context_stream(csdr_context* ctx);
/* Number of kernels this library has launched on the context since creation. */
CSDR_API uint64_t csdr_context_launch_count(const csdr_context* ctx);

/* Iteration limits of the device-side waits (no counterpart in the reference, which has no
 * device). Every wait inside a kernel is a bounded poll: the fused decode GEMV's hand-over of
 * partial results, the mbarrier waits of the tensor-core kernels, and a tensor-parallel rank's
 * wait for its peers' flags. A wait that runs out records a status word, the kernel returns, and
 * the next csdr_context_synchronize answers CSDR_ERR_TIMEOUT; the context stays usable. 0 keeps
 * or restores a default (1e6 polls, 4e6 rounds, 2e6 polls: of the order of a second each). */
CSDR_API int csdr_context_set_wait_limits(csdr_context* ctx, uint32_t gemv_polls,
                                          uint32_t barrier_rounds, uint32_t exchange_polls);
/* Diagnostic: runs the receiving side of a two-rank exchange on a scratch region whose second
 * flag nothing ever raises, then synchronizes. Answers CSDR_ERR_TIMEOUT once the exchange
 * limit is spent (set a small one first) - the proof that a lost peer surfaces as an error code
 * rather than as a hung device. */
CSDR_API int csdr_context_wait_selftest(csdr_context* ctx);

/* Per-kernel device timing for benchmarks. While enabled, every kernel this library
 * launches on the context is bracketed by two CUDA events on the context's stream;
 * csdr_context_profile_read then gives, for one kernel class (0 <= cls < the count
 * csdr_kernel_class_name knows), the launches bracketed since enabling and the sum of
 * their event-to-event durations. Enabling or disabling clears the record. With
 * profiling off, *launches is the class's lifetime launch count and *total_ms is 0. */
CSDR_API int csdr_context_profile(csdr_context* ctx, int enable);
CSDR_API int csdr_context_profile_read(csdr_context* ctx, int cls, uint64_t* launches,
                                       double* total_ms);
CSDR_API const char* csdr_kernel_class_name(int cls); /* "?" past the last class */
/* Phase timeline of the fused decode GEMV, for tuning. While enabled, thread 0 of every CTA
 * of each fused-GEMV launch stores global-timer stamps (ns) in 16 slots: 0 start, 1 weights
 * requested, 2 dependency wait over, 3 activations staged, 4 projection published, 5 hand-over
 * seen, 6 first gather done, 7 end, 8 products done, 9 partials stored, 10 CTA joined; the rest
 * unused. The call first copies the stamps of the LAST launch to `out` (16 words per CTA, may
 * be NULL), then applies `enable`. */
CSDR_API int csdr_context_gemv_trace(csdr_context* ctx, int enable, uint64_t* out, size_t capacity,
                                     size_t* n_out);

/* ---- payload framing (host only) ----
 * Replaces the header parse + checks at the top of matmulRowMajor / decompress
 * (strategies/HierarchicalSDRStrategy.cpp:1262-1299, :1345-1389) and parseCodesStream
 * (:1766-1801). Validates magic, version, stream lengths, and that every packed code
 * names an atom < n_atoms (the reference does not check the last one; a device kernel
 * must never be handed an out-of-range index). */
CSDR_API int csdr_payload_inspect(const void* payload, size_t nbytes, csdr_payload_info* info);

/* ---- device images ---- */
/* From an "HSDR" payload (dictionary embedded). */
CSDR_API int csdr_segment_create(csdr_context* ctx, const void* payload, size_t nbytes,
                                 csdr_segment** out);
/* SharedDictionary (strategies/HierarchicalSDRStrategy.hpp:194-198): atoms is
 * (n_atoms x tile_rows*tile_cols) fp32 row-major, scales has n_stages entries. */
CSDR_API int csdr_dictionary_create(csdr_context* ctx, uint16_t tile_rows, uint16_t tile_cols,
                                    uint16_t n_atoms, uint8_t n_stages, uint8_t k_per_stage,
                                    const float* atoms, const float* scales,
                                    csdr_dictionary** out);
/* From an "HSDC" codes-only payload + its dictionary; geometry is checked as in
 * parseCodesStream (:1781-1787). The dictionary must outlive the segment. */
CSDR_API int csdr_segment_create_shared(csdr_context* ctx, const void* codes, size_t nbytes,
                                        const csdr_dictionary* dict, csdr_segment** out);
CSDR_API int csdr_segment_destroy(csdr_segment* seg);
CSDR_API int csdr_dictionary_destroy(csdr_dictionary* dict);
CSDR_API int csdr_segment_info(const csdr_segment* seg, csdr_payload_info* info);
/* Row-shard for tensor parallelism: keep only output rows [row_begin, row_end) of the
 * code stream (1-D row tiles: any range; 2-D tiles: multiples of tile_rows). The
 * dictionary is shared with `seg`, which must outlive the shard. */
CSDR_API int csdr_segment_shard_rows(csdr_context* ctx, const csdr_segment* seg,
                                     uint32_t row_begin, uint32_t row_end, csdr_segment** out);
/* Column-shard for tensor parallelism (1-D row tiles): keep input columns [col_begin, col_end),
 * multiples of four, of every dictionary atom, copied into a dictionary of the shard's own;
 * the code stream is shared with `seg`, which must outlive the shard. A column shard times
 * the matching slice of x is that slice's share of W x: the shares of all slices add up to
 * the product (no counterpart in the reference, whose matmul is not distributed). */
CSDR_API int csdr_segment_shard_cols(csdr_context* ctx, const csdr_segment* seg,
                                     uint32_t col_begin, uint32_t col_end, csdr_segment** out);

/* ---- sparse-code unpack ----
 * unpackIndexSign (strategies/HierarchicalSDRStrategy.cpp:81-84; loops :1394-1399,
 * :1795-1799): u16 -> (index = v & 0x7FFF, sign = v >> 15 ? -1 : +1), on the device,
 * results copied to host arrays of n_tiles*n_stages*k entries. */
CSDR_API int csdr_unpack_codes(csdr_context* ctx, const csdr_segment* seg, int32_t* idx_out,
                               int8_t* sign_out, size_t capacity);

/* ---- fused matmul ----
 * HierarchicalSDRStrategy::matmulRowMajor (strategies/HierarchicalSDRStrategy.cpp:1257)
 * and ::matmulWithExternalDictionary (:1830): host buffers, reference layout
 * (x: C x batch, y: R x batch, fp32). As the reference, refuses 2-D tiles
 * (CSDR_ERR_GEOMETRY) unless allow_2d != 0, in which case the result equals the
 * reference's decompress() + dense product (SparseInferenceEngine.cpp:1301-1310). */
CSDR_API int csdr_matmul(csdr_context* ctx, const csdr_segment* seg, const float* x,
                         size_t batch, float* y, int allow_2d);
/* Same product with device-resident activations. x_dtype/x_layout/y_layout as the
 * enums above; y is fp32; bias (R floats, device) may be NULL
 * (applyLinearLayer adds it, SparseInferenceEngine.cpp:1509-1511). Asynchronous on the
 * context's stream. */
CSDR_API int csdr_matmul_device_async(csdr_context* ctx, const csdr_segment* seg,
                                      const void* x_dev, int x_dtype, int x_layout,
                                      size_t batch, float* y_dev, int y_layout,
                                      const float* bias_dev);

/* Several compressed weights that consume the SAME activations (q|k|v, gate|up) in as few
 * launches as possible: 1-D row-tile segments of equal column count share one kernel,
 * anything else is issued segment by segment. ys_dev[i] receives segment i's product.
 * The reference issues these as separate matmulHSDR calls
 * (api/cortex_sdk.cpp:1578-1583, :1653-1656). */
CSDR_API int csdr_matmul_group_device_async(csdr_context* ctx, const csdr_segment* const* segs,
                                            size_t n_segs, const void* x_dev, int x_dtype,
                                            int x_layout, size_t batch, float* const* ys_dev,
                                            int y_layout);

/* A list of products in as few launches as possible: the heads of a batch of requests, q|k|v
 * and gate|up of a block, the experts of a routed layer, a chain of layers. Lists whose members
 * are all 1-D row-tile segments with one common batch of 1 to 4 tokens run as one persistent
 * kernel per 32 tasks, in which the weight stream of task n+1 flows under the hand-over and
 * gather of task n (tasks may differ in shape, activations and outputs); any other list is
 * issued task by task, in order. A task whose activations are another task's output names that
 * task in after_task (an index below its own, in the same group of 32; -1: none): its weights
 * still stream ahead, its activations are read once that task's rows are complete. The
 * reference issues one matmulHSDR call per product (SparseInferenceEngine.cpp:1074-1091). */
typedef struct {
    const csdr_segment* seg;
    const void* x_dev;      /* activations, dtype/layout as the enums above */
    int x_dtype, x_layout;
    size_t batch;
    float* y_dev;           /* fp32 */
    int y_layout;
    const float* bias_dev;  /* R floats or NULL */
    int after_task;         /* -1, or the index of the task whose y this task's x_dev is (or depends on) */
} csdr_matmul_task;
CSDR_API int csdr_matmul_queue_device_async(csdr_context* ctx, const csdr_matmul_task* tasks,
                                            size_t n_tasks);

/* The same list with HOST buffers, reference layout (x: C x batch, y: R x batch, fp32): every
 * task's activations cross to the device in one copy, the list runs as above, every result
 * comes back in one copy, one synchronisation in all. Tasks that name the same host x share one
 * staged copy. When the tasks' activations (results) lie one behind the other, in task order
 * and in multiples of 256 bytes, in page-locked host memory (cudaHostAlloc / cudaHostRegister),
 * they are transferred straight from (to) the caller's memory instead of through a staging
 * buffer. 1-D row tiles only, as matmulRowMajor (CSDR_ERR_GEOMETRY otherwise). */
typedef struct {
    const csdr_segment* seg;
    const float* x;
    size_t batch;
    float* y;
} csdr_matmul_host_task;
CSDR_API int csdr_matmul_queue(csdr_context* ctx, const csdr_matmul_host_task* tasks, size_t n_tasks);

/* The same row-tile product for callers that must not allocate. No counterpart in the
 * reference: it exists for hosts that cannot call cudaMalloc while they run - a process
 * whose device memory map is frozen after start-up (real-time or certified systems), a
 * plug-in that lives inside another runtime's memory pool and owns no allocator of its own,
 * or a service that has handed all device memory to its own arena. This call makes no device
 * allocation: no cudaMalloc, no cudaFree, no library routine that allocates device memory (on
 * the host the success path allocates nothing either; an error builds its message string).
 * What the CUDA driver does on its own account still happens once: with lazy module loading the
 * first launch of each kernel variant - one per token-tile width 1, 2, 4, 8, 16, chosen from the
 * batch - and the first address look-up load code onto the device. So warm up, before the memory
 * map freezes and before any stream capture, with one call per tile width the caller will use
 * (batches 1, 2, 4, 8 and 16 cover them all). Every buffer is the caller's,
 * as raw device pointers taken straight from a payload's streams:
 *   dict_dev    n_atoms x cols fp32 (the "HSDR" dictionary stream), 16-byte aligned
 *   codes_dev   rows x n_stages x k_per_stage packed u16 codes, 16-byte aligned, in an
 *               allocation whose length is rounded up to 16 bytes (kernels read it in
 *               128-bit units); every code should name an atom < n_atoms (csdr_payload_inspect
 *               checks that on the host). A code that does not is skipped - it adds nothing to
 *               its row, nothing is read out of bounds - and is reported by
 *               csdr_matmul_rowtiles_noalloc_status
 *   scales_dev  n_stages fp32
 *   x_dev/y_dev activations and fp32 output, dtype and layouts as for csdr_matmul_device_async
 * The one piece of scratch the two-kernel path needs (Dx, n_atoms x 16 floats) sits in a
 * fixed array inside the library's device image: 256 KiB, held by every GPU that loads the
 * library until the process exits. Hence the limit: n_atoms <= 4096 (CSDR_ERR_LIMIT beyond
 * it), 1-D row tiles only, cols a multiple of 4. The first call on a device looks up the
 * array's device address (that device must be current, as for every call); make that first
 * call before starting any stream capture. All calls share the array, and it keeps the last
 * call's contents (nothing in it needs clearing: each call overwrites what it reads): calls
 * that overlap on the GPU - issued on different streams - race on it; calls on one stream are ordered and safe. Asynchronous on `stream`
 * (a cudaStream_t; NULL is the default stream). */
CSDR_API int csdr_matmul_rowtiles_noalloc(const float* dict_dev, const uint16_t* codes_dev,
                                          const float* scales_dev, uint32_t rows, uint32_t cols,
                                          uint32_t n_atoms, uint32_t n_stages, uint32_t k_per_stage,
                                          const void* x_dev, int x_dtype, int x_layout, size_t batch,
                                          float* y_dev, int y_layout, void* stream);
/* Waits for `stream`, then tells whether any allocation-free call on this device since the last
 * query met a code naming an atom >= n_atoms: *bad_codes = 1 and CSDR_ERR_CODE_RANGE if so
 * (the flag is cleared), else 0 and CSDR_OK. Allocates nothing. No counterpart in the reference. */
CSDR_API int csdr_matmul_rowtiles_noalloc_status(void* stream, int* bad_codes);

/* ---- materialise the weight ----
 * HierarchicalSDRStrategy::decompress (:1340) / ::decompressWithExternalDictionary
 * (:1804): fp32 (rows x cols) row-major, edge strips spliced back. */
CSDR_API int csdr_decompress(csdr_context* ctx, const csdr_segment* seg, float* out_host,
                             size_t capacity_floats);
CSDR_API int csdr_decompress_device_async(csdr_context* ctx, const csdr_segment* seg,
                                          float* out_dev);

/* ---- source-dtype dequantisation ----
 * HierarchicalSDRStrategy::dequantizeToFP32 (:1017; body :713-989), HSDR's own
 * element order. fmt: "f32","f16","bf16","i8","q4_0","q8_0","q4_k","q5_k","q6_k".
 * *n_out receives the element count. Bit-exact against the reference. */
CSDR_API int csdr_dequantize(csdr_context* ctx, const char* fmt, const void* data,
                             size_t nbytes, float scale, float zero_point, float* out_host,
                             size_t capacity_floats, size_t* n_out);

/* ---- encoder ----
 * HierarchicalSDRStrategy::compress (strategies/HierarchicalSDRStrategy.cpp:1068-1236) on the
 * device: fitHierarchicalKSVD (:494-607) - a dictionary of n_atoms tiles picked by
 * std::mt19937(0xC0DE), normalised and scaled, one coding pass, then ksvd_iters rounds of
 * atomUpdateStep (:281-489) + coding pass (0 rounds is the reference's fast mode). W is
 * rows x cols fp32 row-major on the host, the result an "HSDR" v2 payload. *n_out receives the
 * payload size (also when the buffer is too small: CSDR_ERR_BUFFER). Header, stage scales, tile
 * picks and edge strips equal the reference encoder's; atoms agree to rounding; a code may differ
 * where a round's two best atoms tie within fp32 rounding (the coding pass works on projections
 * computed once and updated through the Gram matrix instead of re-projecting a residual), and
 * behind such a code the update rounds move the atoms it touches differently: with rounds the
 * two encoders agree in reconstruction error, not atom for atom. */
CSDR_API int csdr_hsdr_encode(csdr_context* ctx, const float* W, uint32_t rows, uint32_t cols,
                              uint16_t tile_rows, uint16_t tile_cols, uint16_t n_atoms,
                              uint8_t n_stages, uint8_t k_per_stage, float stage_decay,
                              uint8_t ksvd_iters, void* payload_out, size_t capacity, size_t* n_out);
/* Several tensors behind ONE dictionary: compressGroupedSegments (:2211-2500) for tensors of one
 * configuration, with the fit on all pooled tiles (max_tiles_for_fit = 0) - the tensors' tiles
 * pooled in order, one fit on the pool (fitSharedDictionary, :1446-1469), every tensor coded
 * against the result (compressFP32WithExternalDictionary, :1691-1754). Every shape must divide
 * by the tile (CSDR_ERR_GEOMETRY otherwise, as the reference throws). dict_out receives the
 * dictionary as a .hsda holds it (20-byte config, counted stage scales, counted atoms:
 * SharedDictArchive::writeToStream, :1972-2002) - also the payload of a shared-dictionary
 * resource segment of a .sdr; codes_out[i] receives tensor i's codes-only "HSDC" stream.
 * dict_bytes and codes_bytes[i] receive the sizes, also when a buffer is missing or too small
 * (CSDR_ERR_BUFFER). The reservoir-sampled fit of the reference (a cap on the pool) is not built. */
CSDR_API int csdr_hsdr_encode_shared(csdr_context* ctx, const float* const* tensors,
                                     const uint32_t* rows, const uint32_t* cols, size_t n_tensors,
                                     uint16_t tile_rows, uint16_t tile_cols, uint16_t n_atoms,
                                     uint8_t n_stages, uint8_t k_per_stage, float stage_decay,
                                     uint8_t ksvd_iters, void* dict_out, size_t dict_capacity,
                                     size_t* dict_bytes, void* const* codes_out,
                                     const size_t* codes_capacity, size_t* codes_bytes);
/* The coding pass alone (hierarchicalBinaryCode, :219-262, over every tile): tiles is
 * (n_tiles x tile_dim) fp32, atoms (n_atoms x tile_dim), both on the host; codes_out receives
 * n_tiles * n_stages * k_per_stage packed codes (packIndexSign, :76-80). */
CSDR_API int csdr_encode_codes(csdr_context* ctx, const float* tiles, size_t n_tiles, size_t tile_dim,
                               const float* atoms, uint16_t n_atoms, uint8_t n_stages,
                               uint8_t k_per_stage, const float* stage_scales, uint16_t* codes_out,
                               size_t capacity);

/* The same block formats as the reference's INFERENCE side widens a stored-raw tensor
 * (decodeSupportedGGUFQuantized, SparseInferenceEngine.cpp:276-469): ggml's element order -
 * q4_k: 32 low nibbles then 32 high nibbles per 64-element group; q6_k: four runs of 32 per
 * 128-element half; q5_k: that function's generic 5-bit fall-back; q4_0, q8_0 sequential.
 * fmt: "q4_0","q8_0","q4_k","q5_k","q6_k". Whole blocks only; at most n_elements values.
 * This is what the decoder applies to strategy-0 tensors; csdr_dequantize above is what the
 * ENCODER applies to its inputs, and the two orders differ for the k-quants. */
CSDR_API int csdr_dequantize_inference(csdr_context* ctx, const char* fmt, const void* data,
                                       size_t nbytes, size_t n_elements, float* out_host,
                                       size_t capacity_floats, size_t* n_out);

/* ---- .sdr archive: SDRModelLoader / SDRInferenceEngine routing ---- */
typedef struct {
    const char* name;           /* owned by the archive */
    const char* data_format;
    const char* layer_type;
    uint8_t original_type;      /* SegmentType, core/ModelSegment.hpp:36-55 */
    uint8_t strategy_id;        /* 5 = HSDR, 0 = stored raw */
    uint64_t original_size, compressed_size, data_offset;
    uint32_t layer_index;
    uint32_t n_dims;
    uint32_t dims[8];
} csdr_segment_header;

/* SDRModelLoader(path) -> loadFromArchive -> AIDecompressor::readArchiveIndex
 * (SparseInferenceEngine.cpp:725-751, :994; core/AIDecompressor.cpp:78-262). */
CSDR_API int csdr_archive_open(csdr_context* ctx, const char* path, csdr_archive** out);
CSDR_API int csdr_archive_close(csdr_archive* ar);
CSDR_API int csdr_archive_num_segments(const csdr_archive* ar, size_t* n);
CSDR_API int csdr_archive_header_at(const csdr_archive* ar, size_t i, csdr_segment_header* h);
/* findSegmentHeader (SparseInferenceEngine.cpp:1066): CSDR_ERR_NOT_FOUND if absent. */
CSDR_API int csdr_archive_find(const csdr_archive* ar, const char* name, csdr_segment_header* h);
/* loadCompressedBytesByName (:1055): raw payload bytes. *n gets the needed size. */
CSDR_API int csdr_archive_read_payload(const csdr_archive* ar, const char* name, void* buf,
                                       size_t capacity, size_t* n);
/* loadSegmentByName (:1044): decoded segment bytes (HSDR -> fp32 matrix via the device
 * decompress kernel; strategy 0 -> stored bytes). Other strategies: CSDR_ERR_UNSUPPORTED. */
CSDR_API int csdr_archive_load_segment(csdr_archive* ar, const char* name, void* buf,
                                       size_t capacity, size_t* n);
/* Device image of a named HSDR segment, uploaded on first use and cached — the step the
 * reference repeats per call (file open + payload read + two copies). Owned by the archive. */
CSDR_API int csdr_archive_segment(csdr_archive* ar, const char* name, const csdr_segment** seg);
/* Drops the cached device image of `name` (NULL: of every segment); the next use uploads it
 * again. The reference's counterpart is its layer cache's eviction
 * (aggressive memory management, SparseInferenceEngine.hpp:414, :455).
 * Images handed out by csdr_archive_segment are dangling after this. */
CSDR_API int csdr_archive_release(csdr_archive* ar, const char* name);
/* Device bytes held by the archive's cached images (dictionaries, codes, scales, edge strips,
 * raw matrices) - SDRInferenceEngine::getCurrentMemoryUsage (SparseInferenceEngine.hpp:415). */
CSDR_API int csdr_archive_resident_bytes(const csdr_archive* ar, size_t* bytes);
/* SDRModelLoader::matmulHSDR (:1074): errors mirror the reference's
 * ("segment not found" -> CSDR_ERR_NOT_FOUND, "is not HSDR-encoded" -> CSDR_ERR_STRATEGY,
 * 2-D tiles -> CSDR_ERR_GEOMETRY). y_capacity in floats; *n_out = R*batch. */
CSDR_API int csdr_archive_matmul_hsdr(csdr_archive* ar, const char* name, const float* x,
                                      size_t batch, float* y, size_t y_capacity, size_t* n_out);
/* SDRInferenceEngine::matmulForLayer (:1271): HSDR route for strategy 5 (any tile
 * geometry; 2-D tiles give the reference's decompress+dense result), dense product on
 * the device for raw fp32 2-D segments, CSDR_ERR_UNSUPPORTED otherwise. */
CSDR_API int csdr_archive_matmul_for_layer(csdr_archive* ar, const char* name, const float* x,
                                           size_t batch, float* y, size_t y_capacity,
                                           size_t* n_out);
/* SDRInferenceEngine::applyLinearLayer, HSDR branches (:1487-1521, :1694-1728):
 * looks up `layer` then `layer + ".weight"`; token-major input (batch x C) and output
 * (batch x R); optional bias (R floats, host). */
CSDR_API int csdr_archive_apply_linear(csdr_archive* ar, const char* layer, const float* input,
                                       size_t input_size, const float* bias, float* output,
                                       size_t capacity, size_t* n_out);

/* ---- .hsda container: HSDAReader (strategies/HierarchicalSDRStrategy.cpp:2506-2550;
 * format :1905-1933, reader :2004-2064) ---- */
CSDR_API int csdr_hsda_open(csdr_context* ctx, const char* path, csdr_hsda** out);
CSDR_API int csdr_hsda_close(csdr_hsda* h);
CSDR_API int csdr_hsda_counts(const csdr_hsda* h, size_t* n_dicts, size_t* n_segments);
CSDR_API int csdr_hsda_has_segment(const csdr_hsda* h, const char* name);
CSDR_API int csdr_hsda_segment(csdr_hsda* h, const char* name, const csdr_segment** seg);
/* HSDAReader::matmul (:2536): 1-D row tiles only unless allow_2d. */
CSDR_API int csdr_hsda_matmul(csdr_hsda* h, const char* name, const float* x, size_t batch,
                              float* y, size_t y_capacity, size_t* n_out, int allow_2d);
/* HSDAReader::decompress (:2523). */
CSDR_API int csdr_hsda_decompress(csdr_hsda* h, const char* name, float* out,
                                  size_t capacity_floats, size_t* n_out);

/* ---- decoder-layer driver ----
 * Device-resident restatement of run_transformer_decode (api/cortex_sdk.cpp:1543-1696):
 * RMSNorm (:1208), RoPE on adjacent pairs (:1363-1423), grouped-query causal attention
 * (:1453-1478; kernels/attention_kernels.cpp:26-113), SwiGLU (:1245), residual adds,
 * final norm, logits (SparseInferenceEngine.cpp:2310-2320) — with a KV cache, which the
 * reference lacks (it recomputes the whole sequence per token). Block tensors are found
 * by the reference's GGUF-style names (cortex_sdk.cpp:456-524): token_embd.weight,
 * blk.<n>.{attn_norm,attn_q,attn_k,attn_v,attn_output,ffn_norm,ffn_gate,ffn_up,ffn_down}.weight,
 * output_norm.weight, output.weight. */
typedef struct {
    uint32_t n_layers, hidden, q_heads, kv_heads, head_dim, inter, vocab;
    uint32_t max_seq;       /* KV-cache capacity in positions, per sequence */
    uint32_t max_batch;     /* sequences decoded together */
    float rms_eps;          /* reference default 1e-5 (cortex_sdk.cpp:1212) */
    float rope_theta;       /* reference default 1e6 (cortex_sdk.cpp:1358) */
    /* tensor parallelism: this rank's index and the number of ranks sharing the model.
     * tp_size == 1 means no sharding. comm is an ncclComm_t (void*) or NULL. */
    uint32_t tp_rank, tp_size;
    void* nccl_comm;
    /* KV cache element type: CSDR_DTYPE_F32 (0, default: the reference's arithmetic),
     * CSDR_DTYPE_F16 or CSDR_DTYPE_BF16 (keys and values rounded to 16 bits when they enter
     * the cache, scores and sums in fp32; half the cache bytes per step; fp16 keeps three more
     * mantissa bits and wants |k|, |v| < 65504). No counterpart in the reference. */
    uint32_t kv_dtype;
} csdr_decoder_config;

CSDR_API int csdr_decoder_create(csdr_archive* ar, const csdr_decoder_config* cfg,
                                 csdr_decoder** out);
CSDR_API int csdr_decoder_destroy(csdr_decoder* d);
CSDR_API int csdr_decoder_reset(csdr_decoder* d);
/* Token selection of the reference's generation loop (select_best_from_logits,
 * api/cortex_sdk.cpp:1005-1030) for the steps: score = logit / temperature (temperature <= 0:
 * unscaled), non-finite scores skipped, 1.5 subtracted for tokens the sequence has produced
 * already, first maximum wins, -1 when nothing is selectable. Off by default (plain argmax).
 * While it is on every token a step selects is recorded for its sequence; note_generated records
 * tokens chosen elsewhere (the one picked from the prefill's logits); csdr_decoder_reset forgets
 * them all. */
CSDR_API int csdr_decoder_selection_policy(csdr_decoder* d, int enable, float temperature);
CSDR_API int csdr_decoder_note_generated(csdr_decoder* d, uint32_t seq, const int32_t* tokens,
                                         size_t n_tokens);
/* Tensor-parallel ranks (2 to 8, one process per GPU) can sum their partial projections through
 * peer memory instead of NCCL for steps of at most 16 tokens: every rank exports a 64-byte CUDA
 * IPC handle of its exchange region, the host program gathers the handles of all ranks
 * (rank-major) and every rank imports them. All ranks must do so, or none (no counterpart in
 * the reference). Waits on peers are bounded; one that runs out surfaces as CSDR_ERR_TIMEOUT
 * from csdr_context_synchronize. */
CSDR_API int csdr_decoder_exchange_export(csdr_decoder* d, void* handle64);
CSDR_API int csdr_decoder_exchange_import(csdr_decoder* d, const void* handles, size_t n_ranks);
/* Set sequence `seq` to `position` without computing anything: the cache rows below it
 * keep whatever they hold (zeros after creation). For throughput measurements at a given
 * context length. */
CSDR_API int csdr_decoder_seek(csdr_decoder* d, uint32_t seq, uint32_t position);
/* Run n_tokens new positions of sequence `seq` (prefill when n_tokens > 1). If
 * logits_out != NULL it receives the vocab logits of the LAST position (host, fp32).
 * If hidden_out != NULL it receives the final-normed hidden state of every new
 * position (n_tokens x hidden, host). */
CSDR_API int csdr_decoder_forward(csdr_decoder* d, uint32_t seq, const int32_t* tokens,
                                  size_t n_tokens, float* logits_out, float* hidden_out);
/* One decode step for `batch` sequences at once (sequence b gets tokens[b]); writes the
 * greedy next token of each to next_out (host). logits_out may be NULL, else
 * (batch x vocab) host fp32. */
CSDR_API int csdr_decoder_step(csdr_decoder* d, const int32_t* tokens, size_t batch,
                               int32_t* next_out, float* logits_out);
/* Same step, nothing copied to the host: tokens_dev in, next_dev out (device int32). */
CSDR_API int csdr_decoder_step_device_async(csdr_decoder* d, const int32_t* tokens_dev,
                                            size_t batch, int32_t* next_dev);

/* ---- NCCL plumbing for tensor parallelism (rank 0 makes the id, the host program
 * broadcasts it, every rank initialises) ---- */
CSDR_API int csdr_nccl_unique_id(void* id128);  /* 128-byte buffer */
CSDR_API int csdr_nccl_comm_create(csdr_context* ctx, const void* id128, int rank, int world,
                                   void** comm_out);
CSDR_API int csdr_nccl_comm_destroy(void* comm);

#ifdef __cplusplus
}
#endif
#endif /* CORTEXSDR_B200_H */
