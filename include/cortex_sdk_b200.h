/*
 * The inference-engine half of the reference's C SDK, re-exported by
 * libcortexsdr_b200.so with the SAME symbol names and signatures
 * (src/ai_compression/api/cortex_sdk.h:110-237, error type api/c_api.hpp:26-29), so a
 * program written against cortex_sdk.h relinks against this library unchanged for the
 * HSDR linear path.
 *
 * Conventions kept from the reference (api/cortex_sdk.cpp):
 *   - CortexError is returned BY VALUE; {NULL, 0} on success; negative codes below.
 *   - Handles are registered in a process-wide table and validated on every call (:1798).
 *   - Output buffers are caller-allocated; when too small, *actual_output_size receives
 *     the needed element count and the code is CORTEX_B200_ERROR_MEMORY (:1873-1876).
 *   - One thread per handle.
 * Differences, all deliberate:
 *   - error messages are owned by the library (thread-local; valid until the next call on
 *     the same thread) — never free them;
 *   - strings handed to the caller (stats JSON) are malloc'ed; release with cortex_free_string;
 *   - layers are LINEAR layers backed by HSDR segments (strategy id 5) or raw fp32 2-D
 *     weights; `run` applies the archive's 2-D weights in index order, each feeding the next
 *     (the reference's interpreter over a LINEAR-only graph);
 *   - this library has no tokenizer: `generate_text` takes the prompt as decimal token ids
 *     separated by blanks and returns the generated ids the same way. The loop, the decoder
 *     shape discovery and the token selection (temperature 0.8, 1.5 off tokens already
 *     generated, first maximum) follow api/cortex_sdk.cpp:1951-2054, :1335-1349, :1005-1030,
 *     on the transformer path with a KV cache.
 */
#ifndef CORTEX_SDK_B200_H
#define CORTEX_SDK_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#ifndef CORTEXSDR_API
#if defined(__GNUC__)
#define CORTEXSDR_API __attribute__((visibility("default")))
#else
#define CORTEXSDR_API
#endif
#endif

/* api/cortex_sdk.cpp:56-64 */
#define CORTEX_B200_SUCCESS 0
#define CORTEX_B200_ERROR_INVALID_ARGUMENT (-1)
#define CORTEX_B200_ERROR_FILE_IO (-2)
#define CORTEX_B200_ERROR_MEMORY (-3)
#define CORTEX_B200_ERROR_UNSUPPORTED_FORMAT (-4)
#define CORTEX_B200_ERROR_DECOMPRESSION (-6)
#define CORTEX_B200_ERROR_INFERENCE (-7)
#define CORTEX_B200_ERROR_UNKNOWN (-99)

#ifndef C_API_HPP /* the reference's own header defines the same struct */
typedef struct {
    const char* message;
    int code;
} CortexError;
#endif

typedef struct CortexInferenceEngine* CortexInferenceEngineHandle;

/* cortex_sdk.h:110 — opens the .sdr index; segments go to the device on first use. */
CORTEXSDR_API CortexError cortex_inference_engine_create(const char* compressed_model_path,
                                                         CortexInferenceEngineHandle* handle);
/* cortex_sdk.h:118-169 — engine settings. batch size: what `run` expects (0 = from the input);
 * mode/dropout: recorded, `run` refuses training with dropout; memory pool: MiB budget for
 * cached device images; aggressive memory: a layer's image is dropped once it has run;
 * layer prefetch: every HSDR segment is uploaded now. */
CORTEXSDR_API CortexError cortex_inference_engine_set_batch_size(CortexInferenceEngineHandle handle, size_t batch_size);
CORTEXSDR_API CortexError cortex_inference_engine_enable_dropout(CortexInferenceEngineHandle handle, int enable);
CORTEXSDR_API CortexError cortex_inference_engine_set_mode(CortexInferenceEngineHandle handle, int training_mode);
CORTEXSDR_API CortexError cortex_inference_engine_init_memory_pool(CortexInferenceEngineHandle handle, size_t max_memory_mb);
CORTEXSDR_API CortexError cortex_inference_engine_enable_aggressive_memory(CortexInferenceEngineHandle handle, int enable);
/* cortex_sdk.h:158 — bytes of device memory held by uploaded segments. */
CORTEXSDR_API CortexError cortex_inference_engine_get_memory_usage(CortexInferenceEngineHandle handle, size_t* bytes);
CORTEXSDR_API CortexError cortex_inference_engine_enable_layer_prefetch(CortexInferenceEngineHandle handle, int enable);
/* cortex_sdk.h:174 — {"total_ms", "layers":[{"name","load_ms","exec_ms","output_size","used_compressed"}...]}. */
CORTEXSDR_API CortexError cortex_inference_engine_get_last_run_stats_json(CortexInferenceEngineHandle handle, char** out_json);
CORTEXSDR_API void cortex_free_string(char* s);
/* cortex_sdk.h:192 — the archive's 2-D weights in index order, token-major (batch x width). */
CORTEXSDR_API CortexError cortex_inference_engine_run(CortexInferenceEngineHandle handle, const float* input_data,
                                                      size_t input_size, float* output_data, size_t output_size,
                                                      size_t* actual_output_size);
/* cortex_sdk.h:204 — one LINEAR layer: token-major input (batch x C), output (batch x R);
 * the segment is `layer_name` or `layer_name + ".weight"` (SparseInferenceEngine.cpp:1489-1494). */
CORTEXSDR_API CortexError cortex_inference_engine_run_layer(CortexInferenceEngineHandle handle, const char* layer_name,
                                                            const float* input_data, size_t input_size,
                                                            float* output_data, size_t output_size,
                                                            size_t* actual_output_size);
/* cortex_sdk.h:220 — token ids in, token ids out (see above); release with cortex_free_string. */
CORTEXSDR_API CortexError cortex_inference_engine_generate_text(CortexInferenceEngineHandle handle, const char* prompt,
                                                                int max_new_tokens, char** out_text);
CORTEXSDR_API CortexError cortex_inference_engine_free(CortexInferenceEngineHandle handle);
CORTEXSDR_API const char* cortex_sdk_version(void);

#ifdef __cplusplus
}
#endif
#endif
