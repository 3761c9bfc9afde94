// The inference-engine functions of the reference's C SDK (api/cortex_sdk.h:110-237),
// same names and signatures, on top of the archive routing in archive.cpp.
#include <chrono>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <sstream>
#include <string>
#include <unordered_set>
#include <vector>

#include "../../../include/cortex_sdk_b200.h"
#include "../internal.hpp"

struct CortexInferenceEngine {
    csdr_context* ctx = nullptr;
    csdr_archive* archive = nullptr;
    size_t batch_size = 1;
    bool dropout = false, training = false, aggressive = false, prefetch = false;
    size_t pool_mb = 0;
    struct LayerStat {
        std::string name;
        double exec_ms;
        bool used_compressed;
    };
    std::vector<LayerStat> last_stats;
};

namespace {

std::mutex g_mu;
std::unordered_set<CortexInferenceEngine*> g_engines;  // api/cortex_sdk.cpp:114
thread_local std::string g_msg;

CortexError ok() { return {nullptr, CORTEX_B200_SUCCESS}; }

CortexError fail(int code, const std::string& msg) {
    g_msg = msg;
    return {g_msg.c_str(), code};
}

CortexError from_status(int rc) {
    switch (rc) {
        case CSDR_OK: return ok();
        case CSDR_ERR_INVALID_ARG: return fail(CORTEX_B200_ERROR_INVALID_ARGUMENT, csdr_last_error());
        case CSDR_ERR_IO: return fail(CORTEX_B200_ERROR_FILE_IO, csdr_last_error());
        case CSDR_ERR_BUFFER: return fail(CORTEX_B200_ERROR_MEMORY, "Output buffer too small");
        case CSDR_ERR_FORMAT:
        case CSDR_ERR_CODE_RANGE: return fail(CORTEX_B200_ERROR_DECOMPRESSION, csdr_last_error());
        case CSDR_ERR_UNSUPPORTED: return fail(CORTEX_B200_ERROR_UNSUPPORTED_FORMAT, csdr_last_error());
        default: return fail(CORTEX_B200_ERROR_INFERENCE, csdr_last_error());
    }
}

CortexInferenceEngine* lookup(CortexInferenceEngineHandle h) {
    std::lock_guard<std::mutex> lk(g_mu);
    return (h && g_engines.count(h)) ? h : nullptr;
}

template <typename F>
CortexError with_engine(CortexInferenceEngineHandle h, F&& f) {
    try {
        CortexInferenceEngine* e = lookup(h);
        if (!e) return fail(CORTEX_B200_ERROR_INVALID_ARGUMENT, "Invalid handle");
        return f(*e);
    } catch (const std::exception& ex) {
        return fail(CORTEX_B200_ERROR_UNKNOWN, ex.what());
    } catch (...) {
        return fail(CORTEX_B200_ERROR_UNKNOWN, "unknown error");
    }
}

}  // namespace

extern "C" {

CORTEXSDR_API CortexError cortex_inference_engine_create(const char* path,
                                                         CortexInferenceEngineHandle* handle) {
    try {
        if (!path || !handle) return fail(CORTEX_B200_ERROR_INVALID_ARGUMENT, "Invalid arguments (null pointers)");
        auto e = std::make_unique<CortexInferenceEngine>();
        int rc = csdr_context_create(-1, nullptr, &e->ctx);
        if (rc) return from_status(rc);
        rc = csdr_archive_open(e->ctx, path, &e->archive);
        if (rc) {
            csdr_context_destroy(e->ctx);
            return from_status(rc);
        }
        std::lock_guard<std::mutex> lk(g_mu);
        g_engines.insert(e.get());
        *handle = e.release();
        return ok();
    } catch (const std::exception& ex) {
        return fail(CORTEX_B200_ERROR_UNKNOWN, ex.what());
    }
}

CORTEXSDR_API CortexError cortex_inference_engine_set_batch_size(CortexInferenceEngineHandle h, size_t n) {
    return with_engine(h, [&](CortexInferenceEngine& e) { e.batch_size = n ? n : 1; return ok(); });
}
CORTEXSDR_API CortexError cortex_inference_engine_enable_dropout(CortexInferenceEngineHandle h, int v) {
    return with_engine(h, [&](CortexInferenceEngine& e) { e.dropout = v != 0; return ok(); });
}
CORTEXSDR_API CortexError cortex_inference_engine_set_mode(CortexInferenceEngineHandle h, int v) {
    return with_engine(h, [&](CortexInferenceEngine& e) { e.training = v != 0; return ok(); });
}
CORTEXSDR_API CortexError cortex_inference_engine_init_memory_pool(CortexInferenceEngineHandle h, size_t mb) {
    return with_engine(h, [&](CortexInferenceEngine& e) { e.pool_mb = mb; return ok(); });
}
CORTEXSDR_API CortexError cortex_inference_engine_enable_aggressive_memory(CortexInferenceEngineHandle h, int v) {
    return with_engine(h, [&](CortexInferenceEngine& e) { e.aggressive = v != 0; return ok(); });
}
CORTEXSDR_API CortexError cortex_inference_engine_enable_layer_prefetch(CortexInferenceEngineHandle h, int v) {
    return with_engine(h, [&](CortexInferenceEngine& e) { e.prefetch = v != 0; return ok(); });
}

CORTEXSDR_API CortexError cortex_inference_engine_get_memory_usage(CortexInferenceEngineHandle h, size_t* bytes) {
    return with_engine(h, [&](CortexInferenceEngine& e) {
        if (!bytes) return fail(CORTEX_B200_ERROR_INVALID_ARGUMENT, "Invalid arguments (null pointers)");
        size_t free_b = 0, total_b = 0;
        cudaSetDevice(e.ctx->device);
        if (cudaMemGetInfo(&free_b, &total_b) != cudaSuccess) return fail(CORTEX_B200_ERROR_INFERENCE, "cudaMemGetInfo failed");
        *bytes = total_b - free_b;
        return ok();
    });
}

CORTEXSDR_API CortexError cortex_inference_engine_get_last_run_stats_json(CortexInferenceEngineHandle h, char** out) {
    return with_engine(h, [&](CortexInferenceEngine& e) {
        if (!out) return fail(CORTEX_B200_ERROR_INVALID_ARGUMENT, "Invalid arguments (null pointers)");
        std::ostringstream js;
        js << "{\"layers\":[";
        for (size_t i = 0; i < e.last_stats.size(); ++i) {
            const auto& s = e.last_stats[i];
            js << (i ? "," : "") << "{\"name\":\"" << s.name << "\",\"load_ms\":0,\"exec_ms\":" << s.exec_ms
               << ",\"used_compressed\":" << (s.used_compressed ? "true" : "false") << "}";
        }
        js << "]}";
        const std::string str = js.str();
        char* buf = static_cast<char*>(std::malloc(str.size() + 1));
        if (!buf) return fail(CORTEX_B200_ERROR_MEMORY, "out of memory");
        std::memcpy(buf, str.c_str(), str.size() + 1);
        *out = buf;
        return ok();
    });
}

CORTEXSDR_API void cortex_free_string(char* s) { std::free(s); }

CORTEXSDR_API CortexError cortex_inference_engine_run(CortexInferenceEngineHandle h, const float*, size_t, float*,
                                                      size_t, size_t*) {
    return with_engine(h, [&](CortexInferenceEngine&) {
        return fail(CORTEX_B200_ERROR_UNSUPPORTED_FORMAT,
                    "whole-graph execution is not part of this library; call "
                    "cortex_inference_engine_run_layer per LINEAR layer");
    });
}

CORTEXSDR_API CortexError cortex_inference_engine_run_layer(CortexInferenceEngineHandle h, const char* layer,
                                                            const float* in, size_t n_in, float* out,
                                                            size_t cap, size_t* actual) {
    return with_engine(h, [&](CortexInferenceEngine& e) {
        if (!layer || !in || !out || !actual)
            return fail(CORTEX_B200_ERROR_INVALID_ARGUMENT, "Invalid arguments (null pointers)");
        const auto t0 = std::chrono::steady_clock::now();
        size_t n = 0;
        const int rc = csdr_archive_apply_linear(e.archive, layer, in, n_in, nullptr, out, cap, &n);
        *actual = n;
        if (rc) return from_status(rc);
        const double ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
        e.last_stats.assign(1, {layer, ms, true});
        return ok();
    });
}

CORTEXSDR_API CortexError cortex_inference_engine_generate_text(CortexInferenceEngineHandle h, const char*, int,
                                                                char**) {
    return with_engine(h, [&](CortexInferenceEngine&) {
        return fail(CORTEX_B200_ERROR_UNSUPPORTED_FORMAT,
                    "text generation needs the reference's tokenizer and sampling policy, which are "
                    "not part of this library; drive csdr_decoder_* with token ids instead");
    });
}

CORTEXSDR_API CortexError cortex_inference_engine_free(CortexInferenceEngineHandle h) {
    CortexInferenceEngine* e = lookup(h);
    if (!e) return fail(CORTEX_B200_ERROR_INVALID_ARGUMENT, "Invalid handle");
    {
        std::lock_guard<std::mutex> lk(g_mu);
        g_engines.erase(e);
    }
    csdr_archive_close(e->archive);
    csdr_context_destroy(e->ctx);
    delete e;
    return ok();
}

CORTEXSDR_API const char* cortex_sdk_version(void) { return "1.0.0-b200"; }

}  // extern "C"
