// The inference-engine functions of the reference's C SDK (api/cortex_sdk.h:110-237),
// same names and signatures, on top of the archive routing in archive.cpp and the
// device-resident decoder in decoder.cu.
//
// What each call does here:
//   create / free         open the .sdr index on a device context; handles live in a registry
//                         and every call checks membership (api/cortex_sdk.cpp:114, :1798)
//   run_layer             one LINEAR layer through the HSDR product (applyLinearLayer route)
//   run                   the archive's 2-D weight segments applied in index order, each
//                         feeding the next, as SDRInferenceEngine::run walks its execution
//                         order (SparseInferenceEngine.cpp:2220, :2911) for a LINEAR-only graph
//   generate_text         the token loop of api/cortex_sdk.cpp:1951-2054 over the transformer
//                         path, with token ids in place of text (the tokenizer is not part of
//                         this library): prompt and result are decimal ids separated by spaces
//   set_batch_size        the batch `run` expects; a mismatch is an argument error
//   set_mode / dropout    recorded; `run` refuses training mode with dropout on (no
//                         stochastic path here), everything else is inference as before
//   init_memory_pool      budget in MiB for cached device images: before a layer runs, images of
//                         other layers are dropped when the budget is exceeded
//   aggressive_memory     drop a layer's device image as soon as the layer has run
//   layer_prefetch        upload the device image of every HSDR segment now
#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdlib>
#include <limits>
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
    size_t batch_size = 0;   // 0: not set, taken from the input size
    bool dropout = false, training = false, aggressive = false, prefetch = false;
    size_t pool_mb = 0;
    struct LayerStat {
        std::string name;
        double load_ms, exec_ms;
        size_t output_size;
        bool used_compressed;
    };
    std::vector<LayerStat> last_stats;
    double last_total_ms = 0.0;
    csdr_decoder* decoder = nullptr;   // built on the first generate_text
    uint32_t decoder_max_seq = 0;
    csdr_decoder_config decoder_cfg{};
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

double ms_since(std::chrono::steady_clock::time_point t0) {
    return std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
}

// A weight the LINEAR route can apply: HSDR-encoded, or stored raw fp32 with 2-D metadata.
bool is_linear_weight(const csdr_segment_header& h) {
    if (h.n_dims != 2) return false;
    if (h.strategy_id == 5) return true;
    return h.strategy_id == 0 && h.compressed_size >= static_cast<uint64_t>(h.dims[0]) * h.dims[1] * 4;
}

// The memory settings, applied before layer `name` runs.
void make_room(CortexInferenceEngine& e, const char* name) {
    if (!e.pool_mb || e.decoder) return;   // a live decoder borrows the archive's images
    size_t held = 0;
    if (csdr_archive_resident_bytes(e.archive, &held) != CSDR_OK) return;
    if (held <= e.pool_mb * (size_t(1) << 20)) return;
    // over budget: keep nothing but what this layer is about to use
    size_t n = 0;
    csdr_archive_num_segments(e.archive, &n);
    for (size_t i = 0; i < n; ++i) {
        csdr_segment_header h{};
        if (csdr_archive_header_at(e.archive, i, &h) == CSDR_OK && std::strcmp(h.name, name) != 0)
            csdr_archive_release(e.archive, h.name);
    }
}

// One LINEAR layer on host buffers, token-major; the reference's route first, the dense
// fallback for raw fp32 weights second (matmulForLayer takes the reference's feature-major
// layout, so batches above one are transposed around it).
int apply_layer(CortexInferenceEngine& e, const char* layer, const float* in, size_t n_in, float* out, size_t cap,
                size_t* n_out, bool* compressed) {
    make_room(e, layer);
    int rc = csdr_archive_apply_linear(e.archive, layer, in, n_in, nullptr, out, cap, n_out);
    *compressed = true;
    if (rc == CSDR_ERR_STRATEGY) {
        csdr_segment_header h{};
        std::string name = layer;
        if (csdr_archive_find(e.archive, name.c_str(), &h) != CSDR_OK) {
            name += ".weight";
            if (csdr_archive_find(e.archive, name.c_str(), &h) != CSDR_OK) return CSDR_ERR_NOT_FOUND;
        }
        if (!is_linear_weight(h)) return rc;
        *compressed = false;
        const size_t C = h.dims[1], R = h.dims[0];
        if (!n_in || n_in % C) {
            csdr::set_last_error("input size is not a multiple of the layer's input width");
            return CSDR_ERR_INVALID_ARG;
        }
        const size_t batch = n_in / C;
        *n_out = batch * R;
        if (cap < batch * R) return CSDR_ERR_BUFFER;
        if (batch == 1) {
            rc = csdr_archive_matmul_for_layer(e.archive, name.c_str(), in, 1, out, cap, n_out);
        } else {
            std::vector<float> xt(n_in), yt(batch * R);
            for (size_t b = 0; b < batch; ++b)
                for (size_t c = 0; c < C; ++c) xt[c * batch + b] = in[b * C + c];
            rc = csdr_archive_matmul_for_layer(e.archive, name.c_str(), xt.data(), batch, yt.data(), yt.size(), n_out);
            if (rc == CSDR_OK)
                for (size_t b = 0; b < batch; ++b)
                    for (size_t r = 0; r < R; ++r) out[b * R + r] = yt[r * batch + b];
        }
    }
    if (rc == CSDR_OK && e.aggressive && !e.decoder) {
        csdr_archive_release(e.archive, layer);
        csdr_archive_release(e.archive, (std::string(layer) + ".weight").c_str());
    }
    return rc;
}

// Decoder shape from the archive's own headers, the way the reference discovers it: blocks by
// their GGUF-style names (api/cortex_sdk.cpp:488-524), the head size by the preference list of
// infer_attention_layout (:1335-1349), eps and theta at the reference's defaults (:1212, :1358).
bool discover_decoder(csdr_archive* ar, csdr_decoder_config* cfg, std::string* why) {
    csdr_segment_header h{};
    auto dims2 = [&](const std::string& name, uint32_t* r, uint32_t* c) {
        if (csdr_archive_find(ar, name.c_str(), &h) != CSDR_OK || h.n_dims != 2) return false;
        *r = h.dims[0];
        *c = h.dims[1];
        return true;
    };
    uint32_t vocab = 0, hidden = 0;
    if (!dims2("token_embd.weight", &vocab, &hidden)) {
        *why = "archive has no 2-D token_embd.weight";
        return false;
    }
    uint32_t layers = 0;
    while (csdr_archive_find(ar, ("blk." + std::to_string(layers) + ".attn_q.weight").c_str(), &h) == CSDR_OK) ++layers;
    if (!layers) {
        *why = "archive has no transformer blocks (blk.<n>.attn_q.weight)";
        return false;
    }
    uint32_t qd = 0, kd = 0, vd = 0, inter = 0, c = 0;
    if (!dims2("blk.0.attn_q.weight", &qd, &c) || !dims2("blk.0.attn_k.weight", &kd, &c) ||
        !dims2("blk.0.attn_v.weight", &vd, &c) || !dims2("blk.0.ffn_gate.weight", &inter, &c)) {
        *why = "block 0 lacks a 2-D attn_q/attn_k/attn_v/ffn_gate weight";
        return false;
    }
    uint32_t head_dim = 0;
    for (uint32_t hd : {128u, 64u, 256u, 32u, 16u}) {
        if (qd % hd || kd % hd || vd % hd) continue;
        const uint32_t qh = qd / hd, kh = kd / hd, vh = vd / hd;
        if (!qh || !kh || !vh || qh < kh || qh < vh || qh % kh || qh % vh) continue;
        head_dim = hd;
        break;
    }
    if (!head_dim || kd != vd) {
        *why = "no head size in {128, 64, 256, 32, 16} fits the q/k/v widths";
        return false;
    }
    *cfg = csdr_decoder_config{};
    cfg->n_layers = layers;
    cfg->hidden = hidden;
    cfg->q_heads = qd / head_dim;
    cfg->kv_heads = kd / head_dim;
    cfg->head_dim = head_dim;
    cfg->inter = inter;
    cfg->vocab = vocab;
    cfg->max_batch = 1;
    cfg->rms_eps = 1e-5f;
    cfg->rope_theta = 1e6f;
    cfg->tp_rank = 0;
    cfg->tp_size = 1;
    return true;
}

// select_best_from_logits, api/cortex_sdk.cpp:1005-1030.
int select_best(const std::vector<float>& logits, const std::unordered_set<int>& produced, float temperature) {
    const float temp_scale = temperature > 0.0f ? (1.0f / temperature) : 1.0f;
    float best = -std::numeric_limits<float>::infinity();
    int tok = -1;
    for (size_t t = 0; t < logits.size(); ++t) {
        float score = logits[t] * temp_scale;
        if (!std::isfinite(score)) continue;
        if (produced.count(static_cast<int>(t))) score -= 1.5f;
        if (score > best) {
            best = score;
            tok = static_cast<int>(t);
        }
    }
    return tok;
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
    return with_engine(h, [&](CortexInferenceEngine& e) { e.batch_size = n; return ok(); });
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
    return with_engine(h, [&](CortexInferenceEngine& e) {
        e.prefetch = v != 0;
        if (!e.prefetch) return ok();
        size_t n = 0;
        csdr_archive_num_segments(e.archive, &n);
        for (size_t i = 0; i < n; ++i) {
            csdr_segment_header hd{};
            if (csdr_archive_header_at(e.archive, i, &hd) != CSDR_OK || hd.strategy_id != 5) continue;
            const csdr_segment* seg = nullptr;
            const int rc = csdr_archive_segment(e.archive, hd.name, &seg);
            if (rc) return from_status(rc);
        }
        return ok();
    });
}

CORTEXSDR_API CortexError cortex_inference_engine_get_memory_usage(CortexInferenceEngineHandle h, size_t* bytes) {
    return with_engine(h, [&](CortexInferenceEngine& e) {
        if (!bytes) return fail(CORTEX_B200_ERROR_INVALID_ARGUMENT, "Invalid arguments (null pointers)");
        return from_status(csdr_archive_resident_bytes(e.archive, bytes));
    });
}

CORTEXSDR_API CortexError cortex_inference_engine_get_last_run_stats_json(CortexInferenceEngineHandle h, char** out) {
    return with_engine(h, [&](CortexInferenceEngine& e) {
        if (!out) return fail(CORTEX_B200_ERROR_INVALID_ARGUMENT, "Invalid argument(s)");
        std::ostringstream js;   // field for field the reference's shape, api/cortex_sdk.cpp:2069-2080
        js << "{\"total_ms\": " << e.last_total_ms << ", \"layers\": [";
        for (size_t i = 0; i < e.last_stats.size(); ++i) {
            const auto& s = e.last_stats[i];
            js << "{\"name\":\"" << s.name << "\",\"load_ms\":" << s.load_ms << ",\"exec_ms\":" << s.exec_ms
               << ",\"output_size\":" << s.output_size << ",\"used_compressed\":" << (s.used_compressed ? "true" : "false")
               << "}";
            if (i + 1 < e.last_stats.size()) js << ",";
        }
        js << "]}";
        const std::string str = js.str();
        char* buf = static_cast<char*>(std::malloc(str.size() + 1));
        if (!buf) return fail(CORTEX_B200_ERROR_MEMORY, "Allocation failure");
        std::memcpy(buf, str.c_str(), str.size() + 1);
        *out = buf;
        return ok();
    });
}

CORTEXSDR_API void cortex_free_string(char* s) { std::free(s); }

CORTEXSDR_API CortexError cortex_inference_engine_run(CortexInferenceEngineHandle h, const float* in, size_t n_in,
                                                      float* out, size_t cap, size_t* actual) {
    return with_engine(h, [&](CortexInferenceEngine& e) {
        if (!in || !out || !actual) return fail(CORTEX_B200_ERROR_INVALID_ARGUMENT, "Invalid arguments (null pointers)");
        if (e.training && e.dropout)
            return fail(CORTEX_B200_ERROR_UNSUPPORTED_FORMAT, "training mode with dropout is not part of this library");
        size_t n = 0;
        csdr_archive_num_segments(e.archive, &n);
        std::vector<float> cur(in, in + n_in), next;
        std::vector<CortexInferenceEngine::LayerStat> stats;
        const auto t_all = std::chrono::steady_clock::now();
        bool first = true;
        for (size_t i = 0; i < n; ++i) {
            csdr_segment_header hd{};
            if (csdr_archive_header_at(e.archive, i, &hd) != CSDR_OK || !is_linear_weight(hd)) continue;
            const size_t C = hd.dims[1], R = hd.dims[0];
            if (cur.empty() || cur.size() % C)
                return fail(CORTEX_B200_ERROR_INFERENCE, std::string("layer '") + hd.name + "' takes " + std::to_string(C) +
                                                             " inputs per sample; got " + std::to_string(cur.size()));
            if (first && e.batch_size && cur.size() / C != e.batch_size)
                return fail(CORTEX_B200_ERROR_INVALID_ARGUMENT, "input size does not match the batch size set on the engine");
            first = false;
            next.assign(cur.size() / C * R, 0.0f);
            size_t got = 0;
            bool compressed = false;
            const std::string name = hd.name;   // the header's strings die with a release
            const auto t0 = std::chrono::steady_clock::now();
            const int rc = apply_layer(e, name.c_str(), cur.data(), cur.size(), next.data(), next.size(), &got, &compressed);
            if (rc) return from_status(rc);
            stats.push_back({name, 0.0, ms_since(t0), got, compressed});
            cur.swap(next);
        }
        if (first) return fail(CORTEX_B200_ERROR_INFERENCE, "archive holds no 2-D weight this library can apply");
        *actual = cur.size();
        if (cur.size() > cap) return fail(CORTEX_B200_ERROR_MEMORY, "Output buffer too small");
        std::memcpy(out, cur.data(), cur.size() * 4);
        e.last_stats = std::move(stats);
        e.last_total_ms = ms_since(t_all);
        return ok();
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
        bool compressed = false;
        const int rc = apply_layer(e, layer, in, n_in, out, cap, &n, &compressed);
        *actual = n;
        if (rc) return from_status(rc);
        e.last_total_ms = ms_since(t0);
        e.last_stats.assign(1, {layer, 0.0, e.last_total_ms, n, compressed});
        return ok();
    });
}

CORTEXSDR_API CortexError cortex_inference_engine_generate_text(CortexInferenceEngineHandle h, const char* prompt,
                                                                int max_new_tokens, char** out_text) {
    return with_engine(h, [&](CortexInferenceEngine& e) {
        if (!prompt || !out_text) return fail(CORTEX_B200_ERROR_INVALID_ARGUMENT, "Invalid argument(s)");
        // the prompt: decimal token ids separated by blanks or commas
        std::vector<int32_t> ids;
        for (const char* p = prompt; *p;) {
            if (*p == ' ' || *p == ',' || *p == '\t' || *p == '\n') {
                ++p;
                continue;
            }
            char* end = nullptr;
            const long v = std::strtol(p, &end, 10);
            if (end == p || v < 0)
                return fail(CORTEX_B200_ERROR_INVALID_ARGUMENT,
                            "this library has no tokenizer: the prompt must be decimal token ids separated by blanks");
            ids.push_back(static_cast<int32_t>(v));
            p = end;
        }
        if (ids.empty()) return fail(CORTEX_B200_ERROR_INFERENCE, "Prompt tokenization produced no tokens");
        const int step_limit = std::max(1, max_new_tokens);
        const uint32_t need_seq = static_cast<uint32_t>(ids.size()) + static_cast<uint32_t>(step_limit) + 1u;
        if (!e.decoder || e.decoder_max_seq < need_seq) {
            if (e.decoder) csdr_decoder_destroy(e.decoder);
            e.decoder = nullptr;
            std::string why;
            if (!discover_decoder(e.archive, &e.decoder_cfg, &why)) return fail(CORTEX_B200_ERROR_INFERENCE, why);
            e.decoder_cfg.max_seq = std::max<uint32_t>(need_seq, 256u);
            const int rc = csdr_decoder_create(e.archive, &e.decoder_cfg, &e.decoder);
            if (rc) return from_status(rc);
            e.decoder_max_seq = e.decoder_cfg.max_seq;
        }
        int rc = csdr_decoder_reset(e.decoder);
        if (rc) return from_status(rc);
        std::vector<float> logits(e.decoder_cfg.vocab);
        std::vector<int> generated;
        std::unordered_set<int> produced;    // the transformer path penalises generated tokens only (:1999-2001)
        const float temperature = 0.8f;      // :2011
        rc = csdr_decoder_forward(e.decoder, 0, ids.data(), ids.size(), logits.data(), nullptr);
        if (rc) return from_status(rc);
        for (int step = 0; step < step_limit; ++step) {
            const int tok = select_best(logits, produced, temperature);
            if (tok < 0) return fail(CORTEX_B200_ERROR_INFERENCE, "Failed to sample next token");
            generated.push_back(tok);
            produced.insert(tok);
            if (step + 1 == step_limit) break;
            const int32_t t32 = tok;
            rc = csdr_decoder_forward(e.decoder, 0, &t32, 1, logits.data(), nullptr);
            if (rc) return from_status(rc);
        }
        std::string text;
        for (size_t i = 0; i < generated.size(); ++i) text += (i ? " " : "") + std::to_string(generated[i]);
        char* buf = static_cast<char*>(std::malloc(text.size() + 1));
        if (!buf) return fail(CORTEX_B200_ERROR_MEMORY, "Allocation failure");
        std::memcpy(buf, text.c_str(), text.size() + 1);
        *out_text = buf;
        return ok();
    });
}

CORTEXSDR_API CortexError cortex_inference_engine_free(CortexInferenceEngineHandle h) {
    CortexInferenceEngine* e = lookup(h);
    if (!e) return fail(CORTEX_B200_ERROR_INVALID_ARGUMENT, "Invalid handle");
    {
        std::lock_guard<std::mutex> lk(g_mu);
        g_engines.erase(e);
    }
    if (e->decoder) csdr_decoder_destroy(e->decoder);
    csdr_archive_close(e->archive);
    csdr_context_destroy(e->ctx);
    delete e;
    return ok();
}

CORTEXSDR_API const char* cortex_sdk_version(void) { return "1.0.0-b200"; }

}  // extern "C"
