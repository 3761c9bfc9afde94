// TEST INFRASTRUCTURE ONLY — never linked into, loaded by, or shipped with the product library.
//
// A second extern "C" face over the UNMODIFIED reference sources, this one over its inference
// engine's translation units (compiled where they lie; see oracle/Makefile, target ref_engine):
//   SDRModelLoader::loadLayerByName      SparseInferenceEngine.cpp (weights of a layer as the
//                                        inference side decodes them: stored-raw tensors in a
//                                        source dtype go through decodeSupportedGGUFQuantized,
//                                        :276-469)
// It pins the oracle's restatement of that decode (orc_dequantize_inference).
#include "ai_compression/SparseInferenceEngine.hpp"

#include <cstring>
#include <string>

using namespace CortexAICompression;

namespace {
thread_local std::string g_err;
}

extern "C" {

const char* ref_engine_last_error() { return g_err.c_str(); }

// fp32 weights of layer `name` of the .sdr at `path`, as SDRModelLoader hands them to the
// interpreter. *n receives the element count; returns 0, or -1 with a message.
int ref_engine_layer_weights(const char* path, const char* name, float* out, size_t capacity, size_t* n) {
    try {
        SDRModelLoader loader(path);
        LayerInfo layer = loader.loadLayerByName(name);
        if (n) *n = layer.weights.size();
        if (out) {
            if (capacity < layer.weights.size()) {
                g_err = "buffer too small";
                return -1;
            }
            std::memcpy(out, layer.weights.data(), layer.weights.size() * sizeof(float));
        }
        return 0;
    } catch (const std::exception& e) {
        g_err = e.what();
        return -1;
    }
}

}  // extern "C"
