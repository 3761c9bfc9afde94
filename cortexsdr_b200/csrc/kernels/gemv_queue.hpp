// A list of decode GEMVs (1-D row-tile segments, at most 4 tokens each) in one persistent launch,
// with the decoder's glue folded into the gather as per-task epilogues: see gemv_queue.cu.
#pragma once

#include <cstddef>
#include <cstdint>

struct csdr_context;
struct csdr_segment;

namespace csdr {

constexpr uint32_t kMaxQueueTasks = 32;   // per launch; longer lists take several launches

struct QueueItem {
    const csdr_segment* seg;
    const void* x;          // device activations of this product
    int x_dtype, x_layout;
    size_t batch;           // the same for every item of a list
    float* y;               // device, fp32
    int y_layout;
    const float* bias;      // device, R floats, or null
    // ---- optional glue (token-major fp32 buffers of [batch][rows]) ----
    const float* residual = nullptr;     // y = W x + residual (may be y itself)
    const float* swiglu_gate = nullptr;  // y = silu(gate) * (W x); gate = y of the task just before, same rows
    int dep = -1;                        // index of the earlier task whose y is this task's x (x == that y)
    const float* norm_weight = nullptr;  // with dep: y = W rmsnorm(x; norm_weight, norm_eps)
    float norm_eps = 0.0f;
};

// Every item a 1-D row-tile image with cols a multiple of 4, one common batch of 1 to 4 tokens;
// dep points backwards within the same group of kMaxQueueTasks.
bool gemv_queue_supported(const csdr_context* ctx, const QueueItem* items, uint32_t n);
void launch_gemv_queue(csdr_context* ctx, const QueueItem* items, uint32_t n);

}  // namespace csdr
