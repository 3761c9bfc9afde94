// A list of independent decode GEMVs (1-D row-tile segments, at most 4 tokens each) in one
// persistent launch: see gemv_queue.cu.
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
};

// Every item a 1-D row-tile image with cols a multiple of 4, one common batch of 1 to 4 tokens.
bool gemv_queue_supported(const csdr_context* ctx, const QueueItem* items, uint32_t n);
void launch_gemv_queue(csdr_context* ctx, const QueueItem* items, uint32_t n);

}  // namespace csdr
