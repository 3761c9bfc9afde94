// Tensor-core (tcgen05 / TMEM) path for wide token tiles of 1-D row-tile HSDR segments.
#pragma once

#include <cuda_bf16.h>

#include <cstddef>
#include <cstdint>

struct csdr_context;
struct csdr_segment;

namespace csdr {

struct MatmulArgs;

// 1-D row tiles, n_atoms a multiple of 128, cols a multiple of 64, batch at least the
// context's tensor-core threshold.
bool tcgen05_supported(const csdr_context* ctx, const csdr_segment* seg, size_t batch);

// The whole batch in one pass: projection on the tensor cores, column-split reduction, gather.
void launch_matmul_tcgen05(csdr_context* ctx, const csdr_segment* seg, const MatmulArgs& a);

// TMA-fed projection (gemm_tma.cu): Dx [n_atoms][dx_stride >= batch] for the whole batch in one
// launch, from bf16 dictionary planes that are built on the first call and cached with the
// dictionary.
bool dx_tma_supported(const csdr_context* ctx, const csdr_segment* seg, size_t batch);
void launch_dx_tma(csdr_context* ctx, const csdr_segment* seg, const MatmulArgs& a, float* dx, uint32_t dx_stride);
// Builds and caches the bf16 planes of the segment's dictionary now (they are otherwise built
// on the first projection); afterwards the fp32 atoms are no longer read by the TMA kernel.
void dx_tma_prepare(csdr_context* ctx, const csdr_segment* seg);


// Activations as token-major bf16 planes [tokens][cols]: hi = bf16(x), lo = bf16(x - hi); lo is
// null when the source was bf16 already.
struct XPlanesView {
    const __nv_bfloat16* hi;
    const __nv_bfloat16* lo;
};
// Planes of a caller's activation matrix: the matrix itself when it is bf16, token-major and
// 16-byte aligned, else a conversion into context scratch (valid until the next conversion).
XPlanesView make_x_planes(csdr_context* ctx, const void* x, int x_dtype, int x_layout, uint32_t M, uint32_t cols);
struct Exchange;
struct NormShares;
// One projection launch for up to four dictionaries over the same activations (q|k|v, gate|up).
// With an exchange (tensor parallelism, at most 16 tokens) the finished rows go into every
// rank's slot for this rank, at the offsets dx[i] - blk_base, `sums` (this rank's per-token sums
// of squares, or null) ride along at offset 0, and the launch's last CTA raises the flags: the
// projection and its share of the collective are one kernel. transposed (one dictionary, no
// exchange): Dx leaves token-major, [token][atom] with dx_stride floats between token rows.
// shares: see NextNorm.
void launch_dx_tma_group(csdr_context* ctx, const csdr_segment* const* segs, uint32_t n_seg, XPlanesView x, uint32_t M,
                         float* const* dx, uint32_t dx_stride, const Exchange* xch, const float* blk_base,
                         const float* sums, bool transposed = false, const NormShares* shares = nullptr);

// Up to four row-tile segments over the same activation planes: one projection launch and, for
// a single token tile (M <= 16), one gather launch for the whole group. y = W x (+ bias)
// (+ residual, which may be y itself).
struct WideOut {
    float* y;
    const float* bias;
    const float* residual;
};
// Per-token factor applied by the gather before bias and residual: 1 / sqrt(sumsq[t] * inv_width
// + eps). With activations w*h (not yet normalised) this is the RMS normalisation of h moved
// behind the product; sumsq == nullptr means no factor.
struct TokenScale {
    const float* sumsq = nullptr;
    float inv_width = 0.0f;
    float eps = 0.0f;
};
// The first half of the NEXT RMS normalisation, riding on a one-member gather over a single token
// tile: beside y the gather writes the bf16 planes of w * y (what the next projection reads) and
// every CTA leaves its share of the per-token sums of y^2 in `partial`. The projection launch
// behind the gather gets the shares as NormShares and one of its CTAs adds them up, in CTA order
// (so the sums do not depend on any order of arrival), into `sumsq`, where the gather behind that
// projection finds them and turns them into 1 / rms.
constexpr uint32_t kNextNormCtas = 1024;
struct NextNorm {
    const float* w = nullptr;       // the next norm's weights, one per row of y
    __nv_bfloat16* hi = nullptr;    // planes of w * y, laid out like y (token-major)
    __nv_bfloat16* lo = nullptr;
    float* partial = nullptr;       // [kNextNormCtas][16] shares, one row per CTA of the gather
};
struct NormShares {
    const float* partial = nullptr;
    uint32_t ctas = 0;              // CTAs of the gather that left shares
    float* sumsq = nullptr;         // [tokens]
};
// Where a group's projections live between the two launches: member i at dx[i], rows `stride`
// floats apart, `floats` in all from `base` (one contiguous block, so that tensor-parallel
// ranks can sum their partial projections with one collective over it).
struct WideDx {
    float* base;
    float* dx[4];
    size_t floats;
    uint32_t stride, tile_mt;
};
// Exchange of partial projections between tensor-parallel ranks through peer memory (one
// process per GPU, regions mapped into each other with CUDA IPC). Every rank owns a region of
// 2 (parity) x ranks slots of `blk_floats` floats plus 2 x ranks flag words. A rank's projection
// kernel stores its finished rows into slot [parity][its rank] of EVERY rank's region (plain peer
// stores), and its last CTA stores the exchange's sequence number into the matching flag word of
// every region. A small launch on each rank waits (bounded) for all flags of the parity to show
// the number and sums the slots in rank order into the local block the gather reads. Two
// parities: a rank can run at most one exchange ahead of a peer, because its next reduce launch
// needs that peer's next push. The sequence number lives in device
// memory and is advanced by the projection kernel, so a captured CUDA graph replays correctly.
constexpr uint32_t kMaxExchangeRanks = 8;
struct Exchange {
    uint32_t ranks = 0;            // 0 or 1: no exchange
    uint32_t rank = 0;
    uint32_t blk_floats = 0;
    float* slots[kMaxExchangeRanks] = {};       // every rank's slot area (index = owner), [2][ranks][blk_floats]
    uint32_t* flags[kMaxExchangeRanks] = {};    // every rank's flag words, [2][ranks]
    uint32_t* seq = nullptr;       // this rank's sequence counter (device)
    uint32_t* done = nullptr;      // this rank's count of finished CTAs of the projection kernel (device)
    int* status = nullptr;         // context status word: a wait that ran out is recorded here
};
// The two halves of launch_matmul_wide_group. dx_base == nullptr: context scratch.
WideDx launch_wide_project(csdr_context* ctx, const csdr_segment* const* segs, uint32_t n, XPlanesView x, uint32_t M,
                           float* dx_base, const Exchange* xch = nullptr, const float* blk_base = nullptr,
                           const float* sums = nullptr, const NormShares* shares = nullptr);
// Returns the number of CTAs that left shares when `next` was given and rode on the gather (one
// member, single token tile, token-major y); 0 leaves the next norm's first half to the caller.
uint32_t launch_wide_gather(csdr_context* ctx, const csdr_segment* const* segs, uint32_t n, const WideDx& w, uint32_t M,
                        const WideOut* outs, int y_layout, const TokenScale& ts, const NextNorm* next = nullptr);
// Receiving side of the exchange: one small launch waits for every rank's flag and adds the
// ranks' slots up, in rank order, over block range [off_floats, off_floats + floats) into the
// local block at dst; the gather behind it reads the sum like any local projection.
void launch_exchange_reduce(csdr_context* ctx, const Exchange& x, uint32_t off_floats, size_t floats, float* dst);
// (gate, up) of a SwiGLU block over at most 16 tokens: one gather launch that writes
// silu(gate) * up, token-major, as bf16 planes for the down projection.
void launch_wide_gather_swiglu(csdr_context* ctx, const csdr_segment* const* gate_up, const WideDx& w, uint32_t M,
                               const TokenScale& ts, __nv_bfloat16* act_hi, __nv_bfloat16* act_lo);
bool wide_group_supported(const csdr_context* ctx, const csdr_segment* const* segs, uint32_t n, size_t batch);
void launch_matmul_wide_group(csdr_context* ctx, const csdr_segment* const* segs, uint32_t n, XPlanesView x,
                              uint32_t M, const WideOut* outs, int y_layout);

}  // namespace csdr
