// Device kernels for the decoder-layer glue around the compressed matmul. Activations are
// fp32, token-major (tokens x features), as in the reference's driver
// (api/cortex_sdk.cpp:1543-1696). What each kernel restates:
//   rmsnorm_kernel        rms_norm, api/cortex_sdk.cpp:1208-1232
//   rope_cache_kernel     get_rope_cache + apply_rope_inplace, :1363-1423 (adjacent pairs
//                         (2i, 2i+1), freq = theta^(-2i/head_dim)), then the K/V cache write
//   attention_kernel      repeat_kv_heads :1453-1478 + multi_head_attention(causal)
//                         kernels/attention_kernels.cpp:26-113 + softmax simd_kernels.cpp:198-217
//   silu_mul_kernel       silu_mul, :1245-1256
//   add_kernel            add_vectors, :1234-1243
//   argmax_kernel         greedy pick over the logits row
#include <cooperative_groups.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <cfloat>
#include <type_traits>

#include "../internal.hpp"
#include "decoder_ops.hpp"

namespace csdr {

namespace {

// bf16 planes of an fp32 value for the tensor-core projection: hi = bf16(v), lo = bf16(v - hi).
__device__ __forceinline__ void store_planes(__nv_bfloat16* hi, __nv_bfloat16* lo, size_t i, float v) {
    const __nv_bfloat16 h = __float2bfloat16_rn(v);
    hi[i] = h;
    lo[i] = __float2bfloat16_rn(v - __bfloat162float(h));
}

// Every glue kernel lets the kernel behind it on the stream start its own prologue at once and
// then waits until everything before it on the stream has completed and is visible; no global
// memory is touched before that wait.
__device__ __forceinline__ void pdl_enter() {
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

// Launch with programmatic stream serialization allowed (the kernel must begin with pdl_enter()).
template <typename... KArgs, typename... Args>
void launch_pdl(csdr_context* ctx, void (*kern)(KArgs...), dim3 grid, dim3 block, Args... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = 0;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = ctx->pdl ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    CSDR_CUDA(cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...));
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, off);
    return v;
}

// One CTA per token.
__global__ void __launch_bounds__(256)
rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ w, uint32_t H, float eps,
               float* __restrict__ out, __nv_bfloat16* __restrict__ hi, __nv_bfloat16* __restrict__ lo) {
    pdl_enter();
    __shared__ float red[8];
    __shared__ float inv_s;
    const float* src = x + static_cast<size_t>(blockIdx.x) * H;
    float* dst = out + static_cast<size_t>(blockIdx.x) * H;
    float ss = 0.0f;
    for (uint32_t i = threadIdx.x; i < H; i += 256) ss = fmaf(src[i], src[i], ss);
    ss = warp_sum(ss);
    if ((threadIdx.x & 31u) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) t += red[i];
        inv_s = 1.0f / sqrtf(t / static_cast<float>(H) + eps);
    }
    __syncthreads();
    const float inv = inv_s;
    if (hi) {
        const size_t o = static_cast<size_t>(blockIdx.x) * H;
        for (uint32_t i = threadIdx.x; i < H; i += 256) store_planes(hi, lo, o + i, src[i] * inv * w[i]);
    } else {
        for (uint32_t i = threadIdx.x; i < H; i += 256) dst[i] = src[i] * inv * w[i];
    }
}

// hidden += delta, then out = rmsnorm(hidden) — the residual add and the next norm in one pass.
// Planes of w * x (not normalised) plus each token's sum of squares over this slice of the
// hidden width: the normalisation itself is applied behind the projection, where a
// tensor-parallel rank has the sums of all slices (rms_norm, api/cortex_sdk.cpp:1208-1232, split
// in two).
__global__ void __launch_bounds__(1024)
scale_sumsq_planes_kernel(const float* __restrict__ x, const float* __restrict__ w, uint32_t H,
                          __nv_bfloat16* __restrict__ hi, __nv_bfloat16* __restrict__ lo,
                          float* __restrict__ sumsq) {
    pdl_enter();
    __shared__ float red[32];
    const size_t o = static_cast<size_t>(blockIdx.x) * H;
    float ss = 0.0f;
    if ((H & 3u) == 0) {
        // four elements per thread and pass: 128-bit loads, 64-bit plane stores
        const float4* x4 = reinterpret_cast<const float4*>(x + o);
        const float4* w4 = reinterpret_cast<const float4*>(w);
        uint2* hi2 = reinterpret_cast<uint2*>(hi + o);
        uint2* lo2 = reinterpret_cast<uint2*>(lo + o);
        for (uint32_t i = threadIdx.x; i < H / 4u; i += blockDim.x) {
            const float4 v = x4[i], ww = w4[i];
            ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
            const float p[4] = {v.x * ww.x, v.y * ww.y, v.z * ww.z, v.w * ww.w};
            __nv_bfloat16 h[4], l[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                h[j] = __float2bfloat16_rn(p[j]);
                l[j] = __float2bfloat16_rn(p[j] - __bfloat162float(h[j]));
            }
            hi2[i] = make_uint2(static_cast<uint32_t>(__bfloat16_as_ushort(h[0])) | (static_cast<uint32_t>(__bfloat16_as_ushort(h[1])) << 16),
                                static_cast<uint32_t>(__bfloat16_as_ushort(h[2])) | (static_cast<uint32_t>(__bfloat16_as_ushort(h[3])) << 16));
            lo2[i] = make_uint2(static_cast<uint32_t>(__bfloat16_as_ushort(l[0])) | (static_cast<uint32_t>(__bfloat16_as_ushort(l[1])) << 16),
                                static_cast<uint32_t>(__bfloat16_as_ushort(l[2])) | (static_cast<uint32_t>(__bfloat16_as_ushort(l[3])) << 16));
        }
    } else {
        for (uint32_t i = threadIdx.x; i < H; i += blockDim.x) {
            const float v = x[o + i];
            ss = fmaf(v, v, ss);
            store_planes(hi, lo, o + i, v * w[i]);
        }
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31u) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.0f;
        for (uint32_t i = 0; i < (blockDim.x + 31u) / 32u; ++i) t += red[i];
        sumsq[blockIdx.x] = t;
    }
}

// out = x * w / rms, with the sum of squares of the whole hidden width given.
__global__ void __launch_bounds__(256)
norm_from_sumsq_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ sumsq,
                       uint32_t H, float inv_width, float eps, float* __restrict__ out) {
    pdl_enter();
    const size_t o = static_cast<size_t>(blockIdx.x) * H;
    const float inv = rsqrtf(sumsq[blockIdx.x] * inv_width + eps);
    for (uint32_t i = threadIdx.x; i < H; i += 256) out[o + i] = x[o + i] * inv * w[i];
}

__global__ void __launch_bounds__(256)
add_rmsnorm_kernel(float* __restrict__ hidden, const float* __restrict__ delta,
                   const float* __restrict__ w, uint32_t H, float eps, float* __restrict__ out) {
    pdl_enter();
    __shared__ float red[8];
    __shared__ float inv_s;
    float* h = hidden + static_cast<size_t>(blockIdx.x) * H;
    const float* d = delta + static_cast<size_t>(blockIdx.x) * H;
    float* dst = out + static_cast<size_t>(blockIdx.x) * H;
    float ss = 0.0f;
    for (uint32_t i = threadIdx.x; i < H; i += 256) {
        const float v = h[i] + d[i];
        h[i] = v;
        ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31u) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) t += red[i];
        inv_s = 1.0f / sqrtf(t / static_cast<float>(H) + eps);
    }
    __syncthreads();
    const float inv = inv_s;
    for (uint32_t i = threadIdx.x; i < H; i += 256) dst[i] = h[i] * inv * w[i];
}

// grid (tokens); rotates q in place, writes rotated k and plain v into the cache slot
// (seq_of[t], pos_of[t]). q (T, QH, HD); k, v (T, KVH, HD); caches (B, max_seq, KVH, HD).
template <typename KV>
__device__ __forceinline__ KV to_kv(float v);
template <>
__device__ __forceinline__ float to_kv<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 to_kv<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ __half to_kv<__half>(float v) { return __float2half_rn(v); }

// One rotary pair. Products and sums are rounded one by one (no fused multiply-add), so that
// every kernel that rotates a row gets the same bits.
__device__ __forceinline__ void rope_rotate(float x0, float x1, float c, float s, float& y0, float& y1) {
    y0 = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s));
    y1 = __fadd_rn(__fmul_rn(x0, s), __fmul_rn(x1, c));
}

template <typename KV>
__global__ void __launch_bounds__(256)
rope_cache_kernel(float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                  KV* __restrict__ kc, KV* __restrict__ vc, const int32_t* __restrict__ seq_of,
                  const int32_t* __restrict__ pos_of, uint32_t QH, uint32_t KVH, uint32_t HD,
                  uint32_t max_seq, float theta) {
    pdl_enter();
    // grid (token, slice of the heads): the few tokens of a decode step still fill a good part of
    // the GPU. A thread keeps one rotary pair index whenever the block size is a multiple of the
    // pairs per head, so the angle's cosine and sine are computed once per thread.
    const uint32_t t = blockIdx.x;
    const int32_t pos = pos_of[t], sq = seq_of[t];
    const uint32_t rotary = HD - (HD & 1u), half = rotary >> 1;
    float* qt = q + static_cast<size_t>(t) * QH * HD;
    const float* kt = k + static_cast<size_t>(t) * KVH * HD;
    const float* vt = v + static_cast<size_t>(t) * KVH * HD;
    const size_t slot = (static_cast<size_t>(sq) * max_seq + static_cast<size_t>(pos)) * KVH * HD;
    const bool in_cache = pos >= 0 && static_cast<uint32_t>(pos) < max_seq && sq >= 0;
    const uint32_t heads = QH + KVH;
    const uint32_t per = (heads + gridDim.y - 1u) / gridDim.y;
    const uint32_t h0 = blockIdx.y * per, h1 = min(heads, h0 + per);
    auto rotate = [&](uint32_t head, uint32_t i, float c, float s) {
        if (head < QH) {
            float* b = qt + head * HD + i;
            rope_rotate(b[0], b[1], c, s, b[0], b[1]);
        } else if (in_cache) {
            const uint32_t kh = head - QH;
            const float* b = kt + kh * HD + i;
            float y0, y1;
            rope_rotate(b[0], b[1], c, s, y0, y1);
            kc[slot + kh * HD + i] = to_kv<KV>(y0);
            kc[slot + kh * HD + i + 1] = to_kv<KV>(y1);
        }
    };
    auto angle_of = [&](uint32_t i, float& c, float& s) {
        const float exponent = static_cast<float>(i) / static_cast<float>(HD);
        const float freq = powf(theta, -exponent);
        const float angle = static_cast<float>(pos) * freq;
        c = cosf(angle);
        s = sinf(angle);
    };
    if (half > 0 && half <= 256u && 256u % half == 0) {
        const uint32_t i = (threadIdx.x % half) * 2u;
        float c, s;
        angle_of(i, c, s);
        for (uint32_t head = h0 + threadIdx.x / half; head < h1; head += 256u / half) rotate(head, i, c, s);
    } else {
        for (uint32_t e = threadIdx.x; e < (h1 - h0) * half; e += 256) {
            const uint32_t head = h0 + e / half, i = (e % half) * 2u;
            float c, s;
            angle_of(i, c, s);
            rotate(head, i, c, s);
        }
    }
    if (in_cache) {
        // this slice's share of the K tail (odd head_dim) and of V: the kv heads it covers
        const uint32_t kv0 = h0 > QH ? h0 - QH : 0u, kv1 = h1 > QH ? h1 - QH : 0u;
        if (HD & 1u)
            for (uint32_t kh = kv0 + threadIdx.x; kh < kv1; kh += 256)
                kc[slot + kh * HD + HD - 1] = to_kv<KV>(kt[kh * HD + HD - 1]);
        for (uint32_t e = kv0 * HD + threadIdx.x; e < kv1 * HD; e += 256) vc[slot + e] = to_kv<KV>(vt[e]);
    }
}

// One CTA (4 warps) per (token, query head). Each warp walks the keys four at a time with the
// head dimension spread over its lanes (VPL floats per lane, 128-bit loads): the eight K and V
// rows of a step are requested before any is used, so a warp keeps 4 KB of cache rows in
// flight. It keeps a running max / sum / weighted V (the softmax of simd_kernels.cpp:198-217
// evaluated in one pass); the four warps' partial states are merged through shared memory.
// Causality: token t sees cache positions 0..pos_of[t] of its own sequence, all of which are
// written before this kernel runs.
constexpr int kAttnKeys = 4;   // keys per warp per step

template <int VPL>
__device__ __forceinline__ void load_row(const float* p, float (&v)[VPL]) {
    if constexpr (VPL == 1) {
        v[0] = __ldg(p);
    } else if constexpr (VPL == 2) {
        const float2 t = __ldg(reinterpret_cast<const float2*>(p));
        v[0] = t.x;
        v[1] = t.y;
    } else {
#pragma unroll
        for (int i = 0; i < VPL / 4; ++i) {
            const float4 t = __ldg(reinterpret_cast<const float4*>(p) + i);
            v[4 * i] = t.x;
            v[4 * i + 1] = t.y;
            v[4 * i + 2] = t.z;
            v[4 * i + 3] = t.w;
        }
    }
}

// A lane's share of one cache row. fp32 cache: the values. 16-bit caches (options: fp16, bf16; scores
// and sums stay fp32): the packed words, widened where they are used, and twice the keys per step
// so that a warp keeps as many bytes in flight.
template <typename KV>
__device__ __forceinline__ float widen16(uint32_t pair, int odd);
template <>
__device__ __forceinline__ float widen16<__nv_bfloat16>(uint32_t pair, int odd) {   // a bf16 is the upper half of its fp32
    return __uint_as_float(odd ? (pair & 0xFFFF0000u) : (pair << 16));
}
template <>
__device__ __forceinline__ float widen16<__half>(uint32_t pair, int odd) {
    return __half2float(__ushort_as_half(static_cast<unsigned short>(odd ? pair >> 16 : pair & 0xFFFFu)));
}
template <typename KV, int VPL>
struct CacheRow {
    uint32_t w[(VPL + 1) / 2];
    __device__ __forceinline__ void load(const KV* p) {
        if constexpr (VPL == 1) {
            w[0] = __ldg(reinterpret_cast<const unsigned short*>(p));
        } else if constexpr (VPL == 2) {
            w[0] = __ldg(reinterpret_cast<const uint32_t*>(p));
        } else if constexpr (VPL == 4) {
            const uint2 t = __ldg(reinterpret_cast<const uint2*>(p));
            w[0] = t.x;
            w[1] = t.y;
        } else {
#pragma unroll
            for (int i = 0; i < VPL / 8; ++i) {
                const uint4 t = __ldg(reinterpret_cast<const uint4*>(p) + i);
                w[4 * i] = t.x;
                w[4 * i + 1] = t.y;
                w[4 * i + 2] = t.z;
                w[4 * i + 3] = t.w;
            }
        }
    }
    __device__ __forceinline__ float get(int e) const { return widen16<KV>(w[e >> 1], e & 1); }
    // the row as the cache would hold it: every value rounded to the cache type
    __device__ __forceinline__ void set(const float (&f)[VPL]) {
#pragma unroll
        for (int i = 0; i < (VPL + 1) / 2; ++i) {
            const KV lo = to_kv<KV>(f[2 * i]);
            const KV hi = to_kv<KV>(2 * i + 1 < VPL ? f[2 * i + 1] : 0.0f);
            w[i] = static_cast<uint32_t>(*reinterpret_cast<const unsigned short*>(&lo)) |
                   (static_cast<uint32_t>(*reinterpret_cast<const unsigned short*>(&hi)) << 16);
        }
    }
};
template <int VPL>
struct CacheRow<float, VPL> {
    float v[VPL];
    __device__ __forceinline__ void load(const float* p) { load_row<VPL>(p, v); }
    __device__ __forceinline__ float get(int e) const { return v[e]; }
    __device__ __forceinline__ void set(const float (&f)[VPL]) {
#pragma unroll
        for (int e = 0; e < VPL; ++e) v[e] = f[e];
    }
};

// Rotary embedding and cache write of a decode step folded into the attention kernel (every
// token of the step belongs to a different sequence, so no token attends to another token of
// the launch): the kernel rotates its query row in registers, takes the newest key and value of
// its sequence from the projection outputs (rotated and rounded as the cache would hold them)
// instead of the cache, and one CTA per (token, kv head) files them in the cache for later steps.
struct StepRope {
    const float* k = nullptr;   // (T, KVH, HD) fresh keys, not yet rotated; null: q and the cache are ready
    const float* v = nullptr;   // (T, KVH, HD) fresh values
    float theta = 0.0f;
};

// cos and sin of the rotary angle of pair (i, i + 1) at a position (apply_rope_inplace,
// api/cortex_sdk.cpp:1363-1423: freq = theta^(-i / head_dim)).
__device__ __forceinline__ void rope_angle(uint32_t i, uint32_t HD, int32_t pos, float theta, float& c, float& s) {
    const float exponent = static_cast<float>(i) / static_cast<float>(HD);
    const float freq = powf(theta, -exponent);
    const float angle = static_cast<float>(pos) * freq;
    c = cosf(angle);
    s = sinf(angle);
}

// Sums over the warp of N values per lane (N = 4 or 8), all N sums back in every lane. The first
// rounds halve the payload instead of carrying every value through every round: lanes whose bit
// `off` is set keep the upper half of the values and hand the lower half over, and the other way
// round; 9 + 8 shuffles for eight values instead of 40.
template <int N>
__device__ __forceinline__ void warp_sums(float (&s)[N], uint32_t lane) {
    static_assert(N == 4 || N == 8, "four or eight values");
    int n = N;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        if (n > 1) {
            const int half = n / 2;
            const bool upper = (lane & static_cast<uint32_t>(off)) != 0u;
#pragma unroll
            for (int i = 0; i < N / 2; ++i) {
                if (i < half) {
                    const float send = upper ? s[i] : s[i + half];
                    const float keep = upper ? s[i + half] : s[i];
                    s[i] = keep + __shfl_xor_sync(0xFFFFFFFFu, send, off);
                }
            }
            n = half;
        } else {
            s[0] += __shfl_xor_sync(0xFFFFFFFFu, s[0], off);
        }
    }
    // lane l now holds the sum of value number (l >> shift) & (N - 1)
    constexpr int shift = N == 8 ? 2 : 3;
    const float mine = s[0];
#pragma unroll
    for (int u = 0; u < N; ++u) s[u] = __shfl_sync(0xFFFFFFFFu, mine, u << shift);
}

// 2^x in one instruction (ex2.approx: relative error 2^-22; 2^-inf = 0).
__device__ __forceinline__ float exp2_fast(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// WARPS warps split the keys of one (token, head); few (token, head) pairs (batched decode
// against a long context) take more warps each so that enough K/V rows are in flight per SM.
// The cache element type of an attention kernel, from its pointer type (host-side launch helper).
template <typename KV, typename... Rest>
KV* kernel_kv(void (*)(const float*, KV*, Rest...)) {
    return nullptr;
}

// kSplit: the keys of one (token, head) are split over the CTAs of a thread-block cluster
// (grid z = cluster size) and the CTAs' partial softmax states are merged by the cluster's first
// CTA through distributed shared memory - for steps with fewer (token, head) pairs than SMs
// (batch-1 decode), where one CTA per pair would walk the whole context alone, one load latency
// after the other.
template <typename KV, int VPL, int kAttnWarps, bool kSplit>
__global__ void __launch_bounds__(kAttnWarps * 32)
attention_kernel(const float* __restrict__ q, KV* __restrict__ kc,
                 KV* __restrict__ vc, const int32_t* __restrict__ seq_of,
                 const int32_t* __restrict__ pos_of, uint32_t QH, uint32_t KVH, uint32_t max_seq,
                 float scale, float* __restrict__ out, __nv_bfloat16* __restrict__ hi,
                 __nv_bfloat16* __restrict__ lo, const StepRope rope) {
    pdl_enter();
    constexpr uint32_t HD = VPL * 32u;
    constexpr int kKeys = kAttnKeys * static_cast<int>(sizeof(float) / sizeof(KV));
    __shared__ float sm_m[kAttnWarps], sm_l[kAttnWarps];
    __shared__ float sm_acc[kAttnWarps][HD];
    const uint32_t t = blockIdx.x, h = blockIdx.y;
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const uint32_t kvh = h / (QH / KVH);
    const int32_t n_keys = min(pos_of[t] + 1, static_cast<int32_t>(max_seq));   // the newest key is the last one
    const size_t row = static_cast<size_t>(KVH) * HD;
    const size_t base = static_cast<size_t>(seq_of[t]) * max_seq * row + kvh * HD + lane * VPL;
    float qv[VPL], acc[VPL];
    load_row<VPL>(q + (static_cast<size_t>(t) * QH + h) * HD + lane * VPL, qv);
    // step with the rotary embedding folded in (VPL >= 2: a lane holds whole pairs): rotate the
    // query, build the newest key and value rows, file them in the cache once per (token, kv head)
    const int32_t pos = pos_of[t];
    const bool fresh = VPL >= 2 && rope.k != nullptr && pos >= 0 && pos < static_cast<int32_t>(max_seq);
    CacheRow<KV, VPL> knew, vnew;
    if (VPL >= 2 && rope.k != nullptr) {
        float kf[VPL], vf[VPL];
        if (fresh) {
            load_row<VPL>(rope.k + (static_cast<size_t>(t) * KVH + kvh) * HD + lane * VPL, kf);
            load_row<VPL>(rope.v + (static_cast<size_t>(t) * KVH + kvh) * HD + lane * VPL, vf);
        }
#pragma unroll
        for (int e = 0; e + 1 < VPL; e += 2) {
            float c, sn;
            rope_angle(lane * VPL + e, HD, pos, rope.theta, c, sn);
            rope_rotate(qv[e], qv[e + 1], c, sn, qv[e], qv[e + 1]);
            if (fresh) rope_rotate(kf[e], kf[e + 1], c, sn, kf[e], kf[e + 1]);
        }
        if (fresh) {
            knew.set(kf);
            vnew.set(vf);
            if (warp == 0 && h == kvh * (QH / KVH) && (!kSplit || blockIdx.z == 0)) {
                const size_t slot = static_cast<size_t>(seq_of[t]) * max_seq * (static_cast<size_t>(KVH) * HD) +
                                    static_cast<size_t>(pos) * (static_cast<size_t>(KVH) * HD) + kvh * HD + lane * VPL;
#pragma unroll
                for (int e = 0; e < VPL; ++e) {
                    kc[slot + e] = to_kv<KV>(kf[e]);
                    vc[slot + e] = to_kv<KV>(vf[e]);
                }
            }
        }
    }
    // scores are kept as log2 of the softmax weights (the query carries scale * log2 e), so that a
    // weight is one ex2 instruction; maxima and running sums are in the same units throughout
    const float qscale = scale * 1.4426950408889634f;
#pragma unroll
    for (int e = 0; e < VPL; ++e) {
        qv[e] *= qscale;
        acc[e] = 0.0f;
    }
    float m = -INFINITY, l = 0.0f;
    const uint32_t crank = kSplit ? blockIdx.z : 0u, csize = kSplit ? gridDim.z : 1u;
    for (int32_t j0 = (crank * kAttnWarps + warp) * kKeys; j0 < n_keys; j0 += csize * kAttnWarps * kKeys) {
        CacheRow<KV, VPL> kv[kKeys], vv[kKeys];
        const bool whole = j0 + kKeys <= n_keys;   // warp-uniform: every step but a warp's last
        if (whole) {
            const KV* k0 = kc + base + static_cast<size_t>(j0) * row;
            const KV* v0 = vc + base + static_cast<size_t>(j0) * row;
#pragma unroll
            for (int u = 0; u < kKeys; ++u) {
                kv[u].load(k0 + static_cast<size_t>(u) * row);
                vv[u].load(v0 + static_cast<size_t>(u) * row);
            }
        } else {
#pragma unroll
            for (int u = 0; u < kKeys; ++u) {
                const int32_t j = min(j0 + u, n_keys - 1);   // clamp: the tail re-reads the last row, unused
                kv[u].load(kc + base + static_cast<size_t>(j) * row);
                vv[u].load(vc + base + static_cast<size_t>(j) * row);
            }
        }
        if (fresh && j0 + kKeys > pos) {      // this step holds the newest key: not from the cache
#pragma unroll
            for (int u = 0; u < kKeys; ++u)
                if (j0 + u == pos) {
                    kv[u] = knew;
                    vv[u] = vnew;
                }
        }
        float s[kKeys];
#pragma unroll
        for (int u = 0; u < kKeys; ++u) {
            float d = 0.0f;
#pragma unroll
            for (int e = 0; e < VPL; ++e) d = fmaf(qv[e], kv[u].get(e), d);
            s[u] = d;
        }
        warp_sums<kKeys>(s, lane);
        // the keys of a step join the running softmax together: one new maximum, one correction of
        // what has been summed so far, then every key's weight
        float m_new = m;
        if (!whole) {
#pragma unroll
            for (int u = 0; u < kKeys; ++u)
                if (j0 + u >= n_keys) s[u] = -INFINITY;
        }
#pragma unroll
        for (int u = 0; u < kKeys; ++u) m_new = fmaxf(m_new, s[u]);
        const float corr = exp2_fast(m - m_new);   // 2^-inf = 0 on the first step; the step's first key is always valid
        float psum = 0.0f;
#pragma unroll
        for (int u = 0; u < kKeys; ++u) {
            s[u] = exp2_fast(s[u] - m_new);        // 2^-inf = 0 for the keys past the end
            psum += s[u];
        }
        l = fmaf(l, corr, psum);
#pragma unroll
        for (int e = 0; e < VPL; ++e) {
            float a = acc[e] * corr;
#pragma unroll
            for (int u = 0; u < kKeys; ++u) a = fmaf(s[u], vv[u].get(e), a);
            acc[e] = a;
        }
        m = m_new;
    }
    if (lane == 0) {
        sm_m[warp] = m;
        sm_l[warp] = l;
    }
#pragma unroll
    for (int e = 0; e < VPL; ++e) sm_acc[warp][lane * VPL + e] = acc[e];
    __syncthreads();
    float M = -INFINITY, L = 0.0f, o[VPL];
#pragma unroll
    for (int e = 0; e < VPL; ++e) o[e] = 0.0f;
    if (warp == 0) {
#pragma unroll
        for (int w = 0; w < kAttnWarps; ++w) M = fmaxf(M, sm_m[w]);
#pragma unroll
        for (int w = 0; w < kAttnWarps; ++w) {
            const float f = sm_m[w] == -INFINITY ? 0.0f : exp2_fast(sm_m[w] - M);
            L = fmaf(sm_l[w], f, L);
#pragma unroll
            for (int e = 0; e < VPL; ++e) o[e] = fmaf(sm_acc[w][lane * VPL + e], f, o[e]);
        }
    }
    if constexpr (kSplit) {
        namespace cg = cooperative_groups;
        cg::cluster_group cluster = cg::this_cluster();
        // this CTA's state where the first CTA can read it: row 0 of the buffers (a lane rewrites
        // only the slots it has just read)
        if (warp == 0) {
            if (lane == 0) {
                sm_m[0] = M;
                sm_l[0] = L;
            }
#pragma unroll
            for (int e = 0; e < VPL; ++e) sm_acc[0][lane * VPL + e] = o[e];
        }
        cluster.sync();
        if (crank == 0 && warp == 0) {
            float Mc = -INFINITY;
            for (uint32_t r = 0; r < csize; ++r) Mc = fmaxf(Mc, cluster.map_shared_rank(&sm_m[0], r)[0]);
            float Lc = 0.0f, oc[VPL];
#pragma unroll
            for (int e = 0; e < VPL; ++e) oc[e] = 0.0f;
            for (uint32_t r = 0; r < csize; ++r) {                       // in rank order: the result does not depend on timing
                const float mr = cluster.map_shared_rank(&sm_m[0], r)[0];
                const float f = mr == -INFINITY ? 0.0f : exp2_fast(mr - Mc);
                Lc = fmaf(cluster.map_shared_rank(&sm_l[0], r)[0], f, Lc);
                const float* ar = cluster.map_shared_rank(&sm_acc[0][0], r);
#pragma unroll
                for (int e = 0; e < VPL; ++e) oc[e] = fmaf(ar[lane * VPL + e], f, oc[e]);
            }
            L = Lc;
#pragma unroll
            for (int e = 0; e < VPL; ++e) o[e] = oc[e];
        }
        cluster.sync();   // the peers' shared memory must outlive the reads above
        if (crank != 0) return;
    }
    if (warp == 0) {
        const float inv = L > 0.0f ? 1.0f / L : 0.0f;
        const size_t o0 = (static_cast<size_t>(t) * QH + h) * HD + lane * VPL;
#pragma unroll
        for (int e = 0; e < VPL; ++e) {
            if (hi) store_planes(hi, lo, o0 + e, o[e] * inv);
            else out[o0 + e] = o[e] * inv;
        }
    }
}

__global__ void silu_mul_kernel(const float* __restrict__ gate, const float* __restrict__ up,
                                size_t n, float* __restrict__ out, __nv_bfloat16* __restrict__ hi,
                                __nv_bfloat16* __restrict__ lo) {
    pdl_enter();
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n; i += stride) {
        const float x = gate[i];
        const float sig = 1.0f / (1.0f + expf(-x));
        const float v = (x * sig) * up[i];
        if (hi) store_planes(hi, lo, i, v);
        else out[i] = v;
    }
}

__global__ void add_kernel(float* __restrict__ a, const float* __restrict__ b, size_t n) {
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n; i += stride)
        a[i] = a[i] + b[i];
}

// Rank-major gathered shards (P, T, W) -> token-major (T, P*W); add != 0 accumulates.
__global__ void unshard_kernel(const float* __restrict__ staged, uint32_t P, uint32_t T, uint32_t W,
                               float* __restrict__ out, int add) {
    const size_t n = static_cast<size_t>(P) * T * W;
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n; i += stride) {
        const uint32_t w = static_cast<uint32_t>(i % W);
        const uint32_t t = static_cast<uint32_t>((i / W) % T);
        const uint32_t p = static_cast<uint32_t>(i / (static_cast<size_t>(W) * T));
        const size_t o = static_cast<size_t>(t) * P * W + static_cast<size_t>(p) * W + w;
        out[o] = add ? out[o] + staged[i] : staged[i];
    }
}

__global__ void gather_rows_kernel(const float* __restrict__ table, uint32_t n_rows, uint32_t H,
                                   const int32_t* __restrict__ ids, float* __restrict__ out) {
    const int32_t r = ids[blockIdx.x];
    float* dst = out + static_cast<size_t>(blockIdx.x) * H;
    const bool ok = r >= 0 && static_cast<uint32_t>(r) < n_rows;
    const float* src = table + static_cast<size_t>(ok ? r : 0) * H;
    for (uint32_t i = threadIdx.x; i < H; i += blockDim.x) dst[i] = ok ? src[i] : 0.0f;
}

// One CTA per logits row; first maximum wins.
__global__ void __launch_bounds__(1024)
argmax_kernel(const float* __restrict__ logits, uint32_t V, int32_t* __restrict__ out, float temp_scale,
              uint32_t* __restrict__ seen, uint32_t seen_words) {
    // seen == nullptr: plain argmax. Else select_best_from_logits (api/cortex_sdk.cpp:1005-1030):
    // score = logit * temp_scale, non-finite scores skipped, 1.5 off for tokens the sequence has
    // produced (bitmap row blockIdx.x), first maximum wins; the pick is recorded in the bitmap.
    __shared__ float bv[32];
    __shared__ int32_t bi[32];
    const float* row = logits + static_cast<size_t>(blockIdx.x) * V;
    uint32_t* mine = seen ? seen + static_cast<size_t>(blockIdx.x) * seen_words : nullptr;
    float best = -INFINITY;
    int32_t idx = 0x7FFFFFFF;
    for (uint32_t i = threadIdx.x; i < V; i += 1024) {
        float v = row[i];
        if (mine) {
            v *= temp_scale;
            if (!isfinite(v)) continue;
            if ((mine[i >> 5] >> (i & 31u)) & 1u) v -= 1.5f;
        }
        if (v > best || (v == best && static_cast<int32_t>(i) < idx)) {
            best = v;
            idx = static_cast<int32_t>(i);
        }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        const float ov = __shfl_xor_sync(0xFFFFFFFFu, best, off);
        const int32_t oi = __shfl_xor_sync(0xFFFFFFFFu, idx, off);
        if (ov > best || (ov == best && oi < idx)) {
            best = ov;
            idx = oi;
        }
    }
    if ((threadIdx.x & 31u) == 0) {
        bv[threadIdx.x >> 5] = best;
        bi[threadIdx.x >> 5] = idx;
    }
    __syncthreads();
    if (threadIdx.x < 32) {
        best = bv[threadIdx.x];
        idx = bi[threadIdx.x];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            const float ov = __shfl_xor_sync(0xFFFFFFFFu, best, off);
            const int32_t oi = __shfl_xor_sync(0xFFFFFFFFu, idx, off);
            if (ov > best || (ov == best && oi < idx)) {
                best = ov;
                idx = oi;
            }
        }
        if (threadIdx.x == 0) {
            // nothing selectable: plain argmax answers token 0, the policy answers -1 like the reference
            out[blockIdx.x] = idx == 0x7FFFFFFF ? (mine ? -1 : 0) : idx;
            if (mine && idx != 0x7FFFFFFF) mine[idx >> 5] |= 1u << (idx & 31);
        }
    }
}

// Records tokens chosen outside a step (e.g. from the prefill's logits) for one sequence.
__global__ void mark_seen_kernel(uint32_t* __restrict__ seen_row, const int32_t* __restrict__ tokens, uint32_t n,
                                 uint32_t V) {
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const int32_t t = tokens[i];
        if (t >= 0 && static_cast<uint32_t>(t) < V) atomicOr(seen_row + (t >> 5), 1u << (t & 31));
    }
}

// positions: pos_of[t] = pos[b] for a batched step, then pos[b] += 1 (all on the device, so a
// captured step replays without host involvement).
__global__ void step_positions_kernel(int32_t* __restrict__ pos, uint32_t B, int32_t* __restrict__ seq_of,
                                      int32_t* __restrict__ pos_of) {
    const uint32_t b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b < B) {
        seq_of[b] = static_cast<int32_t>(b);
        pos_of[b] = pos[b];
        pos[b] = pos[b] + 1;
    }
}

unsigned grid_for(size_t n, csdr_context* ctx) {
    return static_cast<unsigned>(std::min<size_t>((n + 255) / 256, static_cast<size_t>(ctx->sm_count) * 8));
}

}  // namespace

void op_rmsnorm(csdr_context* ctx, const float* x, const float* w, uint32_t T, uint32_t H, float eps,
                float* out) {
    LaunchScope ls(ctx, KC_DECODER_OP);
    launch_pdl(ctx, rmsnorm_kernel, dim3(T), dim3(256), x, w, H, eps, out, nullptr, nullptr);
    ls.done("rmsnorm_kernel");
}

void op_rmsnorm_planes(csdr_context* ctx, const float* x, const float* w, uint32_t T, uint32_t H, float eps,
                       __nv_bfloat16* hi, __nv_bfloat16* lo) {
    LaunchScope ls(ctx, KC_DECODER_OP);
    launch_pdl(ctx, rmsnorm_kernel, dim3(T), dim3(256), x, w, H, eps, nullptr, hi, lo);
    ls.done("rmsnorm_kernel");
}

void op_scale_sumsq_planes(csdr_context* ctx, const float* x, const float* w, uint32_t T, uint32_t H,
                           __nv_bfloat16* hi, __nv_bfloat16* lo, float* sumsq) {
    LaunchScope ls(ctx, KC_DECODER_OP);
    // few tokens: a wide block per token keeps the pass short; many tokens: the grid already fills the GPU
    launch_pdl(ctx, scale_sumsq_planes_kernel, dim3(T), dim3(T <= 64u ? 1024u : 256u), x, w, H, hi, lo, sumsq);
    ls.done("scale_sumsq_planes_kernel");
}

void op_norm_from_sumsq(csdr_context* ctx, const float* x, const float* w, const float* sumsq, uint32_t T,
                        uint32_t H, uint32_t full_width, float eps, float* out) {
    LaunchScope ls(ctx, KC_DECODER_OP);
    launch_pdl(ctx, norm_from_sumsq_kernel, dim3(T), dim3(256), x, w, sumsq, H, 1.0f / static_cast<float>(full_width),
               eps, out);
    ls.done("norm_from_sumsq_kernel");
}

void op_add_rmsnorm(csdr_context* ctx, float* hidden, const float* delta, const float* w, uint32_t T,
                    uint32_t H, float eps, float* out) {
    LaunchScope ls(ctx, KC_DECODER_OP);
    launch_pdl(ctx, add_rmsnorm_kernel, dim3(T), dim3(256), hidden, delta, w, H, eps, out);
    ls.done("add_rmsnorm_kernel");
}

void op_rope_cache(csdr_context* ctx, float* q, const float* k, const float* v, void* kc, void* vc, int kv_dtype,
                   const int32_t* seq_of, const int32_t* pos_of, uint32_t T, uint32_t QH, uint32_t KVH,
                   uint32_t HD, uint32_t max_seq, float theta) {
    LaunchScope ls(ctx, KC_DECODER_OP);
    // slices of the heads per token: enough CTAs for a decode step, one for a long prefill
    const uint32_t slices = T >= 256u ? 1u : std::min<uint32_t>(QH + KVH, std::max(1u, 256u / std::max(T, 1u)));
    if (kv_dtype == CSDR_DTYPE_BF16)
        launch_pdl(ctx, rope_cache_kernel<__nv_bfloat16>, dim3(T, std::min(slices, 16u)), dim3(256), q, k, v,
                   static_cast<__nv_bfloat16*>(kc), static_cast<__nv_bfloat16*>(vc), seq_of, pos_of, QH, KVH, HD, max_seq, theta);
    else if (kv_dtype == CSDR_DTYPE_F16)
        launch_pdl(ctx, rope_cache_kernel<__half>, dim3(T, std::min(slices, 16u)), dim3(256), q, k, v, static_cast<__half*>(kc),
                   static_cast<__half*>(vc), seq_of, pos_of, QH, KVH, HD, max_seq, theta);
    else
        launch_pdl(ctx, rope_cache_kernel<float>, dim3(T, std::min(slices, 16u)), dim3(256), q, k, v, static_cast<float*>(kc),
                   static_cast<float*>(vc), seq_of, pos_of, QH, KVH, HD, max_seq, theta);
    ls.done("rope_cache_kernel");
}

bool attention_step_supported(uint32_t HD) { return HD == 64u || HD == 128u || HD == 256u; }

void op_attention(csdr_context* ctx, const float* q, const void* kc, const void* vc, int kv_dtype,
                  const int32_t* seq_of, const int32_t* pos_of, uint32_t T, uint32_t QH, uint32_t KVH,
                  uint32_t HD, uint32_t max_seq, float* out, __nv_bfloat16* hi, __nv_bfloat16* lo) {
    op_attention_step(ctx, q, nullptr, nullptr, 0.0f, const_cast<void*>(kc), const_cast<void*>(vc), kv_dtype, seq_of, pos_of, T,
                      QH, KVH, HD, max_seq, out, hi, lo);
}

void op_attention_step(csdr_context* ctx, const float* q, const float* k_new, const float* v_new, float theta, void* kc,
                       void* vc, int kv_dtype, const int32_t* seq_of, const int32_t* pos_of, uint32_t T, uint32_t QH,
                       uint32_t KVH, uint32_t HD, uint32_t max_seq, float* out, __nv_bfloat16* hi, __nv_bfloat16* lo) {
    if (HD % 32u || HD > 256u || HD == 96u || HD == 160u || HD == 192u || HD == 224u)
        throw Error(CSDR_ERR_UNSUPPORTED, "attention: head_dim must be 32, 64, 128 or 256");
    if (k_new && !attention_step_supported(HD))
        throw Error(CSDR_ERR_UNSUPPORTED, "attention with the rotary embedding folded in: head_dim must be 64, 128 or 256");
    const StepRope rope{k_new, v_new, theta};
    const float scale = 1.0f / sqrtf(static_cast<float>(HD));
    LaunchScope ls(ctx, KC_ATTENTION);
    const uint32_t pairs = T * QH;
    const uint32_t sms = static_cast<uint32_t>(ctx->sm_count);
    // few pairs: a cluster of 2, 4 or 8 CTAs per pair shares the keys
    uint32_t split = 1;
    while (split < 8u && pairs * split * 2u <= sms) split *= 2u;
    const int warps = pairs >= sms * 8u ? 4 : pairs >= sms * 4u ? 8 : 16;
    auto launch = [&](auto kern, int w) {
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(T, QH, split);
        cfg.blockDim = dim3(static_cast<unsigned>(w) * 32u);
        cfg.stream = ctx->stream;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = ctx->pdl ? 1 : 0;
        cfg.numAttrs = 1;
        if (split > 1) {
            attr[1].id = cudaLaunchAttributeClusterDimension;
            attr[1].val.clusterDim.x = 1;
            attr[1].val.clusterDim.y = 1;
            attr[1].val.clusterDim.z = split;
            cfg.numAttrs = 2;
        }
        cfg.attrs = attr;
        using KVp = std::remove_pointer_t<decltype(kernel_kv(kern))>;
        CSDR_CUDA(cudaLaunchKernelEx(&cfg, kern, q, static_cast<KVp*>(kc), static_cast<KVp*>(vc), seq_of, pos_of, QH, KVH,
                                     max_seq, scale, out, hi, lo, rope));
    };
#define CSDR_ATTN(V, W)                                                                     \
    do {                                                                                    \
        if (kv_dtype == CSDR_DTYPE_BF16) {                                                  \
            if (split > 1) launch(attention_kernel<__nv_bfloat16, V, W, true>, W);          \
            else launch(attention_kernel<__nv_bfloat16, V, W, false>, W);                   \
        } else if (kv_dtype == CSDR_DTYPE_F16) {                                            \
            if (split > 1) launch(attention_kernel<__half, V, W, true>, W);                 \
            else launch(attention_kernel<__half, V, W, false>, W);                          \
        } else {                                                                            \
            if (split > 1) launch(attention_kernel<float, V, W, true>, W);                  \
            else launch(attention_kernel<float, V, W, false>, W);                           \
        }                                                                                   \
    } while (0)
#define CSDR_ATTN_W(V)                        \
    do {                                      \
        if (split > 1) CSDR_ATTN(V, 16);      \
        else if (warps == 4) CSDR_ATTN(V, 4); \
        else if (warps == 8) CSDR_ATTN(V, 8); \
        else CSDR_ATTN(V, 16);                \
    } while (0)
    switch (HD / 32u) {
        case 1: CSDR_ATTN_W(1); break;
        case 2: CSDR_ATTN_W(2); break;
        case 4: CSDR_ATTN_W(4); break;
        default: CSDR_ATTN_W(8); break;
    }
#undef CSDR_ATTN_W
#undef CSDR_ATTN
    ls.done("attention_kernel");
}

void op_silu_mul(csdr_context* ctx, const float* gate, const float* up, size_t n, float* out) {
    LaunchScope ls(ctx, KC_DECODER_OP);
    launch_pdl(ctx, silu_mul_kernel, dim3(grid_for(n, ctx)), dim3(256), gate, up, n, out, nullptr, nullptr);
    ls.done("silu_mul_kernel");
}

void op_silu_mul_planes(csdr_context* ctx, const float* gate, const float* up, size_t n, __nv_bfloat16* hi,
                        __nv_bfloat16* lo) {
    LaunchScope ls(ctx, KC_DECODER_OP);
    launch_pdl(ctx, silu_mul_kernel, dim3(grid_for(n, ctx)), dim3(256), gate, up, n, nullptr, hi, lo);
    ls.done("silu_mul_kernel");
}

void op_add(csdr_context* ctx, float* a, const float* b, size_t n) {
    LaunchScope ls(ctx, KC_DECODER_OP);
    add_kernel<<<grid_for(n, ctx), 256, 0, ctx->stream>>>(a, b, n);
    ls.done("add_kernel");
}

void op_unshard(csdr_context* ctx, const float* staged, uint32_t P, uint32_t T, uint32_t W, float* out,
                bool add) {
    LaunchScope ls(ctx, KC_DECODER_OP);
    unshard_kernel<<<grid_for(static_cast<size_t>(P) * T * W, ctx), 256, 0, ctx->stream>>>(staged, P, T, W, out, add ? 1 : 0);
    ls.done("unshard_kernel");
}

void op_gather_rows(csdr_context* ctx, const float* table, uint32_t n_rows, uint32_t H,
                    const int32_t* ids, uint32_t T, float* out) {
    LaunchScope ls(ctx, KC_DECODER_OP);
    gather_rows_kernel<<<T, 256, 0, ctx->stream>>>(table, n_rows, H, ids, out);
    ls.done("gather_rows_kernel");
}

void op_select(csdr_context* ctx, const float* logits, uint32_t rows, uint32_t V, int32_t* out, float temperature,
               uint32_t* seen, uint32_t seen_words) {
    LaunchScope ls(ctx, KC_DECODER_OP);
    argmax_kernel<<<rows, 1024, 0, ctx->stream>>>(logits, V, out, temperature > 0.0f ? 1.0f / temperature : 1.0f, seen,
                                                  seen_words);
    ls.done("argmax_kernel");
}

void op_mark_seen(csdr_context* ctx, uint32_t* seen_row, const int32_t* tokens_dev, uint32_t n, uint32_t V) {
    if (!n) return;
    LaunchScope ls(ctx, KC_DECODER_OP);
    mark_seen_kernel<<<(n + 255u) / 256u, 256, 0, ctx->stream>>>(seen_row, tokens_dev, n, V);
    ls.done("mark_seen_kernel");
}

void op_argmax(csdr_context* ctx, const float* logits, uint32_t rows, uint32_t V, int32_t* out) {
    LaunchScope ls(ctx, KC_DECODER_OP);
    argmax_kernel<<<rows, 1024, 0, ctx->stream>>>(logits, V, out, 1.0f, nullptr, 0u);
    ls.done("argmax_kernel");
}

void op_step_positions(csdr_context* ctx, int32_t* pos, uint32_t B, int32_t* seq_of, int32_t* pos_of) {
    LaunchScope ls(ctx, KC_DECODER_OP);
    step_positions_kernel<<<(B + 127) / 128, 128, 0, ctx->stream>>>(pos, B, seq_of, pos_of);
    ls.done("step_positions_kernel");
}

}  // namespace csdr
