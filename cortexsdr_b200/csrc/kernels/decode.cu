// Weight materialisation and source-dtype dequantisation kernels for sm_100a.
//
//   hsdr_decode_rows_kernel   HierarchicalSDRStrategy::decompress /
//                             decompressWithExternalDictionary
//                             (strategies/HierarchicalSDRStrategy.cpp:1340-1440, :1804-1828;
//                             decodeAllTiles :612-634, reassembleTiles :119-135, edge splice
//                             :1412-1438) — for all rows, or for a list of rows (the
//                             embedding-row lookup of api/cortex_sdk.cpp:860-876).
//   dequant_*_kernel          dequantizeSegmentToFP32 (:713-989), bit-exact.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstring>

#include "../internal.hpp"

namespace csdr {

namespace {

struct DecodeGeom {
    uint32_t R, C, Rf, Cf, Tr, Tc, n_ct, S, k, K;
};

// One thread per VEC consecutive columns of one output row. The per-element sum runs
// stage-major, slot-minor with one multiply and one add per code, the order and the
// operations of decodeAllTiles, so the result is bit-identical to the reference's.
template <int VEC>
__global__ void __launch_bounds__(256)
hsdr_decode_rows_kernel(const float* __restrict__ D, const uint16_t* __restrict__ codes,
                        const float* __restrict__ scales, const float* __restrict__ edges,
                        DecodeGeom g, const int32_t* __restrict__ rows, float* __restrict__ out) {
    const uint32_t c = (blockIdx.y * 256u + threadIdx.x) * VEC;
    if (c >= g.C) return;
    const size_t oi = static_cast<size_t>(blockIdx.x) * g.C + c;
    const int64_t rr = rows ? static_cast<int64_t>(rows[blockIdx.x]) : static_cast<int64_t>(blockIdx.x);
    float v[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) v[e] = 0.0f;
    if (rr >= 0 && rr < static_cast<int64_t>(g.R)) {
        const uint32_t r = static_cast<uint32_t>(rr);
        if (r >= g.Rf) {
            const float* e0 = edges + static_cast<size_t>(g.Rf) * (g.C - g.Cf) +
                              static_cast<size_t>(r - g.Rf) * g.C + c;
#pragma unroll
            for (int e = 0; e < VEC; ++e) v[e] = e0[e];
        } else if (c >= g.Cf) {
            const float* e0 = edges + static_cast<size_t>(r) * (g.C - g.Cf) + (c - g.Cf);
#pragma unroll
            for (int e = 0; e < VEC; ++e)
                if (c + e < g.C) v[e] = e0[e];
        } else {
            const uint32_t br = r / g.Tr, j = r - br * g.Tr;
            const uint32_t bc = c / g.Tc, i = c - bc * g.Tc;
            const uint32_t slots = g.S * g.k;
            const uint16_t* tc = codes + (static_cast<size_t>(br) * g.n_ct + bc) * slots;
            const size_t T = static_cast<size_t>(g.Tr) * g.Tc;
            const size_t eoff = static_cast<size_t>(j) * g.Tc + i;
            for (uint32_t l = 0; l < g.S; ++l) {
                const float gamma = scales[l];
                for (uint32_t kk = 0; kk < g.k; ++kk) {
                    const uint32_t code = tc[l * g.k + kk];
                    const float scale = (code & 0x8000u) ? -gamma : gamma;
                    const float* atom = D + static_cast<size_t>(code & 0x7FFFu) * T + eoff;
                    if constexpr (VEC == 4) {
                        const float4 a4 = *reinterpret_cast<const float4*>(atom);
                        v[0] = __fadd_rn(v[0], __fmul_rn(scale, a4.x));
                        v[1] = __fadd_rn(v[1], __fmul_rn(scale, a4.y));
                        v[2] = __fadd_rn(v[2], __fmul_rn(scale, a4.z));
                        v[3] = __fadd_rn(v[3], __fmul_rn(scale, a4.w));
                    } else {
                        v[0] = __fadd_rn(v[0], __fmul_rn(scale, atom[0]));
                    }
                }
            }
        }
    }
    if constexpr (VEC == 4) {
        *reinterpret_cast<float4*>(out + oi) = make_float4(v[0], v[1], v[2], v[3]);
    } else {
        out[oi] = v[0];
    }
}

enum Fmt { F32 = 0, F16, BF16, I8, Q4_0, Q8_0, Q4_K, Q5_K, Q6_K };

__global__ void dequant_simple_kernel(int fmt, const uint8_t* __restrict__ p, size_t n_out,
                                      float scale, float zp, float* __restrict__ out) {
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n_out; i += stride) {
        float v;
        switch (fmt) {
            case F32: v = reinterpret_cast<const float*>(p)[i]; break;
            case F16: v = __half2float(__ushort_as_half(reinterpret_cast<const uint16_t*>(p)[i])); break;
            case BF16: v = __uint_as_float(static_cast<uint32_t>(reinterpret_cast<const uint16_t*>(p)[i]) << 16); break;
            case I8: v = __fmul_rn(__fsub_rn(static_cast<float>(static_cast<int8_t>(p[i])), zp), scale); break;
            case Q4_0: {
                const uint8_t* blk = p + (i / 32) * 18;
                const float d = __half2float(__ushort_as_half(static_cast<uint16_t>(blk[0] | (blk[1] << 8))));
                const uint32_t e = static_cast<uint32_t>(i % 32);
                const uint8_t byte = blk[2 + e / 2];
                const int q = (e & 1u) ? static_cast<int>(byte >> 4) - 8 : static_cast<int>(byte & 0x0F) - 8;
                v = __fmul_rn(static_cast<float>(q), d);
                break;
            }
            default: {  // Q8_0
                const uint8_t* blk = p + (i / 32) * 34;
                const float d = __half2float(__ushort_as_half(static_cast<uint16_t>(blk[0] | (blk[1] << 8))));
                v = __fmul_rn(static_cast<float>(static_cast<int8_t>(blk[2 + i % 32])), d);
                break;
            }
        }
        out[i] = v;
    }
}

__device__ __forceinline__ float ld_half(const uint8_t* p) {
    return __half2float(__ushort_as_half(static_cast<uint16_t>(p[0] | (p[1] << 8))));
}

// One warp per 256-element super-block, 8 consecutive elements per lane.
__global__ void __launch_bounds__(256)
dequant_kquant_kernel(int fmt, const uint8_t* __restrict__ data, size_t n_blocks,
                      float* __restrict__ out) {
    const uint32_t lane = threadIdx.x & 31u;
    const size_t warps = static_cast<size_t>(gridDim.x) * 8u;
    for (size_t blk = blockIdx.x * 8ull + (threadIdx.x >> 5); blk < n_blocks; blk += warps) {
        float v[8];
        if (fmt == Q6_K) {
            const uint8_t* p = data + blk * 210;
            const float d = ld_half(p + 208);
            const uint32_t half = lane >> 4, l16 = lane & 15u;
            const int8_t sc = static_cast<int8_t>(p[192 + half * 8 + (l16 >> 1)]);
            const float ds = __fmul_rn(d, static_cast<float>(sc));
            const uint8_t* ql = p + half * 64 + l16 * 4;
            const uint8_t* qh = p + 128 + half * 32 + l16 * 2;
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const uint8_t lb = ql[e >> 1];
                const uint32_t lo = (e & 1) ? (lb >> 4) : (lb & 0x0Fu);
                const uint32_t hi = (qh[e >> 2] >> ((e & 3) * 2)) & 3u;
                const int q = static_cast<int>((hi << 4) | lo) - 32;
                v[e] = __fmul_rn(static_cast<float>(q), ds);
            }
        } else {
            const uint32_t bb = fmt == Q5_K ? 176u : 144u;
            const uint8_t* p = data + blk * bb;
            const float d = ld_half(p), dmin = ld_half(p + 2);
            const uint8_t* s12 = p + 4;
            const uint32_t is = lane >> 2;
            uint32_t sc, mn;
            if (is < 4) {
                sc = s12[is] & 0x3Fu;
                mn = s12[is + 4] & 0x3Fu;
            } else {
                sc = (s12[is + 4] & 0x0Fu) | ((s12[is - 4] >> 6) << 4);
                mn = (s12[is + 4] >> 4) | ((s12[is] >> 6) << 4);
            }
            const float ds = __fmul_rn(d, static_cast<float>(sc));
            const float dm = __fmul_rn(dmin, static_cast<float>(mn));
            const uint8_t* qs = p + (fmt == Q5_K ? 48 : 16) + lane * 4;
            const uint32_t qhb = fmt == Q5_K ? p[16 + lane] : 0u;
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const uint8_t byte = qs[e >> 1];
                uint32_t q = (e & 1) ? (byte >> 4) : (byte & 0x0Fu);
                q |= ((qhb >> e) & 1u) << 4;
                v[e] = __fsub_rn(__fmul_rn(static_cast<float>(q), ds), dm);
            }
        }
        float4* o = reinterpret_cast<float4*>(out + blk * 256 + lane * 8);
        o[0] = make_float4(v[0], v[1], v[2], v[3]);
        o[1] = make_float4(v[4], v[5], v[6], v[7]);
    }
}

// Stored-raw k-quant tensors as the reference's INFERENCE side widens them
// (decodeSupportedGGUFQuantized, SparseInferenceEngine.cpp:276-469): ggml's element order, not
// the encoder's. One thread per output element, 256 elements per super-block.
//   q4_k (:362-383)  64-element groups: 32 low nibbles under scale 2g, then 32 high nibbles
//                    under scale 2g+1; (d*sc)*q - dmin*mn
//   q6_k (:329-360)  128-element halves, four runs of 32: low nibbles of ql[0..31], of ql[32..63],
//                    then the high nibbles; two bits of qh[l] each; d * float(sc[2r] * (q - 32))
//   q5_k (:437-463)  the generic fall-back: 5-bit fields packed from byte 16, (q - 16) * d, with
//                    d replaced by 1 when it is not finite or below 1e-12
__global__ void __launch_bounds__(256)
dequant_inference_kquant_kernel(int fmt, const uint8_t* __restrict__ data, size_t n_out, float* __restrict__ out) {
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n_out; i += stride) {
        const size_t blk = i >> 8;
        const uint32_t e = static_cast<uint32_t>(i & 255u);
        float v;
        if (fmt == Q4_K) {
            const uint8_t* p = data + blk * 144;
            const float d = ld_half(p), dmin = ld_half(p + 2);
            const uint8_t* s12 = p + 4;
            const uint32_t g = e >> 6, hi = (e >> 5) & 1u, l = e & 31u, j = 2u * g + hi;
            uint32_t sc, mn;
            if (j < 4) {
                sc = s12[j] & 0x3Fu;
                mn = s12[j + 4] & 0x3Fu;
            } else {
                sc = (s12[j + 4] & 0x0Fu) | ((s12[j - 4] >> 6) << 4);
                mn = (s12[j + 4] >> 4) | ((s12[j] >> 6) << 4);
            }
            const uint8_t byte = p[16 + g * 32 + l];
            const uint32_t q = hi ? (byte >> 4) : (byte & 0x0Fu);
            v = __fsub_rn(__fmul_rn(__fmul_rn(d, static_cast<float>(sc)), static_cast<float>(q)),
                          __fmul_rn(dmin, static_cast<float>(mn)));
        } else if (fmt == Q6_K) {
            const uint8_t* p = data + blk * 210;
            const float d = ld_half(p + 208);
            const uint32_t half = e >> 7, r = (e >> 5) & 3u, l = e & 31u;
            const uint8_t lb = p[half * 64 + l + (r & 1u) * 32u];
            const uint32_t lo = r >= 2 ? (lb >> 4) : (lb & 0x0Fu);
            const uint32_t hi2 = (p[128 + half * 32 + l] >> (2u * r)) & 3u;
            const int q = static_cast<int>(lo | (hi2 << 4)) - 32;
            const int sc = static_cast<int8_t>(p[192 + half * 8 + 2u * r]);
            v = __fmul_rn(d, static_cast<float>(sc * q));
        } else {  // Q5_K
            const uint8_t* p = data + blk * 176;
            float d = ld_half(p);
            if (!isfinite(d) || fabsf(d) < 1e-12f) d = 1.0f;
            const uint32_t bit = e * 5u;
            const uint8_t* f = p + 16 + (bit >> 3);
            const uint32_t two = static_cast<uint32_t>(f[0]) | (static_cast<uint32_t>((bit >> 3) + 1u < 160u ? f[1] : 0u) << 8);
            const int q = static_cast<int>((two >> (bit & 7u)) & 31u) - 16;
            v = __fmul_rn(static_cast<float>(q), d);
        }
        out[i] = v;
    }
}

}  // namespace

void launch_decode_rows(csdr_context* ctx, const csdr_segment* seg, const int32_t* rows_dev,
                        size_t n_rows, float* out_dev) {
    if (n_rows == 0) return;
    const Geometry& g = seg->g;
    DecodeGeom dg{g.rows, g.cols, g.rows_full, g.cols_full, g.tile_rows, g.tile_cols,
                  g.n_col_tiles, g.n_stages, g.k, g.n_atoms};
    const float* edges = seg->edges ? static_cast<const float*>(seg->edges->ptr) : nullptr;
    const bool vec = (g.cols % 4u == 0) && (g.tile_cols % 4u == 0);
    const uint32_t per_block = 256u * (vec ? 4u : 1u);
    dim3 grid(static_cast<unsigned>(n_rows), (g.cols + per_block - 1u) / per_block, 1);
    LaunchScope ls(ctx, KC_DECODE_ROWS);
    if (vec)
        hsdr_decode_rows_kernel<4><<<grid, 256, 0, ctx->stream>>>(
            static_cast<const float*>(seg->atoms->ptr), seg->codes_ptr(),
            static_cast<const float*>(seg->scales->ptr), edges, dg, rows_dev, out_dev);
    else
        hsdr_decode_rows_kernel<1><<<grid, 256, 0, ctx->stream>>>(
            static_cast<const float*>(seg->atoms->ptr), seg->codes_ptr(),
            static_cast<const float*>(seg->scales->ptr), edges, dg, rows_dev, out_dev);
    ls.done("hsdr_decode_rows_kernel");
}

int dequant_format_id(const char* fmt) {
    static const char* names[] = {"f32", "f16", "bf16", "i8", "q4_0", "q8_0", "q4_k", "q5_k", "q6_k"};
    if (!fmt) return -1;
    for (int i = 0; i < 9; ++i)
        if (std::strcmp(fmt, names[i]) == 0) return i;
    return -1;
}

size_t dequant_output_count(int fmt, size_t nbytes) {
    // Size checks and messages follow dequantizeSegmentToFP32.
    static const size_t unit[] = {4, 2, 2, 1, 18, 34, 144, 176, 210};
    static const size_t per[] = {1, 1, 1, 1, 32, 32, 256, 256, 256};
    static const char* what[] = {"FP32 byte size not a multiple of 4", "FP16 byte size not a multiple of 2",
                                 "BF16 byte size not a multiple of 2", "",
                                 "Q4_0 byte size not a multiple of 18", "Q8_0 byte size not a multiple of 34",
                                 "Q4_K byte size not a multiple of 144", "Q5_K byte size not a multiple of 176",
                                 "Q6_K byte size not a multiple of 210"};
    if (nbytes % unit[fmt]) throw Error(CSDR_ERR_FORMAT, std::string("HSDR dequant: ") + what[fmt]);
    return nbytes / unit[fmt] * per[fmt];
}

void launch_dequantize_inference(csdr_context* ctx, int fmt, const uint8_t* data_dev, size_t nbytes, size_t n_out,
                                 float* out_dev) {
    if (n_out == 0) return;
    if (fmt < Q4_K) {   // sequential formats: both sides of the reference agree on them
        launch_dequantize(ctx, fmt, data_dev, nbytes, n_out, 1.0f, 0.0f, out_dev);
        return;
    }
    LaunchScope ls(ctx, KC_DEQUANT);
    const unsigned grid = static_cast<unsigned>(
        std::min<size_t>((n_out + 255) / 256, static_cast<size_t>(ctx->sm_count) * 16));
    dequant_inference_kquant_kernel<<<grid, 256, 0, ctx->stream>>>(fmt, data_dev, n_out, out_dev);
    ls.done("dequant_inference_kquant_kernel");
}

void launch_dequantize(csdr_context* ctx, int fmt, const uint8_t* data_dev, size_t nbytes,
                       size_t n_out, float scale, float zero_point, float* out_dev) {
    if (n_out == 0) return;
    LaunchScope ls(ctx, KC_DEQUANT);
    if (fmt >= Q4_K) {
        const size_t n_blocks = n_out / 256;
        const unsigned grid = static_cast<unsigned>(
            std::min<size_t>((n_blocks + 7) / 8, static_cast<size_t>(ctx->sm_count) * 16));
        dequant_kquant_kernel<<<grid, 256, 0, ctx->stream>>>(fmt, data_dev, n_blocks, out_dev);
    } else {
        const unsigned grid = static_cast<unsigned>(
            std::min<size_t>((n_out + 255) / 256, static_cast<size_t>(ctx->sm_count) * 16));
        dequant_simple_kernel<<<grid, 256, 0, ctx->stream>>>(fmt, data_dev, n_out, scale, zero_point, out_dev);
    }
    (void)nbytes;
    ls.done("dequant kernel");
}

}  // namespace csdr
