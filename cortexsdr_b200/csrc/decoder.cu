// Device-resident decoder-layer driver: the block loop of run_transformer_decode
// (api/cortex_sdk.cpp:1543-1696) with every linear going through the compressed matmul,
// activations kept on the device, and a KV cache in place of the reference's
// whole-sequence recompute. Tensor parallelism row-shards every compressed weight
// (dictionaries replicated) and rejoins with NCCL all-gathers at the four points per
// block where a full vector is next consumed.
#include <dlfcn.h>
#include <nccl.h>

#include <algorithm>
#include <cctype>
#include <cstdlib>
#include <cstring>
#include <initializer_list>
#include <string>
#include <vector>

#include "internal.hpp"
#include "kernels/decoder_ops.hpp"
#include "kernels/gemm_tcgen05.hpp"
#include "kernels/gemv_fused.hpp"
#include "kernels/gemv_queue.hpp"

using namespace csdr;

namespace {

// ---- NCCL, bound at run time so the library loads (and the single-GPU path runs)
// without it. If a process already holds libnccl.so.2 (PyTorch's), that copy is used. ----
struct NcclApi {
    void* handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
};

NcclApi& nccl() {
    static NcclApi api;
    if (api.handle) return api;
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) throw Error(CSDR_ERR_UNSUPPORTED, std::string("NCCL not available: ") + dlerror());
    auto sym = [&](const char* n) {
        void* p = dlsym(h, n);
        if (!p) throw Error(CSDR_ERR_UNSUPPORTED, std::string("NCCL symbol missing: ") + n);
        return p;
    };
    api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(sym("ncclGetUniqueId"));
    api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(sym("ncclCommInitRank"));
    api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(sym("ncclCommDestroy"));
    api.AllGather = reinterpret_cast<decltype(api.AllGather)>(sym("ncclAllGather"));
    api.AllReduce = reinterpret_cast<decltype(api.AllReduce)>(sym("ncclAllReduce"));
    api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(sym("ncclGetErrorString"));
    api.handle = h;
    return api;
}

void nccl_check(ncclResult_t r, const char* what) {
    if (r != ncclSuccess)
        throw Error(CSDR_ERR_CUDA, std::string(what) + ": " + nccl().GetErrorString(r));
}

void rethrow_last(int rc) {
    if (rc != CSDR_OK) throw Error(rc, csdr_last_error());
}

// One linear layer of the model: an HSDR image (whole or this rank's row shard) or a
// stored-raw fp32 matrix.
struct Linear {
    const csdr_segment* seg = nullptr;  // owned by the archive
    csdr_segment* shard = nullptr;      // owned here
    DevPtr raw;                         // fp32 (rows_local x cols), rows already sliced
    uint32_t rows = 0, cols = 0, rows_local = 0, cols_local = 0;
    const csdr_segment* use() const { return shard ? shard : seg; }
};

struct Layer {
    DevPtr attn_norm, ffn_norm;
    Linear q, k, v, o, gate, up, down;
};

}  // namespace

struct csdr_decoder {
    csdr_archive* ar = nullptr;
    csdr_context* ctx = nullptr;
    csdr_decoder_config cfg{};
    uint32_t P = 1, rank = 0;
    uint32_t QH_l = 0, KVH_l = 0, QD_l = 0, KVD_l = 0, I_l = 0, H_l = 0, V_l = 0;
    uint32_t T_max = 0;
    ncclComm_t comm = nullptr;
    Linear emb, lm_head;
    DevPtr out_norm;
    std::vector<Layer> layers;
    DevPtr kcache, vcache;  // [layer][seq][pos][kv head (local)][head_dim]
    size_t cache_layer_stride = 0;   // elements
    int kv_dtype = CSDR_DTYPE_F32;   // fp32 as the reference computes, or fp16 / bf16 (half the cache traffic; sums stay fp32)
    size_t kv_es = 4;
    std::vector<int32_t> pos_host;
    // token selection of the reference's generation loop (off: plain argmax): temperature and a
    // bitmap of the tokens each sequence has produced, [max_batch][seen_words]
    bool policy = false;
    float temperature = 1.0f;
    DevPtr seen;
    uint32_t seen_words = 0;
    DevPtr pos_dev, tokens_dev, seq_of, pos_of, next_dev;
    DevPtr hidden, normed, q, k, v, att, proj, gate, up, staged, logits, logits_l;
    // projections of a group between its two launches, behind a block of per-token sums of
    // squares: [sum_pad floats][Dx of every member]; tensor-parallel ranks add theirs up in place
    DevPtr dxbuf;
    uint32_t sum_pad = 0;
    // the RMS-norm half that rides on the output and down gathers of a decode step:
    // [kNextNormCtas][16] shares of the sums of squares, and how many CTAs of the last such
    // gather left shares for the projection launch behind it to add up (0: none pending)
    DevPtr norm_scratch;
    uint32_t norm_pending = 0;
    // every token of the pass being run belongs to a different sequence (a decode step, or a
    // one-token forward): set by the entry points before the block loop
    bool distinct_seqs = false;
    // peer-memory exchange of partial projections between tensor-parallel ranks (steps of at
    // most 16 tokens); until the host program has passed the peers' handles in, NCCL sums them
    DevPtr xch_region;
    Exchange xch;                  // ranks == 0 until imported
    bool xch_use = false;          // imported AND chosen: CSDR_TP_EXCHANGE=peer|nccl, default peer from 3 ranks up
    uint32_t xch_blk = 0;
    std::vector<void*> xch_maps;   // peers' regions as mapped here (closed on destroy)
    // bf16 hi/lo planes of the three activation widths the projections consume (hidden,
    // attention output, SwiGLU product) for steps that run on the tensor cores
    DevPtr xp_h, xp_att, xp_act;
    bool planes_capable = false;
    bool queue_capable = false;    // every block linear an HSDR row-tile image the GEMV queue takes
    uint32_t fold_max_mt = 0;      // widest token tile at which the one-launch GEMVs take the blocks' glue (0: never)
    ~csdr_decoder() {
        for (void* m : xch_maps)
            if (m) cudaIpcCloseMemHandle(m);
        auto drop = [](Linear& l) {
            if (l.shard) csdr_segment_destroy(l.shard);
        };
        drop(emb);
        drop(lm_head);
        for (auto& L : layers) {
            drop(L.q); drop(L.k); drop(L.v); drop(L.o); drop(L.gate); drop(L.up); drop(L.down);
        }
    }
};

namespace {

DevPtr dev_alloc(csdr_context* ctx, size_t bytes) { return std::make_shared<DeviceBuffer>(bytes, ctx->device); }
float* F(const DevPtr& p) { return static_cast<float*>(p->ptr); }
int32_t* I32(const DevPtr& p) { return static_cast<int32_t*>(p->ptr); }

std::vector<float> load_raw(csdr_archive* ar, const std::string& name, size_t want_floats) {
    size_t n = 0;
    int rc = csdr_archive_load_segment(ar, name.c_str(), nullptr, 0, &n);
    if (rc != CSDR_OK && rc != CSDR_ERR_BUFFER) rethrow_last(rc);
    std::vector<float> v((n + 3) / 4);
    rethrow_last(csdr_archive_load_segment(ar, name.c_str(), v.data(), v.size() * 4, &n));
    if (want_floats && v.size() < want_floats)
        throw Error(CSDR_ERR_GEOMETRY, "tensor '" + name + "' is smaller than the decoder config needs");
    return v;
}

DevPtr load_vector(csdr_decoder* d, const std::string& name, uint32_t n) {
    std::vector<float> v = load_raw(d->ar, name, n);
    DevPtr p = upload(d->ctx, v.data(), static_cast<size_t>(n) * 4);
    CSDR_CUDA(cudaStreamSynchronize(d->ctx->stream));
    return p;
}

// Resolve a linear by name. A tensor-parallel rank keeps output rows [rank*R/P, (rank+1)*R/P) of
// the code stream (row_shard: q, k, v, gate, up, the head - their input is the replicated
// hidden state, their output stays on the rank) or input columns [rank*C/P, (rank+1)*C/P) of the
// dictionary (col_shard: the output and down projections - their input is the rank's slice of
// the heads / intermediate width; every rank projects its slice, the partial projections are
// summed over the ranks, and every rank gathers all rows into its copy of the hidden state).
Linear load_linear(csdr_decoder* d, const std::string& name, uint32_t rows, uint32_t cols, bool row_shard,
                   bool col_shard) {
    csdr_segment_header h{};
    int rc = csdr_archive_find(d->ar, name.c_str(), &h);
    if (rc == CSDR_ERR_NOT_FOUND) throw Error(CSDR_ERR_NOT_FOUND, "decoder: tensor not in archive: " + name);
    rethrow_last(rc);
    Linear l;
    l.rows = rows;
    l.cols = cols;
    const uint32_t PR = row_shard ? d->P : 1u, PC = col_shard ? d->P : 1u;
    if (rows % PR || cols % PC)
        throw Error(CSDR_ERR_GEOMETRY, "decoder: shape of '" + name + "' does not divide by the tensor-parallel size");
    l.rows_local = rows / PR;
    l.cols_local = cols / PC;
    const uint32_t r0 = (row_shard ? d->rank : 0u) * l.rows_local;
    const uint32_t c0 = (col_shard ? d->rank : 0u) * l.cols_local;
    if (h.strategy_id == kHSDRStrategyId) {
        rethrow_last(csdr_archive_segment(d->ar, name.c_str(), &l.seg));
        if (l.seg->g.rows != rows || l.seg->g.cols != cols)
            throw Error(CSDR_ERR_GEOMETRY, "decoder: shape of '" + name + "' does not match the config");
        csdr_segment* by_cols = nullptr;
        if (PC > 1) rethrow_last(csdr_segment_shard_cols(d->ctx, l.seg, c0, c0 + l.cols_local, &by_cols));
        if (PR > 1) {
            rc = csdr_segment_shard_rows(d->ctx, by_cols ? by_cols : l.seg, r0, r0 + l.rows_local, &l.shard);
            if (by_cols) csdr_segment_destroy(by_cols);   // the row shard shares its dictionary
            rethrow_last(rc);
        } else {
            l.shard = by_cols;
        }
    } else if (h.strategy_id == 0) {
        if (d->P > 1)
            throw Error(CSDR_ERR_UNSUPPORTED, "decoder: tensor-parallel decoding needs HSDR-encoded linears ('" + name +
                                                  "' is stored raw)");
        // stored as it came from the model file: fp32, or a source dtype (f16, bf16, q4_0, q8_0,
        // q4_k, q5_k, q6_k) that is widened to fp32 on the device once, in the element order of
        // the reference's inference side (decodeSupportedGGUFQuantized,
        // SparseInferenceEngine.cpp:276-469) - ggml's order for the k-quants, which differs from
        // the order the encoder's dequantizeSegmentToFP32 assumes
        std::string fmt = h.data_format ? h.data_format : "";
        for (char& ch : fmt) ch = static_cast<char>(std::tolower(static_cast<unsigned char>(ch)));
        const size_t want = static_cast<size_t>(rows) * cols;
        if (fmt.empty() || fmt == "f32" || fmt == "fp32" || fmt == "float32") {
            std::vector<float> w = load_raw(d->ar, name, want);
            l.raw = upload(d->ctx, w.data(), want * 4);
        } else {
            const int id = dequant_format_id(fmt == "fp16" || fmt == "float16" || fmt == "half" ? "f16"
                                             : fmt == "bfloat16"                                ? "bf16"
                                                                                                : fmt.c_str());
            if (id < 0)
                throw Error(CSDR_ERR_UNSUPPORTED, "decoder: tensor '" + name + "' is stored as '" + fmt +
                                                      "', which this library does not widen");
            size_t nbytes = 0;
            int rc2 = csdr_archive_load_segment(d->ar, name.c_str(), nullptr, 0, &nbytes);
            if (rc2 != CSDR_OK && rc2 != CSDR_ERR_BUFFER) rethrow_last(rc2);
            std::vector<uint8_t> bytes(nbytes);
            rethrow_last(csdr_archive_load_segment(d->ar, name.c_str(), bytes.data(), bytes.size(), &nbytes));
            if (dequant_output_count(id, nbytes) < want)
                throw Error(CSDR_ERR_GEOMETRY, "tensor '" + name + "' is smaller than the decoder config needs");
            DevPtr packed = upload(d->ctx, bytes.data(), nbytes);
            l.raw = dev_alloc(d->ctx, dequant_output_count(id, nbytes) * 4);
            launch_dequantize_inference(d->ctx, id, static_cast<const uint8_t*>(packed->ptr), nbytes,
                                        dequant_output_count(id, nbytes), F(l.raw));
        }
        CSDR_CUDA(cudaStreamSynchronize(d->ctx->stream));
    } else {
        throw Error(CSDR_ERR_UNSUPPORTED, "decoder: tensor '" + name + "' uses a strategy this library does not decode");
    }
    return l;
}

// y (T x rows_local) = x (T x cols) * W^T, token-major both sides.
void linear(csdr_decoder* d, const Linear& l, const float* x, uint32_t T, float* y) {
    if (l.raw) {
        MatmulArgs a;
        a.x = x;
        a.x_layout = CSDR_LAYOUT_TOKEN_MAJOR;
        a.batch = T;
        a.y = y;
        a.y_layout = CSDR_LAYOUT_TOKEN_MAJOR;
        launch_dense_matmul(d->ctx, F(l.raw), l.rows_local, l.cols, a);
    } else {
        rethrow_last(csdr_matmul_device_async(d->ctx, l.use(), x, CSDR_DTYPE_F32, CSDR_LAYOUT_TOKEN_MAJOR, T, y,
                                              CSDR_LAYOUT_TOKEN_MAJOR, nullptr));
    }
}

// Several linears over the same x in as few launches as the matmul layer allows.
void linear_group(csdr_decoder* d, std::initializer_list<const Linear*> ls, const float* x, uint32_t T,
                  std::initializer_list<float*> ys) {
    bool all_hsdr = true;
    for (const Linear* l : ls) all_hsdr = all_hsdr && !l->raw;
    if (!all_hsdr) {
        auto y = ys.begin();
        for (const Linear* l : ls) linear(d, *l, x, T, *y++);
        return;
    }
    const csdr_segment* segs[8];
    float* outs[8];
    size_t n = 0;
    auto y = ys.begin();
    for (const Linear* l : ls) {
        segs[n] = l->use();
        outs[n++] = *y++;
    }
    rethrow_last(csdr_matmul_group_device_async(d->ctx, segs, n, x, CSDR_DTYPE_F32, CSDR_LAYOUT_TOKEN_MAJOR, T, outs,
                                                CSDR_LAYOUT_TOKEN_MAJOR));
}

void embed(csdr_decoder* d, uint32_t T) {
    if (d->emb.raw) op_gather_rows(d->ctx, F(d->emb.raw), d->cfg.vocab, d->cfg.hidden, I32(d->tokens_dev), T, F(d->hidden));
    else launch_decode_rows(d->ctx, d->emb.use(), I32(d->tokens_dev), T, F(d->hidden));
}

__nv_bfloat16* BF(const DevPtr& p) { return static_cast<__nv_bfloat16*>(p->ptr); }

// Sum the ranks' partial projections (and, when asked, the block of per-token sums of squares
// in front of them) in place. One collective per group of linears.
void sum_over_ranks(csdr_decoder* d, float* from, size_t floats) {
    if (d->P == 1) return;
    nccl_check(nccl().AllReduce(from, from, floats, ncclFloat, ncclSum, d->comm, d->ctx->stream), "ncclAllReduce");
}

// Rotary embedding of q and k, the cache write and attention of block li over d->q, d->k, d->v:
// one launch when every token of the step belongs to a different sequence (a decode step), else
// the rotary kernel first (tokens of one sequence attend to each other's cache rows).
void attend(csdr_decoder* d, uint32_t li, uint32_t T, float* out, __nv_bfloat16* hi = nullptr, __nv_bfloat16* lo = nullptr) {
    const csdr_decoder_config& c = d->cfg;
    csdr_context* ctx = d->ctx;
    void* kc = static_cast<char*>(d->kcache->ptr) + li * d->cache_layer_stride * d->kv_es;
    void* vc = static_cast<char*>(d->vcache->ptr) + li * d->cache_layer_stride * d->kv_es;
    if (d->distinct_seqs && ctx->attention_rope_fold && attention_step_supported(c.head_dim)) {
        op_attention_step(ctx, F(d->q), F(d->k), F(d->v), c.rope_theta, kc, vc, d->kv_dtype, I32(d->seq_of), I32(d->pos_of), T,
                          d->QH_l, d->KVH_l, c.head_dim, c.max_seq, out, hi, lo);
        return;
    }
    op_rope_cache(ctx, F(d->q), F(d->k), F(d->v), kc, vc, d->kv_dtype, I32(d->seq_of), I32(d->pos_of), T, d->QH_l, d->KVH_l,
                  c.head_dim, c.max_seq, c.rope_theta);
    op_attention(ctx, F(d->q), kc, vc, d->kv_dtype, I32(d->seq_of), I32(d->pos_of), T, d->QH_l, d->KVH_l, c.head_dim, c.max_seq, out,
                 hi, lo);
}

// One group of linears over activation planes: projection launch, rank sum, gather launch.
// `normed`: the planes hold w*h and the gather applies 1/rms from the sums of squares.
// `act_hi`: the group is (gate, up) and, when the step is a single token tile, the gather writes
// silu(gate) * up into these planes and returns true; else the caller applies SiLU itself.
// `partial`: every rank holds a column slice of the dictionaries, so the projections must be
// summed over the ranks before the gather.
// `next_w` (one linear): the first half of the next RMS normalisation of the output - planes of
// next_w * y into the hidden planes, sums of y^2 into the sums block - rides on the gather when
// the step is a single token tile (the gather leaves shares of the sums, the next call's
// projection launch adds them up), and is a launch of its own behind the gather otherwise.
bool wide(csdr_decoder* d, std::initializer_list<const Linear*> ls, const __nv_bfloat16* planes, size_t plane_elems,
          uint32_t T, bool normed, bool partial, const float* sums, std::initializer_list<WideOut> outs,
          __nv_bfloat16* act_hi = nullptr, __nv_bfloat16* act_lo = nullptr, const float* next_w = nullptr) {
    const csdr_segment* segs[4];
    WideOut o[4];
    uint32_t n = 0;
    auto it = outs.begin();
    for (const Linear* l : ls) {
        segs[n] = l->use();
        o[n++] = *it++;
    }
    const XPlanesView xp{planes, planes + plane_elems};
    float* base = F(d->dxbuf);
    TokenScale ts{};
    if (normed) ts = TokenScale{sums, 1.0f / static_cast<float>(d->cfg.hidden), d->cfg.rms_eps};
    NextNorm nn{};
    if (next_w) {
        __nv_bfloat16* h_hi = BF(d->xp_h);
        nn = NextNorm{next_w, h_hi, h_hi + static_cast<size_t>(T) * d->H_l, F(d->norm_scratch)};
    }
    // shares left by the previous call's gather: this call's projection adds them up
    const NormShares shares{F(d->norm_scratch), d->norm_pending, F(d->dxbuf)};
    d->norm_pending = 0;
    auto gather = [&](const WideDx& w) {
        const uint32_t rode = launch_wide_gather(d->ctx, segs, n, w, T, o, CSDR_LAYOUT_TOKEN_MAJOR, ts, next_w ? &nn : nullptr);
        if (next_w && !rode) op_scale_sumsq_planes(d->ctx, o[0].y, next_w, T, d->H_l, nn.hi, nn.lo, F(d->dxbuf));
        d->norm_pending = rode;
    };
    uint32_t total_atoms = 0;
    for (uint32_t i = 0; i < n; ++i) total_atoms += segs[i]->g.n_atoms;
    if (partial && d->xch_use && T <= 16u && d->sum_pad + static_cast<size_t>(total_atoms) * 16u <= d->xch_blk) {
        // the projection kernel stores its finished rows into every rank's exchange slot and
        // raises the flags; a small launch waits for all ranks and sums the slots into the local
        // block; the gather then runs as on one GPU
        const WideDx w = launch_wide_project(d->ctx, segs, n, xp, T, base + d->sum_pad, &d->xch, base, nullptr, &shares);
        launch_exchange_reduce(d->ctx, d->xch, d->sum_pad, w.floats, w.base);
        if (act_hi) {
            launch_wide_gather_swiglu(d->ctx, segs, w, T, ts, act_hi, act_lo);
            return true;
        }
        gather(w);
        return false;
    }
    const WideDx w = launch_wide_project(d->ctx, segs, n, xp, T, base + d->sum_pad, nullptr, nullptr, nullptr, &shares);
    if (partial) sum_over_ranks(d, w.base, w.floats);
    if (act_hi && w.tile_mt) {
        launch_wide_gather_swiglu(d->ctx, segs, w, T, ts, act_hi, act_lo);
        return true;
    }
    gather(w);
    return false;
}

// The block loop on the tensor cores (steps of at least the tensor-core threshold on one GPU;
// every step under tensor parallelism). Every glue kernel hands its result to the next
// projection as bf16 planes; q|k|v and gate|up share a projection launch and a gather launch;
// the residual additions ride on the gathers of the output and down projections; RMS
// normalisation is split into "planes of w*h + sums of squares" before the projection (for single
// token tiles part of the gather that produced h, else a launch of its own) and "times 1/rms" in
// the gather; SwiGLU is folded into the gate|up gather for single token tiles.
// With P ranks the hidden state is replicated; heads, KV cache and intermediate width are sliced
// P ways, q|k|v|gate|up by code rows, and the output and down projections by dictionary columns,
// so that the only exchanges are the sums of those two projections' partial results (K x T
// floats each): two per block, each of them a barrier across the ranks.
// Leaves the final hidden states in d->hidden and the final norm's planes and sums in
// xp_h / dxbuf.
void run_blocks_planes(csdr_decoder* d, uint32_t T) {
    const csdr_decoder_config& c = d->cfg;
    csdr_context* ctx = d->ctx;
    const uint32_t HD = c.head_dim, Hl = d->H_l;
    float* sums = F(d->dxbuf);
    __nv_bfloat16* h_hi = BF(d->xp_h);
    __nv_bfloat16* a_hi = BF(d->xp_att);
    __nv_bfloat16* i_hi = BF(d->xp_act);
    const size_t h_n = static_cast<size_t>(T) * Hl, a_n = static_cast<size_t>(T) * d->QD_l, i_n = static_cast<size_t>(T) * d->I_l;
    op_scale_sumsq_planes(ctx, F(d->hidden), F(d->layers[0].attn_norm), T, Hl, h_hi, h_hi + h_n, sums);
    d->norm_pending = 0;    // a step that ended in an error may have left shares behind
    for (uint32_t li = 0; li < c.n_layers; ++li) {
        Layer& L = d->layers[li];
        wide(d, {&L.q, &L.k, &L.v}, h_hi, h_n, T, true, false, sums,
             {WideOut{F(d->q), nullptr, nullptr}, WideOut{F(d->k), nullptr, nullptr}, WideOut{F(d->v), nullptr, nullptr}});
        attend(d, li, T, nullptr, a_hi, a_hi + a_n);
        wide(d, {&L.o}, a_hi, a_n, T, false, true, nullptr, {WideOut{F(d->hidden), nullptr, F(d->hidden)}}, nullptr, nullptr,
             F(L.ffn_norm));
        if (!wide(d, {&L.gate, &L.up}, h_hi, h_n, T, true, false, sums,
                  {WideOut{F(d->gate), nullptr, nullptr}, WideOut{F(d->up), nullptr, nullptr}}, i_hi, i_hi + i_n))
            op_silu_mul_planes(ctx, F(d->gate), F(d->up), i_n, i_hi, i_hi + i_n);
        // the last block's sums have no projection launch behind them to add shares up
        const bool last = li + 1 == c.n_layers;
        wide(d, {&L.down}, i_hi, i_n, T, false, true, nullptr, {WideOut{F(d->hidden), nullptr, F(d->hidden)}}, nullptr, nullptr,
             last ? nullptr : F(d->layers[li + 1].attn_norm));
        if (last) op_scale_sumsq_planes(ctx, F(d->hidden), F(d->out_norm), T, Hl, h_hi, h_hi + h_n, sums);
    }
}

// Steps of at most four tokens on one GPU: a block is two or three launches. The output projection,
// gate, up and down of block n and q, k, v of block n + 1 run as ONE list on the persistent GEMV
// kernel, with the residual additions and SwiGLU as epilogues of its gather role and the two RMS
// normalisations folded into the products that consume them; attention (with the rotary
// embedding and the cache write inside it on a decode step) stays a kernel of its own between
// two lists.
bool use_queue(const csdr_decoder* d, uint32_t T) {
    return d->queue_capable && d->P == 1 && T <= 4u && d->ctx->gemv_queue && d->ctx->decoder_queue;
}

void run_blocks_queue(csdr_decoder* d, uint32_t T) {
    const csdr_decoder_config& c = d->cfg;
    csdr_context* ctx = d->ctx;
    const uint32_t H = c.hidden, HD = c.head_dim;
    auto item = [&](const Linear& l, const float* x, float* y) {
        return QueueItem{l.use(), x, CSDR_DTYPE_F32, CSDR_LAYOUT_TOKEN_MAJOR, T, y, CSDR_LAYOUT_TOKEN_MAJOR, nullptr};
    };
    float* xn = F(d->normed);   // the first norm is a kernel of its own; the others ride on the lists
    op_rmsnorm(ctx, F(d->hidden), F(d->layers[0].attn_norm), T, H, c.rms_eps, xn);
    {
        const Layer& L = d->layers[0];
        const QueueItem first[3] = {item(L.q, xn, F(d->q)), item(L.k, xn, F(d->k)), item(L.v, xn, F(d->v))};
        launch_gemv_queue(ctx, first, 3);
    }
    for (uint32_t li = 0; li < c.n_layers; ++li) {
        const Layer& L = d->layers[li];
        attend(d, li, T, F(d->att));
        QueueItem list[7];
        uint32_t n = 0;
        list[n] = item(L.o, F(d->att), F(d->hidden));            // 0: h += Wo att
        list[n].residual = F(d->hidden);
        ++n;
        list[n] = item(L.gate, F(d->hidden), F(d->gate));        // 1: gate = Wg norm(h)
        list[n].dep = 0;
        list[n].norm_weight = F(L.ffn_norm);
        ++n;
        list[n] = item(L.up, F(d->hidden), F(d->up));            // 2: act = silu(gate) * (Wu norm(h))
        list[n].dep = 0;
        list[n].norm_weight = F(L.ffn_norm);
        list[n].swiglu_gate = F(d->gate);
        ++n;
        list[n] = item(L.down, F(d->up), F(d->hidden));          // 3: h += Wd act
        list[n].dep = 2;
        list[n].residual = F(d->hidden);
        ++n;
        if (li + 1 < c.n_layers) {
            const Layer& N = d->layers[li + 1];
            const Linear* qkv[3] = {&N.q, &N.k, &N.v};
            float* outs[3] = {F(d->q), F(d->k), F(d->v)};
            for (int j = 0; j < 3; ++j) {                        // 4..6: q, k, v of the next block
                list[n] = item(*qkv[j], F(d->hidden), outs[j]);
                list[n].dep = 3;
                list[n].norm_weight = F(N.attn_norm);
                ++n;
            }
        }
        for (uint32_t i = 0; i < n; ++i) list[i].norm_eps = c.rms_eps;
        launch_gemv_queue(ctx, list, n);
    }
    op_rmsnorm(ctx, F(d->hidden), F(d->out_norm), T, H, c.rms_eps, F(d->normed));
}

// A short step with the glue of api/cortex_sdk.cpp:1569-1679 folded into the one-launch GEMVs: the
// two RMS normalisations ride on the products that consume them (q|k|v, gate|up), the residual
// additions on the output and down projections, SwiGLU on the (gate, up) pair. Five launches per
// block on a decode step (q|k|v, attention with the rotary embedding and the cache write inside,
// output, gate|up, down; six when the rotary kernel runs on its own) instead of nine.
uint32_t token_tile(uint32_t T) { return T <= 1 ? 1u : T <= 2 ? 2u : T <= 4 ? 4u : T <= 8 ? 8u : 16u; }
bool use_folded(const csdr_decoder* d, uint32_t T) {
    return d->P == 1 && T <= 16u && d->ctx->decoder_fold && token_tile(T) <= d->fold_max_mt;
}
void fused_with_glue(csdr_decoder* d, std::initializer_list<const Linear*> ls, const float* x, uint32_t T,
                     std::initializer_list<float*> ys, const FusedGlue& glue) {
    const csdr_segment* segs[kMaxFusedGroup];
    float* outs[kMaxFusedGroup];
    uint32_t n = 0;
    auto y = ys.begin();
    for (const Linear* l : ls) {
        segs[n] = l->use();
        outs[n++] = *y++;
    }
    launch_gemv_fused(d->ctx, segs, n, x, CSDR_DTYPE_F32, CSDR_LAYOUT_TOKEN_MAJOR, T, 0, T, outs, CSDR_LAYOUT_TOKEN_MAJOR,
                      nullptr, static_cast<int>(token_tile(T)), &glue);
}
void run_blocks_folded(csdr_decoder* d, uint32_t T) {
    const csdr_decoder_config& c = d->cfg;
    csdr_context* ctx = d->ctx;
    const uint32_t H = c.hidden, HD = c.head_dim;
    float* h = F(d->hidden);
    for (uint32_t li = 0; li < c.n_layers; ++li) {
        const Layer& L = d->layers[li];
        FusedGlue g_attn;
        g_attn.norm_w = F(L.attn_norm);
        g_attn.norm_eps = c.rms_eps;
        fused_with_glue(d, {&L.q, &L.k, &L.v}, h, T, {F(d->q), F(d->k), F(d->v)}, g_attn);
        attend(d, li, T, F(d->att));
        FusedGlue g_res;
        g_res.residual[0] = h;
        fused_with_glue(d, {&L.o}, F(d->att), T, {h}, g_res);                       // h += Wo att
        FusedGlue g_mlp;
        g_mlp.norm_w = F(L.ffn_norm);
        g_mlp.norm_eps = c.rms_eps;
        g_mlp.swiglu = true;
        fused_with_glue(d, {&L.gate, &L.up}, h, T, {F(d->gate), F(d->up)}, g_mlp);  // up = silu(gate) * up
        fused_with_glue(d, {&L.down}, F(d->up), T, {h}, g_res);                     // h += Wd act
    }
    op_rmsnorm(ctx, h, F(d->out_norm), T, H, c.rms_eps, F(d->normed));
}

bool use_planes(const csdr_decoder* d, uint32_t T) {
    if (d->P > 1) return true;
    const csdr_context* ctx = d->ctx;
    return d->planes_capable && ctx->tensor_cores && ctx->tma && T >= ctx->tc_min_batch;
}

// All blocks over T tokens whose (sequence, position) pairs sit in seq_of/pos_of. On return
// either d->normed holds the final-normed hidden states (fp32 path), or the planes path's state
// described above does.
void run_blocks(csdr_decoder* d, uint32_t T) {
    const csdr_decoder_config& c = d->cfg;
    csdr_context* ctx = d->ctx;
    const uint32_t H = c.hidden, HD = c.head_dim;
    if (use_planes(d, T)) {
        run_blocks_planes(d, T);
        return;
    }
    if (use_queue(d, T)) {
        run_blocks_queue(d, T);
        return;
    }
    if (use_folded(d, T)) {
        run_blocks_folded(d, T);
        return;
    }
    op_rmsnorm(ctx, F(d->hidden), F(d->layers[0].attn_norm), T, H, c.rms_eps, F(d->normed));
    for (uint32_t li = 0; li < c.n_layers; ++li) {
        Layer& L = d->layers[li];
        linear_group(d, {&L.q, &L.k, &L.v}, F(d->normed), T, {F(d->q), F(d->k), F(d->v)});
        attend(d, li, T, F(d->att));
        linear(d, L.o, F(d->att), T, F(d->proj));
        op_add_rmsnorm(ctx, F(d->hidden), F(d->proj), F(L.ffn_norm), T, H, c.rms_eps, F(d->normed));
        linear_group(d, {&L.gate, &L.up}, F(d->normed), T, {F(d->gate), F(d->up)});
        op_silu_mul(ctx, F(d->gate), F(d->up), static_cast<size_t>(T) * d->I_l, F(d->gate));
        linear(d, L.down, F(d->gate), T, F(d->proj));
        const float* next_norm = li + 1 < c.n_layers ? F(d->layers[li + 1].attn_norm) : F(d->out_norm);
        op_add_rmsnorm(ctx, F(d->hidden), F(d->proj), next_norm, T, H, c.rms_eps, F(d->normed));
    }
}

// Final-normed hidden states of all T tokens into d->normed (what forward() hands back); only
// the planes path has work to do here.
void materialise_normed(csdr_decoder* d, uint32_t T) {
    if (!use_planes(d, T)) return;
    op_norm_from_sumsq(d->ctx, F(d->hidden), F(d->out_norm), F(d->dxbuf), T, d->cfg.hidden, d->cfg.hidden, d->cfg.rms_eps,
                       F(d->normed));
}

// logits (n x vocab) of tokens [t0, t0 + n) of the T that run_blocks just processed. Ranks hold
// row shards of the head (whole dictionary, replicated hidden state): the logits are
// all-gathered.
void run_logits(csdr_decoder* d, uint32_t T, uint32_t t0, uint32_t n) {
    if (!use_planes(d, T)) {
        linear(d, d->lm_head, F(d->normed) + static_cast<size_t>(t0) * d->cfg.hidden, n, F(d->logits));
        return;
    }
    // the final norm's planes and sums are in place; rows t0.. of them feed the head
    float* base = F(d->dxbuf);
    const size_t h_n = static_cast<size_t>(T) * d->cfg.hidden;
    const __nv_bfloat16* hi = BF(d->xp_h) + static_cast<size_t>(t0) * d->cfg.hidden;
    const csdr_segment* seg = d->lm_head.use();
    const XPlanesView xp{hi, hi + h_n};
    const WideDx w = launch_wide_project(d->ctx, &seg, 1, xp, n, base + d->sum_pad);
    const TokenScale ts{base + t0, 1.0f / static_cast<float>(d->cfg.hidden), d->cfg.rms_eps};
    const WideOut out{d->P > 1 ? F(d->logits_l) : F(d->logits), nullptr, nullptr};
    launch_wide_gather(d->ctx, &seg, 1, w, n, &out, CSDR_LAYOUT_TOKEN_MAJOR, ts);
    if (d->P > 1) {
        nccl_check(nccl().AllGather(F(d->logits_l), F(d->staged), static_cast<size_t>(n) * d->V_l, ncclFloat, d->comm,
                                    d->ctx->stream),
                   "ncclAllGather");
        op_unshard(d->ctx, F(d->staged), d->P, n, d->V_l, F(d->logits), false);
    }
}

void need(csdr_decoder* d) {
    if (!d) throw Error(CSDR_ERR_INVALID_ARG, "decoder is null");
    require_ctx(d->ctx);
}

}  // namespace

extern "C" {

int csdr_nccl_unique_id(void* id128) {
    return guard([&] {
        if (!id128) throw Error(CSDR_ERR_INVALID_ARG, "null argument");
        static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId is 128 bytes");
        ncclUniqueId id;
        nccl_check(nccl().GetUniqueId(&id), "ncclGetUniqueId");
        std::memcpy(id128, &id, sizeof(id));
    });
}

int csdr_nccl_comm_create(csdr_context* ctx, const void* id128, int rank, int world, void** comm_out) {
    return guard([&] {
        require_ctx(ctx);
        if (!id128 || !comm_out || world < 1 || rank < 0 || rank >= world)
            throw Error(CSDR_ERR_INVALID_ARG, "bad communicator arguments");
        ncclUniqueId id;
        std::memcpy(&id, id128, sizeof(id));
        ncclComm_t comm = nullptr;
        nccl_check(nccl().CommInitRank(&comm, world, id, rank), "ncclCommInitRank");
        *comm_out = comm;
    });
}

int csdr_nccl_comm_destroy(void* comm) {
    return guard([&] {
        if (comm) nccl_check(nccl().CommDestroy(static_cast<ncclComm_t>(comm)), "ncclCommDestroy");
    });
}

int csdr_decoder_create(csdr_archive* ar, const csdr_decoder_config* cfg, csdr_decoder** out) {
    return guard([&] {
        if (!ar || !cfg || !out) throw Error(CSDR_ERR_INVALID_ARG, "null argument");
        const csdr_segment* probe = nullptr;  // also proves the archive has a device context
        auto d = std::make_unique<csdr_decoder>();
        d->ar = ar;
        d->cfg = *cfg;
        const csdr_decoder_config& c = d->cfg;
        if (!c.n_layers || !c.hidden || !c.q_heads || !c.kv_heads || !c.head_dim || !c.inter || !c.vocab ||
            !c.max_seq || !c.max_batch || c.q_heads % c.kv_heads)
            throw Error(CSDR_ERR_INVALID_ARG, "decoder config has a zero or inconsistent field");
        d->P = c.tp_size ? c.tp_size : 1;
        d->rank = c.tp_rank;
        if (d->rank >= d->P) throw Error(CSDR_ERR_INVALID_ARG, "tp_rank out of range");
        if (d->P > 1 && !c.nccl_comm) throw Error(CSDR_ERR_INVALID_ARG, "tensor parallelism needs an NCCL communicator");
        if (c.q_heads % d->P || c.kv_heads % d->P || c.hidden % d->P || c.inter % d->P || c.vocab % d->P)
            throw Error(CSDR_ERR_GEOMETRY, "heads, hidden, intermediate and vocab sizes must divide by the tensor-parallel size");
        d->comm = static_cast<ncclComm_t>(c.nccl_comm);
        // the context comes with the first HSDR image
        int rc = csdr_archive_segment(ar, "token_embd.weight", &probe);
        if (rc == CSDR_OK) d->ctx = probe->ctx;
        else if (rc == CSDR_ERR_STRATEGY) {
            rethrow_last(csdr_archive_segment(ar, "blk.0.attn_q.weight", &probe));
            d->ctx = probe->ctx;
        } else rethrow_last(rc);
        require_ctx(d->ctx);
        const uint32_t H = c.hidden, HD = c.head_dim, QD = c.q_heads * HD, KVD = c.kv_heads * HD;
        d->QH_l = c.q_heads / d->P;
        d->KVH_l = c.kv_heads / d->P;
        d->QD_l = QD / d->P;
        d->KVD_l = KVD / d->P;
        d->I_l = c.inter / d->P;
        d->H_l = H;   // the residual stream is replicated on every rank
        d->V_l = c.vocab / d->P;
        d->emb = load_linear(d.get(), "token_embd.weight", c.vocab, H, false, false);
        {
            csdr_segment_header h{};
            const char* head = csdr_archive_find(ar, "output.weight", &h) == CSDR_OK ? "output.weight"
                               : csdr_archive_find(ar, "lm_head.weight", &h) == CSDR_OK ? "lm_head.weight"
                                                                                        : "token_embd.weight";
            d->lm_head = load_linear(d.get(), head, c.vocab, H, true, false);
        }
        d->out_norm = load_vector(d.get(), "output_norm.weight", H);
        d->layers.resize(c.n_layers);
        for (uint32_t i = 0; i < c.n_layers; ++i) {
            const std::string p = "blk." + std::to_string(i) + ".";
            Layer& L = d->layers[i];
            L.attn_norm = load_vector(d.get(), p + "attn_norm.weight", H);
            L.ffn_norm = load_vector(d.get(), p + "ffn_norm.weight", H);
            L.q = load_linear(d.get(), p + "attn_q.weight", QD, H, true, false);
            L.k = load_linear(d.get(), p + "attn_k.weight", KVD, H, true, false);
            L.v = load_linear(d.get(), p + "attn_v.weight", KVD, H, true, false);
            L.o = load_linear(d.get(), p + "attn_output.weight", H, QD, false, true);
            L.gate = load_linear(d.get(), p + "ffn_gate.weight", c.inter, H, true, false);
            L.up = load_linear(d.get(), p + "ffn_up.weight", c.inter, H, true, false);
            L.down = load_linear(d.get(), p + "ffn_down.weight", H, c.inter, false, true);
        }
        csdr_context* ctx = d->ctx;
        d->T_max = std::max(c.max_seq, c.max_batch);
        const size_t T = d->T_max;
        d->cache_layer_stride = static_cast<size_t>(c.max_batch) * c.max_seq * d->KVD_l;
        if (c.kv_dtype != CSDR_DTYPE_F32 && c.kv_dtype != CSDR_DTYPE_BF16 && c.kv_dtype != CSDR_DTYPE_F16)
            throw Error(CSDR_ERR_INVALID_ARG, "decoder: kv_dtype must be CSDR_DTYPE_F32, CSDR_DTYPE_F16 or CSDR_DTYPE_BF16");
        d->kv_dtype = static_cast<int>(c.kv_dtype);
        d->kv_es = d->kv_dtype == CSDR_DTYPE_F32 ? 4 : 2;
        d->kcache = dev_alloc(ctx, d->cache_layer_stride * c.n_layers * d->kv_es);
        d->vcache = dev_alloc(ctx, d->cache_layer_stride * c.n_layers * d->kv_es);
        d->pos_host.assign(c.max_batch, 0);
        d->pos_dev = dev_alloc(ctx, c.max_batch * 4);
        d->tokens_dev = dev_alloc(ctx, T * 4);
        d->seq_of = dev_alloc(ctx, T * 4);
        d->pos_of = dev_alloc(ctx, T * 4);
        d->next_dev = dev_alloc(ctx, c.max_batch * 4);
        d->hidden = dev_alloc(ctx, T * d->H_l * 4);
        d->normed = dev_alloc(ctx, T * H * 4);
        d->q = dev_alloc(ctx, T * d->QD_l * 4);
        d->k = dev_alloc(ctx, T * d->KVD_l * 4);
        d->v = dev_alloc(ctx, T * d->KVD_l * 4);
        d->att = dev_alloc(ctx, T * d->QD_l * 4);
        d->proj = dev_alloc(ctx, T * d->H_l * 4);
        d->gate = dev_alloc(ctx, T * d->I_l * 4);
        d->up = dev_alloc(ctx, T * d->I_l * 4);
        d->logits = dev_alloc(ctx, static_cast<size_t>(c.max_batch) * c.vocab * 4);
        {
            // the planes path needs every block linear (and the head) to be an HSDR image the
            // grouped tensor-core path takes
            bool ok = !d->lm_head.raw;
            uint32_t widest = 0;   // atoms of the largest group
            auto atoms = [](const Linear& l) { return l.use() ? l.use()->g.n_atoms : 0u; };
            for (const Layer& L : d->layers) {
                const Linear* all[7] = {&L.q, &L.k, &L.v, &L.o, &L.gate, &L.up, &L.down};
                for (const Linear* l : all) {
                    if (l->raw || !l->use()) {
                        ok = false;
                        continue;
                    }
                    const csdr_segment* sgp = l->use();
                    ok = ok && wide_group_supported(ctx, &sgp, 1, ctx->tc_min_batch);
                }
                widest = std::max({widest, atoms(L.q) + atoms(L.k) + atoms(L.v), atoms(L.gate) + atoms(L.up), atoms(L.o),
                                   atoms(L.down)});
            }
            if (ok) {
                const csdr_segment* sgp = d->lm_head.use();
                ok = wide_group_supported(ctx, &sgp, 1, ctx->tc_min_batch);
                widest = std::max(widest, atoms(d->lm_head));
            }
            d->planes_capable = ok;
            {
                bool q_ok = true;
                for (const Layer& L : d->layers) {
                    const Linear* all[7] = {&L.q, &L.k, &L.v, &L.o, &L.gate, &L.up, &L.down};
                    for (const Linear* l : all) {
                        if (l->raw || !l->use()) {
                            q_ok = false;
                            continue;
                        }
                        const QueueItem probe{l->use(), nullptr, CSDR_DTYPE_F32, CSDR_LAYOUT_TOKEN_MAJOR, 4, nullptr,
                                              CSDR_LAYOUT_TOKEN_MAJOR, nullptr};
                        q_ok = q_ok && gemv_queue_supported(ctx, &probe, 1);
                    }
                    q_ok = q_ok && !L.gate.raw && !L.up.raw && L.gate.rows_local == L.up.rows_local;
                }
                d->queue_capable = q_ok;
            }
            if (d->P == 1) {
                // widest token tile at which every group of every block takes the folded glue
                for (uint32_t mt : {16u, 8u, 4u, 2u, 1u}) {
                    bool f_ok = true;
                    for (const Layer& L : d->layers) {
                        const Linear* all[7] = {&L.q, &L.k, &L.v, &L.o, &L.gate, &L.up, &L.down};
                        for (const Linear* l : all) f_ok = f_ok && !l->raw && l->use();
                        if (!f_ok) break;
                        FusedGlue norm, mlp, none;
                        norm.norm_w = mlp.norm_w = F(L.attn_norm);
                        mlp.swiglu = true;
                        const csdr_segment* qkv[3] = {L.q.use(), L.k.use(), L.v.use()};
                        const csdr_segment* gu[2] = {L.gate.use(), L.up.use()};
                        const csdr_segment* o = L.o.use();
                        const csdr_segment* dn = L.down.use();
                        f_ok = gemv_fused_glue_supported(ctx, qkv, 3, mt, norm) && gemv_fused_glue_supported(ctx, gu, 2, mt, mlp) &&
                               gemv_fused_glue_supported(ctx, &o, 1, mt, none) && gemv_fused_glue_supported(ctx, &dn, 1, mt, none);
                    }
                    if (f_ok) {
                        d->fold_max_mt = mt;
                        break;
                    }
                }
            }
            if (d->P > 1 && !ok)
                throw Error(CSDR_ERR_UNSUPPORTED,
                            "decoder: tensor parallelism needs every linear as HSDR row tiles with a multiple of 128 "
                            "atoms and per-rank input widths that are multiples of 64");
            if (ok) {
                d->xp_h = dev_alloc(ctx, T * d->H_l * 4);          // two bf16 planes each
                d->xp_att = dev_alloc(ctx, T * d->QD_l * 4);
                d->xp_act = dev_alloc(ctx, T * d->I_l * 4);
                d->sum_pad = static_cast<uint32_t>((T + 63) / 64 * 64);
                d->dxbuf = dev_alloc(ctx, (d->sum_pad + static_cast<size_t>(widest) * std::max<size_t>(T, 16)) * 4);
                CSDR_CUDA(cudaMemsetAsync(d->dxbuf->ptr, 0, d->dxbuf->bytes, ctx->stream));
                d->norm_scratch = dev_alloc(ctx, static_cast<size_t>(kNextNormCtas) * 16u * 4u);
                CSDR_CUDA(cudaMemsetAsync(d->norm_scratch->ptr, 0, d->norm_scratch->bytes, ctx->stream));
            }
        }
        if (d->P > 1 && d->P <= kMaxExchangeRanks) {
            // exchange region: [2][P] slots of a decode-sized block, then flag words, then this
            // rank's two counters; zeroed (sequence numbers start at 1)
            uint32_t widest = 0;
            auto atoms = [](const Linear& l) { return l.use() ? l.use()->g.n_atoms : 0u; };
            for (const Layer& L : d->layers)
                widest = std::max({widest, atoms(L.q) + atoms(L.k) + atoms(L.v), atoms(L.gate) + atoms(L.up), atoms(L.o),
                                   atoms(L.down)});
            d->xch_blk = d->sum_pad + widest * 16u;
            const size_t slot_bytes = static_cast<size_t>(2) * d->P * d->xch_blk * 4;
            d->xch_region = dev_alloc(ctx, slot_bytes + 1024);
            CSDR_CUDA(cudaMemsetAsync(d->xch_region->ptr, 0, d->xch_region->bytes, ctx->stream));
        }
        if (d->P > 1) {
            d->logits_l = dev_alloc(ctx, static_cast<size_t>(c.max_batch) * d->V_l * 4);
            d->staged = dev_alloc(ctx, std::max<size_t>(T * H, static_cast<size_t>(c.max_batch) * c.vocab) * 4);
        }
        CSDR_CUDA(cudaMemsetAsync(d->kcache->ptr, 0, d->kcache->bytes, ctx->stream));
        CSDR_CUDA(cudaMemsetAsync(d->vcache->ptr, 0, d->vcache->bytes, ctx->stream));
        CSDR_CUDA(cudaMemsetAsync(d->pos_dev->ptr, 0, d->pos_dev->bytes, ctx->stream));
        CSDR_CUDA(cudaStreamSynchronize(ctx->stream));
        *out = d.release();
    });
}

int csdr_decoder_exchange_export(csdr_decoder* d, void* handle64) {
    return guard([&] {
        need(d);
        if (!handle64) throw Error(CSDR_ERR_INVALID_ARG, "handle buffer is null");
        if (!d->xch_region) throw Error(CSDR_ERR_UNSUPPORTED, "this decoder has no exchange region (one rank, or more than 8)");
        static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
        cudaIpcMemHandle_t h;
        CSDR_CUDA(cudaIpcGetMemHandle(&h, d->xch_region->ptr));
        std::memcpy(handle64, &h, 64);
    });
}

int csdr_decoder_exchange_import(csdr_decoder* d, const void* handles, size_t n_ranks) {
    return guard([&] {
        need(d);
        if (!handles || n_ranks != d->P) throw Error(CSDR_ERR_INVALID_ARG, "one 64-byte handle per rank, rank-major");
        if (!d->xch_region) throw Error(CSDR_ERR_UNSUPPORTED, "this decoder has no exchange region (one rank, or more than 8)");
        if (d->xch.ranks) throw Error(CSDR_ERR_INVALID_ARG, "exchange handles were imported already");
        const size_t slot_bytes = static_cast<size_t>(2) * d->P * d->xch_blk * 4;
        Exchange x{};
        d->xch_maps.assign(d->P, nullptr);
        for (uint32_t r = 0; r < d->P; ++r) {
            void* base = d->xch_region->ptr;
            if (r != d->rank) {
                cudaIpcMemHandle_t h;
                std::memcpy(&h, static_cast<const unsigned char*>(handles) + 64u * r, 64);
                CSDR_CUDA(cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess));
                d->xch_maps[r] = base;
            }
            x.slots[r] = static_cast<float*>(base);
            x.flags[r] = reinterpret_cast<uint32_t*>(static_cast<unsigned char*>(base) + slot_bytes);
        }
        unsigned char* mine = static_cast<unsigned char*>(d->xch_region->ptr) + slot_bytes;
        x.seq = reinterpret_cast<uint32_t*>(mine + 512);
        x.done = reinterpret_cast<uint32_t*>(mine + 768);
        x.rank = d->rank;
        x.blk_floats = d->xch_blk;
        x.status = d->ctx->status_word;
        x.ranks = d->P;
        d->xch = x;
        // measured on B200s: 3.92 vs 4.63 ms per step at 8 ranks, 4.53 vs 4.70 at 2 (same box) in
        // favour of the peer exchange over ncclAllReduce; the environment overrides the default
        d->xch_use = true;
        if (const char* e = std::getenv("CSDR_TP_EXCHANGE")) {
            if (std::string(e) == "peer") d->xch_use = true;
            else if (std::string(e) == "nccl") d->xch_use = false;
        }
    });
}

int csdr_decoder_destroy(csdr_decoder* d) {
    return guard([&] {
        if (!d) return;
        cudaSetDevice(d->ctx->device);
        cudaStreamSynchronize(d->ctx->stream);
        delete d;
    });
}

int csdr_decoder_reset(csdr_decoder* d) {
    return guard([&] {
        need(d);
        std::fill(d->pos_host.begin(), d->pos_host.end(), 0);
        CSDR_CUDA(cudaMemsetAsync(d->pos_dev->ptr, 0, d->pos_dev->bytes, d->ctx->stream));
        if (d->seen) CSDR_CUDA(cudaMemsetAsync(d->seen->ptr, 0, d->seen->bytes, d->ctx->stream));
        CSDR_CUDA(cudaStreamSynchronize(d->ctx->stream));
    });
}

int csdr_decoder_selection_policy(csdr_decoder* d, int enable, float temperature) {
    return guard([&] {
        need(d);
        d->policy = enable != 0;
        d->temperature = temperature;
        if (d->policy && !d->seen) {
            d->seen_words = (d->cfg.vocab + 31u) / 32u;
            d->seen = dev_alloc(d->ctx, static_cast<size_t>(d->cfg.max_batch) * d->seen_words * 4);
            CSDR_CUDA(cudaMemsetAsync(d->seen->ptr, 0, d->seen->bytes, d->ctx->stream));
            CSDR_CUDA(cudaStreamSynchronize(d->ctx->stream));
        }
    });
}

int csdr_decoder_note_generated(csdr_decoder* d, uint32_t seq, const int32_t* tokens, size_t n_tokens) {
    return guard([&] {
        need(d);
        if (!d->seen) throw Error(CSDR_ERR_INVALID_ARG, "turn the selection policy on first");
        if (seq >= d->cfg.max_batch || (!tokens && n_tokens)) throw Error(CSDR_ERR_INVALID_ARG, "bad sequence or null tokens");
        if (!n_tokens) return;
        DevPtr t = upload(d->ctx, tokens, n_tokens * 4);
        op_mark_seen(d->ctx, static_cast<uint32_t*>(d->seen->ptr) + static_cast<size_t>(seq) * d->seen_words,
                     static_cast<const int32_t*>(t->ptr), static_cast<uint32_t>(n_tokens), d->cfg.vocab);
        CSDR_CUDA(cudaStreamSynchronize(d->ctx->stream));
    });
}

int csdr_decoder_seek(csdr_decoder* d, uint32_t seq, uint32_t position) {
    return guard([&] {
        need(d);
        if (seq >= d->cfg.max_batch || position > d->cfg.max_seq)
            throw Error(CSDR_ERR_INVALID_ARG, "sequence or position out of range");
        d->pos_host[seq] = static_cast<int32_t>(position);
        CSDR_CUDA(cudaMemcpyAsync(I32(d->pos_dev) + seq, &d->pos_host[seq], 4, cudaMemcpyHostToDevice, d->ctx->stream));
        CSDR_CUDA(cudaStreamSynchronize(d->ctx->stream));
    });
}

int csdr_decoder_forward(csdr_decoder* d, uint32_t seq, const int32_t* tokens, size_t n_tokens,
                         float* logits_out, float* hidden_out) {
    return guard([&] {
        need(d);
        const csdr_decoder_config& c = d->cfg;
        if (!tokens || n_tokens == 0) throw Error(CSDR_ERR_INVALID_ARG, "no tokens");
        if (seq >= c.max_batch) throw Error(CSDR_ERR_INVALID_ARG, "sequence index out of range");
        const int32_t p0 = d->pos_host[seq];
        if (n_tokens > d->T_max || p0 + n_tokens > c.max_seq)
            throw Error(CSDR_ERR_LIMIT, "sequence would exceed the KV-cache capacity (max_seq)");
        for (size_t i = 0; i < n_tokens; ++i)
            if (tokens[i] < 0 || static_cast<uint32_t>(tokens[i]) >= c.vocab)
                throw Error(CSDR_ERR_INVALID_ARG, "token id outside the vocabulary");
        csdr_context* ctx = d->ctx;
        const uint32_t T = static_cast<uint32_t>(n_tokens);
        std::vector<int32_t> so(T, static_cast<int32_t>(seq)), po(T);
        for (uint32_t t = 0; t < T; ++t) po[t] = p0 + static_cast<int32_t>(t);
        CSDR_CUDA(cudaMemcpyAsync(d->tokens_dev->ptr, tokens, T * 4, cudaMemcpyHostToDevice, ctx->stream));
        CSDR_CUDA(cudaMemcpyAsync(d->seq_of->ptr, so.data(), T * 4, cudaMemcpyHostToDevice, ctx->stream));
        CSDR_CUDA(cudaMemcpyAsync(d->pos_of->ptr, po.data(), T * 4, cudaMemcpyHostToDevice, ctx->stream));
        embed(d, T);
        d->distinct_seqs = T == 1u;
        run_blocks(d, T);
        if (hidden_out) {
            materialise_normed(d, T);
            CSDR_CUDA(cudaMemcpyAsync(hidden_out, d->normed->ptr, static_cast<size_t>(T) * c.hidden * 4,
                                      cudaMemcpyDeviceToHost, ctx->stream));
        }
        if (logits_out) {
            run_logits(d, T, T - 1, 1);
            CSDR_CUDA(cudaMemcpyAsync(logits_out, d->logits->ptr, static_cast<size_t>(c.vocab) * 4,
                                      cudaMemcpyDeviceToHost, ctx->stream));
        }
        d->pos_host[seq] = p0 + static_cast<int32_t>(T);
        CSDR_CUDA(cudaMemcpyAsync(I32(d->pos_dev) + seq, &d->pos_host[seq], 4, cudaMemcpyHostToDevice, ctx->stream));
        CSDR_CUDA(cudaStreamSynchronize(ctx->stream));
    });
}

int csdr_decoder_step_device_async(csdr_decoder* d, const int32_t* tokens_dev, size_t batch, int32_t* next_dev) {
    return guard([&] {
        need(d);
        const csdr_decoder_config& c = d->cfg;
        if (!tokens_dev || !next_dev || batch == 0 || batch > c.max_batch)
            throw Error(CSDR_ERR_INVALID_ARG, "bad batch or null buffers");
        for (size_t b = 0; b < batch; ++b)
            if (d->pos_host[b] >= static_cast<int32_t>(c.max_seq))
                throw Error(CSDR_ERR_LIMIT, "sequence would exceed the KV-cache capacity (max_seq)");
        csdr_context* ctx = d->ctx;
        const uint32_t B = static_cast<uint32_t>(batch);
        if (tokens_dev != I32(d->tokens_dev))
            CSDR_CUDA(cudaMemcpyAsync(d->tokens_dev->ptr, tokens_dev, B * 4, cudaMemcpyDeviceToDevice, ctx->stream));
        op_step_positions(ctx, I32(d->pos_dev), B, I32(d->seq_of), I32(d->pos_of));
        embed(d, B);
        d->distinct_seqs = true;
        run_blocks(d, B);
        run_logits(d, B, 0, B);
        if (d->policy)
            op_select(ctx, F(d->logits), B, c.vocab, next_dev, d->temperature, static_cast<uint32_t*>(d->seen->ptr),
                      d->seen_words);
        else
            op_argmax(ctx, F(d->logits), B, c.vocab, next_dev);
        for (size_t b = 0; b < batch; ++b) ++d->pos_host[b];
    });
}

int csdr_decoder_step(csdr_decoder* d, const int32_t* tokens, size_t batch, int32_t* next_out, float* logits_out) {
    return guard([&] {
        need(d);
        if (!tokens || !next_out || batch == 0 || batch > d->cfg.max_batch)
            throw Error(CSDR_ERR_INVALID_ARG, "bad batch or null buffers");
        for (size_t b = 0; b < batch; ++b)
            if (tokens[b] < 0 || static_cast<uint32_t>(tokens[b]) >= d->cfg.vocab)
                throw Error(CSDR_ERR_INVALID_ARG, "token id outside the vocabulary");
        csdr_context* ctx = d->ctx;
        CSDR_CUDA(cudaMemcpyAsync(d->tokens_dev->ptr, tokens, batch * 4, cudaMemcpyHostToDevice, ctx->stream));
        rethrow_last(csdr_decoder_step_device_async(d, I32(d->tokens_dev), batch, I32(d->next_dev)));
        CSDR_CUDA(cudaMemcpyAsync(next_out, d->next_dev->ptr, batch * 4, cudaMemcpyDeviceToHost, ctx->stream));
        if (logits_out)
            CSDR_CUDA(cudaMemcpyAsync(logits_out, d->logits->ptr, batch * d->cfg.vocab * 4, cudaMemcpyDeviceToHost,
                                      ctx->stream));
        CSDR_CUDA(cudaStreamSynchronize(ctx->stream));
    });
}

}  // extern "C"
