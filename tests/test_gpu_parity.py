"""Parity of the CUDA path against the oracle and the committed golden fixtures, through
the C-ABI. Bit-exact for code unpacking, weight materialisation and dequantisation;
1e-3 relative (max-abs over max|ref|, and relative L2) for matmul outputs."""
import os
import zlib

import numpy as np
import pytest

import cortexsdr_b200 as cs
from conftest import GOLDEN, rel_err

pytestmark = pytest.mark.gpu
TOL = 1e-3  # matmul tolerance named by the task: relative, fp32 accumulate


def crc(a):
    return zlib.crc32(np.ascontiguousarray(a).view(np.uint8).reshape(-1).tobytes())


def test_unpack_bit_exact(ctx, oracle, golden):
    for name, key in (("fused_rowtile.npz", "payload"), ("tiles_2d.npz", "edges_payload")):
        pay = golden(name)[key]
        seg = cs.Segment.from_payload(pay, ctx)
        idx, sign = seg.unpack()
        packed, oidx, osign, _ = oracle.codes(pay)
        assert idx.size == packed.size
        assert np.array_equal(idx, oidx) and np.array_equal(sign, osign)


def test_unpack_ragged_tail(ctx, oracle, reference):
    # code counts that are not multiples of 8 exercise the scalar tail of the 128-bit path
    from oracle.bindings import SEG_ATTENTION, Segment, cfg_row1d
    rng = np.random.default_rng(3)
    for R, k in ((37, 3), (65, 5)):
        W = rng.normal(0, 0.05, (R, 64)).astype(np.float32)
        cfg = cfg_row1d(64, 16, k, ksvd_iters=0)
        pay = reference.compress(Segment("t", W, W.shape, SEG_ATTENTION), cfg, cfg)
        idx, sign = cs.Segment.from_payload(pay, ctx).unpack()
        _, oidx, osign, _ = oracle.codes(pay)
        assert (R * 3 * k) % 8 != 0
        assert np.array_equal(idx, oidx) and np.array_equal(sign, osign)


def test_fused_matmul_reference_fixture(ctx, golden):
    g = golden("fused_rowtile.npz")
    y = cs.HierarchicalSDRStrategy(ctx).matmulRowMajor(g["payload"], g["x"], 4)
    assert y.shape == (256, 4)
    assert np.abs(y - g["y_fused"]).max() < 1e-3      # the reference test's own criterion
    e = rel_err(y, g["y_fused"])
    assert e[0] < TOL and e[1] < TOL


@pytest.mark.parametrize("batch", [1, 2, 3, 4, 7, 8, 15, 16, 17, 33])
def test_fused_matmul_batches(ctx, oracle, golden, batch):
    g = golden("fused_rowtile.npz")
    x = np.random.default_rng(batch).normal(0, 1, (512, batch)).astype(np.float32)
    seg = cs.Segment.from_payload(g["payload"], ctx)
    e = rel_err(seg.matmul(x, batch), oracle.matmul(g["payload"], x, batch))
    assert e[0] < TOL and e[1] < TOL, e


def test_fused_matmul_empty_batch(ctx, golden):
    seg = cs.Segment.from_payload(golden("fused_rowtile.npz")["payload"], ctx)
    assert seg.matmul(np.zeros((512, 0), np.float32), 0).shape == (256, 0)


def test_decompress_bit_exact(ctx, golden):
    g = golden("fused_rowtile.npz")
    W = cs.HierarchicalSDRStrategy(ctx).decompress(g["payload"])
    assert crc(W) == int(g["w_crc"])
    t = golden("tiles_2d.npz")
    for label in ("attn_small", "mlp_small", "edges"):
        W = cs.HierarchicalSDRStrategy(ctx).decompress(t[label + "_payload"])
        assert crc(W) == int(t[label + "_w_crc"]), label
        assert np.array_equal(W[t[label + "_w_rows_idx"]], t[label + "_w_rows"])


def test_2d_tiles_refused_like_reference_and_allowed_on_request(ctx, oracle, golden):
    t = golden("tiles_2d.npz")
    for label, C in (("attn_small", 256), ("mlp_small", 320), ("edges", 257)):
        pay = t[label + "_payload"]
        seg = cs.Segment.from_payload(pay, ctx)
        with pytest.raises(cs.CompressionError, match="tile_rows == 1"):
            seg.matmul(np.zeros((C, 1), np.float32), 1)
        W = oracle.decompress(pay)
        for batch in (1, 3, 5):
            x = np.random.default_rng(batch).normal(0, 1, (C, batch)).astype(np.float32)
            e = rel_err(seg.matmul(x, batch, allow_2d=True), oracle.dense_matmul(W, x, batch))
            assert e[0] < TOL and e[1] < TOL, (label, batch, e)


def test_dequant_bit_exact(ctx, golden):
    g = golden("dequant.npz")
    st = cs.HierarchicalSDRStrategy(ctx)
    for fmt in ("q4_k", "q5_k", "q6_k", "q4_0", "q8_0", "f16", "bf16"):
        out = st.dequantizeToFP32(g[fmt + "_in"], fmt)
        assert np.array_equal(out.view(np.uint32), g[fmt + "_out"].view(np.uint32)), fmt
    out = st.dequantizeToFP32(g["i8_in"], "i8", float(g["i8_scale"]), float(g["i8_zp"]))
    assert np.allclose(out, g["i8_out"], rtol=1e-6, atol=0)
    with pytest.raises(cs.CompressionError, match="not a multiple of 144"):
        st.dequantizeToFP32(np.zeros(100, np.uint8), "q4_k")
    with pytest.raises(cs.CompressionError, match="unsupported input dtype"):
        st.dequantizeToFP32(np.zeros(100, np.uint8), "iq2_xs")


def test_dequant_kquant_known_answers(ctx):
    f16 = lambda v: np.array([v], np.float16).view(np.uint8)
    st = cs.HierarchicalSDRStrategy(ctx)
    b = np.zeros(144, np.uint8); b[0:2] = f16(2.0); b[2:4] = f16(1.0); b[4] = 3; b[8] = 4; b[16] = 0x05
    out = st.dequantizeToFP32(b, "q4_k")
    assert out[0] == 26.0 and out[1] == -4.0
    b = np.zeros(176, np.uint8); b[0:2] = f16(1.0); b[4] = 1; b[16] = 0x01; b[48] = 0x02
    assert st.dequantizeToFP32(b, "q5_k")[0] == 18.0
    b = np.zeros(210, np.uint8); b[0] = 0x21; b[128] = 0x03; b[192] = 2; b[208:210] = f16(1.0)
    out = st.dequantizeToFP32(b, "q6_k")
    assert out[0] == 34.0 and out[1] == -60.0


def test_stored_raw_block_formats_in_the_inference_side_order(ctx, oracle, golden):
    # what SDRModelLoader::loadLayerByName made of the same bytes (fixture written through the
    # reference's loader): bit for bit, and unlike the encoder-side order for the k-quants
    g = golden("raw_tensors.npz")
    for fmt in ("q4_k", "q5_k", "q6_k", "q4_0", "q8_0"):
        got = cs.dequantize_inference(g[fmt + "_in"], fmt, ctx=ctx)
        assert np.array_equal(got.view(np.uint32), g[fmt + "_out"].view(np.uint32)), fmt
        assert np.array_equal(got.view(np.uint32), oracle.dequantize_inference(fmt, g[fmt + "_in"]).view(np.uint32))
    # clipped to the element count asked for, trailing partial block ignored
    part = cs.dequantize_inference(np.append(g["q4_k_in"], np.zeros(7, np.uint8)), "q4_k", n_elements=300, ctx=ctx)
    assert np.array_equal(part, g["q4_k_out"][:300])
    enc = cs.HierarchicalSDRStrategy(ctx).dequantizeToFP32(g["q4_k_in"], "q4_k")
    assert not np.array_equal(enc, g["q4_k_out"])
    with pytest.raises(cs.CompressionError):
        cs.dequantize_inference(g["q4_k_in"], "f16", ctx=ctx)


def test_archive_e2e(ctx, golden):
    # src/test_hsdr_archive_e2e.cpp: .sdr written by the reference's AICompressor
    g = golden("archive_e2e.npz")
    ld = cs.SDRModelLoader(os.path.join(GOLDEN, "archive_e2e.sdr"), ctx)
    h = ld.findSegmentHeader("test.layer.weight")
    assert h.compression_strategy_id == cs.HSDR_STRATEGY_ID
    y = ld.matmulHSDR("test.layer.weight", g["x"], 4)
    assert np.abs(y - g["y_fused"]).max() < 1e-3
    W = ld.loadSegmentByName("test.layer.weight").view(np.float32).reshape(128, 512)
    assert crc(W) == int(g["w_crc"])


def test_matmul_routing(ctx, golden):
    # src/test_inference_matmul_routing.cpp:111-182
    g = golden("routing.npz")
    ld = cs.SDRModelLoader(os.path.join(GOLDEN, "routing.sdr"), ctx)
    eng = cs.SDRInferenceEngine(ld)
    y_route = eng.matmulForLayer("layer.hsdr.weight", g["x_hsdr"], 2)
    y_direct = ld.matmulHSDR("layer.hsdr.weight", g["x_hsdr"], 2)
    assert np.abs(y_route - y_direct).max() < 1e-6
    assert np.abs(y_direct - g["y_hsdr"]).max() < 1e-3
    y_raw = eng.matmulForLayer("layer.raw.weight", g["x_raw"], 2)     # dense fallback
    assert np.abs(y_raw - g["y_raw"]).max() < 1e-5
    with pytest.raises(RuntimeError, match="not found"):
        eng.matmulForLayer("does.not.exist", g["x_raw"], 2)
    with pytest.raises(cs.CompressionError, match="2-D tensor_metadata"):
        eng.matmulForLayer("layer.norm.weight", g["x_raw"], 2)
    # applyLinearLayer: token-major, name or name + ".weight", bias added
    bias = np.linspace(-1, 1, 256).astype(np.float32)
    out = eng.applyLinearLayer("layer.hsdr", g["x_hsdr"].T.copy(), bias)
    assert out.shape == (2, 256)
    assert np.abs(out - (y_direct.T + bias)).max() < 1e-5


def test_hsda_reader(ctx, golden):
    # src/test_hsda_reader.cpp: name-indexed decompress + fused matmul, missing-name error
    g = golden("reader_hsda.npz")
    r = cs.HSDAReader.fromFile(os.path.join(GOLDEN, "reader.hsda"), ctx)
    assert r.numDictionaries() == 2
    for i, name in enumerate(g["names"]):
        y = r.matmul(str(name), g["x"], 2)
        assert np.abs(y - g[f"y_{i}"]).max() < 1e-3
        assert crc(r.decompress(str(name))) == int(g[f"w_crc_{i}"])
    with pytest.raises(RuntimeError, match="segment not found"):
        r.matmul("nope", g["x"], 2)


def test_hsda_shared_2d(ctx, oracle, golden):
    g = golden("shared_2d.npz")
    r = cs.HSDAReader.fromFile(os.path.join(GOLDEN, "shared_2d.hsda"), ctx)
    for i, name in enumerate(g["names"]):
        R, C = (int(v) for v in g["shapes"][i])
        W = r.decompress(str(name))
        assert crc(W) == int(g[f"w_crc_{i}"])
        x = np.random.default_rng(i).normal(0, 1, (C, 2)).astype(np.float32)
        with pytest.raises(cs.CompressionError):
            r.matmul(str(name), x, 2)
        e = rel_err(r.matmul(str(name), x, 2, allow_2d=True), oracle.dense_matmul(W, x, 2))
        assert e[0] < TOL and e[1] < TOL


def test_shared_dictionary_geometry_mismatch(ctx, golden):
    import struct
    raw = open(os.path.join(GOLDEN, "reader.hsda"), "rb").read()
    # first dictionary of the container, then a codes stream of the OTHER role
    from test_oracle_golden import _hsda_dicts
    dicts, segs = _hsda_dicts(os.path.join(GOLDEN, "reader.hsda"))
    name = next(n for n, (di, _, _) in segs.items() if di == 1)
    d0 = dicts[0]
    dd = cs.Dictionary(ctx, d0.tile_rows, d0.tile_cols, d0.n_atoms, d0.n_stages, d0.k, d0.atoms, d0.scales)
    with pytest.raises(cs.CompressionError, match="doesn't match dictionary"):
        cs.Segment.from_payload(segs[name][2], ctx, dd)


def test_device_resident_layouts_and_bf16(ctx, oracle, golden):
    import torch
    g = golden("fused_rowtile.npz")
    seg = cs.Segment.from_payload(g["payload"], ctx)
    rng = np.random.default_rng(11)
    for batch in (1, 8):
        xb = torch.from_numpy(rng.normal(0, 1, (batch, 512)).astype(np.float32)).cuda().to(torch.bfloat16)
        x32 = xb.float().cpu().numpy()                     # the oracle sees the bf16-rounded values
        y = torch.empty((batch, 256), dtype=torch.float32, device="cuda")
        bias = torch.linspace(-1, 1, 256, device="cuda")
        torch.cuda.synchronize()
        seg.matmul_device(xb.data_ptr(), cs.DTYPE_BF16, cs.TOKEN_MAJOR, batch, y.data_ptr(),
                          cs.TOKEN_MAJOR, bias.data_ptr())
        ctx.synchronize()
        want = oracle.matmul(g["payload"], x32.T.copy(), batch).T + bias.cpu().numpy()
        e = rel_err(y.cpu().numpy(), want)
        assert e[0] < TOL and e[1] < TOL, e


def test_row_shards_concatenate_to_whole(ctx, oracle, golden):
    g = golden("fused_rowtile.npz")
    seg = cs.Segment.from_payload(g["payload"], ctx)
    x = g["x"]
    whole = seg.matmul(x, 4)
    parts = [seg.shard_rows(b, e).matmul(x, 4) for b, e in ((0, 64), (64, 100), (100, 256))]
    assert np.array_equal(np.concatenate(parts, 0), whole)
    t = golden("tiles_2d.npz")
    seg2 = cs.Segment.from_payload(t["attn_small_payload"], ctx)
    x2 = np.random.default_rng(0).normal(0, 1, (256, 2)).astype(np.float32)
    whole2 = seg2.matmul(x2, 2, allow_2d=True)
    parts2 = [seg2.shard_rows(b, e).matmul(x2, 2, allow_2d=True) for b, e in ((0, 96), (96, 256))]
    assert np.array_equal(np.concatenate(parts2, 0), whole2)
    with pytest.raises(cs.CompressionError, match="tile-row boundaries"):
        seg2.shard_rows(0, 40)


def test_column_shards_add_up_to_the_whole_product(ctx, oracle):
    """Input-column shards (tensor parallelism): each shard times its slice of x is that slice's
    share of W x; shares add up to the oracle's product, on the GEMV path and the tensor-core path."""
    from tests import synth
    pay = synth.hsdr_payload(200, 512, n_atoms=128, k=4, seed=71)
    seg = cs.Segment.from_payload(pay, ctx)
    shards = [seg.shard_cols(b, e) for b, e in ((0, 128), (128, 320), (320, 512))]
    assert [s.cols for s in shards] == [128, 192, 192] and all(s.rows == 200 for s in shards)
    rng = np.random.default_rng(12)
    for batch in (1, 16):
        x = rng.normal(0, 1, (512, batch)).astype(np.float32)
        want = oracle.matmul(pay, x, batch)
        got = sum(s.matmul(np.ascontiguousarray(x[b:e]), batch)
                  for s, (b, e) in zip(shards, ((0, 128), (128, 320), (320, 512))))
        e = rel_err(got, want)
        assert e[0] < TOL and e[1] < TOL, (batch, e)
    # a row shard of a column shard keeps the column shard's dictionary
    both = shards[1].shard_rows(40, 120)
    x = rng.normal(0, 1, (192, 3)).astype(np.float32)
    assert np.array_equal(both.matmul(x, 3), shards[1].matmul(x, 3)[40:120])
    with pytest.raises(cs.CompressionError, match="multiples of four"):
        seg.shard_cols(2, 130)


def test_grouped_matmul_matches_single_calls(ctx, oracle, golden):
    import torch
    from tests import synth
    pays = [synth.hsdr_payload(r, 512, n_atoms=k, k=4, seed=40 + i) for i, (r, k) in enumerate(((256, 64), (96, 32), (130, 64)))]
    segs = [cs.Segment.from_payload(p, ctx) for p in pays]
    rng = np.random.default_rng(9)
    for batch in (1, 5, 16, 21):
        x = torch.from_numpy(rng.normal(0, 1, (batch, 512)).astype(np.float32)).cuda()
        ys = [torch.zeros((batch, s.rows), device="cuda") for s in segs]
        torch.cuda.synchronize()
        cs.Segment.matmul_group_device(segs, x.data_ptr(), cs.DTYPE_F32, cs.TOKEN_MAJOR, batch,
                                       [y.data_ptr() for y in ys], cs.TOKEN_MAJOR)
        ctx.synchronize()
        for p, y in zip(pays, ys):
            want = oracle.matmul(p, np.ascontiguousarray(x.cpu().numpy().T), batch).T
            e = rel_err(y.cpu().numpy(), want)
            assert e[0] < TOL and e[1] < TOL, (batch, e)


def test_grouped_tensor_core_projection_matches_oracle(ctx, oracle):
    """Members with different atom counts and row counts over one activation matrix: one
    projection launch for the group (bf16 planes built once), one gather launch up to 16 tokens."""
    import torch
    from tests import synth
    shapes = ((264, 128), (96, 256), (130, 128))
    # 472 columns: seven 64-column blocks and a ragged eighth
    pays = [synth.hsdr_payload(r, 472, n_atoms=k, k=4, seed=60 + i) for i, (r, k) in enumerate(shapes)]
    segs = [cs.Segment.from_payload(p, ctx) for p in pays]
    rng = np.random.default_rng(11)
    for batch, dtype in ((8, "f32"), (13, "f32"), (16, "bf16"), (21, "f32"), (64, "bf16"), (130, "f32")):
        xf = rng.normal(0, 1, (batch, 472)).astype(np.float32)
        if dtype == "bf16":
            x = torch.from_numpy(xf).cuda().to(torch.bfloat16)
            xf = x.float().cpu().numpy()
            code = cs.DTYPE_BF16
        else:
            x = torch.from_numpy(xf).cuda()
            code = cs.DTYPE_F32
        ys = [torch.zeros((batch, s.rows), device="cuda") for s in segs]
        torch.cuda.synchronize()
        cs.Segment.matmul_group_device(segs, x.data_ptr(), code, cs.TOKEN_MAJOR, batch,
                                       [y.data_ptr() for y in ys], cs.TOKEN_MAJOR)
        ctx.synchronize()
        for p, y in zip(pays, ys):
            want = oracle.matmul(p, np.ascontiguousarray(xf.T), batch).T
            e = rel_err(y.cpu().numpy(), want)
            assert e[0] < TOL and e[1] < TOL, (batch, dtype, e)


def test_fused_and_two_kernel_paths_agree(lib, oracle, golden, monkeypatch):
    g = golden("fused_rowtile.npz")
    x = np.random.default_rng(5).normal(0, 1, (512, 9)).astype(np.float32)
    outs = []
    for flag in ("1", "0"):
        monkeypatch.setenv("CSDR_FUSED_GEMV", flag)
        c = cs.Context(0)
        seg = cs.Segment.from_payload(g["payload"], c)
        outs.append(seg.matmul(x, 9))
        seg.close()
        c.close()
    want = oracle.matmul(g["payload"], x, 9)
    for y in outs:
        e = rel_err(y, want)
        assert e[0] < TOL and e[1] < TOL
    assert np.abs(outs[0] - outs[1]).max() < 1e-5


def test_chained_launches_are_ordered(ctx, oracle, golden):
    # y of one launch feeds the next as x: the dependent launch must see the finished result
    import torch
    from tests import synth
    p1 = synth.hsdr_payload(512, 512, n_atoms=64, k=4, seed=70)
    p2 = synth.hsdr_payload(512, 512, n_atoms=64, k=4, seed=71)
    s1, s2 = cs.Segment.from_payload(p1, ctx), cs.Segment.from_payload(p2, ctx)
    x0 = np.random.default_rng(6).normal(0, 1, (1, 512)).astype(np.float32)
    a = torch.from_numpy(x0).cuda()
    b = torch.empty_like(a)
    torch.cuda.synchronize()
    for _ in range(6):
        s1.matmul_device(a.data_ptr(), cs.DTYPE_F32, cs.TOKEN_MAJOR, 1, b.data_ptr(), cs.TOKEN_MAJOR)
        s2.matmul_device(b.data_ptr(), cs.DTYPE_F32, cs.TOKEN_MAJOR, 1, a.data_ptr(), cs.TOKEN_MAJOR)
    ctx.synchronize()
    v = x0.T.copy()
    for _ in range(6):
        v = oracle.matmul(p2, oracle.matmul(p1, v, 1), 1)
    e = rel_err(a.cpu().numpy().T, v)
    assert e[0] < 1e-3, e


def test_graph_replay_sees_new_activations(ctx, oracle):
    # One fused GEMV captured in a CUDA graph, replayed with x changed in place between the
    # replays: the hand-over tag is advanced on the device, so no replay may accept the
    # partial results an earlier replay left in the scratch words.
    import torch
    from tests import synth
    pay = synth.hsdr_payload(768, 2048, n_atoms=256, k=6, seed=90)
    stream = torch.cuda.Stream()
    c = cs.Context(0, stream.cuda_stream)
    seg = cs.Segment.from_payload(pay, c)
    x = torch.zeros((1, 2048), device="cuda")
    y = torch.zeros((1, 768), device="cuda")
    rng = np.random.default_rng(12)
    with torch.cuda.stream(stream):
        seg.matmul_device(x.data_ptr(), cs.DTYPE_F32, cs.TOKEN_MAJOR, 1, y.data_ptr(), cs.TOKEN_MAJOR)
        c.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            seg.matmul_device(x.data_ptr(), cs.DTYPE_F32, cs.TOKEN_MAJOR, 1, y.data_ptr(), cs.TOKEN_MAJOR)
        for i in range(6):
            xh = rng.normal(0, 1 + i, (1, 2048)).astype(np.float32)
            x.copy_(torch.from_numpy(xh), non_blocking=False)
            g.replay()
            c.synchronize()
            want = oracle.matmul(pay, np.ascontiguousarray(xh.T), 1).T
            e = rel_err(y.cpu().numpy(), want)
            assert e[0] < TOL and e[1] < TOL, (i, e)
    seg.close()
    c.close()


def test_a_wait_that_runs_out_is_an_error_code_not_a_hang(lib, oracle, golden):
    # The receiving side of a tensor-parallel exchange waits on a flag that nothing raises; with
    # a limit of a thousand polls it gives up within microseconds, the next synchronize says
    # TIMEOUT, and the same context computes correctly afterwards.
    from cortexsdr_b200 import _lib
    c = cs.Context(0)
    c.set_wait_limits(exchange_polls=1000)
    assert c.wait_selftest() == _lib.ERR_TIMEOUT
    assert b"wait ran out" in lib.csdr_last_error()
    c.set_wait_limits()            # defaults again
    c.synchronize()                # the status word was cleared with the report
    g = golden("fused_rowtile.npz")
    seg = cs.Segment.from_payload(g["payload"], c)
    x = np.random.default_rng(5).normal(0, 1, (512, 3)).astype(np.float32)
    e = rel_err(seg.matmul(x, 3), oracle.matmul(g["payload"], x, 3))
    assert e[0] < TOL and e[1] < TOL
    seg.close()
    c.close()


def _queue_case(ctx, oracle, specs, batch, dtype="f32", layout="token", with_bias=False, replays=0):
    """specs: (rows, cols, atoms, k) per task; every task gets its own activations."""
    import torch
    from tests import synth
    rng = np.random.default_rng(len(specs) * 100 + batch)
    segs, pays, xs, ys, xhs, biases, tasks = [], [], [], [], [], [], []
    for i, (r, c, a, k) in enumerate(specs):
        pay = synth.hsdr_payload(r, c, n_atoms=a, k=k, seed=500 + i)
        seg = cs.Segment.from_payload(pay, ctx)
        xh = rng.normal(0, 1, (batch, c)).astype(np.float32)
        xt = torch.from_numpy(xh).cuda()
        if dtype == "bf16":
            xt = xt.to(torch.bfloat16)
            xh = xt.float().cpu().numpy()
        lay = cs.TOKEN_MAJOR
        if layout == "feature":
            xt, lay = xt.t().contiguous(), cs.FEATURE_MAJOR
        y = torch.full((r, batch) if layout == "feature" else (batch, r), float("nan"), device="cuda")
        b = torch.from_numpy(rng.normal(0, 1, r).astype(np.float32)).cuda() if with_bias else None
        segs.append(seg); pays.append(pay); xs.append(xt); ys.append(y); xhs.append(xh); biases.append(b)
        tasks.append((seg, xt.data_ptr(), cs.DTYPE_BF16 if dtype == "bf16" else cs.DTYPE_F32, lay, batch,
                      y.data_ptr(), lay, b.data_ptr() if with_bias else 0))
    torch.cuda.synchronize()
    for _ in range(1 + replays):
        cs.Segment.matmul_queue_device(tasks)
    ctx.synchronize()
    for i, pay in enumerate(pays):
        want = oracle.matmul(pay, np.ascontiguousarray(xhs[i].T), batch)          # (R, batch)
        if with_bias:
            want = want + biases[i].cpu().numpy()[:, None]
        got = ys[i].cpu().numpy()
        got = got if layout == "feature" else got.T
        e = rel_err(got, want)
        assert e[0] < TOL and e[1] < TOL, (i, specs[i], batch, dtype, layout, e)
    for s_ in segs:
        s_.close()


@pytest.mark.parametrize("batch", [1, 2, 3, 4])
def test_queue_of_products_mixed_shapes(ctx, oracle, batch):
    # different rows, widths (not multiples of the 1024-column slab), dictionary sizes (not
    # multiples of the 8 atoms of a work unit) and code counts in one list
    specs = [(384, 1024, 128, 6), (200, 4096, 512, 8), (77, 1540, 100, 5), (1000, 256, 64, 4), (16, 2052, 9, 3)]
    _queue_case(ctx, oracle, specs, batch)


def test_queue_longer_than_one_launch_with_bias_and_replays(ctx, oracle):
    # 70 tasks = three launches of at most 32; bias added; run three times back to back (the
    # second and third pass find the previous pass's tagged words in the scratch buffer)
    specs = [(96 + 8 * (i % 5), 512 + 256 * (i % 3), 64, 4) for i in range(70)]
    _queue_case(ctx, oracle, specs, 1, with_bias=True, replays=2)


@pytest.mark.parametrize("dtype,layout", [("bf16", "token"), ("f32", "feature"), ("bf16", "feature")])
def test_queue_activation_formats(ctx, oracle, dtype, layout):
    _queue_case(ctx, oracle, [(264, 1536, 192, 5), (128, 1536, 64, 8), (512, 640, 128, 6)], 3, dtype=dtype, layout=layout)


def test_queue_falls_back_for_wide_batches_and_2d_tiles(ctx, oracle):
    import torch
    from tests import synth
    _queue_case(ctx, oracle, [(264, 1536, 192, 5), (128, 512, 64, 8)], 9)      # nine tokens: issued one by one
    pay = synth.hsdr_payload(128, 192, tile_rows=32, tile_cols=32, n_atoms=32, k=4, seed=3)
    seg = cs.Segment.from_payload(pay, ctx)
    xh = np.random.default_rng(1).normal(0, 1, (2, 192)).astype(np.float32)
    x, y = torch.from_numpy(xh).cuda(), torch.zeros((2, 128), device="cuda")
    cs.Segment.matmul_queue_device([(seg, x.data_ptr(), cs.DTYPE_F32, cs.TOKEN_MAJOR, 2, y.data_ptr(), cs.TOKEN_MAJOR)])
    ctx.synchronize()
    want = oracle.dense_matmul(oracle.decompress(pay), np.ascontiguousarray(xh.T), 2).T
    e = rel_err(y.cpu().numpy(), want)
    assert e[0] < TOL and e[1] < TOL


def test_queue_graph_replay_with_changed_activations(ctx, oracle):
    import torch
    from tests import synth
    stream = torch.cuda.Stream()
    c = cs.Context(0, stream.cuda_stream)
    pays = [synth.hsdr_payload(300 + 20 * i, 2048, n_atoms=256, k=6, seed=40 + i) for i in range(5)]
    segs = [cs.Segment.from_payload(p, c) for p in pays]
    x = torch.zeros((1, 2048), device="cuda")
    ys = [torch.zeros((1, s.rows), device="cuda") for s in segs]
    tasks = [(s, x.data_ptr(), cs.DTYPE_F32, cs.TOKEN_MAJOR, 1, y.data_ptr(), cs.TOKEN_MAJOR) for s, y in zip(segs, ys)]
    rng = np.random.default_rng(3)
    with torch.cuda.stream(stream):
        cs.Segment.matmul_queue_device(tasks)
        c.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            cs.Segment.matmul_queue_device(tasks)
        for i in range(4):
            xh = rng.normal(0, 1 + i, (1, 2048)).astype(np.float32)
            x.copy_(torch.from_numpy(xh))
            g.replay()
            c.synchronize()
            for p, y in zip(pays, ys):
                e = rel_err(y.cpu().numpy(), oracle.matmul(p, np.ascontiguousarray(xh.T), 1).T)
                assert e[0] < TOL and e[1] < TOL, (i, e)
    for s_ in segs:
        s_.close()
    c.close()


def test_queue_on_host_buffers(ctx, oracle):
    # the same list through the host-buffer call: one upload, one download; two tasks share
    # their activations (one staged copy), one has a batch of its own kind
    from tests import synth
    rng = np.random.default_rng(21)
    pays = [synth.hsdr_payload(r, c, n_atoms=a, k=k, seed=60 + i)
            for i, (r, c, a, k) in enumerate([(300, 1024, 128, 6), (520, 1024, 256, 8), (77, 1540, 100, 5)])]
    segs = [cs.Segment.from_payload(p, ctx) for p in pays]
    x01 = rng.normal(0, 1, (1024, 2)).astype(np.float32)
    x2 = rng.normal(0, 1, (1540, 2)).astype(np.float32)
    outs = [np.full((s.rows, 2), np.nan, np.float32) for s in segs]
    prepared = cs.Segment.matmul_queue([(segs[0], x01, 2, outs[0]), (segs[1], x01, 2, outs[1]), (segs[2], x2, 2, outs[2])])
    for p, x, out in zip(pays, (x01, x01, x2), outs):
        e = rel_err(out, oracle.matmul(p, x, 2))
        assert e[0] < TOL and e[1] < TOL
    x01 *= 2.0                                               # same arrays, new values, prepared list reused
    cs.Segment.matmul_queue(None, prepared)
    e = rel_err(outs[1], oracle.matmul(pays[1], x01, 2))
    assert e[0] < TOL and e[1] < TOL
    # mixed batches are issued one by one, 2-D tiles are refused as the reference's fused call refuses them
    y9 = np.zeros((300, 9), np.float32)
    x9 = rng.normal(0, 1, (1024, 9)).astype(np.float32)
    cs.Segment.matmul_queue([(segs[0], x9, 9, y9), (segs[1], x01, 2, outs[1])])
    e = rel_err(y9, oracle.matmul(pays[0], x9, 9))
    assert e[0] < TOL and e[1] < TOL
    seg2d = cs.Segment.from_payload(synth.hsdr_payload(64, 64, tile_rows=32, tile_cols=32, n_atoms=16, k=2, seed=1), ctx)
    with pytest.raises(cs.CompressionError, match="tile_rows == 1"):
        cs.Segment.matmul_queue([(seg2d, np.zeros((64, 1), np.float32), 1, np.zeros((64, 1), np.float32))])


def test_queue_on_page_locked_host_buffers(ctx, oracle):
    """Activations and results one behind the other in page-locked memory, in task order and in
    multiples of 256 bytes: moved straight from and to the caller's memory. Same results as
    through the staging buffer (pageable arrays), and as the oracle's; a list whose results are
    NOT contiguous takes the staged way for them."""
    import torch
    from tests import synth
    rng = np.random.default_rng(23)
    n, R, Cc = 6, 320, 1024                                    # 320 * 4 and 1024 * 4 are multiples of 256
    pays = [synth.hsdr_payload(R, Cc, n_atoms=128, k=6, seed=80 + i) for i in range(n)]
    segs = [cs.Segment.from_payload(p, ctx) for p in pays]
    x_pin = torch.empty((n, Cc), dtype=torch.float32, pin_memory=True)
    y_pin = torch.full((n, R), float("nan"), dtype=torch.float32, pin_memory=True)
    xa, ya = x_pin.numpy(), y_pin.numpy()
    xa[:] = rng.normal(0, 1, (n, Cc)).astype(np.float32)
    cs.Segment.matmul_queue([(segs[i], xa[i].reshape(Cc, 1), 1, ya[i].reshape(R, 1)) for i in range(n)])
    plain = [np.full((R, 1), np.nan, np.float32) for _ in range(n)]
    cs.Segment.matmul_queue([(segs[i], xa[i].copy().reshape(Cc, 1), 1, plain[i]) for i in range(n)])
    for i in range(n):
        want = oracle.matmul(pays[i], xa[i].reshape(Cc, 1), 1)
        e = rel_err(ya[i].reshape(R, 1), want)
        assert e[0] < TOL and e[1] < TOL, i
        assert np.array_equal(ya[i].reshape(R, 1), plain[i])
    # results in reverse order: page-locked, not consecutive
    y2 = torch.full((n, R), float("nan"), dtype=torch.float32, pin_memory=True).numpy()
    cs.Segment.matmul_queue([(segs[i], xa[i].reshape(Cc, 1), 1, y2[n - 1 - i].reshape(R, 1)) for i in range(n)])
    for i in range(n):
        assert np.array_equal(y2[n - 1 - i].reshape(R, 1), plain[i])


@pytest.mark.parametrize("batch", [1, 3])
def test_queue_chain_of_dependent_products(ctx, oracle, batch):
    # y1 = W1 x, y2 = W2 y1, y3 = W3 y2 and, beside the chain, y4 = W4 x: one list, one launch; the
    # later tasks name the task whose rows they read
    import torch
    from tests import synth
    dims = [(640, 1024), (384, 640), (200, 384), (96, 1024)]
    pays = [synth.hsdr_payload(r, c, n_atoms=128, k=5, seed=80 + i, weight_std=0.05) for i, (r, c) in enumerate(dims)]
    segs = [cs.Segment.from_payload(p, ctx) for p in pays]
    xh = np.random.default_rng(batch).normal(0, 1, (batch, 1024)).astype(np.float32)
    x = torch.from_numpy(xh).cuda()
    ys = [torch.full((batch, r), float("nan"), device="cuda") for r, _ in dims]
    F, T = cs.DTYPE_F32, cs.TOKEN_MAJOR
    tasks = [(segs[0], x.data_ptr(), F, T, batch, ys[0].data_ptr(), T, 0, -1),
             (segs[3], x.data_ptr(), F, T, batch, ys[3].data_ptr(), T, 0, -1),
             (segs[1], ys[0].data_ptr(), F, T, batch, ys[1].data_ptr(), T, 0, 0),
             (segs[2], ys[1].data_ptr(), F, T, batch, ys[2].data_ptr(), T, 0, 2)]
    torch.cuda.synchronize()
    for _ in range(3):                       # back to back: alternate counter sets, cleared by the launch before
        prepared = cs.Segment.matmul_queue_device(tasks)
    ctx.synchronize()
    w1 = oracle.matmul(pays[0], np.ascontiguousarray(xh.T), batch)
    w2 = oracle.matmul(pays[1], w1, batch)
    w3 = oracle.matmul(pays[2], w2, batch)
    w4 = oracle.matmul(pays[3], np.ascontiguousarray(xh.T), batch)
    for got, want in zip(ys, (w1, w2, w3, w4)):
        e = rel_err(got.cpu().numpy().T, want)
        assert e[0] < TOL and e[1] < TOL, e
    with pytest.raises(Exception):           # a task may only point backwards
        cs.Segment.matmul_queue_device([(segs[0], x.data_ptr(), F, T, batch, ys[0].data_ptr(), T, 0, 0)])
    del prepared


@pytest.mark.parametrize("batch", [1, 3, 7, 13])
def test_2d_tile_products_on_the_tensor_cores(ctx, oracle, batch, monkeypatch):
    """2-D tiles below 16 tokens, no column edge strip, tile width a multiple of 8 and
    n_atoms * tile_rows a multiple of 128: every tile product comes from ONE tensor-core GEMM
    (dictionary as n_atoms * tile_rows rows of tile_cols columns against batch * n_col_tiles
    "tokens"), written token-major for the gather. Against decompress + dense of the oracle, and
    against the CUDA-core projection (CSDR_TILE_TC=0) on the same payload; a row edge strip and
    bf16 token-major activations on device pointers included."""
    import torch
    from tests import synth
    pay = synth.hsdr_payload(200, 256, tile_rows=32, tile_cols=64, n_atoms=32, k=4, seed=21)   # 8 edge rows
    W = oracle.decompress(pay)
    x = np.random.default_rng(batch).normal(0, 1, (256, batch)).astype(np.float32)
    want = oracle.dense_matmul(W, x, batch)
    seg = cs.Segment.from_payload(pay, ctx)
    l0 = ctx.launch_count
    got = seg.matmul(x, batch, allow_2d=True)
    launches_tc = ctx.launch_count - l0
    e = rel_err(got, want)
    assert e[0] < TOL and e[1] < TOL, e
    # bf16 activations, token-major, on device pointers
    xt = torch.from_numpy(np.ascontiguousarray(x.T)).cuda().to(torch.bfloat16)
    yt = torch.empty((batch, 200), device="cuda", dtype=torch.float32)
    seg.matmul_device(xt.data_ptr(), cs.DTYPE_BF16, cs.TOKEN_MAJOR, batch, yt.data_ptr(), cs.TOKEN_MAJOR)
    ctx.synchronize()
    want16 = oracle.dense_matmul(W, np.ascontiguousarray(xt.float().cpu().numpy().T), batch)
    e = rel_err(yt.cpu().numpy().T, want16)
    assert e[0] < TOL and e[1] < TOL, e
    seg.close()
    monkeypatch.setenv("CSDR_TILE_TC", "0")
    plain = cs.Context(0)
    seg2 = cs.Segment.from_payload(pay, plain)
    l0 = plain.launch_count
    got2 = seg2.matmul(x, batch, allow_2d=True)
    launches_plain = plain.launch_count - l0
    e = rel_err(got2, want)
    assert e[0] < TOL and e[1] < TOL, e
    assert np.abs(got - got2).max() <= 1e-4 * np.abs(want).max()
    assert launches_tc != launches_plain or batch <= 4      # the two routes differ in their launches
    seg2.close()
    plain.close()
