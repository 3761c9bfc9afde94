"""BASELINE-sized cases on the GPU: config 1 (4096x4096, batch 1, both tile geometries),
config 2 (11008x4096, M in {1, 8, 64, 512}, bf16 activations) and config 5 (a q4_K source
tensor pair 14336x4096 / 4096x14336 behind one shared dictionary, M in {1, 128}), encoded by the reference's
own encoder where oracle/_ref is present (ksvd_iters=0: the legal fast mode; parity is
against the reference decoding the SAME archive), else by the synthetic writer. Checked
against the oracle and through size-independent properties."""
import os
import zlib

import numpy as np
import pytest

import cortexsdr_b200 as cs
from tests import synth
from conftest import rel_err

pytestmark = pytest.mark.gpu
TOL = 1e-3
CACHE = os.path.join(os.environ.get("TMPDIR", "/tmp"), "cortexsdr_b200_tests")


def _payload(tag, R, C, seed, geometry, seg_type):
    """geometry: 'row' = forRow1D(C) (K=512, 3x8); 'tile' = the reference's default 2-D config
    (128x128; K=256 k=5, or forMLP K=512 k=8 for FEED_FORWARD segments)."""
    os.makedirs(CACHE, exist_ok=True)
    path = os.path.join(CACHE, f"{tag}.hsdr")
    if os.path.exists(path):
        return open(path, "rb").read()
    from oracle.bindings import SEG_FEED_FORWARD, Reference, Segment, cfg_default, cfg_mlp, cfg_row1d
    mlp = seg_type == SEG_FEED_FORWARD
    if Reference.available():
        W = np.random.default_rng(seed).normal(0, 0.02, (R, C)).astype(np.float32)
        if geometry == "row":
            a = m = cfg_row1d(C, ksvd_iters=0)
        else:
            a, m = cfg_default(ksvd_iters=0), cfg_mlp(ksvd_iters=0)
        pay = Reference().compress(Segment(tag + ".weight", W, (R, C), seg_type), a, m)
    elif geometry == "row":
        pay = synth.hsdr_payload(R, C, seed=seed)
    else:
        pay = synth.hsdr_payload(R, C, tile_rows=128, tile_cols=128, n_atoms=512 if mlp else 256,
                                 k=8 if mlp else 5, seed=seed)
    open(path, "wb").write(pay)
    return pay


def test_config1_row_tiles(ctx, oracle):
    from oracle.bindings import SEG_WEIGHTS_FP32
    pay = _payload("cfg1_row", 4096, 4096, 0, "row", SEG_WEIGHTS_FP32)
    info = cs.inspect_payload(pay)
    assert (info.n_atoms, info.n_stages, info.k_per_stage, info.tile_rows) == (512, 3, 8, 1)
    assert len(pay) == 8585264                       # 36 + 12 + 4*512*4096 + 2*4096*24
    seg = cs.Segment.from_payload(pay, ctx)
    idx, sign = seg.unpack()
    _, oidx, osign, _ = oracle.codes(pay)
    assert np.array_equal(idx, oidx) and np.array_equal(sign, osign)
    x = np.random.default_rng(1).normal(0, 1, (4096, 1)).astype(np.float32)
    y = seg.matmul(x, 1)
    e = rel_err(y, oracle.matmul(pay, x, 1))
    assert e[0] < TOL and e[1] < TOL, e
    # the decompress + dense route of the reference agrees with the fused one
    W = seg.decompress()
    assert zlib.crc32(W.tobytes()) == zlib.crc32(oracle.decompress(pay).tobytes())
    e = rel_err(y, oracle.dense_matmul(W, x, 1))
    assert e[0] < TOL and e[1] < TOL, e
    # linearity of the whole path
    x2 = np.random.default_rng(2).normal(0, 1, (4096, 1)).astype(np.float32)
    lin = seg.matmul(x + 2 * x2, 1) - (y + 2 * seg.matmul(x2, 1))
    assert np.abs(lin).max() < 1e-4 * np.abs(y).max()


def test_config1_default_2d_tiles(ctx, oracle):
    from oracle.bindings import SEG_WEIGHTS_FP32
    pay = _payload("cfg1_tile", 4096, 4096, 0, "tile", SEG_WEIGHTS_FP32)
    info = cs.inspect_payload(pay)
    assert (info.tile_rows, info.tile_cols, info.n_atoms, info.k_per_stage) == (128, 128, 256, 5)
    assert len(pay) == 16807984
    seg = cs.Segment.from_payload(pay, ctx)
    W = seg.decompress()
    Wo = oracle.decompress(pay)
    assert np.array_equal(W, Wo)
    x = np.random.default_rng(1).normal(0, 1, (4096, 1)).astype(np.float32)
    with pytest.raises(cs.CompressionError):
        seg.matmul(x, 1)                             # the reference refuses 2-D tiles here
    e = rel_err(seg.matmul(x, 1, allow_2d=True), oracle.dense_matmul(Wo, x, 1))
    assert e[0] < TOL and e[1] < TOL, e


@pytest.mark.parametrize("M", [1, 8, 64, 512])
def test_config2_mlp_projection_sweep(ctx, oracle, M):
    import torch
    from oracle.bindings import SEG_FEED_FORWARD
    pay = _payload("cfg2_row", 11008, 4096, 2, "row", SEG_FEED_FORWARD)
    seg = cs.Segment.from_payload(pay, ctx)
    g = torch.Generator(device="cuda").manual_seed(3)
    xb = torch.randn((M, 4096), generator=g, device="cuda").to(torch.bfloat16)
    y = torch.empty((M, 11008), device="cuda", dtype=torch.float32)
    torch.cuda.synchronize()
    seg.matmul_device(xb.data_ptr(), cs.DTYPE_BF16, cs.TOKEN_MAJOR, M, y.data_ptr(), cs.TOKEN_MAJOR)
    ctx.synchronize()
    x32 = xb.float().cpu().numpy()                   # the bf16-rounded values, widened
    want = oracle.matmul(pay, np.ascontiguousarray(x32.T), M).T
    e = rel_err(y.cpu().numpy(), want)
    assert e[0] < TOL and e[1] < TOL, (M, e)


def test_config2_default_2d_tiles_mlp(ctx, oracle):
    from oracle.bindings import SEG_FEED_FORWARD
    pay = _payload("cfg2_tile", 11008, 4096, 2, "tile", SEG_FEED_FORWARD)
    info = cs.inspect_payload(pay)
    assert (info.n_atoms, info.k_per_stage, info.n_tiles) == (512, 8, 86 * 32)
    seg = cs.Segment.from_payload(pay, ctx)
    Wo = oracle.decompress(pay)
    assert np.array_equal(seg.decompress(), Wo)
    for M in (1, 4, 64, 512):
        x = np.random.default_rng(M).normal(0, 1, (4096, M)).astype(np.float32)
        e = rel_err(seg.matmul(x, M, allow_2d=True), oracle.dense_matmul(Wo, x, M))
        assert e[0] < TOL and e[1] < TOL, (M, e)


def test_config5_kquant_source_shared_dictionary(ctx, oracle, tmp_path):
    """Two k-quant (q4_K) source tensors, 14336x4096 and 4096x14336: dequantised on the device
    bit for bit like the oracle, then - as the reference does for quantised GGUF tensors, whose
    blocks are source dtypes, not coefficient packing - HSDR-encoded from the fp32 values by the
    reference encoder into an .hsda whose FEED_FORWARD role shares one 128x128-tile dictionary.
    Default density here (8 atoms per stage); the sparsity sweep is test_config5_sparsity_sweep."""
    import torch
    from oracle.bindings import SEG_FEED_FORWARD, Reference, Segment, cfg_default, cfg_mlp
    if not Reference.available():
        pytest.skip("needs the compiled reference (oracle/_ref) to write the shared-dictionary archive")
    ref = Reference()
    st = cs.HierarchicalSDRStrategy(ctx)
    rng = np.random.default_rng(55)
    shapes = ((14336, 4096), (4096, 14336))
    segs = []
    for i, (R, C) in enumerate(shapes):
        nblk = R * C // 256
        raw = rng.integers(0, 256, size=(nblk, 144), dtype=np.uint8)
        # fp16 super-scale d and super-min dmin of every block: small, finite
        raw[:, 0:4] = rng.normal(0, 0.002, size=(nblk, 2)).astype(np.float16).view(np.uint8).reshape(nblk, 4)
        raw = raw.reshape(-1)
        w = st.dequantizeToFP32(raw, "q4_k")
        assert w.size == R * C
        want = oracle.dequantize("q4_k", raw)
        assert zlib.crc32(w.tobytes()) == zlib.crc32(want.tobytes())          # bit-exact at full size
        segs.append(Segment(f"blk.{i}.ffn.weight", w.reshape(R, C), (R, C), SEG_FEED_FORWARD, layer_index=i))
    path = str(tmp_path / "cfg5.hsda")
    n_dicts = ref.hsda_write(segs, path, cfg_default(ksvd_iters=0), cfg_mlp(ksvd_iters=0))
    assert n_dicts == 1                                                       # one dictionary for both tensors
    r = cs.HSDAReader.fromFile(path, ctx)
    assert r.numDictionaries() == 1
    for i, (R, C) in enumerate(shapes):
        name = f"blk.{i}.ffn.weight"
        W = r.decompress(name)
        assert zlib.crc32(W.tobytes()) == zlib.crc32(ref.hsda_decompress(path, name, R, C).tobytes())
        Wd = torch.from_numpy(W).cuda()
        for M in (1, 128):
            xb = torch.randn((C, M), generator=torch.Generator().manual_seed(M + i)).to(torch.bfloat16).float()
            x = np.ascontiguousarray(xb.numpy())
            with pytest.raises(cs.CompressionError):
                r.matmul(name, x, M)                                          # the reference refuses 2-D tiles here
            y = r.matmul(name, x, M, allow_2d=True)
            want = (Wd.double() @ xb.cuda().double()).float().cpu().numpy()  # dense product of the decoded weights
            e = rel_err(y, want)
            assert e[0] < TOL and e[1] < TOL, (name, M, e)
        del Wd


@pytest.mark.parametrize("sparsity,k", [(0.01, 2), (0.02, 3), (0.05, 9)])
def test_config5_sparsity_sweep(ctx, oracle, tmp_path, sparsity, k):
    """The sparsity settings of the k-quant configuration. HSDR ignores the archive-level sparsity
    option, so the sweep is mapped onto the codec's own density: active atoms per stage
    k = max(1, round(sparsity * n_atoms / n_stages)) = 2, 3, 9 for 512 atoms in 3 stages (this
    mapping is this repository's, not the reference's). Both tensors share one dictionary of
    128x128 tiles; products at M = 1 and 128 against the dense product of the weights the
    reference decodes from the same archive."""
    import torch
    from oracle.bindings import SEG_FEED_FORWARD, Reference, Segment, cfg_default, cfg_mlp
    if not Reference.available():
        pytest.skip("needs the compiled reference (oracle/_ref) to write the shared-dictionary archive")
    assert k == max(1, round(sparsity * 512 / 3))
    ref = Reference()
    shapes = ((14336, 4096), (4096, 14336))
    segs = [Segment(f"blk.{i}.ffn.weight", np.random.default_rng(10 + i).normal(0, 0.02, s).astype(np.float32), s,
                    SEG_FEED_FORWARD, layer_index=i) for i, s in enumerate(shapes)]
    path = str(tmp_path / f"cfg5_k{k}.hsda")
    assert ref.hsda_write(segs, path, cfg_default(ksvd_iters=0), cfg_mlp(ksvd_iters=0, k=k)) == 1
    del segs
    r = cs.HSDAReader.fromFile(path, ctx)
    for i, (R, C) in enumerate(shapes):
        name = f"blk.{i}.ffn.weight"
        W = r.decompress(name)
        assert zlib.crc32(W.tobytes()) == zlib.crc32(ref.hsda_decompress(path, name, R, C).tobytes())
        Wd = torch.from_numpy(W).cuda()
        for M in (1, 128):
            xb = torch.randn((C, M), generator=torch.Generator().manual_seed(M + i)).to(torch.bfloat16).float()
            y = r.matmul(name, np.ascontiguousarray(xb.numpy()), M, allow_2d=True)
            want = (Wd.double() @ xb.cuda().double()).float().cpu().numpy()
            e = rel_err(y, want)
            assert e[0] < TOL and e[1] < TOL, (name, k, M, e)
        del Wd
