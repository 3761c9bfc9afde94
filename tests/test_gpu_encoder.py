"""The encoder on the GPU (fast mode and dictionary-update rounds) against the oracle's restatement of the reference encoder
(pinned to the reference's own payloads in test_oracle_golden.py) and against the payloads the
reference encoder wrote (tests/golden/encoder_coding.npz).

The device codes the tiles from projections computed once and updated through the Gram matrix;
the reference re-projects a residual every round. The two are equal in exact arithmetic, so the
bar is: header, stage scales, tile picks and edge strips identical; atoms within 2e-6 of the
largest atom value; codes identical except where a round's best candidates tie within rounding
(at least 99.5 % identical here), and a reconstruction error within 1e-4 (relative) of the
reference's."""
import numpy as np
import pytest

import cortexsdr_b200 as cs

pytestmark = pytest.mark.gpu


def _tiles_of(W, tile_rows, tile_cols):
    # extractTiles order (strategies/HierarchicalSDRStrategy.cpp:95-116)
    nr, nc = W.shape[0] // tile_rows, W.shape[1] // tile_cols
    return np.stack([W[a * tile_rows:(a + 1) * tile_rows, b * tile_cols:(b + 1) * tile_cols].reshape(-1)
                     for a in range(nr) for b in range(nc)])


def _rebuild(tiles_shape, D, scales, codes):
    # decodeAllTiles (:612-634) on the host, in double
    n, T = tiles_shape
    out = np.zeros((n, T))
    idx, sgn = (codes & 0x7FFF).astype(np.int64), np.where(codes & 0x8000, -1.0, 1.0)
    for l in range(codes.shape[1]):
        for s in range(codes.shape[2]):
            out += (scales[l] * sgn[:, l, s])[:, None] * D[idx[:, l, s]].astype(np.float64)
    return out


def _compare_codes(tiles, D, scales, mine, ref):
    same = float((mine == ref).mean())
    assert same >= 0.995, same
    err_m = np.linalg.norm(tiles - _rebuild(tiles.shape, D, scales, mine)) / np.linalg.norm(tiles)
    err_r = np.linalg.norm(tiles - _rebuild(tiles.shape, D, scales, ref)) / np.linalg.norm(tiles)
    assert abs(err_m - err_r) <= 1e-4 * max(err_r, 1e-12), (err_m, err_r)
    # an atom is used at most once per stage (used_this_stage, :229-241)
    per_stage = (mine & 0x7FFF).reshape(-1, mine.shape[2])
    assert all(len(set(r)) == mine.shape[2] for r in per_stage.tolist())
    return same


@pytest.mark.parametrize("label", ["row_fast", "row_fit", "tiles_2d"])
def test_coding_pass_against_reference_payloads(ctx, oracle, golden, label):
    g = golden("encoder_coding.npz")
    W, pay = g[label + "_w"], g[label + "_payload"]
    v = oracle.parse(pay)
    T = v.tile_rows * v.tile_cols
    D = pay[v.off_dict:v.off_dict + 4 * v.n_atoms * T].view(np.float32).reshape(v.n_atoms, T)
    packed, _, _, scales = oracle.codes(pay)
    tiles = _tiles_of(W, v.tile_rows, v.tile_cols)
    mine = cs.HierarchicalSDRStrategy(ctx).encode_codes(tiles, D, scales, v.k)
    _compare_codes(tiles, D, scales, mine, packed.reshape(mine.shape))


@pytest.mark.parametrize("shape,tile,atoms,k", [((96, 128), (1, 128), 32, 4), ((100, 150), (16, 16), 32, 4),
                                                 ((512, 1024), (1, 1024), 128, 6), ((640, 512), (32, 64), 128, 5)])
def test_fast_mode_payload_against_the_oracle(ctx, oracle, shape, tile, atoms, k):
    # the last two shapes have 128 atoms and tile widths that are multiples of 8: projections and
    # Gram matrix on the tensor cores; the first two run on the CUDA cores
    W = np.random.default_rng(shape[0]).normal(0, 0.05, shape).astype(np.float32)
    st = cs.HierarchicalSDRStrategy(ctx)
    mine = np.frombuffer(st.compress(W, tile_rows=tile[0], tile_cols=tile[1], n_atoms=atoms, k=k), np.uint8)
    want = oracle.encode_fast(W, tile[0], tile[1], atoms, 3, k, 0.5, 0)
    v = oracle.parse(want)
    assert mine.size == want.size
    assert np.array_equal(mine[:v.off_dict], want[:v.off_dict])                      # header + stage scales
    T = tile[0] * tile[1]
    Dw = want[v.off_dict:v.off_codes].view(np.float32).reshape(atoms, T)
    Dm = mine[v.off_dict:v.off_codes].view(np.float32).reshape(atoms, T)
    assert np.abs(Dw - Dm).max() <= 2e-6 * np.abs(Dw).max()                          # same tiles picked, same scale
    assert np.array_equal(mine[v.off_edges:], want[v.off_edges:])                    # edge strips
    n = v.n_tiles * v.n_stages * v.k
    cm = mine[v.off_codes:v.off_codes + 2 * n].view(np.uint16).reshape(v.n_tiles, v.n_stages, v.k)
    cw = want[v.off_codes:v.off_codes + 2 * n].view(np.uint16).reshape(v.n_tiles, v.n_stages, v.k)
    scales = want[v.off_scales:v.off_scales + 4 * v.n_stages].view(np.float32)
    tiles = _tiles_of(W, *tile)
    _compare_codes(tiles, Dw, scales, cm, cw)
    # what this library encoded, it and the oracle decode alike
    seg = cs.Segment.from_payload(mine.tobytes(), ctx)
    assert np.array_equal(seg.decompress(), oracle.decompress(mine))
    seg.close()


def test_encoder_refusals(ctx):
    st = cs.HierarchicalSDRStrategy(ctx)
    W = np.zeros((8, 64), np.float32)
    with pytest.raises(cs.CompressionError, match="smaller than one tile"):
        st.compress(W, tile_rows=16, tile_cols=16, n_atoms=4)
    with pytest.raises(cs.CompressionError, match="not enough tiles"):
        st.compress(W, tile_rows=1, tile_cols=64, n_atoms=16)


def _parts(pay, oracle):
    v = oracle.parse(pay)
    T = v.tile_rows * v.tile_cols
    D = pay[v.off_dict:v.off_codes].view(np.float32).reshape(v.n_atoms, T)
    n = v.n_tiles * v.n_stages * v.k
    codes = pay[v.off_codes:v.off_codes + 2 * n].view(np.uint16).reshape(v.n_tiles, v.n_stages, v.k)
    return v, D, codes


def _rel_error(W, pay, oracle):
    return float(np.linalg.norm(W - oracle.decompress(pay)) / np.linalg.norm(W))


@pytest.mark.parametrize("shape,tile,atoms,k,iters", [((96, 128), (1, 128), 32, 4, 1), ((96, 128), (1, 128), 32, 4, 3),
                                                       ((100, 150), (16, 16), 32, 4, 2), ((512, 1024), (1, 1024), 128, 6, 1),
                                                       ((512, 1024), (1, 1024), 128, 6, 3), ((256, 4608), (1, 4608), 128, 4, 2)])
def test_dictionary_update_rounds_against_the_oracle(ctx, oracle, shape, tile, atoms, k, iters):
    """fitHierarchicalKSVD with update rounds (atomUpdateStep, strategies/HierarchicalSDRStrategy.cpp:281-489,
    then the coding pass again, :573-577). A round's atoms are a function of the round's codes, and
    the device's coding pass may differ from the reference's where two candidates tie within
    rounding (see above), after which the two fits drift apart on the atoms that tile uses. So:
    header, scales and edge strips identical; after ONE round nearly all atoms within 2e-5 of the
    largest atom value and nearly all codes equal; after any number of rounds the same
    reconstruction error (within 2e-3 relative) as the oracle's fit, and a better one than the
    fast mode's. The last shape is wider than one column block of the update kernel."""
    W = np.random.default_rng(shape[0] + iters).normal(0, 0.05, shape).astype(np.float32)
    st = cs.HierarchicalSDRStrategy(ctx)
    kw = dict(tile_rows=tile[0], tile_cols=tile[1], n_atoms=atoms, k=k)
    mine = np.frombuffer(st.compress(W, **kw, ksvd_iters=iters), np.uint8)
    fast = np.frombuffer(st.compress(W, **kw, ksvd_iters=0), np.uint8)
    want = oracle.encode_fast(W, tile[0], tile[1], atoms, 3, k, 0.5, iters)
    v, Dw, cw = _parts(want, oracle)
    _, Dm, cm = _parts(mine, oracle)
    assert mine.size == want.size
    assert np.array_equal(mine[:v.off_dict], want[:v.off_dict]) and np.array_equal(mine[v.off_edges:], want[v.off_edges:])
    assert np.isfinite(Dm).all()
    if iters == 1:
        close = np.abs(Dw - Dm).max(axis=1) <= 2e-5 * np.abs(Dw).max()
        assert close.mean() >= 0.9, close.mean()
        assert float((cm == cw).mean()) >= 0.98
    err_m, err_w, err_f = _rel_error(W, mine, oracle), _rel_error(W, want, oracle), _rel_error(W, fast, oracle)
    assert abs(err_m - err_w) <= 2e-3 * err_w, (err_m, err_w)
    assert err_m < err_f, (err_m, err_f)
    seg = cs.Segment.from_payload(mine.tobytes(), ctx)
    assert np.array_equal(seg.decompress(), oracle.decompress(mine))
    seg.close()


def test_unused_atoms_are_replaced_as_the_reference_replaces_them(ctx, oracle):
    """One code per tile and as many atoms as tiles: most atoms have no user after the coding pass
    and become a random tile scaled to the target norm (:406-428), drawn from a generator seeded
    per atom. Codes of such a tiny problem have no near ties, so the whole payload follows the
    oracle: atoms within 2e-6, codes equal."""
    W = np.random.default_rng(5).normal(0, 0.05, (64, 64)).astype(np.float32)
    st = cs.HierarchicalSDRStrategy(ctx)
    mine = np.frombuffer(st.compress(W, tile_rows=1, tile_cols=64, n_atoms=64, n_stages=1, k=1, ksvd_iters=2), np.uint8)
    want = oracle.encode_fast(W, 1, 64, 64, 1, 1, 0.5, 2)
    v, Dw, cw = _parts(want, oracle)
    _, Dm, cm = _parts(mine, oracle)
    used_first = np.unique(_parts(oracle.encode_fast(W, 1, 64, 64, 1, 1, 0.5, 0), oracle)[2] & 0x7FFF).size
    assert used_first < 64                                   # the case does leave atoms unused
    assert np.abs(Dw - Dm).max() <= 2e-6 * np.abs(Dw).max()
    assert np.array_equal(cm, cw)


def _hsda_parts(raw):
    import struct
    raw = bytes(raw)
    assert raw[:4] == b"HSDA"
    _, nd, ns = struct.unpack_from("<III", raw, 4)
    assert nd == 1
    o = 16
    record_at = o
    tr, tc, K, S, k = struct.unpack_from("<HHHBB", raw, o)
    o += 20
    (n_sc,) = struct.unpack_from("<I", raw, o)
    o += 4 + 4 * n_sc
    (n_at,) = struct.unpack_from("<I", raw, o)
    o += 4 + 4 * n_at
    record = raw[record_at:o]
    codes = []
    for _ in range(ns):
        (ln,) = struct.unpack_from("<I", raw, o)
        o += 4 + ln
        _, _, _, clen = struct.unpack_from("<IQBI", raw, o)
        o += 17
        codes.append(raw[o:o + clen])
        o += clen
    return (tr, tc, K, S, k), record, codes


@pytest.mark.parametrize("label,iters", [("rows", 2), ("tiles", 0)])
def test_grouped_encoder_against_the_reference_archive(ctx, oracle, golden, label, iters):
    """Several tensors behind one dictionary (compressGroupedSegments, :2211-2500) on the device,
    against the .hsda the reference wrote from the same weights: the dictionary record's config and
    stage scales byte for byte (the reference's ksvd_iters and max_tiles_for_fit fields included),
    atoms within 2e-6 of the largest, every tensor's codes-only payload with its header equal and
    its codes equal except at rounding ties (>= 99.5 %), and the same reconstruction."""
    from tests import synth
    from oracle.bindings import SharedDict
    g = golden("grouped_encoder.npz")
    (tr, tc, K, S, k), record, ref_codes = _hsda_parts(g[label + "_hsda"])
    Ws = [g[f"{label}_w{i}"] for i in range(int(g[label + "_n"]))]
    rec, pays = cs.HierarchicalSDRStrategy(ctx).compress_shared(Ws, tile_rows=tr, tile_cols=tc, n_atoms=K, n_stages=S, k=k,
                                                                ksvd_iters=iters)
    assert len(rec) == len(record)
    head = 24 + 4 * S + 4                                   # config, counted scales, atom count
    # bytes 9..11 are padding inside the reference's raw struct (whatever its stack held); zero here
    assert rec[:9] == record[:9] and rec[12:head] == record[12:head] and rec[9:12] == bytes(3)
    mine, want = synth.read_dictionary_record(rec), synth.read_dictionary_record(record)
    assert np.abs(mine[5] - want[5]).max() <= 2e-6 * np.abs(want[5]).max()
    d_ref = SharedDict(*want)
    for W, pay, ref_pay in zip(Ws, pays, ref_codes):
        assert pay[:32] == ref_pay[:32] and len(pay) == len(ref_pay)
        a, b = np.frombuffer(pay, np.uint16, offset=32), np.frombuffer(ref_pay, np.uint16, offset=32)
        assert float((a == b).mean()) >= 0.995
        err_m = np.linalg.norm(W - oracle.hsdc_decompress(pay, SharedDict(*mine))) / np.linalg.norm(W)
        err_r = np.linalg.norm(W - oracle.hsdc_decompress(ref_pay, d_ref)) / np.linalg.norm(W)
        assert abs(err_m - err_r) <= 1e-4 * err_r, (err_m, err_r)


def test_grouped_encoder_to_an_archive_with_shared_dictionaries(ctx, oracle, tmp_path):
    """From weights to products through a shared dictionary, all on this library: three tensors
    encoded behind one dictionary on the device, written as a .sdr whose dictionary is a resource
    segment and whose tensors are codes-only segments naming it, opened and multiplied; against
    the oracle's grouped encoder and its external-dictionary product."""
    from tests import synth
    from oracle.bindings import SharedDict
    rng = np.random.default_rng(31)
    Ws = [rng.normal(0, 0.05, (r, 256)).astype(np.float32) for r in (128, 64, 192)]
    kw = dict(tile_rows=1, tile_cols=256, n_atoms=128, n_stages=3, k=4)
    st = cs.HierarchicalSDRStrategy(ctx)
    rec, pays = st.compress_shared(Ws, **kw, ksvd_iters=1)
    d_want, pays_want = oracle.encode_shared(Ws, 1, 256, 128, 3, 4, 0.5, 1)
    mine = synth.read_dictionary_record(rec)
    assert np.array_equal(mine[6], d_want.scales)
    segs = [dict(name="hsdr.shared_dict/ffn_up", payload=rec, strategy_id=0, original_type=synth.SEG_CONFIG, dims=(128, 256),
                 original_size=128 * 256 * 4, data_format=synth.SHARED_DICT_FORMAT, layer_type="", layer_index=0)]
    for i, (W, pay) in enumerate(zip(Ws, pays)):
        segs.append(dict(name=f"blk.{i}.ffn_up.weight", payload=pay, strategy_id=5, original_type=synth.SEG_FEED_FORWARD,
                         dims=W.shape, original_size=W.nbytes, data_format="hsdc@hsdr.shared_dict/ffn_up", layer_index=i))
    path = str(tmp_path / "grouped.sdr")
    synth.write_sdr(path, segs)
    ld = cs.SDRModelLoader(path, ctx)
    x = rng.normal(0, 1, (256, 3)).astype(np.float32)
    d_mine = SharedDict(*mine)
    for i, (W, pay) in enumerate(zip(Ws, pays)):
        y = ld.matmulHSDR(f"blk.{i}.ffn_up.weight", x, 3)
        want = oracle.hsdc_matmul(pay, d_mine, x, 3)                         # this archive, decoded by the oracle
        assert np.abs(y - want).max() <= 1e-3 * np.abs(want).max()
        # and the fit is as good as the oracle's own grouped fit of the same weights
        err_m = np.linalg.norm(W - oracle.hsdc_decompress(pay, d_mine)) / np.linalg.norm(W)
        err_w = np.linalg.norm(W - oracle.hsdc_decompress(pays_want[i], d_want)) / np.linalg.norm(W)
        assert abs(err_m - err_w) <= 2e-3 * err_w, (err_m, err_w)
    ld.close()
    with pytest.raises(cs.CompressionError, match="not divisible"):
        st.compress_shared([np.zeros((10, 100), np.float32)], tile_rows=4, tile_cols=32, n_atoms=2)
