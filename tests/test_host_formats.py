"""Host logic behind the C-ABI that needs no GPU: the library loads and exports every
declared symbol, payload framing and validation, the .sdr index and .hsda container
readers, and the loud failure of compute calls when no device is present."""
import ctypes as C
import os
import re

import numpy as np
import pytest

import cortexsdr_b200 as cs
from cortexsdr_b200 import _lib
from conftest import GOLDEN, ROOT


def test_library_exports_every_declared_symbol(lib):
    header = open(os.path.join(ROOT, "include", "cortexsdr_b200.h")).read()
    declared = set(re.findall(r"CSDR_API\s+[\w\s\*]+?\b(csdr_\w+)\s*\(", header))
    assert len(declared) >= 40
    assert declared == set(_lib.SIGNATURES), declared ^ set(_lib.SIGNATURES)
    for name in declared:
        assert hasattr(lib, name), name
    sdk = open(os.path.join(ROOT, "include", "cortex_sdk_b200.h")).read()
    for name in set(re.findall(r"\b(cortex_\w+)\s*\(", sdk)):
        assert hasattr(lib, name), name


def test_payload_inspect_rowtile(golden):
    g = golden("fused_rowtile.npz")
    i = cs.inspect_payload(g["payload"])
    assert (i.kind, i.rows, i.cols, i.n_tiles, i.tile_rows, i.tile_cols) == (0, 256, 512, 256, 1, 512)
    assert (i.n_atoms, i.n_stages, i.k_per_stage, i.stage_decay, i.edge_bytes) == (128, 3, 6, 0.5, 0)
    assert i.off_scales == 36 and i.off_dict == 48 and i.off_codes == 48 + 4 * 128 * 512
    assert i.payload_bytes == g["payload"].size


def test_payload_inspect_edges(golden):
    g = golden("tiles_2d.npz")
    i = cs.inspect_payload(g["edges_payload"])
    assert (i.rows, i.cols, i.n_tiles, i.edge_bytes) == (290, 257, 72, 4 * (288 + 2 * 257))
    assert i.off_edges + i.edge_bytes == i.payload_bytes


@pytest.mark.parametrize("mutate,exc", [
    (lambda p: p[:20], cs.CompressionError),                                   # truncated header
    (lambda p: np.concatenate([np.frombuffer(b"XSDR", np.uint8), p[4:]]), cs.CompressionError),  # magic
    (lambda p: np.concatenate([p[:4], np.array([9, 0, 0, 0], np.uint8), p[8:]]), cs.CompressionError),  # version
    (lambda p: p[:-7], cs.CompressionError),                                   # truncated stream
])
def test_payload_rejects_malformed(golden, mutate, exc):
    p = golden("fused_rowtile.npz")["payload"].copy()
    with pytest.raises(exc):
        cs.inspect_payload(mutate(p))


def test_payload_rejects_out_of_range_atom_index(golden):
    p = golden("fused_rowtile.npz")["payload"].copy()
    i = cs.inspect_payload(p)
    p[i.off_codes:i.off_codes + 2] = np.array([200], np.uint16).view(np.uint8)  # K is 128
    with pytest.raises(cs.CompressionError, match="atom index"):
        cs.inspect_payload(p)
    p[i.off_codes:i.off_codes + 2] = np.array([0x8000 | 127], np.uint16).view(np.uint8)  # sign bit is not index
    cs.inspect_payload(p)


def test_sdr_index_reader():
    ld = cs.SDRModelLoader(os.path.join(GOLDEN, "routing.sdr"), index_only=True)
    hs = ld.getSegmentHeaders()
    assert [h.name for h in hs] == ["layer.hsdr.weight", "layer.raw.weight", "layer.norm.weight"]
    assert [h.compression_strategy_id for h in hs] == [5, 0, 0]
    assert hs[0].dimensions == (256, 512) and hs[0].original_size == 256 * 512 * 4
    assert hs[2].dimensions == (256,)
    assert ld.findSegmentHeader("missing") is None
    pay = ld.loadCompressedBytesByName("layer.hsdr.weight")
    assert len(pay) == hs[0].compressed_size and pay[:4] == b"HSDR"
    raw = ld.loadSegmentByName("layer.norm.weight")           # strategy 0: stored bytes
    assert np.array_equal(raw.view(np.float32), np.ones(256, np.float32))
    with pytest.raises(RuntimeError, match="Segment not found"):
        ld.loadCompressedBytesByName("missing")


def test_sdr_rejects_bad_archives(tmp_path):
    p = tmp_path / "bad.sdr"
    p.write_bytes(b"NOTCORTX" + b"\0" * 32)
    with pytest.raises(cs.CompressionError, match="magic"):
        cs.SDRModelLoader(str(p), index_only=True)
    good = open(os.path.join(GOLDEN, "routing.sdr"), "rb").read()
    p.write_bytes(good[:len(good) - 40])                      # index cut short
    with pytest.raises(cs.CompressionError):
        cs.SDRModelLoader(str(p), index_only=True)
    with pytest.raises(RuntimeError):
        cs.SDRModelLoader(str(tmp_path / "absent.sdr"), index_only=True)


def test_hsda_reader_structure():
    r = cs.HSDAReader.fromFile(os.path.join(GOLDEN, "reader.hsda"), index_only=True)
    assert (r.numDictionaries(), r.numSegments()) == (2, 8)
    assert r.hasSegment("model.layers.4.attn.q_proj.weight")
    assert not r.hasSegment("model.layers.9.attn.q_proj.weight")


def test_hsda_rejects_truncation(tmp_path):
    good = open(os.path.join(GOLDEN, "reader.hsda"), "rb").read()
    p = tmp_path / "cut.hsda"
    p.write_bytes(good[:len(good) // 2])
    with pytest.raises(cs.CompressionError):
        cs.HSDAReader.fromFile(str(p), index_only=True)


def test_compute_fails_loudly_without_device():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    with pytest.raises(cs.CudaError, match="no CPU path"):
        cs.Context()
    ld = cs.SDRModelLoader(os.path.join(GOLDEN, "routing.sdr"), index_only=True)
    with pytest.raises(cs.CudaError):
        ld.matmulHSDR("layer.hsdr.weight", np.zeros((512, 1), np.float32), 1)


def test_shared_dictionary_resources_in_the_index(tmp_path, oracle):
    """An .sdr with shared-dictionary resource segments is an ordinary archive to the index reader:
    the dictionary is a stored-raw segment whose payload is one .hsda dictionary record, a tensor
    coded against it carries a codes-only payload and names the dictionary in its data_format."""
    from tests import synth
    from oracle.bindings import SharedDict
    cfg = dict(n_layers=2, hidden=64, q_heads=2, kv_heads=1, head_dim=32, inter=128, vocab=50)
    path = str(tmp_path / "shared.sdr")
    synth.decoder_archive(path, **cfg, k=3, n_atoms=16, kv_atoms=8, shared_dicts=True)
    ld = cs.SDRModelLoader(path, index_only=True)
    names = [h.name for h in ld.getSegmentHeaders()]
    assert sum(n.startswith("hsdr.shared_dict/") for n in names) == 7          # one per block role, not per block
    d = ld.findSegmentHeader("hsdr.shared_dict/ffn_down")
    assert (d.data_format, d.compression_strategy_id) == ("hsdr_dict", 0)
    tr, tc, K, S, k, atoms, scales = synth.read_dictionary_record(ld.loadSegmentByName(d.name))
    assert (tr, tc, K, S, k) == (1, cfg["inter"], 16, 3, 3) and atoms.shape == (16, cfg["inter"])
    for blk in (0, 1):
        h = ld.findSegmentHeader(f"blk.{blk}.ffn_down.weight")
        assert (h.data_format, h.compression_strategy_id) == ("hsdc@hsdr.shared_dict/ffn_down", 5)
        pay = ld.loadCompressedBytesByName(h.name)
        assert bytes(pay[:4]) == b"HSDC" and cs.inspect_payload(pay).kind == 1   # CSDR_KIND_HSDC
        w = oracle.hsdc_decompress(pay, SharedDict(tr, tc, K, S, k, atoms, scales))
        assert w.shape == (cfg["hidden"], cfg["inter"]) and np.isfinite(w).all()


def test_routing_errors_before_any_compute():
    ld = cs.SDRModelLoader(os.path.join(GOLDEN, "routing.sdr"), index_only=True)
    with pytest.raises(RuntimeError, match="matmulHSDR: segment not found"):
        ld.matmulHSDR("missing", np.zeros((512, 1), np.float32), 1)
    with pytest.raises(RuntimeError, match=r"is not HSDR-encoded \(strategy_id=0\)"):
        ld.matmulHSDR("layer.raw.weight", np.zeros((256, 1), np.float32), 1)


def test_payload_reader_agrees_with_an_independent_writer(oracle):
    # payloads framed by the oracle's restatement of the reference encoder (a writer that shares no
    # code with the library's reader): every geometry is accepted and every field agrees,
    # including the edge-strip offsets; a truncated or over-long index in any of them is rejected
    rng = np.random.default_rng(21)
    for R, Cc, tr, tc, K, S, k in ((40, 64, 1, 64, 16, 3, 2), (70, 52, 16, 16, 8, 2, 3), (33, 48, 8, 24, 4, 1, 1),
                                   (64, 64, 32, 32, 4, 3, 4), (19, 130, 1, 128, 16, 4, 2)):
        W = rng.normal(0, 0.05, (R, Cc)).astype(np.float32)
        pay = oracle.encode_fast(W, tr, tc, K, S, k, 0.5)
        i = cs.inspect_payload(pay)
        n_tiles = (R // tr) * (Cc // tc)
        edge = 4 * ((R // tr) * tr * (Cc - (Cc // tc) * tc) + (R - (R // tr) * tr) * Cc)
        assert (i.kind, i.rows, i.cols, i.n_tiles, i.tile_rows, i.tile_cols) == (0, R, Cc, n_tiles, tr, tc)
        assert (i.n_atoms, i.n_stages, i.k_per_stage, i.stage_decay, i.edge_bytes) == (K, S, k, 0.5, edge)
        assert i.off_scales == 36 and i.off_dict == 36 + 4 * S
        assert i.off_codes == i.off_dict + 4 * K * tr * tc and i.off_edges == i.off_codes + 2 * n_tiles * S * k
        assert i.payload_bytes == pay.size == i.off_edges + edge
        with pytest.raises(cs.CompressionError):
            cs.inspect_payload(pay[:-1])
        bad = pay.copy()
        bad[i.off_codes:i.off_codes + 2] = np.array([K], np.uint16).view(np.uint8)     # first index past the table
        with pytest.raises(cs.CompressionError, match="atom index"):
            cs.inspect_payload(bad)
