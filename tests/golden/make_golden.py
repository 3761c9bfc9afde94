"""Regenerates the golden fixtures in this folder by running the UNMODIFIED reference
(oracle/_ref/libcortexsdr_ref.so, built by oracle/Makefile from the reference tree).

Run from the repository root, where the reference tree is available:
    python tests/golden/make_golden.py

Seeds, shapes and encoder settings are those of the reference's own tests
(src/test_hsdr_roundtrip.cpp, test_hsdr_archive_e2e.cpp, test_inference_matmul_routing.cpp,
test_hsda_reader.cpp, test_hsdr_kquants.cpp), drawn with the same libstdc++
mt19937 + normal_distribution sequence. The encoder is multi-threaded with -ffast-math, so
archives are generated once here and shared by every implementation under test.
"""
import os
import sys
import zlib

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle.bindings import (SEG_ATTENTION, SEG_FEED_FORWARD, SEG_LAYER_NORM,  # noqa: E402
                             SEG_WEIGHTS_FP32, SEG_WEIGHTS_INT8, Reference, Segment, cfg_default,
                             cfg_row1d)

OUT = os.path.dirname(os.path.abspath(__file__))


def crc(a: np.ndarray) -> int:
    return zlib.crc32(np.ascontiguousarray(a).view(np.uint8).reshape(-1).tobytes())


def sample_rows(W, n=8):
    rows = np.linspace(0, W.shape[0] - 1, n).astype(np.int64)
    return rows, W[rows].copy()


def main():
    ref = Reference()
    tiny = cfg_default(tile_rows=32, tile_cols=32, n_atoms=32, k=4, ksvd_iters=4)

    # --- test_hsdr_roundtrip.cpp:184-265: fused vs dense, 256x512, K=128, k=6, batch 4
    w, x = ref.mt19937_normal(0xFAFA, [(256 * 512, 0, 0.05), (512 * 4, 0, 1.0)])
    cfg = cfg_row1d(512, 128, 6, ksvd_iters=6)
    pay = ref.compress(Segment("fused.matmul.test", w.reshape(256, 512), (256, 512), SEG_ATTENTION), cfg, cfg)
    W = ref.decompress(pay, 256, 512)
    rows, Wrows = sample_rows(W)
    np.savez_compressed(os.path.join(OUT, "fused_rowtile.npz"), payload=np.frombuffer(pay, np.uint8),
                        x=x.reshape(512, 4), y_fused=ref.matmul(pay, x, 4, 256), w_crc=crc(W),
                        w_rows_idx=rows, w_rows=Wrows)

    # --- test_hsdr_roundtrip.cpp:124-176: 2-D tiles; 290x257 has edge strips
    cases = {}
    for label, R, C, seed, st in (("attn_small", 256, 256, 0xC0FFEE, SEG_ATTENTION),
                                  ("mlp_small", 192, 320, 0xBEEF, SEG_FEED_FORWARD),
                                  ("edges", 290, 257, 0xEDF0001, SEG_ATTENTION)):
        (w,) = ref.mt19937_normal(seed, [(R * C, 0, 0.05)])
        pay = ref.compress(Segment(label, w.reshape(R, C), (R, C), st), tiny, tiny)
        W = ref.decompress(pay, R, C)
        rows, Wrows = sample_rows(W)
        cases[label + "_payload"] = np.frombuffer(pay, np.uint8)
        cases[label + "_w_crc"] = crc(W)
        cases[label + "_w_rows_idx"] = rows
        cases[label + "_w_rows"] = Wrows
        cases[label + "_w_colsum"] = W.astype(np.float64).sum(axis=0)
    np.savez_compressed(os.path.join(OUT, "tiles_2d.npz"), **cases)

    # --- test_hsdr_archive_e2e.cpp: 128x512, K=64, k=6, iters 6, batch 4, through AICompressor
    w, x = ref.mt19937_normal(0xC0FFEE, [(128 * 512, 0, 0.05), (512 * 4, 0, 1.0)])
    cfg = cfg_row1d(512, 64, 6, ksvd_iters=6)
    path = os.path.join(OUT, "archive_e2e.sdr")
    ref.sdr_write([Segment("test.layer.weight", w.reshape(128, 512), (128, 512), SEG_WEIGHTS_FP32)], path, cfg, cfg)
    W = ref.sdr_decompress(path, "test.layer.weight", 128 * 512).reshape(128, 512)
    np.savez_compressed(os.path.join(OUT, "archive_e2e.npz"), x=x.reshape(512, 4),
                        y_fused=ref.sdr_matmul(path, "test.layer.weight", x, 4, 128), w_crc=crc(W))

    # --- test_inference_matmul_routing.cpp: HSDR segment (seed 0xA1, 256x512, K=64, k=6) plus a
    # segment that stays stored raw (strategy 0), plus a 1-D norm vector; x seed 0xDEAD.
    (w1,) = ref.mt19937_normal(0xA1, [(256 * 512, 0, 0.05)])
    (w2,) = ref.mt19937_normal(0xB2, [(96 * 256, 0, 0.05)])
    path = os.path.join(OUT, "routing.sdr")
    ref.sdr_write([Segment("layer.hsdr.weight", w1.reshape(256, 512), (256, 512), SEG_WEIGHTS_FP32),
                   Segment("layer.raw.weight", w2.reshape(96, 256), (96, 256), SEG_LAYER_NORM),
                   Segment("layer.norm.weight", np.ones(256, np.float32), (256,), SEG_LAYER_NORM)],
                  path, cfg, cfg)
    (x1,) = ref.mt19937_normal(0xDEAD, [(512 * 2, 0, 1.0)])
    (x2,) = ref.mt19937_normal(0xDEAD, [(256 * 2, 0, 1.0)])
    y_raw = (w2.reshape(96, 256).astype(np.float64) @ x2.reshape(256, 2).astype(np.float64)).astype(np.float32)
    np.savez_compressed(os.path.join(OUT, "routing.npz"), x_hsdr=x1.reshape(512, 2),
                        y_hsdr=ref.sdr_matmul(path, "layer.hsdr.weight", x1, 2, 256),
                        x_raw=x2.reshape(256, 2), y_raw=y_raw)

    # --- test_hsda_reader.cpp: 5 attention + 3 mlp segments, 96x256, two dictionaries
    segs = []
    for i in range(5):
        (w,) = ref.mt19937_normal(0xAA00 + i, [(96 * 256, 0, 0.05)])
        segs.append(Segment(f"model.layers.{i}.attn.q_proj.weight", w.reshape(96, 256), (96, 256),
                            SEG_ATTENTION, layer_index=i))
    for i in range(3):
        (w,) = ref.mt19937_normal(0xBB00 + i, [(96 * 256, 0, 0.05)])
        segs.append(Segment(f"model.layers.{i}.mlp.down_proj.weight", w.reshape(96, 256), (96, 256),
                            SEG_FEED_FORWARD, layer_index=i))
    attn = cfg_row1d(256, 64, 4, ksvd_iters=4)
    mlp = cfg_row1d(256, 80, 6, ksvd_iters=4)
    path = os.path.join(OUT, "reader.hsda")
    n_dicts = ref.hsda_write(segs, path, attn, mlp)
    (x,) = ref.mt19937_normal(0xDEAD, [(256 * 2, 0, 1.0)])
    out = {"x": x.reshape(256, 2), "n_dicts": n_dicts, "names": np.array([s.name for s in segs])}
    for i, s in enumerate(segs):
        out[f"y_{i}"] = ref.hsda_matmul(path, s.name, x, 2, 96)
        out[f"w_crc_{i}"] = crc(ref.hsda_decompress(path, s.name, 96, 256))
    np.savez_compressed(os.path.join(OUT, "reader_hsda.npz"), **out)

    # --- a 2-D shared dictionary (.hsda with 32x32 tiles), the container config 5 needs
    segs = []
    for i, (R, C) in enumerate(((256, 128), (128, 256))):
        (w,) = ref.mt19937_normal(0xCC00 + i, [(R * C, 0, 0.05)])
        segs.append(Segment(f"blk.{i}.ffn.weight", w.reshape(R, C), (R, C), SEG_FEED_FORWARD, layer_index=i))
    path = os.path.join(OUT, "shared_2d.hsda")
    n_dicts = ref.hsda_write(segs, path, tiny, tiny)
    out = {"n_dicts": n_dicts, "names": np.array([s.name for s in segs]),
           "shapes": np.array([s.dims for s in segs])}
    for i, s in enumerate(segs):
        out[f"w_crc_{i}"] = crc(ref.hsda_decompress(path, s.name, *s.dims))
    np.savez_compressed(os.path.join(OUT, "shared_2d.npz"), **out)

    # --- dequantizeToFP32 on random blocks of every supported source dtype
    rng = np.random.default_rng(1234)
    out = {}
    for fmt, unit, per, nblk in (("q4_k", 144, 256, 24), ("q5_k", 176, 256, 24), ("q6_k", 210, 256, 24),
                                 ("q4_0", 18, 32, 64), ("q8_0", 34, 32, 64)):
        raw = rng.integers(0, 256, size=unit * nblk, dtype=np.uint8)
        # keep the fp16 super-scales finite and modest: overwrite them with small normal halves
        blk = raw.reshape(nblk, unit)
        halves = rng.normal(0, 0.05, size=(nblk, 2)).astype(np.float16).view(np.uint8).reshape(nblk, 4)
        if fmt in ("q4_k", "q5_k"):
            blk[:, 0:4] = halves
        elif fmt == "q6_k":
            blk[:, 208:210] = halves[:, 0:2]
        else:
            blk[:, 0:2] = halves[:, 0:2]
        n = per * nblk
        seg = Segment("q", raw, (n // per, per), SEG_WEIGHTS_INT8, data_format=fmt)
        out[fmt + "_in"] = raw
        out[fmt + "_out"] = ref.dequantize(seg, n).copy()
    h = rng.normal(0, 1, 512).astype(np.float16)
    h[:8] = np.array([0, -0.0, 6e-8, -6e-5, 65504, 1e-7, 5.96e-8, 1.0], np.float16)  # zeros, subnormals, max
    out["f16_in"] = h.view(np.uint8)
    out["f16_out"] = ref.dequantize(Segment("h", h.view(np.uint8), (2, 256), 2, data_format="f16"), 512).copy()
    b = (rng.normal(0, 1, 512).astype(np.float32).view(np.uint32) >> 16).astype(np.uint16)
    out["bf16_in"] = b.view(np.uint8)
    out["bf16_out"] = ref.dequantize(Segment("b", b.view(np.uint8), (2, 256), 2, data_format="bf16"), 512).copy()
    i8 = rng.integers(-128, 128, 512, dtype=np.int8)
    out["i8_in"] = i8.view(np.uint8)
    out["i8_scale"], out["i8_zp"] = np.float32(0.0123), np.float32(3.0)
    out["i8_out"] = ref.dequantize(Segment("i", i8.view(np.uint8), (2, 256), SEG_WEIGHTS_INT8, data_format="i8",
                                           scale=0.0123, zero_point=3.0), 512).copy()
    np.savez_compressed(os.path.join(OUT, "dequant.npz"), **out)
    encoder_coding(ref)
    attention_cases(ref)
    raw_tensor_cases()
    grouped_encoder(ref)
    print("golden fixtures written to", OUT)
    for f in sorted(os.listdir(OUT)):
        print(f"  {f:24s} {os.path.getsize(os.path.join(OUT, f)):>9d} B")


def encoder_coding(ref):
    """The encoder's final coding pass: weights in, the payload the reference encoder made of
    them out. Whatever the number of dictionary-update iterations, the codes of a payload are
    hierarchicalBinaryCode (HierarchicalSDRStrategy.cpp:219-262) of the weights against the
    payload's own dictionary (encode_all is the last thing fitHierarchicalKSVD runs, :552-571)."""
    out = {}
    for label, R, C, seed, cfg in (
            ("row_fast", 64, 128, 0xE0C0, cfg_row1d(128, 32, 4, ksvd_iters=0)),
            ("row_fit", 64, 128, 0xE0C1, cfg_row1d(128, 32, 4, ksvd_iters=3)),
            ("tiles_2d", 128, 192, 0xE0C2, cfg_default(tile_rows=16, tile_cols=16, n_atoms=32, k=4, ksvd_iters=2)),
            ("edges_fast", 100, 150, 0xE0C3, cfg_default(tile_rows=16, tile_cols=16, n_atoms=32, k=4, ksvd_iters=0))):
        (w,) = ref.mt19937_normal(seed, [(R * C, 0, 0.05)])
        pay = ref.compress(Segment("enc." + label, w.reshape(R, C), (R, C), SEG_ATTENTION), cfg, cfg)
        out[label + "_w"] = w.reshape(R, C).copy()
        out[label + "_payload"] = np.frombuffer(pay, np.uint8)
    np.savez_compressed(os.path.join(OUT, "encoder_coding.npz"), **out)


def grouped_encoder(ref):
    """compressGroupedSegments (HierarchicalSDRStrategy.cpp:2211-2500): weights in, the .hsda bytes the
    reference made of them out - three row-tile tensors behind one dictionary after two update
    rounds, and two tensors of 16 x 16 tiles behind another in fast mode. The fit runs on all pooled
    tiles (max_tiles_for_fit = 0)."""
    import tempfile
    out = {}
    cases = (("rows", [(48, 128)] * 3, cfg_row1d(128, 16, 3, ksvd_iters=2, max_tiles_for_fit=0)),
             ("tiles", [(64, 96), (32, 64)], cfg_default(tile_rows=16, tile_cols=16, n_atoms=16, k=3, ksvd_iters=0,
                                                          max_tiles_for_fit=0)))
    for label, shapes, cfg in cases:
        segs = []
        for i, (R, C) in enumerate(shapes):
            (w,) = ref.mt19937_normal(0xE100 + 16 * len(out) + i, [(R * C, 0, 0.05)])
            segs.append(Segment(f"blk.{i}.attn_q.weight", w.reshape(R, C), (R, C), SEG_ATTENTION, layer_index=i))
            out[f"{label}_w{i}"] = w.reshape(R, C)
        with tempfile.TemporaryDirectory() as tmp:
            path = os.path.join(tmp, "g.hsda")
            assert ref.hsda_write(segs, path, cfg, cfg) == 1
            out[label + "_hsda"] = np.frombuffer(open(path, "rb").read(), np.uint8)
        out[label + "_n"] = len(shapes)
    np.savez_compressed(os.path.join(OUT, "grouped_encoder.npz"), **out)


def attention_cases(ref):
    """Causal attention of the decoder driver by the reference's own kernel
    (kernels/attention_kernels.cpp multi_head_attention + kernels/simd_kernels.cpp softmax),
    kv heads repeated as api/cortex_sdk.cpp:1453-1478 does: one head per kv head, and grouped
    query heads in the 0.5B-shaped ratio (14 : 2, head size 64)."""
    rng = np.random.default_rng(77)
    out = {}
    for label, seq, qh, kvh, hd in (("mha", 9, 4, 4, 16), ("gqa", 21, 14, 2, 64)):
        q, k, v = (rng.normal(0, 1, (seq, h, hd)).astype(np.float32) for h in (qh, kvh, kvh))
        out.update({label + "_q": q, label + "_k": k, label + "_v": v, label + "_out": ref.attention(q, k, v)})
    np.savez_compressed(os.path.join(OUT, "attention.npz"), **out)


def raw_tensor_cases(_ref=None):
    """Stored-raw tensors in GGUF block formats as the reference's INFERENCE side widens them
    (SDRModelLoader::loadLayerByName -> decodeSupportedGGUFQuantized,
    SparseInferenceEngine.cpp:276-469): random blocks with modest fp16 super-scales, written into
    a .sdr as strategy-0 segments and read back through the reference's loader."""
    import tempfile
    from oracle.bindings import ReferenceEngine
    from tests import synth
    eng = ReferenceEngine()
    rng = np.random.default_rng(4321)
    out = {}
    with tempfile.TemporaryDirectory() as d:
        for fmt, unit, per, nblk in (("q4_k", 144, 256, 16), ("q5_k", 176, 256, 16), ("q6_k", 210, 256, 16),
                                     ("q4_0", 18, 32, 64), ("q8_0", 34, 32, 64)):
            raw = rng.integers(0, 256, size=unit * nblk, dtype=np.uint8)
            blk = raw.reshape(nblk, unit)
            halves = rng.normal(0, 0.05, size=(nblk, 2)).astype(np.float16).view(np.uint8).reshape(nblk, 4)
            if fmt == "q6_k":
                blk[:, 208:210] = halves[:, 0:2]
            else:
                blk[:, 0:4 if fmt in ("q4_k", "q5_k") else 2] = halves[:, 0:4 if fmt in ("q4_k", "q5_k") else 2]
            n = per * nblk
            path = os.path.join(d, fmt + ".sdr")
            synth.write_sdr(path, [synth.raw_segment("blk.0.ffn_down.weight", raw, synth.SEG_FEED_FORWARD,
                                                     data_format=fmt, dims=(n // 256, 256))])
            out[fmt + "_in"] = raw
            out[fmt + "_out"] = eng.layer_weights(path, "blk.0.ffn_down.weight")
            assert out[fmt + "_out"].size == n
    np.savez_compressed(os.path.join(OUT, "raw_tensors.npz"), **out)


if __name__ == "__main__":
    only = {"encoder_coding": encoder_coding, "attention": attention_cases, "raw_tensors": raw_tensor_cases,
            "grouped_encoder": grouped_encoder}
    if len(sys.argv) == 2 and sys.argv[1] in only:      # only this fixture, the others untouched
        only[sys.argv[1]](Reference() if sys.argv[1] != "raw_tensors" else None)
    else:
        main()
