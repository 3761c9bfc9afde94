"""Seeded synthetic HSDR payloads and .sdr archives, byte-compatible with the reference
writer (strategies/HierarchicalSDRStrategy.cpp:1198-1235; core/AICompressor.cpp:233-312).

The reference encoder needs seconds to minutes per tensor; benchmarks, the smoke check and
large decoder-shaped archives use these stand-ins instead: a Gaussian dictionary and
uniformly random (atom, sign) codes, scaled so the reconstructed weight has the standard
deviation asked for. Decoding cost does not depend on which atoms the codes name.
"""
from __future__ import annotations

import struct

import numpy as np

SEG_WEIGHTS_FP32, SEG_CONFIG, SEG_ATTENTION, SEG_FEED_FORWARD, SEG_EMBEDDING, SEG_LAYER_NORM = 1, 10, 11, 12, 13, 14


def hsdr_payload(rows: int, cols: int, *, tile_rows: int = 1, tile_cols: int | None = None,
                 n_atoms: int = 512, n_stages: int = 3, k: int = 8, decay: float = 0.5,
                 seed: int = 0, weight_std: float = 0.02) -> bytes:
    tile_cols = cols if tile_cols is None else tile_cols
    rng = np.random.default_rng(seed)
    rf, cf = rows // tile_rows * tile_rows, cols // tile_cols * tile_cols
    n_tiles = (rf // tile_rows) * (cf // tile_cols)
    scales = np.array([decay ** l for l in range(n_stages)], np.float32)
    atom_std = weight_std / np.sqrt(k * float((scales.astype(np.float64) ** 2).sum()))
    atoms = rng.standard_normal((n_atoms, tile_rows * tile_cols), dtype=np.float32) * np.float32(atom_std)
    n_codes = n_tiles * n_stages * k
    codes = (rng.integers(0, n_atoms, n_codes, dtype=np.uint16)
             | (rng.integers(0, 2, n_codes, dtype=np.uint16) << 15)).astype(np.uint16)
    n_edge = rf * (cols - cf) + (rows - rf) * cols
    edges = rng.standard_normal(n_edge, dtype=np.float32) * np.float32(weight_std)
    hdr = struct.pack("<4sIIIIHHHBBfI", b"HSDR", 2, rows, cols, n_tiles, tile_rows, tile_cols,
                      n_atoms, n_stages, k, decay, 4 * n_edge)
    return b"".join((hdr, scales.tobytes(), atoms.tobytes(), codes.tobytes(), edges.tobytes()))


def shared_dictionary(tile_rows: int, tile_cols: int, *, n_atoms: int = 512, n_stages: int = 3, k: int = 8,
                      decay: float = 0.5, seed: int = 0, weight_std: float = 0.02):
    """(atoms fp32 [n_atoms][tile_rows*tile_cols], stage scales) of a dictionary several tensors share
    (SharedDictionary, strategies/HierarchicalSDRStrategy.hpp:194-198)."""
    rng = np.random.default_rng(seed)
    scales = np.array([decay ** l for l in range(n_stages)], np.float32)
    atom_std = weight_std / np.sqrt(k * float((scales.astype(np.float64) ** 2).sum()))
    atoms = rng.standard_normal((n_atoms, tile_rows * tile_cols), dtype=np.float32) * np.float32(atom_std)
    return atoms, scales


def hsdc_payload(rows: int, cols: int, *, tile_rows: int, tile_cols: int, n_atoms: int = 512, n_stages: int = 3,
                 k: int = 8, decay: float = 0.5, seed: int = 0) -> bytes:
    """A codes-only "HSDC" stream (HSDRCodesHeader, strategies/HierarchicalSDRStrategy.cpp:675-692) with
    uniformly random (atom, sign) codes; the shape must divide by the tile."""
    assert rows % tile_rows == 0 and cols % tile_cols == 0
    rng = np.random.default_rng(seed)
    n_tiles = (rows // tile_rows) * (cols // tile_cols)
    n_codes = n_tiles * n_stages * k
    codes = (rng.integers(0, n_atoms, n_codes, dtype=np.uint16)
             | (rng.integers(0, 2, n_codes, dtype=np.uint16) << 15)).astype(np.uint16)
    hdr = struct.pack("<4sIIIIHHHBBf", b"HSDC", 1, rows, cols, n_tiles, tile_rows, tile_cols, n_atoms, n_stages, k, decay)
    return hdr + codes.tobytes()


def _s(x: str) -> bytes:
    b = x.encode()
    return struct.pack("<I", len(b)) + b


def write_sdr(path: str, segments) -> None:
    """segments: iterable of dicts {name, payload(bytes), strategy_id, original_type, dims,
    original_size, data_format='f32', layer_type='LINEAR', layer_index=0}. Layout of
    AICompressor::compressModel (archive version 2)."""
    segments = list(segments)
    with open(path, "wb") as f:
        f.write(b"CORTEXSR" + struct.pack("<IQQ", 2, len(segments), 0))
        offsets = []
        for s in segments:
            offsets.append(f.tell())
            f.write(s["payload"])
        index_offset = f.tell()
        for s, off in zip(segments, offsets):
            dims = tuple(s["dims"])
            f.write(_s(s["name"]) + _s(s.get("data_format", "f32")) + _s(s.get("layer_type", "LINEAR")))
            f.write(struct.pack("<BBQQQ", s["original_type"], s["strategy_id"], s["original_size"],
                                len(s["payload"]), off))
            f.write(_s(s["name"]) + struct.pack("<I", s.get("layer_index", 0)))
            f.write(struct.pack("<BB", 1, len(dims)) + struct.pack(f"<{len(dims)}I", *dims))
            f.write(struct.pack("<fBBB", 0.0, 0, 0, 0))
            if len(dims) == 2:
                f.write(struct.pack("<BBII", 1, 2, 1, dims[1]) + struct.pack("<BBII", 1, 2, 1, dims[0]))
            else:
                f.write(struct.pack("<BB", 0, 0))
        f.seek(8 + 4 + 8)
        f.write(struct.pack("<Q", index_offset))


def hsdr_segment(name: str, rows: int, cols: int, seg_type: int = SEG_WEIGHTS_FP32, layer_index: int = 0,
                 **kw) -> dict:
    return dict(name=name, payload=hsdr_payload(rows, cols, **kw), strategy_id=5, original_type=seg_type,
                dims=(rows, cols), original_size=rows * cols * 4, layer_index=layer_index)


def raw_segment(name: str, array: np.ndarray, seg_type: int = SEG_LAYER_NORM, layer_index: int = 0,
                data_format: str = "f32", dims=None) -> dict:
    """A stored-raw segment (strategy 0). With data_format other than "f32", `array` holds the
    packed bytes of that source dtype (f16, bf16, q8_0, q4_k, ...) and `dims` the logical shape."""
    if data_format == "f32":
        a = np.ascontiguousarray(array, dtype=np.float32)
        dims = a.shape
    else:
        a = np.ascontiguousarray(array).view(np.uint8).reshape(-1)
    return dict(name=name, payload=a.tobytes(), strategy_id=0, original_type=seg_type, dims=tuple(dims),
                original_size=a.nbytes, layer_index=layer_index, data_format=data_format,
                layer_type="" if len(dims) < 2 else "LINEAR")


def pack_source_dtype(w: np.ndarray, fmt: str) -> np.ndarray:
    """fp32 values -> packed bytes of a source dtype the reference widens at load: "f16", "bf16"
    (round to nearest even), "q8_0" (blocks of 32: fp16 scale d = max|x| / 127, then 32 int8
    quants), or the k-quants "q4_k", "q5_k", "q6_k" in the block layouts its inference side reads."""
    w = np.ascontiguousarray(w, np.float32).reshape(-1)
    if fmt == "f16":
        return w.astype(np.float16).view(np.uint8)
    if fmt == "bf16":
        u = w.view(np.uint32).astype(np.uint64)
        u = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
        return u.astype(np.uint16).view(np.uint8)
    if fmt == "q8_0":
        b = w.reshape(-1, 32)
        d = (np.abs(b).max(1) / 127.0).astype(np.float16)
        q = np.where(d[:, None] > 0, np.rint(b / np.maximum(d.astype(np.float32), 1e-30)[:, None]), 0)
        out = np.empty((b.shape[0], 34), np.uint8)
        out[:, 0:2] = d.view(np.uint8).reshape(-1, 2)
        out[:, 2:] = np.clip(q, -127, 127).astype(np.int8).view(np.uint8)
        return out.reshape(-1)
    if fmt == "q4_k":
        return _pack_q4_k(w)
    if fmt == "q6_k":
        return _pack_q6_k(w)
    if fmt == "q5_k":
        # the reference's inference side reads q5_k blocks through a generic 5-bit fall-back
        # (fp16 scale at byte 0, 256 five-bit fields from byte 16, value (q - 16) * d): pack for that
        b = w.reshape(-1, 256)
        d = (np.abs(b).max(1) / 15.0).astype(np.float16)
        q = np.clip(np.rint(b / np.maximum(d.astype(np.float32), 1e-30)[:, None]) + 16, 0, 31).astype(np.uint64)
        out = np.zeros((b.shape[0], 176), np.uint8)
        out[:, 0:2] = d.view(np.uint8).reshape(-1, 2)
        bits = ((q[:, :, None] >> np.arange(5, dtype=np.uint64)) & 1).astype(np.uint8).reshape(b.shape[0], 1280)
        out[:, 16:] = np.packbits(bits, axis=1, bitorder="little")
        return out.reshape(-1)
    raise ValueError(f"no packer for source dtype {fmt!r}")


def _pack_q4_k(w: np.ndarray) -> np.ndarray:
    """A plain min/max quantiser writing ggml's q4_K block layout (144 bytes per 256 values:
    fp16 d, fp16 dmin, 12 bytes of 6-bit scales and mins, 128 bytes of nibbles; 64-value groups
    hold 32 low nibbles then 32 high nibbles). Harness code: it only has to produce valid blocks."""
    b = w.reshape(-1, 8, 32).astype(np.float32)
    lo = np.minimum(b.min(2), 0.0)
    scale = (b.max(2) - lo) / 15.0
    d = (scale.max(1) / 63.0).astype(np.float16)
    dmin = ((-lo).max(1) / 63.0).astype(np.float16)
    df, dmf = np.maximum(d.astype(np.float32), 1e-30), np.maximum(dmin.astype(np.float32), 1e-30)
    sc = np.clip(np.rint(scale / df[:, None]), 0, 63).astype(np.uint8)
    mn = np.clip(np.rint(-lo / dmf[:, None]), 0, 63).astype(np.uint8)
    eff = np.maximum(df[:, None] * sc, 1e-30)
    q = np.clip(np.rint((b + (dmf[:, None] * mn)[:, :, None]) / eff[:, :, None]), 0, 15).astype(np.uint8)
    out = np.zeros((b.shape[0], 144), np.uint8)
    out[:, 0:2] = d.view(np.uint8).reshape(-1, 2)
    out[:, 2:4] = dmin.view(np.uint8).reshape(-1, 2)
    for j in range(4):
        out[:, 4 + j] = (sc[:, j] & 63) | ((sc[:, j + 4] >> 4) << 6)
        out[:, 8 + j] = (mn[:, j] & 63) | ((mn[:, j + 4] >> 4) << 6)
        out[:, 12 + j] = (sc[:, j + 4] & 15) | ((mn[:, j + 4] & 15) << 4)
    for g in range(4):
        out[:, 16 + 32 * g:48 + 32 * g] = q[:, 2 * g] | (q[:, 2 * g + 1] << 4)
    return out.reshape(-1)


def _pack_q6_k(w: np.ndarray) -> np.ndarray:
    """ggml's q6_K block layout (210 bytes per 256 values: 128 bytes of low nibbles, 64 bytes of
    high bit pairs, 16 int8 scales, fp16 d), one scale per run of 32 written to both scale slots
    of the run. Harness code."""
    b = w.reshape(-1, 2, 4, 32).astype(np.float32)           # block, half, run, element
    s = np.abs(b).max(3) / 31.0
    d = (s.max((1, 2)) / 127.0).astype(np.float16)
    df = np.maximum(d.astype(np.float32), 1e-30)
    sc = np.clip(np.rint(s / df[:, None, None]), 1, 127).astype(np.int8)
    q = np.clip(np.rint(b / (df[:, None, None] * sc)[..., None]) + 32, 0, 63).astype(np.uint8)
    out = np.zeros((b.shape[0], 210), np.uint8)
    for h in range(2):
        ql = out[:, h * 64:h * 64 + 64]
        ql[:, 0:32] = (q[:, h, 0] & 15) | ((q[:, h, 2] & 15) << 4)
        ql[:, 32:64] = (q[:, h, 1] & 15) | ((q[:, h, 3] & 15) << 4)
        out[:, 128 + h * 32:160 + h * 32] = ((q[:, h, 0] >> 4) | ((q[:, h, 1] >> 4) << 2) | ((q[:, h, 2] >> 4) << 4)
                                             | ((q[:, h, 3] >> 4) << 6))
        for r in range(4):
            out[:, 192 + h * 8 + 2 * r] = sc[:, h, r].view(np.uint8)
            out[:, 192 + h * 8 + 2 * r + 1] = sc[:, h, r].view(np.uint8)
    out[:, 208:210] = d.view(np.uint8).reshape(-1, 2)
    return out.reshape(-1)


def dictionary_record(atoms: np.ndarray, scales: np.ndarray, *, tile_rows: int, tile_cols: int, k: int,
                      decay: float = 0.5) -> bytes:
    """One dictionary as a .hsda holds it (SharedDictArchive::writeToStream,
    strategies/HierarchicalSDRStrategy.cpp:1972-2002): the 20-byte raw HierarchicalSDRConfig, then
    counted stage scales and atoms. Also the payload of a shared-dictionary resource segment."""
    n_atoms, n_stages = atoms.shape[0], len(scales)
    cfg = struct.pack("<HHHBBBxxxfI", tile_rows, tile_cols, n_atoms, n_stages, k, 0, decay, 0)
    assert len(cfg) == 20
    return (cfg + struct.pack("<I", n_stages) + np.asarray(scales, np.float32).tobytes()
            + struct.pack("<I", atoms.size) + np.ascontiguousarray(atoms, np.float32).tobytes())


def read_dictionary_record(b: bytes):
    """Inverse of dictionary_record: (tile_rows, tile_cols, n_atoms, n_stages, k, atoms, scales)."""
    b = bytes(b)
    tile_rows, tile_cols, n_atoms, n_stages, k = struct.unpack_from("<HHHBB", b, 0)
    (n_scales,) = struct.unpack_from("<I", b, 20)
    scales = np.frombuffer(b, np.float32, n_scales, 24).copy()
    (n_floats,) = struct.unpack_from("<I", b, 24 + 4 * n_scales)
    atoms = np.frombuffer(b, np.float32, n_floats, 28 + 4 * n_scales).reshape(n_atoms, tile_rows * tile_cols).copy()
    return tile_rows, tile_cols, n_atoms, n_stages, k, atoms, scales


SHARED_DICT_FORMAT = "hsdr_dict"


def decoder_archive(path: str, *, n_layers, hidden, q_heads, kv_heads, head_dim, inter, vocab, seed=100,
                    geometry="row", n_atoms=512, k=8, kv_atoms=None, raw=None, shared_dicts=False) -> None:
    """A decoder-shaped .sdr with the reference's GGUF-style tensor names
    (api/cortex_sdk.cpp:456-524): every linear an HSDR segment, norm vectors stored raw.
    `raw` maps tensor names to a source dtype ("f32", "f16", "bf16", "q8_0"): those linears are
    stored uncompressed (strategy 0) in that dtype instead, as a converter leaves protected or
    unsuitable tensors. `shared_dicts`: the seven block roles (attn_q ... ffn_down) each share ONE
    dictionary over all blocks - a resource segment "hsdr.shared_dict/<role>" (stored raw,
    data_format "hsdr_dict", one .hsda dictionary record) and per block a codes-only "HSDC"
    payload whose data_format names it ("hsdc@hsdr.shared_dict/<role>")."""
    segs, sd = [], seed
    kw = dict(n_atoms=n_atoms, k=k)
    raw = raw or {}
    role_dicts = {}

    def lin(name, r, c, t, li, atoms=None):
        nonlocal sd
        sd += 1
        role = name.split(".")[2] if name.startswith("blk.") else None
        if shared_dicts and role and name not in raw and geometry == "row":
            K = atoms or n_atoms
            dname = f"hsdr.shared_dict/{role}"
            if role not in role_dicts:
                d_atoms, d_scales = shared_dictionary(1, c, n_atoms=K, k=k, seed=seed + 7919 * (len(role_dicts) + 1))
                role_dicts[role] = dname
                segs.append(dict(name=dname, payload=dictionary_record(d_atoms, d_scales, tile_rows=1, tile_cols=c, k=k),
                                 strategy_id=0, original_type=SEG_CONFIG, dims=(K, c), original_size=d_atoms.nbytes,
                                 data_format=SHARED_DICT_FORMAT, layer_type="", layer_index=0))
            pay = hsdc_payload(r, c, tile_rows=1, tile_cols=c, n_atoms=K, k=k, seed=sd)
            segs.append(dict(name=name, payload=pay, strategy_id=5, original_type=t, dims=(r, c), original_size=r * c * 4,
                             data_format="hsdc@" + dname, layer_index=li))
            return
        if name in raw:
            w = np.random.default_rng(sd).normal(0, 0.02, (r, c)).astype(np.float32)
            fmt = raw[name]
            segs.append(raw_segment(name, w if fmt == "f32" else pack_source_dtype(w, fmt), t, li, data_format=fmt,
                                    dims=(r, c)))
            return
        a = dict(kw, n_atoms=atoms or n_atoms)
        if geometry != "row":
            a.update(tile_rows=geometry[0], tile_cols=geometry[1])
        segs.append(hsdr_segment(name, r, c, t, li, seed=sd, **a))

    lin("token_embd.weight", vocab, hidden, SEG_EMBEDDING, 0)
    for i in range(n_layers):
        p = f"blk.{i}."
        segs.append(raw_segment(p + "attn_norm.weight", np.ones(hidden, np.float32), layer_index=i))
        lin(p + "attn_q.weight", q_heads * head_dim, hidden, SEG_ATTENTION, i)
        lin(p + "attn_k.weight", kv_heads * head_dim, hidden, SEG_ATTENTION, i, kv_atoms)
        lin(p + "attn_v.weight", kv_heads * head_dim, hidden, SEG_ATTENTION, i, kv_atoms)
        lin(p + "attn_output.weight", hidden, q_heads * head_dim, SEG_ATTENTION, i)
        segs.append(raw_segment(p + "ffn_norm.weight", np.ones(hidden, np.float32), layer_index=i))
        lin(p + "ffn_gate.weight", inter, hidden, SEG_FEED_FORWARD, i)
        lin(p + "ffn_up.weight", inter, hidden, SEG_FEED_FORWARD, i)
        lin(p + "ffn_down.weight", hidden, inter, SEG_FEED_FORWARD, i)
    segs.append(raw_segment("output_norm.weight", np.ones(hidden, np.float32)))
    lin("output.weight", vocab, hidden, SEG_EMBEDDING, 0)
    write_sdr(path, segs)
