"""ctypes bindings for the two CPU checkers. TEST INFRASTRUCTURE ONLY.

* ``Oracle``  — liboracle_hsdr.so, this repository's plain-C restatement.
* ``Reference`` — _ref/libcortexsdr_ref.so, the unmodified reference sources behind
  ref_shim.cpp (present only where it was built; ``Reference.available()``).

Only tests, the smoke check and the bench's CPU-baseline leg import this module.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from dataclasses import dataclass

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(_HERE, "liboracle_hsdr.so")
REF_SO = os.path.join(_HERE, "_ref", "libcortexsdr_ref.so")
REF_ENGINE_SO = os.path.join(_HERE, "_ref", "libcortexsdr_ref_engine.so")

# SegmentType values, core/ModelSegment.hpp:36-55 of the reference.
SEG_WEIGHTS_FP32 = 1
SEG_WEIGHTS_FP16 = 2
SEG_WEIGHTS_INT8 = 3
SEG_ATTENTION = 11
SEG_FEED_FORWARD = 12
SEG_EMBEDDING = 13
SEG_LAYER_NORM = 14


def reference_tree():
    """Where the reference sources lie: $CORTEXSDR_REF, else a checkout named ``reference``
    beside this repository. None when neither holds a ``src`` folder."""
    cands = [os.environ.get("CORTEXSDR_REF"),
             os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")]
    for c in cands:
        if c and os.path.isdir(os.path.join(c, "src")):
            return os.path.abspath(c)
    return None


def build(ref: bool = True) -> None:
    """Compile the C oracle and, when the reference tree is present, oracle/_ref."""
    subprocess.check_call(["make", "-s", "-C", _HERE, "oracle"])
    tree = reference_tree() if ref else None
    if tree:
        subprocess.check_call(["make", "-s", "-C", _HERE, "ref", "ref_engine", "REF=" + tree])


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _ptr(a, t=C.c_float):
    return a.ctypes.data_as(C.POINTER(t))


class _View(C.Structure):
    _fields_ = [("kind", C.c_int), ("rows", C.c_uint32), ("cols", C.c_uint32),
                ("n_tiles", C.c_uint32), ("tile_rows", C.c_uint16), ("tile_cols", C.c_uint16),
                ("n_atoms", C.c_uint16), ("n_stages", C.c_uint8), ("k", C.c_uint8),
                ("decay", C.c_float), ("edge_bytes", C.c_uint32), ("off_scales", C.c_size_t),
                ("off_dict", C.c_size_t), ("off_codes", C.c_size_t), ("off_edges", C.c_size_t)]


class _DecoderCfg(C.Structure):
    _fields_ = [("n_layers", C.c_uint32), ("hidden", C.c_uint32), ("q_heads", C.c_uint32),
                ("kv_heads", C.c_uint32), ("head_dim", C.c_uint32), ("inter", C.c_uint32),
                ("vocab", C.c_uint32), ("eps", C.c_float), ("theta", C.c_float)]


class _BlockWeights(C.Structure):
    _fields_ = [(n, C.POINTER(C.c_float)) for n in
                ("attn_norm", "wq", "wk", "wv", "wo", "ffn_norm", "w_gate", "w_up", "w_down")]


@dataclass
class SharedDict:
    """External dictionary of an .hsda container (HierarchicalSDRStrategy.hpp:194-198)."""
    tile_rows: int
    tile_cols: int
    n_atoms: int
    n_stages: int
    k: int
    atoms: np.ndarray
    scales: np.ndarray


class Oracle:
    def __init__(self):
        if not os.path.exists(ORACLE_SO):
            build(ref=False)
        self.lib = C.CDLL(ORACLE_SO)
        L = self.lib
        L.orc_dequantize.restype = C.c_long
        L.orc_fp16_to_fp32.restype = C.c_float

    @staticmethod
    def _bytes(payload):
        a = np.frombuffer(payload, dtype=np.uint8) if not isinstance(payload, np.ndarray) else payload
        return np.ascontiguousarray(a)

    def parse(self, payload):
        p = self._bytes(payload)
        v = _View()
        rc = self.lib.orc_hsdr_parse(_ptr(p, C.c_uint8), C.c_size_t(p.size), C.byref(v))
        if rc:
            raise ValueError(f"orc_hsdr_parse rc={rc}")
        return v

    def unpack(self, packed):
        packed = np.ascontiguousarray(packed, dtype=np.uint16)
        idx = np.empty(packed.size, np.int32)
        sign = np.empty(packed.size, np.int8)
        self.lib.orc_unpack_codes(_ptr(packed, C.c_uint16), C.c_size_t(packed.size),
                                  _ptr(idx, C.c_int32), _ptr(sign, C.c_int8))
        return idx, sign

    def codes(self, payload):
        """(packed u16 codes, idx, sign, scales) of a payload."""
        p = self._bytes(payload)
        v = self.parse(p)
        n = v.n_tiles * v.n_stages * v.k
        packed = p[v.off_codes:v.off_codes + 2 * n].view(np.uint16).copy()
        idx, sign = self.unpack(packed)
        scales = (p[v.off_scales:v.off_scales + 4 * v.n_stages].view(np.float32).copy()
                  if v.kind == 0 else None)
        return packed, idx, sign, scales

    def matmul(self, payload, x, batch):
        """x (C, batch) -> y (R, batch); matmulRowMajor."""
        p = self._bytes(payload)
        v = self.parse(p)
        x = _f32(x)
        y = np.empty((v.rows, batch), np.float32)
        rc = self.lib.orc_hsdr_matmul(_ptr(p, C.c_uint8), C.c_size_t(p.size), _ptr(x),
                                      C.c_size_t(batch), _ptr(y))
        if rc:
            raise ValueError(f"orc_hsdr_matmul rc={rc}")
        return y

    def decompress(self, payload):
        p = self._bytes(payload)
        v = self.parse(p)
        out = np.empty((v.rows, v.cols), np.float32)
        rc = self.lib.orc_hsdr_decompress(_ptr(p, C.c_uint8), C.c_size_t(p.size), _ptr(out))
        if rc:
            raise ValueError(f"orc_hsdr_decompress rc={rc}")
        return out

    def code_tiles(self, tiles, atoms, gammas, k):
        """Coding pass of the encoder over tiles (n_tiles, T) against atoms (K, T): packed u16
        codes (n_tiles, S, k)."""
        tiles, atoms, gammas = _f32(tiles), _f32(atoms), _f32(gammas)
        n, T = tiles.shape
        K, S = atoms.shape[0], gammas.size
        assert atoms.shape[1] == T
        out = np.empty((n, S, k), np.uint16)
        self.lib.orc_hsdr_code_tiles(_ptr(tiles), C.c_size_t(n), C.c_size_t(T), _ptr(atoms), C.c_uint16(K),
                                     C.c_uint8(S), C.c_uint8(k), _ptr(gammas), _ptr(out, C.c_uint16))
        return out

    def encode_fast(self, W, tile_rows, tile_cols, n_atoms, n_stages=3, k=8, decay=0.5, ksvd_iters=0):
        """HSDR payload of W by the encoder; ksvd_iters = 0 is its fast mode (no dictionary-update
        iterations)."""
        W = _f32(W)
        R, Cc = W.shape
        cap = 36 + 4 * n_stages + 4 * n_atoms * tile_rows * tile_cols + 2 * R * Cc * n_stages * k + 4 * R * Cc
        out = np.empty(cap, np.uint8)
        self.lib.orc_hsdr_encode.restype = C.c_long
        n = self.lib.orc_hsdr_encode(_ptr(W), C.c_uint32(R), C.c_uint32(Cc), C.c_uint16(tile_rows),
                                     C.c_uint16(tile_cols), C.c_uint16(n_atoms), C.c_uint8(n_stages),
                                     C.c_uint8(k), C.c_float(decay), C.c_uint8(ksvd_iters),
                                     _ptr(out, C.c_uint8), C.c_size_t(cap))
        if n < 0:
            raise ValueError(f"orc_hsdr_encode rc={n}")
        return out[:n].copy()

    def encode_shared(self, Ws, tile_rows, tile_cols, n_atoms, n_stages=3, k=8, decay=0.5, ksvd_iters=0):
        """compressGroupedSegments (strategies/HierarchicalSDRStrategy.cpp:2211-2500) for tensors of
        one configuration with the fit on all tiles (max_tiles_for_fit = 0): the tensors' tiles
        pooled in order, ONE fit on the pool (fitSharedDictionary, :1446-1469), every tensor coded
        against the result (compressFP32WithExternalDictionary, :1691-1754). Shapes must divide by
        the tile. Returns (SharedDict, [codes-only "HSDC" payload per tensor])."""
        import struct
        T = tile_rows * tile_cols
        pools = []
        for W in Ws:
            W = _f32(W)
            R, Cc = W.shape
            if R % tile_rows or Cc % tile_cols:
                raise ValueError("shape not divisible by tile size")
            nr, nc = R // tile_rows, Cc // tile_cols                    # extractTiles order, :95-116
            pools.append(np.ascontiguousarray(W.reshape(nr, tile_rows, nc, tile_cols).transpose(0, 2, 1, 3).reshape(nr * nc, T)))
        pool = np.ascontiguousarray(np.concatenate(pools))
        D = np.empty((n_atoms, T), np.float32)
        gam = np.empty(n_stages, np.float32)
        codes = np.empty((pool.shape[0], n_stages, k), np.uint16)
        self.lib.orc_hsdr_fit_tiles.restype = C.c_int
        rc = self.lib.orc_hsdr_fit_tiles(_ptr(pool), C.c_uint32(pool.shape[0]), C.c_size_t(T), C.c_uint16(n_atoms),
                                         C.c_uint8(n_stages), C.c_uint8(k), C.c_float(decay), C.c_uint8(ksvd_iters),
                                         _ptr(D), _ptr(gam), _ptr(codes, C.c_uint16))
        if rc:
            raise ValueError(f"orc_hsdr_fit_tiles rc={rc}")
        d = SharedDict(tile_rows, tile_cols, n_atoms, n_stages, k, D, gam)
        payloads = []
        for W, tiles in zip(Ws, pools):
            R, Cc = W.shape
            packed = self.code_tiles(tiles, D, gam, k)
            hdr = struct.pack("<4sIIIIHHHBBf", b"HSDC", 1, R, Cc, tiles.shape[0], tile_rows, tile_cols, n_atoms, n_stages, k, decay)
            payloads.append(np.frombuffer(hdr + packed.tobytes(), np.uint8).copy())
        return d, payloads

    def _dict_args(self, d: SharedDict):
        return (_ptr(d.atoms), _ptr(d.scales), C.c_uint16(d.tile_rows), C.c_uint16(d.tile_cols),
                C.c_uint16(d.n_atoms), C.c_uint8(d.n_stages), C.c_uint8(d.k))

    def hsdc_matmul(self, codes, d: SharedDict, x, batch):
        p = self._bytes(codes)
        v = self.parse(p)
        x = _f32(x)
        y = np.empty((v.rows, batch), np.float32)
        rc = self.lib.orc_hsdc_matmul(_ptr(p, C.c_uint8), C.c_size_t(p.size), *self._dict_args(d),
                                      _ptr(x), C.c_size_t(batch), _ptr(y))
        if rc:
            raise ValueError(f"orc_hsdc_matmul rc={rc}")
        return y

    def hsdc_decompress(self, codes, d: SharedDict):
        p = self._bytes(codes)
        v = self.parse(p)
        out = np.empty((v.rows, v.cols), np.float32)
        rc = self.lib.orc_hsdc_decompress(_ptr(p, C.c_uint8), C.c_size_t(p.size),
                                          *self._dict_args(d), _ptr(out))
        if rc:
            raise ValueError(f"orc_hsdc_decompress rc={rc}")
        return out

    def dense_matmul(self, W, x, batch):
        W = _f32(W)
        x = _f32(x)
        R, Cc = W.shape
        y = np.empty((R, batch), np.float32)
        self.lib.orc_dense_matmul(_ptr(W), C.c_size_t(R), C.c_size_t(Cc), _ptr(x),
                                  C.c_size_t(batch), _ptr(y))
        return y

    def dequantize(self, fmt, data, scale=1.0, zero_point=0.0):
        p = self._bytes(data)
        per = {"f32": (4, 1), "f16": (2, 1), "bf16": (2, 1), "i8": (1, 1), "q4_0": (18, 32),
               "q8_0": (34, 32), "q4_k": (144, 256), "q5_k": (176, 256), "q6_k": (210, 256)}[fmt]
        cap = (p.size // per[0] + 1) * per[1]
        out = np.empty(cap, np.float32)
        n = self.lib.orc_dequantize(fmt.encode(), _ptr(p, C.c_uint8), C.c_size_t(p.size),
                                    C.c_float(scale), C.c_float(zero_point), _ptr(out),
                                    C.c_size_t(cap))
        if n < 0:
            raise ValueError(f"orc_dequantize rc={n}")
        return out[:n].copy()

    def dequantize_inference(self, fmt, data, n_elements=None):
        """Stored-raw tensor in a GGUF block format as the reference's inference side widens it."""
        p = self._bytes(data)
        bb, be = {"q4_0": (18, 32), "q8_0": (34, 32), "q4_k": (144, 256), "q5_k": (176, 256), "q6_k": (210, 256)}[fmt]
        cap = p.size // bb * be
        n_elements = cap if n_elements is None else n_elements
        out = np.empty(max(cap, 1), np.float32)
        self.lib.orc_dequantize_inference.restype = C.c_long
        n = self.lib.orc_dequantize_inference(fmt.encode(), _ptr(p, C.c_uint8), C.c_size_t(p.size),
                                              C.c_size_t(n_elements), _ptr(out), C.c_size_t(cap))
        if n < 0:
            raise ValueError(f"orc_dequantize_inference rc={n}")
        return out[:n].copy()

    def rms_norm(self, x, w, eps):
        x = _f32(x)
        w = _f32(w)
        out = np.empty_like(x)
        self.lib.orc_rms_norm(_ptr(x), _ptr(w), C.c_size_t(x.shape[0]), C.c_size_t(x.shape[1]),
                              C.c_float(eps), _ptr(out))
        return out

    def rope(self, t, theta, pos0=0):
        t = _f32(t).copy()
        seq, heads, hd = t.shape
        self.lib.orc_rope(_ptr(t), C.c_size_t(seq), C.c_size_t(heads), C.c_size_t(hd),
                          C.c_float(theta), C.c_size_t(pos0))
        return t

    def silu_mul(self, g, u):
        g = _f32(g)
        u = _f32(u)
        out = np.empty_like(g)
        self.lib.orc_silu_mul(_ptr(g), _ptr(u), C.c_size_t(g.size), _ptr(out))
        return out

    def attention(self, q, k, v):
        q, k, v = _f32(q), _f32(k), _f32(v)
        seq, qh, hd = q.shape
        out = np.empty((seq, qh * hd), np.float32)
        self.lib.orc_attention(_ptr(q), _ptr(k), _ptr(v), C.c_size_t(seq), C.c_size_t(qh),
                               C.c_size_t(k.shape[1]), C.c_size_t(hd), _ptr(out))
        return out

    def select_best_from_logits(self, logits, generated, temperature):
        """generated: iterable of token ids already produced."""
        lg = np.ascontiguousarray(logits, np.float32)
        flags = np.zeros(lg.size, np.uint8)
        for t in generated:
            if 0 <= int(t) < lg.size:
                flags[int(t)] = 1
        self.lib.orc_select_best_from_logits.restype = C.c_int
        return int(self.lib.orc_select_best_from_logits(_ptr(lg), C.c_size_t(lg.size),
                                                         flags.ctypes.data_as(C.c_void_p), C.c_float(temperature)))

    def decoder_forward(self, cfg: dict, tok_embd, blocks, out_norm, lm_head, tokens):
        """blocks: list of dicts with the nine dense fp32 arrays. Returns (hidden, logits)."""
        c = _DecoderCfg(cfg["n_layers"], cfg["hidden"], cfg["q_heads"], cfg["kv_heads"],
                        cfg["head_dim"], cfg["inter"], cfg["vocab"], cfg["eps"], cfg["theta"])
        keep = []
        bw = (_BlockWeights * len(blocks))()
        for i, b in enumerate(blocks):
            for name, _ in _BlockWeights._fields_:
                a = _f32(b[name])
                keep.append(a)
                setattr(bw[i], name, _ptr(a))
        tok_embd = _f32(tok_embd)
        out_norm = _f32(out_norm)
        lm_head = _f32(lm_head)
        tokens = np.ascontiguousarray(tokens, dtype=np.int32)
        hidden = np.empty((tokens.size, cfg["hidden"]), np.float32)
        logits = np.empty(cfg["vocab"], np.float32)
        rc = self.lib.orc_decoder_forward(C.byref(c), _ptr(tok_embd), bw, _ptr(out_norm),
                                          _ptr(lm_head), _ptr(tokens, C.c_int32),
                                          C.c_size_t(tokens.size), _ptr(hidden), _ptr(logits))
        if rc:
            raise ValueError(f"orc_decoder_forward rc={rc}")
        return hidden, logits


class _RefCfg(C.Structure):
    _fields_ = [("tile_rows", C.c_uint16), ("tile_cols", C.c_uint16), ("n_atoms", C.c_uint16),
                ("n_stages", C.c_uint8), ("k", C.c_uint8), ("ksvd_iters", C.c_uint8),
                ("pad", C.c_uint8), ("decay", C.c_float), ("max_tiles_for_fit", C.c_uint32)]


class _SegDesc(C.Structure):
    _fields_ = [("data", C.c_void_p), ("nbytes", C.c_uint64), ("name", C.c_char_p),
                ("data_format", C.c_char_p), ("seg_type", C.c_int32), ("layer_index", C.c_uint32),
                ("ndims", C.c_uint32), ("dims", C.c_uint32 * 4), ("has_scale", C.c_int32),
                ("scale", C.c_float), ("zero_point", C.c_float)]


def cfg_default(**kw):
    """HierarchicalSDRConfig{} defaults (HierarchicalSDRStrategy.hpp:44-58)."""
    d = dict(tile_rows=128, tile_cols=128, n_atoms=256, n_stages=3, k=5, ksvd_iters=8,
             decay=0.5, max_tiles_for_fit=0)
    d.update(kw)
    return d


def cfg_mlp(**kw):
    """forMLP() (HierarchicalSDRStrategy.hpp:61-67)."""
    return cfg_default(**{**dict(n_atoms=512, k=8, ksvd_iters=12), **kw})


def cfg_row1d(row_width, n_atoms=512, k=8, **kw):
    """forRow1D() (HierarchicalSDRStrategy.hpp:77-89)."""
    return cfg_default(**{**dict(tile_rows=1, tile_cols=row_width, n_atoms=n_atoms, k=k,
                                 n_stages=3, ksvd_iters=12, decay=0.5), **kw})


@dataclass
class Segment:
    name: str
    data: np.ndarray            # raw bytes (uint8) or an fp32 matrix
    dims: tuple
    seg_type: int = SEG_WEIGHTS_FP32
    data_format: str = "f32"
    layer_index: int = 0
    scale: float | None = None
    zero_point: float = 0.0


class Reference:
    @staticmethod
    def available():
        return os.path.exists(REF_SO)

    def __init__(self):
        if not self.available():
            raise FileNotFoundError(REF_SO)
        self.lib = C.CDLL(REF_SO)
        L = self.lib
        for f in ("ref_hsdr_compress", "ref_hsdr_decompress", "ref_hsdr_matmul",
                  "ref_hsdr_matmul_timed", "ref_hsdr_decompress_dense_timed", "ref_dequantize",
                  "ref_hsda_write", "ref_hsda_matmul", "ref_hsda_decompress", "ref_sdr_write",
                  "ref_sdr_decompress", "ref_sdr_matmul"):
            getattr(L, f).restype = C.c_long
        L.ref_last_error.restype = C.c_char_p
        L.ref_free.argtypes = [C.c_void_p]

    def _err(self, what):
        return RuntimeError(f"{what}: {self.lib.ref_last_error().decode(errors='replace')}")

    @staticmethod
    def _cfg(d):
        if d is None:
            return None
        return _RefCfg(d["tile_rows"], d["tile_cols"], d["n_atoms"], d["n_stages"], d["k"],
                       d["ksvd_iters"], 0, d["decay"], d["max_tiles_for_fit"])

    @staticmethod
    def _seg(s: Segment, keep):
        raw = s.data
        if raw.dtype != np.uint8:
            raw = np.ascontiguousarray(raw, dtype=np.float32).view(np.uint8).reshape(-1)
        raw = np.ascontiguousarray(raw)
        keep.append(raw)
        d = _SegDesc()
        d.data = raw.ctypes.data
        d.nbytes = raw.size
        d.name = s.name.encode()
        d.data_format = s.data_format.encode()
        d.seg_type = s.seg_type
        d.layer_index = s.layer_index
        d.ndims = len(s.dims)
        for i, v in enumerate(s.dims):
            d.dims[i] = v
        d.has_scale = 1 if s.scale is not None else 0
        d.scale = s.scale or 0.0
        d.zero_point = s.zero_point
        return d

    def _cfg_ptrs(self, attn_cfg, mlp_cfg, keep):
        a, m = self._cfg(attn_cfg), self._cfg(mlp_cfg)
        keep += [a, m]
        return (C.byref(a) if a is not None else None, C.byref(m) if m is not None else None)

    def mt19937_normal(self, seed, specs):
        """specs: list of (count, mean, std); one engine, one fresh distribution each."""
        counts = np.array([s[0] for s in specs], np.uint64)
        means = np.array([s[1] for s in specs], np.float32)
        stds = np.array([s[2] for s in specs], np.float32)
        out = np.empty(int(counts.sum()), np.float32)
        self.lib.ref_mt19937_normal(C.c_uint32(seed), C.c_uint32(len(specs)),
                                    _ptr(counts, C.c_uint64), _ptr(means), _ptr(stds), _ptr(out))
        res, o = [], 0
        for c in counts:
            res.append(out[o:o + int(c)].copy())
            o += int(c)
        return res

    def attention(self, q, k, v):
        """Causal multi-head attention by the reference's kernel. q (seq, q_heads, hd); k, v
        (seq, kv_heads, hd), repeated here to q_heads as the reference's decoder driver does
        (repeat_kv_heads, api/cortex_sdk.cpp:1453-1478). Returns (seq, q_heads*hd)."""
        q, k, v = _f32(q), _f32(k), _f32(v)
        seq, qh, hd = q.shape
        rep = qh // k.shape[1]
        k, v = _f32(np.repeat(k, rep, axis=1)), _f32(np.repeat(v, rep, axis=1))
        out = np.empty((seq, qh * hd), np.float32)
        self.lib.ref_multi_head_attention.restype = C.c_long
        n = self.lib.ref_multi_head_attention(_ptr(q), _ptr(k), _ptr(v), _ptr(out), C.c_uint64(1), C.c_uint64(seq),
                                              C.c_uint64(qh * hd), C.c_uint64(qh), C.c_int(1))
        if n < 0:
            raise self._err("multi_head_attention")
        return out

    def compress(self, seg: Segment, attn_cfg=None, mlp_cfg=None) -> bytes:
        keep = []
        d = self._seg(seg, keep)
        a, m = self._cfg_ptrs(attn_cfg, mlp_cfg, keep)
        out = C.c_void_p()
        n = self.lib.ref_hsdr_compress(C.byref(d), a, m, C.byref(out))
        if n < 0:
            raise self._err("compress")
        b = C.string_at(out, n)
        self.lib.ref_free(out)
        return b

    def decompress(self, payload, rows, cols):
        p = np.frombuffer(payload, np.uint8)
        out = np.empty((rows, cols), np.float32)
        n = self.lib.ref_hsdr_decompress(_ptr(p, C.c_uint8), C.c_uint64(p.size),
                                         C.c_uint64(rows * cols * 4), _ptr(out))
        if n < 0:
            raise self._err("decompress")
        return out

    def matmul(self, payload, x, batch, rows):
        p = np.frombuffer(payload, np.uint8)
        x = _f32(x)
        y = np.empty((rows, batch), np.float32)
        n = self.lib.ref_hsdr_matmul(_ptr(p, C.c_uint8), C.c_uint64(p.size), _ptr(x),
                                     C.c_uint64(batch), _ptr(y), C.c_uint64(y.size))
        if n < 0:
            raise self._err("matmulRowMajor")
        return y

    def matmul_timed(self, payload, x, batch, rows, iters=5):
        p = np.frombuffer(payload, np.uint8)
        x = _f32(x)
        y = np.empty((rows, batch), np.float32)
        sec = C.c_double()
        n = self.lib.ref_hsdr_matmul_timed(_ptr(p, C.c_uint8), C.c_uint64(p.size), _ptr(x),
                                           C.c_uint64(batch), C.c_int(iters), C.byref(sec),
                                           _ptr(y), C.c_uint64(y.size))
        if n < 0:
            raise self._err("matmulRowMajor(timed)")
        return sec.value, y

    def decompress_dense_timed(self, payload, rows, cols, x_tm, batch, iters=3):
        """x_tm token-major (batch, C). Returns (seconds, y_tm (batch, R))."""
        p = np.frombuffer(payload, np.uint8)
        x_tm = _f32(x_tm)
        y = np.empty((batch, rows), np.float32)
        sec = C.c_double()
        n = self.lib.ref_hsdr_decompress_dense_timed(
            _ptr(p, C.c_uint8), C.c_uint64(p.size), C.c_uint64(rows), C.c_uint64(cols),
            _ptr(x_tm), C.c_uint64(batch), C.c_int(iters), C.byref(sec), _ptr(y))
        if n < 0:
            raise self._err("decompress+linear_forward(timed)")
        return sec.value, y

    def dequantize(self, seg: Segment, n_out):
        keep = []
        d = self._seg(seg, keep)
        out = np.empty(n_out, np.float32)
        n = self.lib.ref_dequantize(C.byref(d), _ptr(out), C.c_uint64(n_out))
        if n < 0:
            raise self._err("dequantizeToFP32")
        return out[:n]

    def _seg_array(self, segs, keep):
        arr = (_SegDesc * len(segs))()
        for i, s in enumerate(segs):
            arr[i] = self._seg(s, keep)
        return arr

    def hsda_write(self, segs, path, attn_cfg=None, mlp_cfg=None):
        keep = []
        arr = self._seg_array(segs, keep)
        a, m = self._cfg_ptrs(attn_cfg, mlp_cfg, keep)
        n = self.lib.ref_hsda_write(arr, C.c_uint32(len(segs)), a, m, path.encode())
        if n < 0:
            raise self._err("compressGroupedSegments")
        return n

    def hsda_matmul(self, path, name, x, batch, rows):
        x = _f32(x)
        y = np.empty((rows, batch), np.float32)
        n = self.lib.ref_hsda_matmul(path.encode(), name.encode(), _ptr(x), C.c_uint64(batch),
                                     _ptr(y), C.c_uint64(y.size))
        if n < 0:
            raise self._err("HSDAReader::matmul")
        return y

    def hsda_decompress(self, path, name, rows, cols):
        out = np.empty((rows, cols), np.float32)
        n = self.lib.ref_hsda_decompress(path.encode(), name.encode(), _ptr(out),
                                         C.c_uint64(out.nbytes))
        if n < 0:
            raise self._err("HSDAReader::decompress")
        return out

    def sdr_write(self, segs, path, attn_cfg=None, mlp_cfg=None):
        keep = []
        arr = self._seg_array(segs, keep)
        a, m = self._cfg_ptrs(attn_cfg, mlp_cfg, keep)
        n = self.lib.ref_sdr_write(arr, C.c_uint32(len(segs)), a, m, path.encode())
        if n < 0:
            raise self._err("AICompressor::compressModel")
        return n

    def sdr_decompress(self, path, name, n_floats):
        out = np.empty(n_floats, np.float32)
        n = self.lib.ref_sdr_decompress(path.encode(), name.encode(), _ptr(out),
                                        C.c_uint64(out.nbytes))
        if n < 0:
            raise self._err("decompressSegment")
        return out[:n // 4]

    def sdr_matmul(self, path, name, x, batch, rows):
        x = _f32(x)
        y = np.empty((rows, batch), np.float32)
        n = self.lib.ref_sdr_matmul(path.encode(), name.encode(), _ptr(x), C.c_uint64(batch),
                                    _ptr(y), C.c_uint64(y.size))
        if n < 0:
            raise self._err("matmulHSDR")
        return y


class ReferenceEngine:
    """The reference's inference engine (SDRModelLoader) behind ref_engine_shim.cpp, where built."""

    @staticmethod
    def available() -> bool:
        return os.path.exists(REF_ENGINE_SO)

    def __init__(self):
        self.lib = C.CDLL(REF_ENGINE_SO)
        self.lib.ref_engine_last_error.restype = C.c_char_p

    def layer_weights(self, path: str, name: str) -> np.ndarray:
        """fp32 weights of a layer as SDRModelLoader::loadLayerByName decodes them."""
        n = C.c_size_t()
        if self.lib.ref_engine_layer_weights(path.encode(), name.encode(), None, C.c_size_t(0), C.byref(n)):
            raise RuntimeError(self.lib.ref_engine_last_error().decode())
        out = np.empty(n.value, np.float32)
        if self.lib.ref_engine_layer_weights(path.encode(), name.encode(), _ptr(out), C.c_size_t(out.size), C.byref(n)):
            raise RuntimeError(self.lib.ref_engine_last_error().decode())
        return out
