"""cortexsdr_b200 — B200-native HSDR on-demand inference matmul.

Python face of libcortexsdr_b200.so. The classes mirror, name for name, the part of the
reference's interface that sits on this path (paths inside the reference tree,
src/ai_compression/):

* ``HierarchicalSDRStrategy`` — decompress / matmulRowMajor /
  decompressWithExternalDictionary / matmulWithExternalDictionary / dequantizeToFP32
  (strategies/HierarchicalSDRStrategy.hpp:157-333)
* ``SDRModelLoader`` — findSegmentHeader / loadCompressedBytesByName / loadSegmentByName /
  matmulHSDR (SparseInferenceEngine.hpp:129-192)
* ``SDRInferenceEngine`` — matmulForLayer / applyLinearLayer (SparseInferenceEngine.hpp:305-307)
* ``HSDAReader`` — fromFile / hasSegment / decompress / matmul
  (strategies/HierarchicalSDRStrategy.hpp:368-405)

Errors follow the reference: ``CompressionError`` for malformed or refused payloads,
``RuntimeError`` for lookups ("segment not found", "is not HSDR-encoded").
All arithmetic runs on the GPU; nothing here falls back to the CPU.
"""
from __future__ import annotations

import ctypes as C
import weakref
from dataclasses import dataclass

import numpy as np

from . import _lib
from ._lib import (DTYPE_BF16, DTYPE_F32, FEATURE_MAJOR, TOKEN_MAJOR, DecoderConfig, PayloadInfo,
                   SegmentHeader)

__all__ = ["CompressionError", "Context", "Segment", "Dictionary", "HierarchicalSDRStrategy",
           "SDRModelLoader", "SDRInferenceEngine", "HSDAReader", "Decoder", "default_context",
           "HSDR_STRATEGY_ID", "NcclComm", "nccl_unique_id"]

HSDR_STRATEGY_ID = 5


class CompressionError(Exception):
    """strategies/CompressionStrategy.hpp:33-36"""


class CudaError(RuntimeError):
    pass


def _raise(rc: int):
    msg = _lib.load().csdr_last_error().decode(errors="replace")
    if rc in (_lib.ERR_FORMAT, _lib.ERR_GEOMETRY, _lib.ERR_CODE_RANGE, _lib.ERR_UNSUPPORTED):
        raise CompressionError(msg)
    if rc in (_lib.ERR_CUDA, _lib.ERR_TIMEOUT):
        raise CudaError(msg)
    if rc == _lib.ERR_BUFFER:
        raise BufferError(msg)
    if rc in (_lib.ERR_INVALID_ARG, _lib.ERR_LIMIT):
        raise ValueError(msg)
    raise RuntimeError(msg)  # NOT_FOUND, STRATEGY, IO


def _check(rc: int):
    if rc != _lib.OK:
        _raise(rc)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _fp(a: np.ndarray):
    return a.ctypes.data_as(C.POINTER(C.c_float))


def _bytes(b) -> np.ndarray:
    if isinstance(b, np.ndarray):
        return np.ascontiguousarray(b.view(np.uint8).reshape(-1))
    return np.frombuffer(bytes(b), dtype=np.uint8)


class Context:
    """One device + one stream. `stream` may be a raw cudaStream_t (int) to share, e.g.
    ``torch.cuda.current_stream().cuda_stream``."""

    def __init__(self, device: int = -1, stream: int | None = None):
        self._lib = _lib.load()
        h = C.c_void_p()
        _check(self._lib.csdr_context_create(device, C.c_void_p(stream) if stream else None,
                                             C.byref(h)))
        self._h = h
        # Everything created on this context; closed before the context itself, whatever order
        # the interpreter finalises objects in (at shutdown the cyclic collector picks any).
        self._children = weakref.WeakSet()

    def _adopt(self, child):
        self._children.add(child)

    def synchronize(self):
        _check(self._lib.csdr_context_synchronize(self._h))

    @property
    def stream(self) -> int:
        return self._lib.csdr_context_stream(self._h) or 0

    @property
    def launch_count(self) -> int:
        return int(self._lib.csdr_context_launch_count(self._h))

    def set_wait_limits(self, gemv_polls: int = 0, barrier_rounds: int = 0, exchange_polls: int = 0):
        """Iteration limits of the bounded device-side waits; 0 restores a default."""
        _check(self._lib.csdr_context_set_wait_limits(self._h, gemv_polls, barrier_rounds, exchange_polls))

    def wait_selftest(self) -> int:
        """Status of a wait on a flag nothing raises (ERR_TIMEOUT once the exchange limit is spent)."""
        return int(self._lib.csdr_context_wait_selftest(self._h))

    def profile(self, enable: bool):
        """Bracket every kernel launch with CUDA events (benchmarks only)."""
        _check(self._lib.csdr_context_profile(self._h, 1 if enable else 0))

    def profile_read(self) -> dict:
        """{kernel class: (launches, total_ms)} since profiling was enabled."""
        out, cls = {}, 0
        while True:
            name = self._lib.csdr_kernel_class_name(cls).decode()
            if name == "?":
                return out
            n, ms = C.c_uint64(), C.c_double()
            _check(self._lib.csdr_context_profile_read(self._h, cls, C.byref(n), C.byref(ms)))
            if n.value:
                out[name] = (int(n.value), float(ms.value))
            cls += 1

    def gemv_trace(self, enable: bool = True):
        """Phase stamps (ns) of the last fused-GEMV launch as an (n_ctas, 8) array, then set tracing."""
        buf = np.zeros(16 * 2048, np.uint64)
        n = C.c_size_t()
        _check(self._lib.csdr_context_gemv_trace(self._h, 1 if enable else 0,
                                                 buf.ctypes.data_as(C.POINTER(C.c_uint64)), buf.size,
                                                 C.byref(n)))
        return buf[:n.value].reshape(-1, 16)

    def close(self):
        if getattr(self, "_h", None):
            for child in sorted(list(self._children), key=lambda c: getattr(c, "_close_rank", 1)):
                try:
                    child.close()
                except Exception:
                    pass
            self._lib.csdr_context_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class _NoDevice:
    """Stands where a Context would when an archive is opened for its index only."""

    def __init__(self):
        self._lib = _lib.load()
        self._h = None

    def _adopt(self, child):
        pass


_default_ctx: Context | None = None


def default_context() -> Context:
    global _default_ctx
    if _default_ctx is None:
        _default_ctx = Context()
    return _default_ctx


def inspect_payload(payload) -> PayloadInfo:
    """Header fields + stream offsets of an HSDR/HSDC payload (host only, no GPU needed)."""
    p = _bytes(payload)
    info = PayloadInfo()
    _check(_lib.load().csdr_payload_inspect(p.ctypes.data_as(C.c_void_p), p.size, C.byref(info)))
    return info


class Dictionary:
    """SharedDictionary (strategies/HierarchicalSDRStrategy.hpp:194-198) on the device."""

    def __init__(self, ctx: Context, tile_rows, tile_cols, n_atoms, n_stages, k, atoms, scales):
        self.ctx = ctx
        atoms, scales = _f32(atoms).reshape(-1), _f32(scales).reshape(-1)
        if atoms.size != n_atoms * tile_rows * tile_cols or scales.size != n_stages:
            raise CompressionError("dictionary arrays do not match its config")
        h = C.c_void_p()
        _check(ctx._lib.csdr_dictionary_create(ctx._h, tile_rows, tile_cols, n_atoms, n_stages, k,
                                               _fp(atoms), _fp(scales), C.byref(h)))
        self._h = h
        ctx._adopt(self)

    def close(self):
        if getattr(self, "_h", None) and self.ctx._h:
            self.ctx._lib.csdr_dictionary_destroy(self._h)
        self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Segment:
    """Device image of one compressed weight."""

    def __init__(self, ctx: Context, handle, owned=True, keep=None):
        self.ctx, self._h, self._owned, self._keep = ctx, handle, owned, keep
        self._close_rank = 0          # segments and shards go first
        ctx._adopt(self)
        info = PayloadInfo()
        _check(ctx._lib.csdr_segment_info(handle, C.byref(info)))
        self.info = info

    @classmethod
    def from_payload(cls, payload, ctx: Context | None = None, dictionary: Dictionary | None = None):
        ctx = ctx or default_context()
        p = _bytes(payload)
        h = C.c_void_p()
        if dictionary is None:
            _check(ctx._lib.csdr_segment_create(ctx._h, p.ctypes.data_as(C.c_void_p), p.size,
                                                C.byref(h)))
        else:
            _check(ctx._lib.csdr_segment_create_shared(ctx._h, p.ctypes.data_as(C.c_void_p), p.size,
                                                       dictionary._h, C.byref(h)))
        return cls(ctx, h, True, dictionary)

    rows = property(lambda s: s.info.rows)
    cols = property(lambda s: s.info.cols)

    @property
    def n_codes(self):
        return self.info.n_tiles * self.info.n_stages * self.info.k_per_stage

    def shard_rows(self, begin: int, end: int) -> "Segment":
        h = C.c_void_p()
        _check(self.ctx._lib.csdr_segment_shard_rows(self.ctx._h, self._h, begin, end, C.byref(h)))
        return Segment(self.ctx, h, True, self)

    def shard_cols(self, begin: int, end: int) -> "Segment":
        """Input columns [begin, end) of a row-tile segment: its product with x[begin:end] is that
        slice's share of W x."""
        h = C.c_void_p()
        _check(self.ctx._lib.csdr_segment_shard_cols(self.ctx._h, self._h, begin, end, C.byref(h)))
        return Segment(self.ctx, h, True, self)

    def unpack(self):
        """(int32 indices, int8 signs), produced by the device unpack kernel."""
        n = self.n_codes
        idx, sign = np.empty(n, np.int32), np.empty(n, np.int8)
        _check(self.ctx._lib.csdr_unpack_codes(self.ctx._h, self._h,
                                               idx.ctypes.data_as(C.POINTER(C.c_int32)),
                                               sign.ctypes.data_as(C.POINTER(C.c_int8)), n))
        return idx, sign

    def matmul(self, x, batch: int, allow_2d: bool = False, out: np.ndarray | None = None) -> np.ndarray:
        """x (C, batch) row-major fp32 -> y (R, batch), host arrays. `out` (fp32, C-contiguous,
        rows*batch elements) receives the result when given, so that a caller in a loop does
        not pay for an allocation per call."""
        if not (type(x) is np.ndarray and x.dtype == np.float32 and x.flags.c_contiguous):
            x = _f32(x)
        if x.size != self.cols * batch:
            raise ValueError("x must hold cols*batch floats")
        if out is None:
            out = np.empty((self.rows, batch), np.float32)
        elif not (out.dtype == np.float32 and out.flags.c_contiguous and out.size == self.rows * batch):
            raise ValueError("out must be a C-contiguous fp32 array of rows*batch elements")
        _check(self.ctx._lib.csdr_matmul(self.ctx._h, self._h, x.__array_interface__["data"][0], batch,
                                         out.__array_interface__["data"][0], 1 if allow_2d else 0))
        return out

    def matmul_device(self, x_ptr: int, x_dtype: int, x_layout: int, batch: int, y_ptr: int,
                      y_layout: int, bias_ptr: int = 0):
        """Asynchronous product on raw device pointers (e.g. torch tensors' data_ptr())."""
        _check(self.ctx._lib.csdr_matmul_device_async(
            self.ctx._h, self._h, C.c_void_p(x_ptr), x_dtype, x_layout, batch, C.c_void_p(y_ptr),
            y_layout, C.c_void_p(bias_ptr) if bias_ptr else None))

    @staticmethod
    def matmul_group_device(segs, x_ptr: int, x_dtype: int, x_layout: int, batch: int, y_ptrs,
                            y_layout: int):
        """Segments sharing one activation (q|k|v, gate|up) in as few launches as possible."""
        ctx = segs[0].ctx
        n = len(segs)
        hs = (C.c_void_p * n)(*[s._h for s in segs])
        ys = (C.c_void_p * n)(*[C.c_void_p(p) for p in y_ptrs])
        _check(ctx._lib.csdr_matmul_group_device_async(ctx._h, hs, n, C.c_void_p(x_ptr), x_dtype,
                                                       x_layout, batch, ys, y_layout))

    @staticmethod
    def matmul_queue_device(tasks, prepared=None):
        """Independent products in as few launches as possible. tasks: iterable of
        (segment, x_ptr, x_dtype, x_layout, batch, y_ptr, y_layout[, bias_ptr[, after_task]]); after_task
        is the index of the earlier task whose output this task reads (-1: none). Returns the ctypes
        array; pass it back as `prepared` to issue the same list again without rebuilding it."""
        if prepared is None:
            tasks = list(tasks)
            prepared = (_lib.MatmulTask * len(tasks))()
            for i, t in enumerate(tasks):
                prepared[i].seg, prepared[i].x_dev, prepared[i].x_dtype, prepared[i].x_layout = t[0]._h, t[1], t[2], t[3]
                prepared[i].batch, prepared[i].y_dev, prepared[i].y_layout = t[4], t[5], t[6]
                prepared[i].bias_dev = t[7] if len(t) > 7 and t[7] else None
                prepared[i].after_task = t[8] if len(t) > 8 else -1
            prepared._ctx = tasks[0][0].ctx
        ctx = prepared._ctx
        _check(ctx._lib.csdr_matmul_queue_device_async(ctx._h, prepared, len(prepared)))
        return prepared

    @staticmethod
    def matmul_queue(tasks, prepared=None):
        """Independent products on host arrays, reference layout: tasks is an iterable of
        (segment, x (C, batch) fp32, batch, out (R, batch) fp32). One upload, one launch per 32
        tasks, one download. Returns the ctypes array; pass it back as `prepared` to run the same
        list again without rebuilding it (the arrays must stay alive and in place)."""
        if prepared is None:
            tasks = list(tasks)
            prepared = (_lib.MatmulHostTask * len(tasks))()
            for i, (seg, x, batch, out) in enumerate(tasks):
                if not (x.dtype == np.float32 and x.flags.c_contiguous and x.size == seg.cols * batch):
                    raise ValueError("x must be C-contiguous fp32 with cols*batch elements")
                if not (out.dtype == np.float32 and out.flags.c_contiguous and out.size == seg.rows * batch):
                    raise ValueError("out must be C-contiguous fp32 with rows*batch elements")
                prepared[i].seg, prepared[i].batch = seg._h, batch
                prepared[i].x, prepared[i].y = x.__array_interface__["data"][0], out.__array_interface__["data"][0]
            prepared._ctx = tasks[0][0].ctx
        ctx = prepared._ctx
        _check(ctx._lib.csdr_matmul_queue(ctx._h, prepared, len(prepared)))
        return prepared

    def decompress(self) -> np.ndarray:
        out = np.empty((self.rows, self.cols), np.float32)
        _check(self.ctx._lib.csdr_decompress(self.ctx._h, self._h, _fp(out), out.size))
        return out

    def decompress_device(self, out_ptr: int):
        _check(self.ctx._lib.csdr_decompress_device_async(self.ctx._h, self._h, C.c_void_p(out_ptr)))

    def close(self):
        if getattr(self, "_h", None) and self._owned and self.ctx._h:
            self.ctx._lib.csdr_segment_destroy(self._h)
        self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


@dataclass
class SharedDictionary:
    """Host-side SharedDictionary as the reference passes it around."""
    tile_rows: int
    tile_cols: int
    n_atoms: int
    n_stages: int
    k: int
    atoms: np.ndarray
    scales: np.ndarray


class HierarchicalSDRStrategy:
    """The strategy plug-in (id 5): the decode side and the encoder (fast mode and dictionary-update
    rounds)."""

    def __init__(self, ctx: Context | None = None):
        self.ctx = ctx or default_context()

    def compress(self, W, *, tile_rows: int = 128, tile_cols: int = 128, n_atoms: int = 256, n_stages: int = 3,
                 k: int = 5, decay: float = 0.5, ksvd_iters: int = 0) -> bytes:
        """HSDR payload of the fp32 matrix W (compress, strategies/HierarchicalSDRStrategy.cpp:1068-1236),
        encoded on the device. Defaults are the reference's HierarchicalSDRConfig{} geometry."""
        W = _f32(W)
        if W.ndim != 2:
            raise CompressionError("HSDR: expected a 2-D tensor")
        n = C.c_size_t()
        lib, h = self.ctx._lib, self.ctx._h
        args = (h, _fp(W), W.shape[0], W.shape[1], tile_rows, tile_cols, n_atoms, n_stages, k, decay, ksvd_iters)
        rc = lib.csdr_hsdr_encode(*args, None, 0, C.byref(n))
        if rc != _lib.ERR_BUFFER:
            _check(rc)
        out = np.empty(n.value, np.uint8)
        _check(lib.csdr_hsdr_encode(*args, out.ctypes.data_as(C.c_void_p), out.size, C.byref(n)))
        return out.tobytes()

    def compress_shared(self, tensors, *, tile_rows: int, tile_cols: int, n_atoms: int, n_stages: int = 3, k: int = 8,
                        decay: float = 0.5, ksvd_iters: int = 0):
        """Several fp32 matrices behind ONE dictionary (compressGroupedSegments,
        strategies/HierarchicalSDRStrategy.cpp:2211-2500, fit on all pooled tiles), encoded on the
        device. Returns (dictionary record bytes - the .hsda record, also the payload of a
        shared-dictionary resource segment of a .sdr -, [codes-only "HSDC" payload per tensor])."""
        Ws = [_f32(W) for W in tensors]
        if any(W.ndim != 2 for W in Ws):
            raise CompressionError("HSDR: expected 2-D tensors")
        n = len(Ws)
        ptrs = (C.POINTER(C.c_float) * n)(*[_fp(W) for W in Ws])
        rows = (C.c_uint32 * n)(*[W.shape[0] for W in Ws])
        cols = (C.c_uint32 * n)(*[W.shape[1] for W in Ws])
        dict_n = C.c_size_t()
        code_n = (C.c_size_t * n)()
        lib, h = self.ctx._lib, self.ctx._h
        head = (h, ptrs, rows, cols, n, tile_rows, tile_cols, n_atoms, n_stages, k, decay, ksvd_iters)
        rc = lib.csdr_hsdr_encode_shared(*head, None, 0, C.byref(dict_n), None, None, code_n)
        if rc != _lib.ERR_BUFFER:
            _check(rc)
        dict_out = np.empty(dict_n.value, np.uint8)
        outs = [np.empty(code_n[i], np.uint8) for i in range(n)]
        out_ptrs = (C.c_void_p * n)(*[o.ctypes.data for o in outs])
        caps = (C.c_size_t * n)(*[o.size for o in outs])
        _check(lib.csdr_hsdr_encode_shared(*head, dict_out.ctypes.data_as(C.c_void_p), dict_out.size, C.byref(dict_n), out_ptrs,
                                           caps, code_n))
        return dict_out.tobytes(), [o.tobytes() for o in outs]

    def encode_codes(self, tiles, atoms, stage_scales, k: int) -> np.ndarray:
        """The coding pass alone: packed u16 codes (n_tiles, n_stages, k)."""
        tiles, atoms, stage_scales = _f32(tiles), _f32(atoms), _f32(stage_scales)
        n, T = tiles.shape
        out = np.empty((n, stage_scales.size, k), np.uint16)
        _check(self.ctx._lib.csdr_encode_codes(self.ctx._h, _fp(tiles), n, T, _fp(atoms), atoms.shape[0], stage_scales.size, k,
                                               _fp(stage_scales), out.ctypes.data_as(C.POINTER(C.c_uint16)), out.size))
        return out

    def decompress(self, compressedData, originalType=None, originalSize: int = 0) -> np.ndarray:
        info = inspect_payload(compressedData)
        if originalSize and originalSize > info.rows * info.cols * 4:
            raise CompressionError("HSDR decompress: originalSize does not match shape")
        seg = Segment.from_payload(compressedData, self.ctx)
        try:
            return seg.decompress()
        finally:
            seg.close()

    def matmulRowMajor(self, compressedData, x, batch: int) -> np.ndarray:
        seg = Segment.from_payload(compressedData, self.ctx)
        try:
            return seg.matmul(x, batch)
        finally:
            seg.close()

    def _dict(self, d: SharedDictionary) -> Dictionary:
        return Dictionary(self.ctx, d.tile_rows, d.tile_cols, d.n_atoms, d.n_stages, d.k, d.atoms,
                          d.scales)

    def decompressWithExternalDictionary(self, codes_bytes, dict_: SharedDictionary,
                                         originalSize: int) -> np.ndarray:
        info = inspect_payload(codes_bytes)
        if info.rows * info.cols * 4 != originalSize:
            raise CompressionError("decompressWithExternalDictionary: originalSize mismatch")
        dd = self._dict(dict_)
        seg = Segment.from_payload(codes_bytes, self.ctx, dd)
        try:
            return seg.decompress()
        finally:
            seg.close()
            dd.close()

    def matmulWithExternalDictionary(self, codes_bytes, dict_: SharedDictionary, x, batch: int):
        dd = self._dict(dict_)
        seg = Segment.from_payload(codes_bytes, self.ctx, dd)
        try:
            return seg.matmul(x, batch)
        finally:
            seg.close()
            dd.close()

    def dequantizeToFP32(self, data, data_format: str, scale: float = 1.0,
                         zero_point: float = 0.0) -> np.ndarray:
        p = _bytes(data)
        fmt = {"fp32": "f32", "float32": "f32", "fp16": "f16", "float16": "f16", "half": "f16",
               "bfloat16": "bf16", "int8": "i8"}.get(data_format.lower(), data_format.lower())
        n = C.c_size_t()
        per = {"f32": (4, 1), "f16": (2, 1), "bf16": (2, 1), "i8": (1, 1), "q4_0": (18, 32),
               "q8_0": (34, 32), "q4_k": (144, 256), "q5_k": (176, 256), "q6_k": (210, 256)}
        unit, cnt = per.get(fmt, (1, 1))
        out = np.empty((p.size // unit + 1) * cnt, np.float32)
        _check(self.ctx._lib.csdr_dequantize(self.ctx._h, fmt.encode(), p.ctypes.data_as(C.c_void_p),
                                             p.size, scale, zero_point, _fp(out), out.size,
                                             C.byref(n)))
        return out[:n.value].copy()


def dequantize_inference(data, data_format: str, n_elements: int | None = None, ctx: Context | None = None) -> np.ndarray:
    """A stored-raw tensor in a GGUF block format, widened the way the reference's inference side
    does it (decodeSupportedGGUFQuantized, SparseInferenceEngine.cpp:276-469)."""
    ctx = ctx or default_context()
    p = _bytes(data)
    bb, be = {"q4_0": (18, 32), "q8_0": (34, 32), "q4_k": (144, 256), "q5_k": (176, 256),
              "q6_k": (210, 256)}.get(data_format.lower(), (1, 0))
    cap = p.size // bb * be
    out = np.empty(max(cap, 1), np.float32)
    n = C.c_size_t()
    _check(ctx._lib.csdr_dequantize_inference(ctx._h, data_format.lower().encode(), p.ctypes.data_as(C.c_void_p), p.size,
                                              cap if n_elements is None else n_elements, _fp(out), out.size,
                                              C.byref(n)))
    return out[:n.value].copy()


@dataclass
class CompressedSegmentHeader:
    """core/AICompressor.hpp:51-65"""
    name: str
    data_format: str
    layer_type: str
    original_type: int
    compression_strategy_id: int
    original_size: int
    compressed_size: int
    data_offset: int
    layer_index: int
    dimensions: tuple


def _hdr(h: SegmentHeader) -> CompressedSegmentHeader:
    return CompressedSegmentHeader(h.name.decode(), h.data_format.decode(), h.layer_type.decode(),
                                   h.original_type, h.strategy_id, h.original_size,
                                   h.compressed_size, h.data_offset, h.layer_index,
                                   tuple(h.dims[i] for i in range(h.n_dims)))


class SDRModelLoader:
    def __init__(self, archive_path: str, ctx: Context | None = None, index_only: bool = False):
        """index_only: open without a device (headers and raw payload reads only)."""
        self.ctx = _NoDevice() if index_only else (ctx or default_context())
        h = C.c_void_p()
        _check(self.ctx._lib.csdr_archive_open(self.ctx._h, archive_path.encode(), C.byref(h)))
        self._h = h
        self._index_only = index_only
        self._close_rank = 2          # after the decoders that borrow its device images
        self.ctx._adopt(self)
        self.archive_path = archive_path

    def getSegmentHeaders(self):
        n = C.c_size_t()
        _check(self.ctx._lib.csdr_archive_num_segments(self._h, C.byref(n)))
        out = []
        for i in range(n.value):
            h = SegmentHeader()
            _check(self.ctx._lib.csdr_archive_header_at(self._h, i, C.byref(h)))
            out.append(_hdr(h))
        return out

    def findSegmentHeader(self, name: str):
        h = SegmentHeader()
        rc = self.ctx._lib.csdr_archive_find(self._h, name.encode(), C.byref(h))
        if rc == _lib.ERR_NOT_FOUND:
            return None
        _check(rc)
        return _hdr(h)

    def loadCompressedBytesByName(self, name: str) -> bytes:
        n = C.c_size_t()
        rc = self.ctx._lib.csdr_archive_read_payload(self._h, name.encode(), None, 0, C.byref(n))
        if rc not in (_lib.OK, _lib.ERR_BUFFER):
            _raise(rc)
        buf = np.empty(n.value, np.uint8)
        _check(self.ctx._lib.csdr_archive_read_payload(self._h, name.encode(),
                                                       buf.ctypes.data_as(C.c_void_p), buf.size,
                                                       C.byref(n)))
        return buf.tobytes()

    def loadSegmentByName(self, name: str) -> np.ndarray:
        """Decoded segment bytes (uint8). HSDR segments come back as the fp32 matrix."""
        n = C.c_size_t()
        rc = self.ctx._lib.csdr_archive_load_segment(self._h, name.encode(), None, 0, C.byref(n))
        if rc not in (_lib.OK, _lib.ERR_BUFFER):
            _raise(rc)
        buf = np.empty(n.value, np.uint8)
        _check(self.ctx._lib.csdr_archive_load_segment(self._h, name.encode(),
                                                       buf.ctypes.data_as(C.c_void_p), buf.size,
                                                       C.byref(n)))
        return buf

    def segment(self, name: str) -> Segment:
        """Cached device image of a named HSDR segment (owned by the loader)."""
        h = C.c_void_p()
        _check(self.ctx._lib.csdr_archive_segment(self._h, name.encode(), C.byref(h)))
        return Segment(self.ctx, h, owned=False, keep=self)

    def _mm(self, fn, name, x, batch):
        x = _f32(x)
        n = C.c_size_t()
        hdr = self.findSegmentHeader(name)
        rows = hdr.dimensions[0] if hdr and hdr.dimensions else 0
        y = np.empty(max(1, rows * batch), np.float32)
        _check(fn(self._h, name.encode(), _fp(x), batch, _fp(y), y.size, C.byref(n)))
        return y[:n.value].reshape(-1, batch) if batch else y[:0]

    def matmulHSDR(self, segment_name: str, x, batch: int) -> np.ndarray:
        return self._mm(self.ctx._lib.csdr_archive_matmul_hsdr, segment_name, x, batch)

    def resident_bytes(self) -> int:
        """Device bytes of the images built so far; a dictionary several tensors share counts once."""
        n = C.c_size_t()
        _check(self.ctx._lib.csdr_archive_resident_bytes(self._h, C.byref(n)))
        return n.value

    def close(self):
        if getattr(self, "_h", None) and (self._index_only or self.ctx._h):
            self.ctx._lib.csdr_archive_close(self._h)
        self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class SDRInferenceEngine:
    def __init__(self, model_loader: SDRModelLoader):
        self.loader_ = model_loader
        self.last_layer_used_compressed_ = False

    def matmulForLayer(self, segment_name: str, x, batch: int) -> np.ndarray:
        ld = self.loader_
        return ld._mm(ld.ctx._lib.csdr_archive_matmul_for_layer, segment_name, x, batch)

    def applyLinearLayer(self, layer_name: str, input_, biases=None) -> np.ndarray:
        """Token-major (batch, C) in, (batch, R) out; HSDR route only."""
        ld = self.loader_
        x = _f32(input_).reshape(-1)
        hdr = ld.findSegmentHeader(layer_name) or ld.findSegmentHeader(layer_name + ".weight")
        if hdr is None:
            raise RuntimeError("Segment not found: " + layer_name)
        rows, cols = hdr.dimensions[0], hdr.dimensions[1]
        batch = x.size // cols if cols else 0
        out = np.empty(max(1, batch * rows), np.float32)
        n = C.c_size_t()
        b = _f32(biases) if biases is not None else None
        _check(ld.ctx._lib.csdr_archive_apply_linear(ld._h, layer_name.encode(), _fp(x), x.size,
                                                     _fp(b) if b is not None else None, _fp(out),
                                                     out.size, C.byref(n)))
        self.last_layer_used_compressed_ = True
        return out[:n.value].reshape(batch, rows)


class HSDAReader:
    def __init__(self, handle, ctx: Context, path: str):
        self._h, self.ctx, self.path = handle, ctx, path
        self._index_only = isinstance(ctx, _NoDevice)
        self._close_rank = 2
        ctx._adopt(self)

    @classmethod
    def fromFile(cls, path: str, ctx: Context | None = None, index_only: bool = False) -> "HSDAReader":
        ctx = _NoDevice() if index_only else (ctx or default_context())
        h = C.c_void_p()
        _check(ctx._lib.csdr_hsda_open(ctx._h, path.encode(), C.byref(h)))
        return cls(h, ctx, path)

    def _counts(self):
        a, b = C.c_size_t(), C.c_size_t()
        _check(self.ctx._lib.csdr_hsda_counts(self._h, C.byref(a), C.byref(b)))
        return a.value, b.value

    def numDictionaries(self):
        return self._counts()[0]

    def numSegments(self):
        return self._counts()[1]

    def hasSegment(self, name: str) -> bool:
        return bool(self.ctx._lib.csdr_hsda_has_segment(self._h, name.encode()))

    def segment(self, name: str) -> Segment:
        h = C.c_void_p()
        _check(self.ctx._lib.csdr_hsda_segment(self._h, name.encode(), C.byref(h)))
        return Segment(self.ctx, h, owned=False, keep=self)

    def decompress(self, name: str) -> np.ndarray:
        seg = self.segment(name)
        out = np.empty((seg.rows, seg.cols), np.float32)
        n = C.c_size_t()
        _check(self.ctx._lib.csdr_hsda_decompress(self._h, name.encode(), _fp(out), out.size,
                                                  C.byref(n)))
        return out

    def matmul(self, name: str, x, batch: int, allow_2d: bool = False) -> np.ndarray:
        seg = self.segment(name)
        x = _f32(x)
        y = np.empty((seg.rows, batch), np.float32)
        n = C.c_size_t()
        _check(self.ctx._lib.csdr_hsda_matmul(self._h, name.encode(), _fp(x), batch, _fp(y),
                                              max(1, y.size), C.byref(n), 1 if allow_2d else 0))
        return y

    def close(self):
        if getattr(self, "_h", None) and (self._index_only or self.ctx._h):
            self.ctx._lib.csdr_hsda_close(self._h)
        self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def nccl_unique_id() -> bytes:
    """128-byte NCCL id made on one rank; broadcast it to the others by any host-side means."""
    buf = C.create_string_buffer(128)
    _check(_lib.load().csdr_nccl_unique_id(buf))
    return buf.raw


class NcclComm:
    """One rank's communicator for the tensor-parallel decoder."""

    def __init__(self, ctx: Context, unique_id: bytes, rank: int, world: int):
        self.ctx = ctx
        h = C.c_void_p()
        _check(ctx._lib.csdr_nccl_comm_create(ctx._h, unique_id, rank, world, C.byref(h)))
        self._h, self.rank, self.world = h, rank, world
        self._close_rank = 3
        ctx._adopt(self)

    def close(self):
        if getattr(self, "_h", None) and self.ctx._h:
            self.ctx._lib.csdr_nccl_comm_destroy(self._h)
        self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Decoder:
    """Device-resident decoder-layer driver over an opened archive (run_transformer_decode,
    api/cortex_sdk.cpp:1543-1696, with a KV cache)."""

    def __init__(self, loader: SDRModelLoader, *, n_layers, hidden, q_heads, kv_heads, head_dim,
                 inter, vocab, max_seq, max_batch=1, rms_eps=1e-5, rope_theta=1e6, comm: "NcclComm | None" = None,
                 all_gather=None, kv_dtype="f32"):
        """kv_dtype: "f32" (the reference's arithmetic), "f16" or "bf16" (cache rows rounded to 16 bits, sums fp32).
        all_gather: a callable bytes -> list[bytes] (one entry per rank, rank order) supplied by
        the host program, e.g. built on torch.distributed.all_gather_object. When given with a
        communicator of 2 to 8 ranks, the ranks exchange CUDA IPC handles through it and sum their
        partial projections through peer memory for steps of at most 16 tokens."""
        self.loader, self.ctx, self.comm = loader, loader.ctx, comm
        self.cfg = DecoderConfig(n_layers, hidden, q_heads, kv_heads, head_dim, inter, vocab,
                                 max_seq, max_batch, rms_eps, rope_theta, comm.rank if comm else 0,
                                 comm.world if comm else 1, comm._h if comm else None,
                                 {"f32": 0, "bf16": 1, "f16": 2}[kv_dtype])
        h = C.c_void_p()
        _check(self.ctx._lib.csdr_decoder_create(loader._h, C.byref(self.cfg), C.byref(h)))
        self._h = h
        self._close_rank = 1
        self.ctx._adopt(self)
        if comm is not None and all_gather is not None and 2 <= comm.world <= 8:
            mine = C.create_string_buffer(64)
            _check(self.ctx._lib.csdr_decoder_exchange_export(self._h, mine))
            handles = all_gather(mine.raw)
            if len(handles) != comm.world or any(len(b) != 64 for b in handles):
                raise ValueError("all_gather must return one 64-byte handle per rank")
            _check(self.ctx._lib.csdr_decoder_exchange_import(self._h, b"".join(handles), comm.world))

    def reset(self):
        _check(self.ctx._lib.csdr_decoder_reset(self._h))

    def selection_policy(self, enable: bool = True, temperature: float = 1.0):
        """The reference's select_best_from_logits for the steps (temperature scale, 1.5 off for
        tokens the sequence has produced, first maximum) instead of plain argmax."""
        _check(self.ctx._lib.csdr_decoder_selection_policy(self._h, 1 if enable else 0, temperature))

    def note_generated(self, tokens, seq: int = 0):
        t = np.ascontiguousarray(tokens, dtype=np.int32).reshape(-1)
        _check(self.ctx._lib.csdr_decoder_note_generated(self._h, seq, t.ctypes.data_as(C.POINTER(C.c_int32)), t.size))

    def seek(self, seq: int, position: int):
        _check(self.ctx._lib.csdr_decoder_seek(self._h, seq, position))

    def forward(self, tokens, seq: int = 0, want_logits=True, want_hidden=False):
        t = np.ascontiguousarray(tokens, dtype=np.int32)
        logits = np.empty(self.cfg.vocab, np.float32) if want_logits else None
        hidden = np.empty((t.size, self.cfg.hidden), np.float32) if want_hidden else None
        _check(self.ctx._lib.csdr_decoder_forward(
            self._h, seq, t.ctypes.data_as(C.POINTER(C.c_int32)), t.size,
            _fp(logits) if want_logits else None, _fp(hidden) if want_hidden else None))
        return logits, hidden

    def step(self, tokens, want_logits=False):
        t = np.ascontiguousarray(tokens, dtype=np.int32)
        nxt = np.empty(t.size, np.int32)
        logits = np.empty((t.size, self.cfg.vocab), np.float32) if want_logits else None
        _check(self.ctx._lib.csdr_decoder_step(
            self._h, t.ctypes.data_as(C.POINTER(C.c_int32)), t.size,
            nxt.ctypes.data_as(C.POINTER(C.c_int32)), _fp(logits) if want_logits else None))
        return nxt, logits

    def step_device(self, tokens_ptr: int, batch: int, next_ptr: int):
        _check(self.ctx._lib.csdr_decoder_step_device_async(self._h, C.c_void_p(tokens_ptr), batch,
                                                            C.c_void_p(next_ptr)))

    def close(self):
        if getattr(self, "_h", None) and self.ctx._h and self.loader._h:
            self.ctx._lib.csdr_decoder_destroy(self._h)
        self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
