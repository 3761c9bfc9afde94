"""ctypes binding of libcortexsdr_b200.so (the C-ABI declared in include/cortexsdr_b200.h).

There is no CPU path: if the shared library is missing, or no B200 is present when a
compute entry point is called, the call fails loudly.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libcortexsdr_b200.so")

OK = 0
ERR_INVALID_ARG = -1
ERR_FORMAT = -2
ERR_GEOMETRY = -3
ERR_NOT_FOUND = -4
ERR_STRATEGY = -5
ERR_CUDA = -6
ERR_TIMEOUT = -7
ERR_IO = -8
ERR_UNSUPPORTED = -9
ERR_BUFFER = -10
ERR_CODE_RANGE = -11
ERR_LIMIT = -12

DTYPE_F32, DTYPE_BF16 = 0, 1
FEATURE_MAJOR, TOKEN_MAJOR = 0, 1


class PayloadInfo(C.Structure):
    _fields_ = [("kind", C.c_int32), ("rows", C.c_uint32), ("cols", C.c_uint32),
                ("n_tiles", C.c_uint32), ("tile_rows", C.c_uint16), ("tile_cols", C.c_uint16),
                ("n_atoms", C.c_uint16), ("n_stages", C.c_uint8), ("k_per_stage", C.c_uint8),
                ("stage_decay", C.c_float), ("edge_bytes", C.c_uint32),
                ("off_scales", C.c_uint64), ("off_dict", C.c_uint64), ("off_codes", C.c_uint64),
                ("off_edges", C.c_uint64), ("payload_bytes", C.c_uint64)]


class SegmentHeader(C.Structure):
    _fields_ = [("name", C.c_char_p), ("data_format", C.c_char_p), ("layer_type", C.c_char_p),
                ("original_type", C.c_uint8), ("strategy_id", C.c_uint8),
                ("original_size", C.c_uint64), ("compressed_size", C.c_uint64),
                ("data_offset", C.c_uint64), ("layer_index", C.c_uint32), ("n_dims", C.c_uint32),
                ("dims", C.c_uint32 * 8)]


class MatmulTask(C.Structure):
    _fields_ = [("seg", C.c_void_p), ("x_dev", C.c_void_p), ("x_dtype", C.c_int), ("x_layout", C.c_int),
                ("batch", C.c_size_t), ("y_dev", C.c_void_p), ("y_layout", C.c_int), ("bias_dev", C.c_void_p),
                ("after_task", C.c_int)]


class MatmulHostTask(C.Structure):
    _fields_ = [("seg", C.c_void_p), ("x", C.c_void_p), ("batch", C.c_size_t), ("y", C.c_void_p)]


class DecoderConfig(C.Structure):
    _fields_ = [("n_layers", C.c_uint32), ("hidden", C.c_uint32), ("q_heads", C.c_uint32),
                ("kv_heads", C.c_uint32), ("head_dim", C.c_uint32), ("inter", C.c_uint32),
                ("vocab", C.c_uint32), ("max_seq", C.c_uint32), ("max_batch", C.c_uint32),
                ("rms_eps", C.c_float), ("rope_theta", C.c_float), ("tp_rank", C.c_uint32),
                ("tp_size", C.c_uint32), ("nccl_comm", C.c_void_p), ("kv_dtype", C.c_uint32)]


_P = C.c_void_p
_SZ = C.c_size_t
_F = C.POINTER(C.c_float)

# name -> (restype, argtypes). Every symbol the public header declares.
SIGNATURES = {
    "csdr_last_error": (C.c_char_p, []),
    "csdr_version": (C.c_char_p, []),
    "csdr_context_create": (C.c_int, [C.c_int, _P, C.POINTER(_P)]),
    "csdr_context_destroy": (C.c_int, [_P]),
    "csdr_context_synchronize": (C.c_int, [_P]),
    "csdr_context_stream": (_P, [_P]),
    "csdr_context_launch_count": (C.c_uint64, [_P]),
    "csdr_context_set_wait_limits": (C.c_int, [_P, C.c_uint32, C.c_uint32, C.c_uint32]),
    "csdr_context_wait_selftest": (C.c_int, [_P]),
    "csdr_context_profile": (C.c_int, [_P, C.c_int]),
    "csdr_context_profile_read": (C.c_int, [_P, C.c_int, C.POINTER(C.c_uint64),
                                            C.POINTER(C.c_double)]),
    "csdr_kernel_class_name": (C.c_char_p, [C.c_int]),
    "csdr_context_gemv_trace": (C.c_int, [_P, C.c_int, C.POINTER(C.c_uint64), _SZ, C.POINTER(_SZ)]),
    "csdr_payload_inspect": (C.c_int, [_P, _SZ, C.POINTER(PayloadInfo)]),
    "csdr_segment_create": (C.c_int, [_P, _P, _SZ, C.POINTER(_P)]),
    "csdr_dictionary_create": (C.c_int, [_P, C.c_uint16, C.c_uint16, C.c_uint16, C.c_uint8,
                                         C.c_uint8, _F, _F, C.POINTER(_P)]),
    "csdr_segment_create_shared": (C.c_int, [_P, _P, _SZ, _P, C.POINTER(_P)]),
    "csdr_segment_destroy": (C.c_int, [_P]),
    "csdr_dictionary_destroy": (C.c_int, [_P]),
    "csdr_segment_info": (C.c_int, [_P, C.POINTER(PayloadInfo)]),
    "csdr_segment_shard_rows": (C.c_int, [_P, _P, C.c_uint32, C.c_uint32, C.POINTER(_P)]),
    "csdr_segment_shard_cols": (C.c_int, [_P, _P, C.c_uint32, C.c_uint32, C.POINTER(_P)]),
    "csdr_unpack_codes": (C.c_int, [_P, _P, C.POINTER(C.c_int32), C.POINTER(C.c_int8), _SZ]),
    "csdr_matmul": (C.c_int, [_P, _P, _P, _SZ, _P, C.c_int]),   # float* passed as raw addresses
    "csdr_matmul_device_async": (C.c_int, [_P, _P, _P, C.c_int, C.c_int, _SZ, _P, C.c_int, _P]),
    "csdr_matmul_group_device_async": (C.c_int, [_P, C.POINTER(_P), _SZ, _P, C.c_int, C.c_int, _SZ,
                                                 C.POINTER(_P), C.c_int]),
    "csdr_matmul_queue_device_async": (C.c_int, [_P, C.POINTER(MatmulTask), _SZ]),
    "csdr_matmul_queue": (C.c_int, [_P, C.POINTER(MatmulHostTask), _SZ]),
    "csdr_matmul_rowtiles_noalloc": (C.c_int, [_P, _P, _P, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32,
                                               C.c_uint32, _P, C.c_int, C.c_int, _SZ, _P, C.c_int, _P]),
    "csdr_matmul_rowtiles_noalloc_status": (C.c_int, [_P, C.POINTER(C.c_int)]),
    "csdr_decompress": (C.c_int, [_P, _P, _F, _SZ]),
    "csdr_decompress_device_async": (C.c_int, [_P, _P, _P]),
    "csdr_dequantize": (C.c_int, [_P, C.c_char_p, _P, _SZ, C.c_float, C.c_float, _F, _SZ,
                                  C.POINTER(_SZ)]),
    "csdr_hsdr_encode": (C.c_int, [_P, _F, C.c_uint32, C.c_uint32, C.c_uint16, C.c_uint16, C.c_uint16, C.c_uint8,
                                   C.c_uint8, C.c_float, C.c_uint8, _P, _SZ, C.POINTER(_SZ)]),
    "csdr_encode_codes": (C.c_int, [_P, _F, _SZ, _SZ, _F, C.c_uint16, C.c_uint8, C.c_uint8, _F,
                                    C.POINTER(C.c_uint16), _SZ]),
    "csdr_hsdr_encode_shared": (C.c_int, [_P, C.POINTER(_F), C.POINTER(C.c_uint32), C.POINTER(C.c_uint32), _SZ,
                                          C.c_uint16, C.c_uint16, C.c_uint16, C.c_uint8, C.c_uint8, C.c_float,
                                          C.c_uint8, _P, _SZ, C.POINTER(_SZ), C.POINTER(_P), C.POINTER(_SZ),
                                          C.POINTER(_SZ)]),
    "csdr_dequantize_inference": (C.c_int, [_P, C.c_char_p, _P, _SZ, _SZ, _F, _SZ, C.POINTER(_SZ)]),
    "csdr_archive_open": (C.c_int, [_P, C.c_char_p, C.POINTER(_P)]),
    "csdr_archive_close": (C.c_int, [_P]),
    "csdr_archive_num_segments": (C.c_int, [_P, C.POINTER(_SZ)]),
    "csdr_archive_header_at": (C.c_int, [_P, _SZ, C.POINTER(SegmentHeader)]),
    "csdr_archive_find": (C.c_int, [_P, C.c_char_p, C.POINTER(SegmentHeader)]),
    "csdr_archive_read_payload": (C.c_int, [_P, C.c_char_p, _P, _SZ, C.POINTER(_SZ)]),
    "csdr_archive_load_segment": (C.c_int, [_P, C.c_char_p, _P, _SZ, C.POINTER(_SZ)]),
    "csdr_archive_segment": (C.c_int, [_P, C.c_char_p, C.POINTER(_P)]),
    "csdr_archive_release": (C.c_int, [_P, C.c_char_p]),
    "csdr_archive_resident_bytes": (C.c_int, [_P, C.POINTER(_SZ)]),
    "csdr_archive_matmul_hsdr": (C.c_int, [_P, C.c_char_p, _F, _SZ, _F, _SZ, C.POINTER(_SZ)]),
    "csdr_archive_matmul_for_layer": (C.c_int, [_P, C.c_char_p, _F, _SZ, _F, _SZ, C.POINTER(_SZ)]),
    "csdr_archive_apply_linear": (C.c_int, [_P, C.c_char_p, _F, _SZ, _F, _F, _SZ, C.POINTER(_SZ)]),
    "csdr_hsda_open": (C.c_int, [_P, C.c_char_p, C.POINTER(_P)]),
    "csdr_hsda_close": (C.c_int, [_P]),
    "csdr_hsda_counts": (C.c_int, [_P, C.POINTER(_SZ), C.POINTER(_SZ)]),
    "csdr_hsda_has_segment": (C.c_int, [_P, C.c_char_p]),
    "csdr_hsda_segment": (C.c_int, [_P, C.c_char_p, C.POINTER(_P)]),
    "csdr_hsda_matmul": (C.c_int, [_P, C.c_char_p, _F, _SZ, _F, _SZ, C.POINTER(_SZ), C.c_int]),
    "csdr_hsda_decompress": (C.c_int, [_P, C.c_char_p, _F, _SZ, C.POINTER(_SZ)]),
    "csdr_decoder_create": (C.c_int, [_P, C.POINTER(DecoderConfig), C.POINTER(_P)]),
    "csdr_decoder_destroy": (C.c_int, [_P]),
    "csdr_decoder_reset": (C.c_int, [_P]),
    "csdr_decoder_selection_policy": (C.c_int, [_P, C.c_int, C.c_float]),
    "csdr_decoder_note_generated": (C.c_int, [_P, C.c_uint32, C.POINTER(C.c_int32), _SZ]),
    "csdr_decoder_exchange_export": (C.c_int, [_P, _P]),
    "csdr_decoder_exchange_import": (C.c_int, [_P, _P, _SZ]),
    "csdr_decoder_seek": (C.c_int, [_P, C.c_uint32, C.c_uint32]),
    "csdr_decoder_forward": (C.c_int, [_P, C.c_uint32, C.POINTER(C.c_int32), _SZ, _F, _F]),
    "csdr_decoder_step": (C.c_int, [_P, C.POINTER(C.c_int32), _SZ, C.POINTER(C.c_int32), _F]),
    "csdr_decoder_step_device_async": (C.c_int, [_P, _P, _SZ, _P]),
    "csdr_nccl_unique_id": (C.c_int, [_P]),
    "csdr_nccl_comm_create": (C.c_int, [_P, _P, C.c_int, C.c_int, C.POINTER(_P)]),
    "csdr_nccl_comm_destroy": (C.c_int, [_P]),
}

_lib = None


def load(build_if_missing: bool = False) -> C.CDLL:
    """Load the shared library and attach prototypes. Raises if it is absent."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        if build_if_missing:
            from . import build as _build
            _build.build()
        else:
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m cortexsdr_b200.build` "
                "(nvcc, sm_100a). cortexsdr_b200 has no CPU or PyTorch fallback.")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here = header and library disagree
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib
