"""The reference's own C SDK names (api/cortex_sdk.h:110-232), called the way a program
written against that header calls them: CortexError returned BY VALUE, opaque handles checked
against a registry, caller-allocated output buffers with the too-small convention
(api/cortex_sdk.cpp:1873-1876), strings released with cortex_free_string. Archives are the
reference-written fixtures of the routing and end-to-end tests."""
import ctypes as C
import json
import os

import numpy as np
import pytest

from conftest import GOLDEN

pytestmark = pytest.mark.gpu

# api/cortex_sdk.cpp:56-64 - a relinked caller compares against these numbers
CORTEX_SUCCESS, INVALID_ARGUMENT, FILE_IO, MEMORY, UNSUPPORTED_FORMAT = 0, -1, -2, -3, -4
DECOMPRESSION, INFERENCE, UNKNOWN = -6, -7, -99


class CortexError(C.Structure):                      # api/c_api.hpp:26-29
    _fields_ = [("message", C.c_char_p), ("code", C.c_int)]


@pytest.fixture(scope="module")
def sdk(lib):
    H, F, SZ = C.c_void_p, C.POINTER(C.c_float), C.c_size_t
    sig = {
        "cortex_inference_engine_create": [C.c_char_p, C.POINTER(H)],
        "cortex_inference_engine_set_batch_size": [H, SZ],
        "cortex_inference_engine_enable_dropout": [H, C.c_int],
        "cortex_inference_engine_set_mode": [H, C.c_int],
        "cortex_inference_engine_init_memory_pool": [H, SZ],
        "cortex_inference_engine_enable_aggressive_memory": [H, C.c_int],
        "cortex_inference_engine_get_memory_usage": [H, C.POINTER(SZ)],
        "cortex_inference_engine_enable_layer_prefetch": [H, C.c_int],
        "cortex_inference_engine_get_last_run_stats_json": [H, C.POINTER(C.c_void_p)],
        "cortex_inference_engine_run": [H, F, SZ, F, SZ, C.POINTER(SZ)],
        "cortex_inference_engine_run_layer": [H, C.c_char_p, F, SZ, F, SZ, C.POINTER(SZ)],
        "cortex_inference_engine_generate_text": [H, C.c_char_p, C.c_int, C.POINTER(C.c_void_p)],
        "cortex_inference_engine_free": [H],
    }
    for name, args in sig.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = CortexError, args
    lib.cortex_free_string.restype, lib.cortex_free_string.argtypes = None, [C.c_void_p]
    lib.cortex_sdk_version.restype = C.c_char_p
    return lib


def fp(a):
    return a.ctypes.data_as(C.POINTER(C.c_float))


def open_engine(sdk, path):
    h = C.c_void_p()
    err = sdk.cortex_inference_engine_create(path.encode(), C.byref(h))
    assert (err.code, err.message) == (CORTEX_SUCCESS, None)
    return h


def take_string(sdk, p):
    s = C.string_at(p).decode()
    sdk.cortex_free_string(p)
    return s


def test_run_layer_stats_and_buffer_convention(sdk, golden):
    g = golden("archive_e2e.npz")
    h = open_engine(sdk, os.path.join(GOLDEN, "archive_e2e.sdr"))
    x = np.ascontiguousarray(g["x"].T)                       # token-major (4 x 512)
    y = np.zeros((4, 128), np.float32)
    n = C.c_size_t(0)
    err = sdk.cortex_inference_engine_run_layer(h, b"test.layer", fp(x), x.size, fp(y), y.size, C.byref(n))
    assert err.code == CORTEX_SUCCESS and err.message is None and n.value == 4 * 128
    assert np.abs(y.T - g["y_fused"]).max() < 1e-3           # the reference's own fused result
    js = C.c_void_p()
    assert sdk.cortex_inference_engine_get_last_run_stats_json(h, C.byref(js)).code == CORTEX_SUCCESS
    stats = json.loads(take_string(sdk, js))
    assert stats["layers"][0]["name"] == "test.layer" and stats["layers"][0]["used_compressed"] is True
    assert stats["layers"][0]["output_size"] == 512 and stats["total_ms"] > 0
    # too small a buffer: the needed element count comes back with CORTEX_ERROR_MEMORY
    small = np.zeros(100, np.float32)
    err = sdk.cortex_inference_engine_run_layer(h, b"test.layer.weight", fp(x), x.size, fp(small), small.size, C.byref(n))
    assert err.code == MEMORY and n.value == 512 and b"too small" in err.message
    # argument errors
    err = sdk.cortex_inference_engine_run_layer(h, b"no.such.layer", fp(x), x.size, fp(y), y.size, C.byref(n))
    assert err.code == INFERENCE and b"not found" in err.message
    err = sdk.cortex_inference_engine_run_layer(h, None, fp(x), x.size, fp(y), y.size, C.byref(n))
    assert err.code == INVALID_ARGUMENT
    err = sdk.cortex_inference_engine_run_layer(h, b"test.layer", fp(x), 511, fp(y), y.size, C.byref(n))
    assert err.code == INVALID_ARGUMENT
    used = C.c_size_t(0)
    assert sdk.cortex_inference_engine_get_memory_usage(h, C.byref(used)).code == CORTEX_SUCCESS
    assert used.value >= 64 * 512 * 4                        # at least the dictionary is resident
    assert sdk.cortex_inference_engine_free(h).code == CORTEX_SUCCESS
    # a freed handle is refused by every call, as the registry lookup of the reference does
    err = sdk.cortex_inference_engine_run_layer(h, b"test.layer", fp(x), x.size, fp(y), y.size, C.byref(n))
    assert err.code == INVALID_ARGUMENT and err.message == b"Invalid handle"
    assert sdk.cortex_inference_engine_free(h).code == INVALID_ARGUMENT
    assert sdk.cortex_inference_engine_set_batch_size(h, 2).code == INVALID_ARGUMENT


def test_create_errors(sdk):
    h = C.c_void_p()
    err = sdk.cortex_inference_engine_create(b"/nonexistent/model.sdr", C.byref(h))
    assert err.code == FILE_IO and err.message
    assert sdk.cortex_inference_engine_create(None, C.byref(h)).code == INVALID_ARGUMENT
    assert sdk.cortex_sdk_version().startswith(b"1.0.0")


def test_run_chains_the_linear_layers_and_settings_act(sdk, golden):
    g = golden("routing.npz")
    h = open_engine(sdk, os.path.join(GOLDEN, "routing.sdr"))
    # layer.hsdr.weight (256 x 512) then layer.raw.weight (96 x 256); the 1-D norm vector is no layer
    x = np.ascontiguousarray(g["x_hsdr"].T)                  # (2 x 512)
    out = np.zeros((2, 96), np.float32)
    n = C.c_size_t(0)
    assert sdk.cortex_inference_engine_enable_layer_prefetch(h, 1).code == CORTEX_SUCCESS
    used = C.c_size_t(0)
    sdk.cortex_inference_engine_get_memory_usage(h, C.byref(used))
    assert used.value >= 64 * 512 * 4                        # prefetch uploaded the HSDR image
    assert sdk.cortex_inference_engine_set_batch_size(h, 3).code == CORTEX_SUCCESS
    err = sdk.cortex_inference_engine_run(h, fp(x), x.size, fp(out), out.size, C.byref(n))
    assert err.code == INVALID_ARGUMENT and b"batch size" in err.message
    assert sdk.cortex_inference_engine_set_batch_size(h, 2).code == CORTEX_SUCCESS
    err = sdk.cortex_inference_engine_run(h, fp(x), x.size, fp(out), out.size, C.byref(n))
    assert err.code == CORTEX_SUCCESS and n.value == 2 * 96
    import cortexsdr_b200 as cs
    ld = cs.SDRModelLoader(os.path.join(GOLDEN, "routing.sdr"), index_only=True)
    w_raw = ld.loadSegmentByName("layer.raw.weight").view(np.float32).reshape(96, 256)
    want = (w_raw.astype(np.float64) @ g["y_hsdr"].astype(np.float64)).T     # reference's fused y through the raw layer
    assert np.abs(out - want).max() < 1e-3
    js = C.c_void_p()
    sdk.cortex_inference_engine_get_last_run_stats_json(h, C.byref(js))
    stats = json.loads(take_string(sdk, js))
    assert [l["name"] for l in stats["layers"]] == ["layer.hsdr.weight", "layer.raw.weight"]
    assert [l["used_compressed"] for l in stats["layers"]] == [True, False]
    # too-small buffer on the whole run
    tiny = np.zeros(10, np.float32)
    err = sdk.cortex_inference_engine_run(h, fp(x), x.size, fp(tiny), tiny.size, C.byref(n))
    assert err.code == MEMORY and n.value == 192
    # aggressive memory: nothing stays resident behind a run
    assert sdk.cortex_inference_engine_enable_aggressive_memory(h, 1).code == CORTEX_SUCCESS
    assert sdk.cortex_inference_engine_run(h, fp(x), x.size, fp(out), out.size, C.byref(n)).code == CORTEX_SUCCESS
    sdk.cortex_inference_engine_get_memory_usage(h, C.byref(used))
    assert used.value == 0
    assert np.abs(out - want).max() < 1e-3
    # training mode with dropout has no implementation here
    sdk.cortex_inference_engine_set_mode(h, 1)
    sdk.cortex_inference_engine_enable_dropout(h, 1)
    assert sdk.cortex_inference_engine_run(h, fp(x), x.size, fp(out), out.size, C.byref(n)).code == UNSUPPORTED_FORMAT
    assert sdk.cortex_inference_engine_free(h).code == CORTEX_SUCCESS


def test_generate_text_on_token_ids(sdk, ctx, oracle, tmp_path):
    """The generation loop of api/cortex_sdk.cpp:1951-2054 with token ids in place of text: the
    decoder shape is discovered from the archive, every step's pick follows
    select_best_from_logits at temperature 0.8 over the tokens generated so far."""
    import cortexsdr_b200 as cs
    from tests import synth
    # a head size the reference's discovery finds: it tries 128, 64, 256, 32, 16 in that order on
    # the q/k/v widths (api/cortex_sdk.cpp:1335-1349), so 128-wide q and 64-wide k/v mean heads of 64
    cfg = dict(n_layers=2, hidden=128, q_heads=2, kv_heads=1, head_dim=64, inter=256, vocab=300)
    path = str(tmp_path / "gen.sdr")
    synth.decoder_archive(path, **cfg, k=3, seed=11, n_atoms=32, kv_atoms=16)
    prompt = [5, 17, 250, 3, 99]
    # what the loop must produce, from this library's decoder driven step by step with the
    # oracle's restatement of the selection rule (the decoder itself is checked against the
    # oracle in test_gpu_decoder.py); eps and theta are the reference's defaults
    dec = cs.Decoder(cs.SDRModelLoader(path, ctx), **cfg, max_seq=64, rms_eps=1e-5, rope_theta=1e6)
    logits, _ = dec.forward(np.array(prompt))
    want, history = [], []
    for _ in range(6):
        tok = oracle.select_best_from_logits(logits, history, 0.8)
        want.append(tok)
        history.append(tok)
        logits, _ = dec.forward(np.array([tok]))
    h = open_engine(sdk, path)
    out = C.c_void_p()
    err = sdk.cortex_inference_engine_generate_text(h, b"5 17 250 3 99", 6, C.byref(out))
    assert err.code == CORTEX_SUCCESS, err.message
    assert [int(t) for t in take_string(sdk, out).split()] == want
    err = sdk.cortex_inference_engine_generate_text(h, b"hello world", 4, C.byref(out))
    assert err.code == INVALID_ARGUMENT and b"token ids" in err.message
    err = sdk.cortex_inference_engine_generate_text(h, b"5 9999", 4, C.byref(out))
    assert err.code == INVALID_ARGUMENT                      # id outside the vocabulary
    assert sdk.cortex_inference_engine_free(h).code == CORTEX_SUCCESS
    # an archive without transformer blocks says so
    h2 = open_engine(sdk, os.path.join(GOLDEN, "routing.sdr"))
    err = sdk.cortex_inference_engine_generate_text(h2, b"1 2 3", 2, C.byref(out))
    assert err.code == INFERENCE
    sdk.cortex_inference_engine_free(h2)
