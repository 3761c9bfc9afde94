"""The allocation-free entry point, for hosts that may not call cudaMalloc once they run (a
frozen device memory map, a plug-in inside another runtime's pool, an arena that holds it all).
It must give what the ordinary entry point gives, on two calls in a row - the second call
reuses the fixed scratch array with the first call's contents still in it. Collected last, so
a run that stops at the first failure has already been through every other test."""
import ctypes as C

import numpy as np
import pytest

import cortexsdr_b200 as cs
from cortexsdr_b200 import _lib
from tests import synth

pytestmark = pytest.mark.gpu
TOL = 1e-3  # the matmul tolerance used throughout these tests (relative, fp32 accumulate)


def _streams(payload):
    info = cs.inspect_payload(payload)
    p = np.frombuffer(payload, np.uint8)
    n_codes = info.n_tiles * info.n_stages * info.k_per_stage
    scales = p[info.off_scales:info.off_scales + 4 * info.n_stages].view(np.float32).copy()
    atoms = p[info.off_dict:info.off_codes].view(np.float32).copy()
    codes = p[info.off_codes:info.off_codes + 2 * n_codes].view(np.uint16).copy()
    return info, scales, atoms, codes


@pytest.mark.parametrize("rows,cols,atoms,k", [(384, 1024, 128, 6), (200, 4096, 512, 8)])
def test_noalloc_matches_ordinary_entry_point(ctx, rows, cols, atoms, k):
    import torch
    lib = _lib.load()
    payload = synth.hsdr_payload(rows, cols, n_atoms=atoms, k=k, seed=rows)
    info, scales, dictionary, codes = _streams(payload)
    seg = cs.Segment.from_payload(payload, ctx)
    # the caller's own buffers, made before the calls under test; the code buffer is padded to 16 bytes
    d_dict = torch.from_numpy(dictionary).cuda()
    d_scales = torch.from_numpy(scales).cuda()
    padded = np.zeros((codes.size + 7) // 8 * 8, np.uint16)
    padded[:codes.size] = codes
    d_codes = torch.from_numpy(padded.view(np.int16)).cuda()
    rng = np.random.default_rng(1)
    stream = torch.cuda.current_stream().cuda_stream
    for call, batch in enumerate((1, 5)):          # two calls in a row, different widths
        x = torch.from_numpy(rng.normal(0, 1, (batch, cols)).astype(np.float32)).cuda()
        want = torch.empty((batch, rows), device="cuda")
        got = torch.full((batch, rows), float("nan"), device="cuda")
        torch.cuda.synchronize()
        seg.matmul_device(x.data_ptr(), cs.DTYPE_F32, cs.TOKEN_MAJOR, batch, want.data_ptr(), cs.TOKEN_MAJOR)
        ctx.synchronize()
        rc = lib.csdr_matmul_rowtiles_noalloc(
            C.c_void_p(d_dict.data_ptr()), C.c_void_p(d_codes.data_ptr()), C.c_void_p(d_scales.data_ptr()),
            rows, cols, info.n_atoms, info.n_stages, info.k_per_stage, C.c_void_p(x.data_ptr()),
            cs.DTYPE_F32, cs.TOKEN_MAJOR, batch, C.c_void_p(got.data_ptr()), cs.TOKEN_MAJOR,
            C.c_void_p(stream))
        assert rc == 0, lib.csdr_last_error()
        torch.cuda.synchronize()
        w, g = want.cpu().numpy().astype(np.float64), got.cpu().numpy().astype(np.float64)
        assert np.isfinite(g).all(), f"call {call}: output not fully written"
        assert np.abs(g - w).max() <= TOL * np.abs(w).max(), f"call {call}"
        assert np.linalg.norm(g - w) <= TOL * np.linalg.norm(w), f"call {call}"


def test_noalloc_rejects_sizes_beyond_its_scratch(ctx):
    import torch
    lib = _lib.load()
    buf = torch.zeros(4096, device="cuda")
    args = lambda atoms, cols: (C.c_void_p(buf.data_ptr()), C.c_void_p(buf.data_ptr()), C.c_void_p(buf.data_ptr()),
                                8, cols, atoms, 3, 8, C.c_void_p(buf.data_ptr()), cs.DTYPE_F32, cs.TOKEN_MAJOR, 1,
                                C.c_void_p(buf.data_ptr()), cs.TOKEN_MAJOR, None)
    assert lib.csdr_matmul_rowtiles_noalloc(*args(4097, 64)) == _lib.ERR_LIMIT
    assert b"4096" in lib.csdr_last_error()
    assert lib.csdr_matmul_rowtiles_noalloc(*args(64, 66)) == _lib.ERR_LIMIT
