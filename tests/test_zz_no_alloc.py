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


@pytest.mark.parametrize("batch,dtype,layout", [(21, "bf16", "token"), (7, "f32", "feature"), (40, "f32", "token")])
def test_noalloc_wide_batches_layouts_and_bf16(ctx, oracle, batch, dtype, layout):
    # more than sixteen tokens walks the chunk loop with the 16-wide tile; bf16 and the
    # reference's feature-major layout go through the generic activation reader
    import torch
    lib = _lib.load()
    rows, cols = 264, 1536
    payload = synth.hsdr_payload(rows, cols, n_atoms=192, k=5, seed=77)
    info, scales, dictionary, codes = _streams(payload)
    d_dict, d_scales = torch.from_numpy(dictionary).cuda(), torch.from_numpy(scales).cuda()
    padded = np.zeros((codes.size + 7) // 8 * 8, np.uint16)
    padded[:codes.size] = codes
    d_codes = torch.from_numpy(padded.view(np.int16)).cuda()
    xh = np.random.default_rng(3).normal(0, 1, (batch, cols)).astype(np.float32)
    xt = torch.from_numpy(xh).cuda()
    if dtype == "bf16":
        xt = xt.to(torch.bfloat16)
        xh = xt.float().cpu().numpy()
    x_layout = cs.TOKEN_MAJOR
    if layout == "feature":
        xt, x_layout = xt.t().contiguous(), cs.FEATURE_MAJOR
    got = torch.full((rows, batch) if layout == "feature" else (batch, rows), float("nan"), device="cuda")
    rc = lib.csdr_matmul_rowtiles_noalloc(
        C.c_void_p(d_dict.data_ptr()), C.c_void_p(d_codes.data_ptr()), C.c_void_p(d_scales.data_ptr()),
        rows, cols, info.n_atoms, info.n_stages, info.k_per_stage, C.c_void_p(xt.data_ptr()),
        cs.DTYPE_BF16 if dtype == "bf16" else cs.DTYPE_F32, x_layout, batch, C.c_void_p(got.data_ptr()), x_layout,
        C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, lib.csdr_last_error()
    torch.cuda.synchronize()
    g = got.cpu().numpy().astype(np.float64)
    if layout == "token":
        g = g.T
    w = oracle.matmul(payload, np.ascontiguousarray(xh.T), batch).astype(np.float64)
    assert np.isfinite(g).all()
    assert np.abs(g - w).max() <= TOL * np.abs(w).max()
    bad = C.c_int(-1)
    assert lib.csdr_matmul_rowtiles_noalloc_status(C.c_void_p(torch.cuda.current_stream().cuda_stream), C.byref(bad)) == 0
    assert bad.value == 0


def test_noalloc_skips_and_reports_a_code_beyond_the_dictionary(ctx, oracle):
    # raw device streams are not checked on the host: a code naming atom >= n_atoms must read
    # nothing out of bounds, add nothing to its row, and be reported by the status query
    import torch
    lib = _lib.load()
    rows, cols = 96, 512
    payload = synth.hsdr_payload(rows, cols, n_atoms=64, k=4, seed=5)
    info, scales, dictionary, codes = _streams(payload)
    slots = info.n_stages * info.k_per_stage
    victim = 10 * slots + 3
    broken = codes.copy()
    broken[victim] = (broken[victim] & 0x8000) | 0x7FFF        # atom 32767 of 64
    d_dict, d_scales = torch.from_numpy(dictionary).cuda(), torch.from_numpy(scales).cuda()
    padded = np.zeros((broken.size + 7) // 8 * 8, np.uint16)
    padded[:broken.size] = broken
    d_codes = torch.from_numpy(padded.view(np.int16)).cuda()
    xh = np.random.default_rng(4).normal(0, 1, (2, cols)).astype(np.float32)
    xt = torch.from_numpy(xh).cuda()
    got = torch.full((2, rows), float("nan"), device="cuda")
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert lib.csdr_matmul_rowtiles_noalloc(
        C.c_void_p(d_dict.data_ptr()), C.c_void_p(d_codes.data_ptr()), C.c_void_p(d_scales.data_ptr()),
        rows, cols, info.n_atoms, info.n_stages, info.k_per_stage, C.c_void_p(xt.data_ptr()), cs.DTYPE_F32,
        cs.TOKEN_MAJOR, 2, C.c_void_p(got.data_ptr()), cs.TOKEN_MAJOR, st) == 0
    bad = C.c_int(0)
    assert lib.csdr_matmul_rowtiles_noalloc_status(st, C.byref(bad)) == _lib.ERR_CODE_RANGE
    assert bad.value == 1
    g = got.cpu().numpy().T
    assert np.isfinite(g).all()
    # every other row is untouched by the bad code; row 10 lacks exactly that code's term
    w = oracle.matmul(payload, np.ascontiguousarray(xh.T), 2)
    others = np.arange(rows) != 10
    assert np.abs(g[others] - w[others]).max() <= TOL * np.abs(w).max()
    dx = dictionary.reshape(info.n_atoms, cols) @ xh.T
    c = int(codes[victim])
    term = (-1.0 if c & 0x8000 else 1.0) * scales[3 // info.k_per_stage] * dx[c & 0x7FFF]
    assert np.abs(g[10] - (w[10] - term)).max() <= TOL * np.abs(w).max()
    assert lib.csdr_matmul_rowtiles_noalloc_status(st, C.byref(bad)) == 0 and bad.value == 0   # cleared


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
