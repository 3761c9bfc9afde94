"""Tensor-parallel host logic on CPU ranks (gloo, world size 2): each rank takes its slice of
the code stream of a compressed weight, runs the oracle on it, and the rank-major
all-gather followed by the shard-interleave reproduces the unsharded result. This is the
index arithmetic csdr_segment_shard_rows and the decoder's rejoin step rely on."""
import os
import struct
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def shard_payload(pay: bytes, r0: int, r1: int) -> bytes:
    """Rows [r0, r1) of a 1-D row-tile HSDR payload as a payload of its own (same dictionary)."""
    hdr = list(struct.unpack("<4sIIIIHHHBBfI", pay[:36]))
    _, _, rows, cols, n_tiles, tr, tc, K, S, k, _, edge = hdr
    assert tr == 1 and tc == cols and edge == 0
    off_codes = 36 + 4 * S + 4 * K * cols
    slots = S * k
    hdr[2] = hdr[4] = r1 - r0
    return (struct.pack("<4sIIIIHHHBBfI", *hdr) + pay[36:off_codes]
            + pay[off_codes + 2 * r0 * slots: off_codes + 2 * r1 * slots])


def unshard(staged: np.ndarray) -> np.ndarray:
    """(P, T, W) rank-major -> (T, P*W) token-major: the device unshard kernel's index map."""
    P, T, W = staged.shape
    return np.ascontiguousarray(staged.transpose(1, 0, 2)).reshape(T, P * W)


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from cortexsdr_b200 import synth
        from oracle.bindings import Oracle
        orc = Oracle()
        R, C, T = 96, 64, 5
        pay = synth.hsdr_payload(R, C, n_atoms=16, k=3, seed=11)
        x = np.random.default_rng(4).normal(0, 1, (T, C)).astype(np.float32)      # token-major
        W = R // world
        local = orc.matmul(shard_payload(pay, rank * W, (rank + 1) * W), np.ascontiguousarray(x.T), T).T
        parts = [torch.empty(T, W) for _ in range(world)]
        dist.all_gather(parts, torch.from_numpy(np.ascontiguousarray(local)))
        full = unshard(torch.stack(parts).numpy())
        want = orc.matmul(pay, np.ascontiguousarray(x.T), T).T
        q.put((rank, bool(np.array_equal(full, want)), float(np.abs(full - want).max())))
    finally:
        dist.destroy_process_group()


def test_row_shards_rejoin_on_two_cpu_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    res = sorted(q.get(timeout=5) for _ in range(2))
    assert [r[0] for r in res] == [0, 1]
    assert all(r[1] for r in res), res


def test_unshard_index_map():
    P, T, W = 3, 4, 5
    staged = np.arange(P * T * W, dtype=np.float32).reshape(P, T, W)
    out = unshard(staged)
    for p in range(P):
        for t in range(T):
            assert np.array_equal(out[t, p * W:(p + 1) * W], staged[p, t])
