"""Tensor-parallel host logic on CPU ranks (gloo, world size 2): each rank takes its slice of
the code stream of a compressed weight, runs the oracle on it, and the rank-major
all-gather followed by the shard-interleave reproduces the unsharded result. This is the
index arithmetic csdr_segment_shard_rows and the decoder's logits rejoin rely on. A second case
covers the column-sharded projection (csdr_segment_shard_cols; the decoder's output and down
projections) in its most general form: dictionary columns and input width sliced per rank,
partial projections and per-token sums of squares added up with one all-reduce, RMS
normalisation applied behind the projection, each rank gathering its own output rows."""
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
        from tests import synth
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


def col_shard_payload(pay: bytes, c0: int, c1: int) -> bytes:
    """Input columns [c0, c1) of a 1-D row-tile HSDR payload as a payload of its own (same codes)."""
    hdr = list(struct.unpack("<4sIIIIHHHBBfI", pay[:36]))
    _, _, rows, cols, n_tiles, tr, tc, K, S, k, _, edge = hdr
    assert tr == 1 and tc == cols and edge == 0
    off_dict = 36 + 4 * S
    off_codes = off_dict + 4 * K * cols
    D = np.frombuffer(pay, np.float32, K * cols, off_dict).reshape(K, cols)
    hdr[3] = c1 - c0
    hdr[6] = c1 - c0
    return (struct.pack("<4sIIIIHHHBBfI", *hdr) + pay[36:off_dict]
            + np.ascontiguousarray(D[:, c0:c1]).tobytes() + pay[off_codes:])


def _tp_worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from tests import synth
        from oracle.bindings import Oracle
        orc = Oracle()
        R, C, T, K, eps = 96, 64, 5, 16, 1e-6
        pay = synth.hsdr_payload(R, C, n_atoms=K, k=3, seed=21)
        rng = np.random.default_rng(8)
        h = rng.normal(0, 1, (T, C)).astype(np.float32)           # hidden states, token-major
        w = rng.normal(1, 0.1, C).astype(np.float32)              # norm weight
        Cl, Rl = C // world, R // world
        c0, r0 = rank * Cl, rank * Rl
        # this rank: its slice of the hidden width, of the dictionary columns and of the code rows
        mine = shard_payload(col_shard_payload(pay, c0, c0 + Cl), r0, r0 + Rl)
        hdr = struct.unpack("<4sIIIIHHHBBfI", mine[:36])
        S, k = hdr[8], hdr[9]
        gam = np.frombuffer(mine, np.float32, S, 36)
        D = np.frombuffer(mine, np.float32, K * Cl, 36 + 4 * S).reshape(K, Cl)
        codes = np.frombuffer(mine, np.uint16, Rl * S * k, 36 + 4 * S + 4 * K * Cl).reshape(Rl, S, k)
        hs = h[:, c0:c0 + Cl]
        block = np.concatenate([(hs.astype(np.float64) ** 2).sum(1), (D.astype(np.float64) @ (hs * w[c0:c0 + Cl]).T.astype(np.float64)).ravel()])
        t = torch.from_numpy(block)
        dist.all_reduce(t)                                         # sums of squares | projection, one collective
        block = t.numpy()
        inv = 1.0 / np.sqrt(block[:T] / C + eps)
        dx = block[T:].reshape(K, T)
        idx, sign = codes & 0x7FFF, np.where(codes >> 15, -1.0, 1.0)
        y_local = np.einsum("rsk,rskt->rt", sign * gam[None, :, None], dx[idx]) * inv[None, :]     # (Rl, T)
        parts = [torch.empty(T, Rl, dtype=torch.float64) for _ in range(world)]
        dist.all_gather(parts, torch.from_numpy(np.ascontiguousarray(y_local.T)))
        full = unshard(torch.stack(parts).numpy())
        # what one rank computes: rms-normalise, then the oracle's matmul on the whole payload
        hn = (h / np.sqrt((h.astype(np.float64) ** 2).mean(1, keepdims=True) + eps) * w).astype(np.float32)
        want = orc.matmul(pay, np.ascontiguousarray(hn.T), T).T
        q.put((rank, float(np.abs(full - want).max() / np.abs(want).max())))
    finally:
        dist.destroy_process_group()


def test_column_sharded_projection_with_folded_norm_on_two_cpu_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 31500 + os.getpid() % 2000
    procs = [ctx.Process(target=_tp_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    res = sorted(q.get(timeout=5) for _ in range(2))
    assert [r[0] for r in res] == [0, 1]
    assert all(r[1] < 1e-5 for r in res), res


def test_unshard_index_map():
    P, T, W = 3, 4, 5
    staged = np.arange(P * T * W, dtype=np.float32).reshape(P, T, W)
    out = unshard(staged)
    for p in range(P):
        for t in range(T):
            assert np.array_equal(out[t, p * W:(p + 1) * W], staged[p, t])
