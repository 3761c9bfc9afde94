"""Tensor-parallel decoder on two GPUs: every compressed weight sharded by output rows (codes)
and input columns (dictionary), the ranks' partial projections summed with one NCCL all-reduce
per group of linears, logits equal to the single-GPU decoder's within the matmul tolerance.
Needs two B200s; skipped otherwise. Ranks run as child processes, one per GPU, with in-switch
reduction off (NCCL_NVLS_ENABLE=0)."""
import os
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CFG = dict(n_layers=2, hidden=128, q_heads=4, kv_heads=2, head_dim=32, inter=256, vocab=300)


LLAMA_W = dict(n_layers=1, hidden=4096, q_heads=32, kv_heads=32, head_dim=128, inter=11008, vocab=32000)


def _rank_wide(rank, world, port, path, q):
    """The 7B-shaped widths (one block): sixteen sequences with different prefilled contexts step
    together on two ranks - the 16-token exchange through peer memory - and on one."""
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch
    import torch.distributed as dist
    import cortexsdr_b200 as cs
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        ctx = cs.Context(rank)
        ids = [cs.nccl_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)
        comm = cs.NcclComm(ctx, ids[0], rank, world)
        ld = cs.SDRModelLoader(path, ctx)

        def all_gather(b):
            out = [None] * world
            dist.all_gather_object(out, b)
            return out
        rng = np.random.default_rng(8)
        lens = [3, 9, 5, 12, 1, 7, 4, 10, 2, 8, 6, 11, 3, 5, 9, 7]
        prompts = [rng.integers(0, LLAMA_W["vocab"], n) for n in lens]
        new = rng.integers(0, LLAMA_W["vocab"], 16)

        def run(dec):
            for s_, p_ in enumerate(prompts):
                dec.forward(p_, seq=s_, want_logits=False)
            nxt, lg = dec.step(new, want_logits=True)
            nxt2, lg2 = dec.step(nxt, want_logits=True)
            ctx.synchronize()
            return dict(nxt=[int(t) for t in nxt], lg=lg, nxt2=[int(t) for t in nxt2], lg2=lg2)
        os.environ["CSDR_TP_EXCHANGE"] = "peer"
        out = {}
        dec = cs.Decoder(ld, **LLAMA_W, max_seq=32, max_batch=16, rms_eps=1e-5, comm=comm, all_gather=all_gather)
        out["tp"] = run(dec)
        dec.close()
        if rank == 0:
            single = cs.Decoder(ld, **LLAMA_W, max_seq=32, max_batch=16, rms_eps=1e-5)
            out["single"] = run(single)
            single.close()
        dist.barrier()
        comm.close()
        q.put((rank, out))
    finally:
        dist.destroy_process_group()


def _rank(rank, world, port, path, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch
    import torch.distributed as dist
    import cortexsdr_b200 as cs
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)   # host-side plumbing only
    try:
        ctx = cs.Context(rank)
        ids = [cs.nccl_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)
        comm = cs.NcclComm(ctx, ids[0], rank, world)
        ld = cs.SDRModelLoader(path, ctx)
        def all_gather(b):
            out = [None] * world
            dist.all_gather_object(out, b)
            return out

        out = {}
        tokens = np.random.default_rng(0).integers(0, CFG["vocab"], 12)
        long_tokens = np.random.default_rng(1).integers(0, CFG["vocab"], 21)
        # "nccl": no IPC handles given, partial projections summed by ncclAllReduce; "peer": pushed
        # into peer memory by the projection and summed by the reduce launch (steps of at most 16
        # tokens; the 21-token pass still takes NCCL)
        os.environ["CSDR_TP_EXCHANGE"] = "peer"      # explicit, whatever the default
        for tag, kw in (("nccl", {}), ("peer", dict(all_gather=all_gather))):
            dec = cs.Decoder(ld, **CFG, max_seq=64, max_batch=2, rms_eps=1e-6, comm=comm, **kw)
            logits, hidden = dec.forward(tokens, want_hidden=True)
            nxt, step_logits = dec.step([int(logits.argmax())], want_logits=True)
            dec.reset()
            wide_logits, _ = dec.forward(long_tokens)
            ctx.synchronize()
            out[tag] = dict(logits=logits, hidden=hidden, step=step_logits[0], nxt=int(nxt[0]), wide=wide_logits)
            dec.close()
        if rank == 0:
            single = cs.Decoder(ld, **CFG, max_seq=64, max_batch=2, rms_eps=1e-6)
            l1, h1 = single.forward(tokens, want_hidden=True)
            n1, s1 = single.step([int(l1.argmax())], want_logits=True)
            single.reset()
            w1, _ = single.forward(long_tokens)
            out["single"] = dict(logits=l1, hidden=h1, step=s1[0], nxt=int(n1[0]), wide=w1)
        dist.barrier()
        comm.close()
        q.put((rank, out))
    finally:
        dist.destroy_process_group()


def test_two_rank_decoder_matches_single_gpu(tmp_path):
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from tests import synth
    path = str(tmp_path / "tp.sdr")
    synth.decoder_archive(path, **CFG, n_atoms=128, k=3, kv_atoms=128, seed=7)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29600 + os.getpid() % 1000
    procs = [ctx.Process(target=_rank, args=(r, 2, port, path, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=300) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    r0, r1 = res[0], res[1]
    one = r0["single"]
    for tag in ("nccl", "peer"):
        got = r0[tag]
        assert np.abs(got["logits"] - one["logits"]).max() < 1e-3, tag
        assert np.abs(got["hidden"] - one["hidden"]).max() < 1e-3, tag
        assert np.abs(got["step"] - one["step"]).max() < 1e-3 and got["nxt"] == one["nxt"], tag
        assert np.abs(got["wide"] - one["wide"]).max() < 1e-3, tag
        assert np.array_equal(got["logits"], r1[tag]["logits"]), tag      # same result on every rank
        assert np.array_equal(got["step"], r1[tag]["step"]), tag


def test_two_rank_decoder_at_the_7b_widths(tmp_path):
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from tests import synth
    path = str(tmp_path / "tpw.sdr")
    synth.decoder_archive(path, **LLAMA_W, n_atoms=512, k=8, seed=7)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29700 + os.getpid() % 1000
    procs = [ctx.Process(target=_rank_wide, args=(r, 2, port, path, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=600) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    tp, one = res[0]["tp"], res[0]["single"]
    assert np.isfinite(tp["lg"]).all() and np.isfinite(tp["lg2"]).all()
    assert np.abs(tp["lg"] - one["lg"]).max() < 2e-2 and tp["nxt"] == one["nxt"]
    assert np.abs(tp["lg2"] - one["lg2"]).max() < 2e-2 and tp["nxt2"] == one["nxt2"]
    assert np.array_equal(tp["lg"], res[1]["tp"]["lg"])                   # every rank holds the same logits
