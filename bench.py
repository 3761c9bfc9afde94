#!/usr/bin/env python
"""Benchmark of the HSDR compressed-weight matmul on B200.

    python bench.py --gpus N --steps K --warmup W            # this library
    python bench.py --impl reference --steps K --warmup W    # the reference's CPU code

Workload (N=1): the MLP-projection case — W 11008x4096, HSDR 1-D row tiles (K=512, 3x8),
decode GEMV at batch 1. One step = one pass over SEGS distinct device-resident copies of
the compressed weight (SEGS * payload > 2 * L2, so every pass reads HBM, not L2), issued as ONE
list of independent products (csdr_matmul_queue_device_async: one persistent launch).
`value` = algorithmic compressed bytes processed per second with inputs resident in HBM;
`e2e` = the same list through the host-buffer C-ABI call (csdr_matmul_queue: H2D of x and D2H of y
inside the timed region). The same pass as a chain of single dependent launches, the grouped
launches and the M sweep {1, 8, 64, 512} are reported beside it.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

R, C, K, S, KPS = 11008, 4096, 512, 3, 8
SEGS = 32                      # 32 * 8.9 MB = 285 MB  >  2 * 126 MB L2
CACHE = os.path.join(os.environ.get("TMPDIR", "/tmp"), "cortexsdr_b200_bench")


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


def workload_payload():
    """The 11008x4096 weight, N(0, 0.02) seed 2, encoded by the reference's own encoder
    (forRow1D, ksvd_iters=0) when oracle/_ref is present, else a synthetic stand-in."""
    os.makedirs(CACHE, exist_ok=True)
    path = os.path.join(CACHE, f"w{R}x{C}_k{K}.hsdr")
    if os.path.exists(path):
        return open(path, "rb").read(), open(path + ".src").read()
    from oracle.bindings import SEG_FEED_FORWARD, Reference, Segment, cfg_row1d
    if Reference.available():
        W = np.random.default_rng(2).normal(0, 0.02, (R, C)).astype(np.float32)
        cfg = cfg_row1d(C, K, KPS, ksvd_iters=0)
        pay = Reference().compress(Segment("blk.0.ffn_gate.weight", W, (R, C), SEG_FEED_FORWARD), cfg, cfg)
        src = "reference encoder (forRow1D, ksvd_iters=0)"
    else:
        from tests import synth
        pay = synth.hsdr_payload(R, C, n_atoms=K, n_stages=S, k=KPS, seed=2)
        src = "synthetic payload (reference encoder not built here)"
    with open(path + ".tmp", "wb") as f:
        f.write(pay)
    os.replace(path + ".tmp", path)
    open(path + ".src", "w").write(src)
    return pay, src


def alg_bytes(payload_len: int, m: int, x_bytes: int = 4) -> int:
    """payload + activations + outputs, the algorithmic traffic of one matmul."""
    return payload_len + C * m * x_bytes + R * m * 4


class ClockSampler:
    """nvidia-smi clocks and throttle reasons during the timed region."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.rows, self.proc, self.index = [], None, index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *a):
        if self.proc:
            time.sleep(0.15)
            self.proc.terminate()
            self.t.join(timeout=2)

    def summary(self):
        sm = [float(r[0]) for r in self.rows if r and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) > 1 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 7 for n, v in zip(names, r[3:7]) if v == "Active"})
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def cpu_baseline(pay: bytes, iters: int = 7):
    """The reference's matmulRowMajor (single-threaded by construction) on the same payload,
    batch 1, payload bytes already in memory; falls back to the C oracle port."""
    from oracle.bindings import Oracle, Reference
    x = np.random.default_rng(3).normal(0, 1, (C, 1)).astype(np.float32)
    if Reference.available():
        sec, _ = Reference().matmul_timed(pay, x, 1, R, iters=iters)
        kind = "reference"
    else:
        orc = Oracle()
        ts = []
        for _ in range(iters):
            t0 = time.perf_counter()
            orc.matmul(pay, x, 1)
            ts.append(time.perf_counter() - t0)
        sec, kind = statistics.median(ts), "port"
    out = {"value": alg_bytes(len(pay), 1) / sec / 1e9, "unit": "GB/s", "cores": 1, "kind": kind,
           "sample": f"1 of {SEGS} segments, batch 1, median of {iters} calls after 2 warm-ups",
           "ms_per_matmul": sec * 1e3}
    if Reference.available():
        # the reference's other route: decompress() then the dense product (linear_forward: one
        # std::thread per hardware thread at batch 1, no BLAS in this build)
        try:
            sec2, _ = Reference().decompress_dense_timed(pay, R, C, np.ascontiguousarray(x.T), 1, iters=3)
            model = ""
            try:
                for line in open("/proc/cpuinfo"):
                    if line.startswith("model name"):
                        model = line.split(":", 1)[1].strip()
                        break
            except OSError:
                pass
            out["decompress_plus_dense"] = {"value": alg_bytes(len(pay), 1) / sec2 / 1e9, "unit": "GB/s",
                                            "ms_per_matmul": sec2 * 1e3, "threads": os.cpu_count(), "cpu": model,
                                            "note": "decompress single-threaded, dense product over all hardware threads"}
        except Exception as e:
            out["decompress_plus_dense"] = {"error": f"{type(e).__name__}: {e}"[:160]}
    return out


DECODERS = {
    # config 3: Qwen2-0.5B shape, batch 1, 512-token prompt then 128 greedy steps
    "qwen0.5b": dict(cfg=dict(n_layers=24, hidden=896, q_heads=14, kv_heads=2, head_dim=64, inter=4864,
                              vocab=151936), kv_atoms=128, batch=1, context=512, steps=128, eps=1e-6, prefill=True),
    # config 4: Llama-7B shape, batch 16 at context 1024
    "llama7b": dict(cfg=dict(n_layers=32, hidden=4096, q_heads=32, kv_heads=32, head_dim=128, inter=11008,
                             vocab=32000), kv_atoms=None, batch=16, context=1024, steps=32, eps=1e-5, prefill=True),
    # two blocks of config 4 (every launch of a block at its full size, a few hundred MB on the
    # device): the case for kernel profilers, not a reported figure
    "llama7b_2blocks": dict(cfg=dict(n_layers=2, hidden=4096, q_heads=32, kv_heads=32, head_dim=128, inter=11008,
                                     vocab=32000), kv_atoms=None, batch=16, context=1024, steps=12, eps=1e-5,
                            prefill=False),
}


FUSED_GEMV_DRAM_BYTES_NCU = 8996000   # per launch, cfg2 shape, batch 1 (8.996 MB read, 0 written)
QUEUE_DRAM_BYTES_PER_TASK_NCU = 9207000   # per product of the list kernel, cfg2 shape, batch 1 (147.3 MB per 16-product launch)


def decoder_bench(name, cs, torch, dist, ctx, stream, rank, world, comm, use_graph=True, kv_dtype="f32",
                  shared_dicts=False):
    """Decode tokens/s of a decoder-shaped synthetic archive (every linear an HSDR row-tile segment
    with its own dictionary, K=512 3x8; random-init stand-in for the config's weights).
    With more than one rank the decoder is tensor parallel; CSDR_BENCH_NCCL_ONLY=1 withholds the
    ranks' IPC handles so that the partial sums go through ncclAllReduce (the comparison arm)."""
    from tests import synth
    spec = DECODERS[name]
    cfg = spec["cfg"]
    os.makedirs(CACHE, exist_ok=True)
    # shared_dicts: a different archive of the same shapes - every block role (attn_q ... ffn_down)
    # shares ONE dictionary over all blocks (resource segments inside the .sdr), so a step reads
    # seven dictionaries and the codes instead of a dictionary per tensor
    path = os.path.join(CACHE, f"{name}{'_shared' if shared_dicts else ''}.sdr")
    if rank == 0 and not os.path.exists(path):
        synth.decoder_archive(path + ".tmp", **cfg, kv_atoms=spec["kv_atoms"], seed=100, shared_dicts=shared_dicts)
        os.replace(path + ".tmp", path)
    if world > 1:
        dist.barrier()
    B, ctxlen, steps = spec["batch"], spec["context"], spec["steps"]
    ld = cs.SDRModelLoader(path, ctx)
    ag = None
    if world > 1:
        def ag(b):
            got = [None] * world
            dist.all_gather_object(got, b)
            return got
    dec = cs.Decoder(ld, **cfg, max_seq=ctxlen + steps + 8, max_batch=B, rms_eps=spec["eps"], comm=comm,
                     all_gather=None if os.environ.get("CSDR_BENCH_NCCL_ONLY") else ag, kv_dtype=kv_dtype)
    rng = np.random.default_rng(7)
    out = {"batch": B, "context": ctxlen, "steps": steps, "tp": world, "kv_cache": kv_dtype,
           "dictionaries": "one per block role, shared by all blocks" if shared_dicts else "one per tensor"}
    if world > 1:
        peer = not os.environ.get("CSDR_BENCH_NCCL_ONLY") and 2 <= world <= 8
        if os.environ.get("CSDR_TP_EXCHANGE") in ("peer", "nccl") and not os.environ.get("CSDR_BENCH_NCCL_ONLY") and world <= 8:
            peer = os.environ["CSDR_TP_EXCHANGE"] == "peer"
        out["partial_sums"] = "peer memory (in-kernel)" if peer else "ncclAllReduce"
    with torch.cuda.stream(stream):
        if spec["prefill"]:
            prompts = rng.integers(0, cfg["vocab"], (B, ctxlen))
            dec.forward(prompts[0], seq=0, want_logits=False)   # first pass builds per-dictionary caches
            dec.reset()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            logits, _ = dec.forward(prompts[0], seq=0)
            e1.record(stream)
            torch.cuda.synchronize()
            out["prefill_ms"] = e0.elapsed_time(e1)
            out["prefill_tokens_per_s"] = ctxlen / (out["prefill_ms"] / 1e3)
            firsts = [int(logits.argmax())]
            for b in range(1, B):        # every sequence gets a real, different context
                lg, _ = dec.forward(prompts[b], seq=b)
                firsts.append(int(lg.argmax()))
            if not np.isfinite(logits).all():
                raise RuntimeError("prefill produced non-finite logits")
            first = np.array(firsts, np.int32)
            out["first_tokens"] = firsts[:4]
        else:
            for b in range(B):          # context without prefill: the cache rows below hold zeros;
                dec.seek(b, ctxlen)     # decode cost does not depend on their content
            first = rng.integers(0, cfg["vocab"], B).astype(np.int32)
            out["note"] = "KV cache positioned at the context length without a prefill pass"
        tok = torch.from_numpy(first).cuda()
        torch.cuda.synchronize()

        def one():
            dec.step_device(tok.data_ptr(), B, tok.data_ptr())   # greedy token fed straight back
        for _ in range(3):
            one()
        ctx.synchronize()
        mode, run = "eager", one
        if use_graph:
            try:
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=stream):
                    one()
                mode, run = "cuda graph", g.replay
            except Exception as e:
                mode = f"eager (graph capture failed: {type(e).__name__})"
                torch.cuda.synchronize()
        run()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n = steps - 5
        e0.record(stream)
        for _ in range(n):
            run()
        e1.record(stream)
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    out.update(launch=mode, ms_per_step=ms / n, tokens_per_s=B * n / (ms / 1e3))
    # a sanity signal on the timed path: one more step through the host-buffer call, logits read back
    with torch.cuda.stream(stream):
        nxt, lg = dec.step(tok.cpu().numpy(), want_logits=True)
    # where a step's time goes: events around every launch of three eager steps (launches do not
    # overlap in this mode, so the sum exceeds the step time above; shares are what it shows)
    ctx.profile(True)
    with torch.cuda.stream(stream):
        for _ in range(3):
            one()
    out["kernels_per_step"] = {k: {"launches": v[0] // 3, "us_each": round(v[1] / v[0] * 1e3, 2)} for k, v in ctx.profile_read().items()}
    ctx.profile(False)
    out["logits_finite"] = bool(np.isfinite(lg).all())
    out["next_tokens"] = [int(t) for t in nxt[:4]]
    if not out["logits_finite"]:
        raise RuntimeError("decode step produced non-finite logits")
    dec.close()
    ld.close()
    return out


def other_configs(cs, torch, ctx, stream, timed, hbm_peak, tf_peak, args):
    """Configurations 1, 2 (2-D tiles) and 5 beside the headline: microseconds per product with the
    operands resident, every pass over more distinct weight copies than L2 holds unless noted.
    Payloads are synthetic stand-ins of the configurations' shapes (timing does not depend on
    which atoms the codes name). frac_hbm counts the compressed bytes a product has to read."""
    from tests import synth
    out = {}
    gen = torch.Generator(device="cuda").manual_seed(5)

    def run(label, make_seg, n_copies, rows, cols, payload_bytes, batches, shared_bytes=0, dtype=torch.bfloat16):
        ent = {}
        try:
            copies = [make_seg(i) for i in range(n_copies)]
            for m in batches:
                x = torch.randn((m, cols), generator=gen, device="cuda").to(dtype)
                y = torch.empty((n_copies, m, rows), device="cuda")
                dt = cs.DTYPE_BF16 if dtype == torch.bfloat16 else cs.DTYPE_F32

                def step():
                    for i, sg in enumerate(copies):
                        sg.matmul_device(x.data_ptr(), dt, cs.TOKEN_MAJOR, m, y[i].data_ptr(), cs.TOKEN_MAJOR)
                step()
                ctx.synchronize()
                st = max(3, args.steps // (4 if m >= 64 else 2))
                ms = timed(step, st, 3)
                per = ms / st / n_copies * 1e-3
                alg = payload_bytes + shared_bytes / n_copies + cols * m * x.element_size() + rows * m * 4
                e = {"us_per_matmul": per * 1e6, "GBps_compressed": alg / per / 1e9, "frac_hbm": alg / per / 1e9 / hbm_peak,
                     "TFLOPs_dense_equiv": 2.0 * rows * cols * m / per / 1e12}
                e["frac_bf16_peak"] = e["TFLOPs_dense_equiv"] / tf_peak
                ctx.profile(True)                       # one pass with events around every launch
                step()
                e["kernel_us"] = {k: round(v[1] / v[0] * 1e3, 2) for k, v in ctx.profile_read().items()}
                ctx.profile(False)
                ent[f"M{m}"] = e
                del x, y
            for sg in copies:
                sg.close()
        except Exception as ex:
            ent["error"] = f"{type(ex).__name__}: {ex}"[:200]
            torch.cuda.synchronize()
        out[label] = ent
        torch.cuda.empty_cache()

    # config 1: 4096 x 4096, batch 1 - row tiles, and the reference's default 128 x 128 tiles
    p1 = synth.hsdr_payload(4096, 4096, seed=0)
    run("cfg1_row_tiles", lambda i: cs.Segment.from_payload(p1, ctx), 32, 4096, 4096, len(p1), (1,), dtype=torch.float32)
    p1t = synth.hsdr_payload(4096, 4096, tile_rows=128, tile_cols=128, n_atoms=256, k=5, seed=0)
    run("cfg1_tiles_128x128", lambda i: cs.Segment.from_payload(p1t, ctx), 16, 4096, 4096, len(p1t), (1,), dtype=torch.float32)
    # config 2 in 2-D tiles (forMLP: 512 atoms, 8 per stage): decode batches on the factored kernels,
    # wide batches on the tensor cores over planes rebuilt once per segment
    p2t = synth.hsdr_payload(R, C, tile_rows=128, tile_cols=128, n_atoms=512, k=8, seed=2)
    run("cfg2_tiles_128x128", lambda i: cs.Segment.from_payload(p2t, ctx), 8, R, C, len(p2t), (1, 64, 512))
    # config 5: two tensors behind ONE shared dictionary of 128 x 128 tiles (33.5 MB: L2-resident)
    atoms, scales = synth.shared_dictionary(128, 128, seed=5)
    dic = cs.Dictionary(ctx, 128, 128, 512, 3, 8, atoms, scales)
    for label, (r5, c5) in (("cfg5_14336x4096_shared", (14336, 4096)), ("cfg5_4096x14336_shared", (4096, 14336))):
        codes = synth.hsdc_payload(r5, c5, tile_rows=128, tile_cols=128, seed=r5)
        run(label, lambda i: cs.Segment.from_payload(codes, ctx, dic), 2, r5, c5, len(codes), (1, 128), shared_bytes=atoms.nbytes)
        if "error" not in out[label]:
            out[label]["note"] = "the shared dictionary stays in L2 between products: not an HBM figure"
    dic.close()
    return out


def encoder_bench(cs, ctx, args):
    """The encoder on config 1's shape (4096 x 4096, row tiles, 512 atoms, 3 x 8 codes): wall time of
    csdr_hsdr_encode with host buffers (the 64 MB tensor crosses to the device inside the call, the
    payload comes back), fast mode and with two dictionary-update rounds; beside it the reference
    encoder on the host cores for the fast mode."""
    out = {"shape": "4096x4096, row tiles, 512 atoms, 3x8 codes"}
    W = np.random.default_rng(0).normal(0, 0.02, (4096, 4096)).astype(np.float32)
    st = cs.HierarchicalSDRStrategy(ctx)
    kw = dict(tile_rows=1, tile_cols=4096, n_atoms=512, n_stages=3, k=8)
    try:
        for label, iters in (("fast", 0), ("two_update_rounds", 2)):
            st.compress(W, **kw, ksvd_iters=iters)              # warm-up: kernels loaded, scratch sized
            best = None
            for _ in range(2):
                t0 = time.perf_counter()
                pay = st.compress(W, **kw, ksvd_iters=iters)
                dt = (time.perf_counter() - t0) * 1e3
                best = dt if best is None else min(best, dt)
            out[label + "_ms"] = best
            out[label + "_payload_bytes"] = len(pay)
    except Exception as e:
        out["error"] = f"{type(e).__name__}: {e}"[:200]
    if not args.no_cpu:
        try:
            from oracle.bindings import SEG_FEED_FORWARD, Reference, Segment, cfg_row1d
            if Reference.available():
                cfg = cfg_row1d(4096, 512, 8, ksvd_iters=0)
                t0 = time.perf_counter()
                Reference().compress(Segment("blk.0.ffn_gate.weight", W, (4096, 4096), SEG_FEED_FORWARD), cfg, cfg)
                out["cpu_reference_fast_ms"] = (time.perf_counter() - t0) * 1e3
                out["cpu_threads"] = os.cpu_count()
        except Exception as e:
            out["cpu_reference_error"] = f"{type(e).__name__}: {e}"[:160]
    return out


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    pay, src = workload_payload()
    from oracle.bindings import Reference
    x = np.random.default_rng(3).normal(0, 1, (C, 1)).astype(np.float32)
    # matmulRowMajor itself is single-threaded; the pass is 32 independent products, so the host
    # arm runs one product per hardware thread at a time (ctypes releases the GIL during the call):
    # a bounded sample of the pass, every host thread busy
    from concurrent.futures import ThreadPoolExecutor
    threads = max(1, min(os.cpu_count() or 1, SEGS))
    per_step = threads
    pool = ThreadPoolExecutor(max_workers=threads)
    if Reference.available():
        refs = [Reference() for _ in range(threads)]
        one, kind = (lambda i: refs[i].matmul(pay, x, 1, R)), "reference"
    else:
        from oracle.bindings import Oracle
        orcs = [Oracle() for _ in range(threads)]
        one, kind = (lambda i: orcs[i].matmul(pay, x, 1)), "port"

    def fn():
        t0 = time.perf_counter()
        list(pool.map(one, range(threads)))
        return time.perf_counter() - t0
    for _ in range(args.warmup):
        fn()
    secs = [fn() for _ in range(args.steps)]
    total = sum(secs)
    val = alg_bytes(len(pay), 1) * per_step * args.steps / total / 1e9
    line = {"impl": "reference", "metric": "compressed_weight_matmul_GBps", "value": val, "unit": "GB/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": total / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": f"synthetic N(0,0.02) weight; {src}",
            "config": {"workload": f"cfg2 MLP projection {R}x{C} HSDR row tiles K={K} {S}x{KPS}, GEMV batch 1"},
            "cpu_baseline": {"value": val, "unit": "GB/s", "cores": threads, "kind": kind,
                             "sample": f"{per_step} of {SEGS} products per step, one per host thread at a time "
                                       "(matmulRowMajor itself is single-threaded), payload bytes in memory"},
            "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--segs", type=int, default=SEGS)
    ap.add_argument("--no-sweep", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--decoder", default="qwen0.5b,llama7b", help="comma list of decoder shapes to time, or none")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)

    import torch
    import torch.distributed as dist
    import cortexsdr_b200 as cs

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        # keep stdout to the one JSON line: NCCL prints its version banner there at the VERSION level
        if os.environ.get("NCCL_DEBUG", "VERSION").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    hbm_peak, tf_peak, peak_src = peaks()

    if rank == 0:
        pay, src = workload_payload()
    if world > 1:
        dist.barrier()
    if rank != 0:
        pay, src = workload_payload()

    stream = torch.cuda.Stream()
    ctx = cs.Context(local, stream.cuda_stream)
    nseg = args.segs
    segs = [cs.Segment.from_payload(pay, ctx) for _ in range(nseg)]
    gen = torch.Generator(device="cuda").manual_seed(3)
    bytes1 = alg_bytes(len(pay), 1)

    def make_io(m, dtype):
        x = torch.randn((m, C), generator=gen, device="cuda", dtype=torch.float32).to(dtype)
        y = torch.empty((nseg, m, R), device="cuda", dtype=torch.float32)
        return x, y

    def step(x, y, m, dt):
        for i, s in enumerate(segs):
            s.matmul_device(x.data_ptr(), dt, cs.TOKEN_MAJOR, m, y[i].data_ptr(), cs.TOKEN_MAJOR)

    def timed(fn, steps, warmup):
        with torch.cuda.stream(stream):
            for _ in range(warmup):
                fn()
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(steps):
                fn()
            e1.record(stream)
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    # ---- headline: GEMV, batch 1, fp32 activations resident in HBM, the pass as one list ----
    x1, y1 = make_io(1, torch.float32)
    queue = cs.Segment.matmul_queue_device(
        [(s, x1.data_ptr(), cs.DTYPE_F32, cs.TOKEN_MAJOR, 1, y1[i].data_ptr(), cs.TOKEN_MAJOR) for i, s in enumerate(segs)])
    ctx.synchronize()

    def qstep():
        cs.Segment.matmul_queue_device(None, queue)
    eager_ms = timed(qstep, args.steps, max(3, args.warmup))
    run_step, launch_mode = qstep, "eager (one C-ABI call per pass)"
    if not args.no_graph:
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                qstep()
            # consecutive eager launches overlap through programmatic dependent launch (the next
            # launch's CTAs move in as this one's leave), replays of a one-kernel graph do not: keep
            # whichever form is faster on this box
            graph.replay()
            graph_ms = timed(graph.replay, args.steps, 3)
            if graph_ms < eager_ms:
                run_step, launch_mode = graph.replay, f"CUDA graph replay of the pass ({nseg} products, one list)"
            else:
                launch_mode = (f"one C-ABI call per pass ({nseg} products, one list), consecutive launches overlapping; "
                               f"graph replay {graph_ms / args.steps:.4f} ms per step")
        except Exception as e:  # capture not possible: keep the eager loop
            launch_mode += f"; graph capture failed: {type(e).__name__}"
            torch.cuda.synchronize()
    with ClockSampler(local) as clk:
        ms = timed(run_step, args.steps, max(3, args.warmup))
        # keep the sampler busy long enough to see the clocks under load
        t_end = time.time() + 1.0
        while time.time() < t_end:
            with torch.cuda.stream(stream):
                run_step()
            ctx.synchronize()
    launches = None
    value = bytes1 * nseg * args.steps * world / (ms / 1e3) / 1e9
    # launch count of exactly the timed region
    l0 = ctx.launch_count
    qstep()
    ctx.synchronize()
    launches_per_step = ctx.launch_count - l0
    launches = launches_per_step * args.steps

    # ---- the same pass as a chain of single launches (each waits for the one before it) ----
    chain = {}
    try:
        cfn = lambda: step(x1, y1, 1, cs.DTYPE_F32)
        cfn()
        ctx.synchronize()
        if not args.no_graph:
            cg = torch.cuda.CUDAGraph()
            with torch.cuda.graph(cg, stream=stream):
                step(x1, y1, 1, cs.DTYPE_F32)
            cfn = cg.replay
        cms = timed(cfn, args.steps, 3)
        cgb = bytes1 * nseg * args.steps / (cms / 1e3) / 1e9
        chain = {"GBps_compressed": cgb, "frac_hbm": cgb / hbm_peak, "us_per_launch": cms / args.steps / nseg * 1e3,
                 "note": "one csdr_matmul_device_async per product, programmatic dependent launches"}
    except Exception as e:
        chain = {"error": f"{type(e).__name__}: {e}"[:200]}
        torch.cuda.synchronize()

    # ---- per-kernel durations over the same steps (events around every launch) ----
    ctx.profile(True)
    with torch.cuda.stream(stream):
        for _ in range(min(args.steps, 20)):
            qstep()
    prof = ctx.profile_read()
    ctx.profile(False)
    if "hsdr_gemv_queue" in prof:
        # one launch per pass: its duration between two events on the stream, averaged
        # the launch's duration: the timed region (CUDA events around it on the launching stream)
        # divided by the launches in it; beside it one launch bracketed by events, nothing overlapping
        n_q, ms_q = prof["hsdr_gemv_queue"]
        us_isolated = ms_q / max(n_q, 1) * 1e3
        us_launch = ms / args.steps / launches_per_step * 1e3
        per_launch = bytes1 * nseg / launches_per_step
        achieved = per_launch / (us_launch * 1e-6) / 1e9
        roofline = {"bound": "hbm", "kernel": "hsdr_gemv_queue_kernel", "achieved": achieved, "peak": hbm_peak,
                    "unit": "GB/s", "frac": achieved / hbm_peak, "peak_source": peak_src,
                    # dram__bytes_read.sum + dram__bytes_write.sum of one launch, scaled from the ncu
                    # capture summarised in profiles/gemv_queue_cfg2_m1.md (traffic grows with the tasks)
                    "traffic": QUEUE_DRAM_BYTES_PER_TASK_NCU * nseg / launches_per_step
                    if (R, C) == (11008, 4096) and QUEUE_DRAM_BYTES_PER_TASK_NCU else None,
                    "alg_bytes_per_launch": per_launch, "us_per_launch": us_launch,
                    "us_per_launch_isolated": us_isolated,
                    "tasks_per_launch": nseg / launches_per_step,
                    "note": "achieved = algorithmic bytes of one launch / (timed region / launches in it); "
                            "isolated = one launch between two events, nothing overlapping it"}
    elif "hsdr_gemv_fused" in prof:
        # one kernel per matmul: its launches overlap (programmatic dependent launch), so the
        # per-launch duration is the timed region divided by the launches in it
        us_launch = ms / args.steps / nseg * 1e3
        achieved = bytes1 / (us_launch * 1e-6) / 1e9
        n_f, ms_f = prof["hsdr_gemv_fused"]
        roofline = {"bound": "hbm", "kernel": "hsdr_gemv_fused_kernel", "achieved": achieved, "peak": hbm_peak,
                    "unit": "GB/s", "frac": achieved / hbm_peak, "peak_source": peak_src,
                    # dram__bytes_read.sum + dram__bytes_write.sum of one launch of this kernel on this
                    # workload, from the ncu capture summarised in profiles/gemv_fused_cfg2_m1.md
                    "traffic": FUSED_GEMV_DRAM_BYTES_NCU if (R, C) == (11008, 4096) else None,
                    "alg_bytes_per_launch": bytes1, "us_per_launch": us_launch,
                    "us_per_launch_isolated": ms_f / max(n_f, 1) * 1e3,
                    "note": "us_per_launch = timed region / launches (launches overlap); isolated = one "
                            "launch bracketed by events, nothing overlapping it"}
    else:
        n_dx, ms_dx = prof.get("hsdr_dx", (0, 0.0))
        n_g, ms_g = prof.get("hsdr_gather", (0, 0.0))
        dict_bytes = 4 * K * C + C * 4 + K * 4      # dictionary + x in, Dx out: the Dx kernel's share
        dx_us = ms_dx / max(n_dx, 1) * 1e3
        achieved = dict_bytes / (dx_us * 1e-6) / 1e9 if n_dx else None
        roofline = {"bound": "hbm", "kernel": "hsdr_dx_kernel", "achieved": achieved, "peak": hbm_peak,
                    "unit": "GB/s", "frac": (achieved / hbm_peak) if achieved else None, "peak_source": peak_src,
                    "traffic": None, "alg_bytes_per_launch": dict_bytes, "us_per_launch": dx_us,
                    "gather_us_per_launch": ms_g / max(n_g, 1) * 1e3,
                    "whole_matmul_frac": value / world / hbm_peak}

    # ---- segments that share x (gate|up, q|k|v) in one launch ----
    grouped = {}
    for gsz in (2, 4):
        if nseg % gsz:
            continue
        ptrs = [[y1[i + j].data_ptr() for j in range(gsz)] for i in range(0, nseg, gsz)]

        def gstep():
            for gi, i in enumerate(range(0, nseg, gsz)):
                cs.Segment.matmul_group_device(segs[i:i + gsz], x1.data_ptr(), cs.DTYPE_F32, cs.TOKEN_MAJOR, 1,
                                               ptrs[gi], cs.TOKEN_MAJOR)
        try:
            gstep()
            ctx.synchronize()
            fn = gstep
            if not args.no_graph:
                gg = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gg, stream=stream):
                    gstep()
                fn = gg.replay
            gms = timed(fn, args.steps, 3)
            gb = bytes1 * nseg * args.steps / (gms / 1e3) / 1e9
            grouped[f"x{gsz}"] = {"GBps_compressed": gb, "frac_hbm": gb / hbm_peak,
                                  "us_per_launch": gms / args.steps / (nseg // gsz) * 1e3}
        except Exception as e:
            grouped[f"x{gsz}"] = {"error": f"{type(e).__name__}: {e}"[:200]}
            torch.cuda.synchronize()

    # ---- e2e: host buffers through the C-ABI (csdr_matmul), H2D + D2H inside the timed region ----
    xh = np.random.default_rng(3).normal(0, 1, (C, 1)).astype(np.float32)

    yh = np.empty((R, 1), np.float32)

    # every product brings its own host activations; activations and results live in page-locked
    # host memory, one product's behind the other's, so that each way is one copy-engine transfer
    x_pin = torch.empty((nseg, C), dtype=torch.float32, pin_memory=True)
    y_pin = torch.empty((nseg, R), dtype=torch.float32, pin_memory=True)
    x_all, y_all = x_pin.numpy(), y_pin.numpy()
    x_all[:] = xh.reshape(1, C)
    xhs = [x_all[i].reshape(C, 1) for i in range(nseg)]
    yhs = [y_all[i].reshape(R, 1) for i in range(nseg)]
    hq = cs.Segment.matmul_queue([(s, xhs[i], 1, yhs[i]) for i, s in enumerate(segs)])

    def e2e_step():
        cs.Segment.matmul_queue(None, hq)
    for _ in range(2):
        e2e_step()
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    n_e2e = max(3, min(args.steps, 10))
    for _ in range(n_e2e):
        e2e_step()
    e2e_s = time.perf_counter() - t0
    if world > 1:
        t = torch.tensor([e2e_s], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e = {"value": bytes1 * nseg * n_e2e * world / e2e_s / 1e9, "unit": "GB/s",
           "h2d_bytes_per_step": nseg * C * 4, "d2h_bytes_per_step": nseg * R * 4,
           "api": "csdr_matmul_queue (host x, host y in page-locked memory), one call per pass"}
    # the same through one host-buffer call per product
    t0 = time.perf_counter()
    for _ in range(3):
        for s in segs:
            s.matmul(xh, 1, out=yh)
    e2e["per_product_calls_GBps"] = bytes1 * nseg * 3 / (time.perf_counter() - t0) / 1e9

    # ---- M sweep of the same workload (bf16 activations, token-major) ----
    sweep = {}
    if not args.no_sweep:
        for m in (1, 8, 64, 512):
            xm, ym = make_io(m, torch.bfloat16)
            st = max(3, args.steps // (4 if m >= 64 else 1))
            sfn, how = (lambda: step(xm, ym, m, cs.DTYPE_BF16)), "eager"
            if not args.no_graph:
                try:
                    with torch.cuda.stream(stream):
                        sfn()                    # builds per-dictionary caches outside the capture
                    ctx.synchronize()
                    sg = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(sg, stream=stream):
                        step(xm, ym, m, cs.DTYPE_BF16)
                    sfn, how = sg.replay, "cuda graph"
                except Exception as e:
                    how = f"eager (graph capture failed: {type(e).__name__})"
                    torch.cuda.synchronize()
            msm = timed(sfn, st, 3)
            per = msm / st / nseg * 1e-3
            ent = {"us_per_matmul": per * 1e6, "launch": how}
            if m <= 16:
                ent["GBps_compressed"] = alg_bytes(len(pay), m, 2) / per / 1e9
                ent["frac_hbm"] = ent["GBps_compressed"] / hbm_peak
            ent["TFLOPs_dense_equiv"] = 2.0 * R * C * m / per / 1e12
            ent["frac_bf16_peak"] = ent["TFLOPs_dense_equiv"] / tf_peak
            if m >= 8:
                # events around every launch: where the time of one wide matmul goes
                ctx.profile(True)
                with torch.cuda.stream(stream):
                    step(xm, ym, m, cs.DTYPE_BF16)
                ent["kernel_us"] = {k: round(v[1] / v[0] * 1e3, 2) for k, v in ctx.profile_read().items()}
                ctx.profile(False)
            sweep[f"M{m}"] = ent
            del xm, ym

    # ---- the other matmul configurations (device-resident, synthetic payloads of their shapes) ----
    other = {}
    if not args.no_sweep and world == 1:
        for s_ in segs:
            s_.close()
        segs.clear()
        torch.cuda.empty_cache()
        other = other_configs(cs, torch, ctx, stream, timed, hbm_peak, tf_peak, args)
        other["encoder"] = encoder_bench(cs, ctx, args)

    # ---- decoder-shaped decode tokens/s (tensor-parallel over the ranks when world > 1) ----
    decode = {}
    for s_ in segs:
        s_.close()
    segs.clear()
    del y1
    torch.cuda.empty_cache()
    comm = None
    if world > 1:
        ids = [cs.nccl_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)
        comm = cs.NcclComm(ctx, ids[0], rank, world)
    for name in [n for n in args.decoder.split(",") if n and n != "none"]:
        try:
            if DECODERS[name]["cfg"]["kv_heads"] % world:
                decode[name] = {"skipped": f"{DECODERS[name]['cfg']['kv_heads']} kv heads do not divide over {world} ranks"}
                continue
            decode[name] = decoder_bench(name, cs, torch, dist, ctx, stream, rank, world, comm, not args.no_graph)
        except Exception as e:
            decode[name] = {"error": f"{type(e).__name__}: {e}"[:300]}
            torch.cuda.synchronize()
            continue
        if world > 1:
            continue        # the option lines are single-GPU figures
        for kvd in ("f16", "bf16"):
            try:
                # the 16-bit cache OPTIONS as lines of their own (rows rounded on entry, sums fp32); the
                # figures above stay on the fp32 cache, the reference's arithmetic
                decode[f"{name}_{kvd}_kv"] = decoder_bench(name, cs, torch, dist, ctx, stream, rank, world, comm,
                                                           not args.no_graph, kv_dtype=kvd)
            except Exception as e:
                decode[f"{name}_{kvd}_kv"] = {"error": f"{type(e).__name__}: {e}"[:300]}
                torch.cuda.synchronize()
        if world == 1:
            try:
                decode[name + "_shared_dicts"] = decoder_bench(name, cs, torch, dist, ctx, stream, rank, world, comm,
                                                               not args.no_graph, shared_dicts=True)
            except Exception as e:
                decode[name + "_shared_dicts"] = {"error": f"{type(e).__name__}: {e}"[:300]}
                torch.cuda.synchronize()

    line = {"metric": "compressed_weight_matmul_GBps", "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": f"synthetic N(0,0.02) weight; {src}",
            "config": {"workload": f"cfg2 MLP projection {R}x{C} HSDR row tiles K={K} {S}x{KPS}, GEMV batch 1",
                       "segments_per_step": nseg, "payload_bytes": len(pay),
                       "l2": f"{nseg} distinct device copies = {nseg * len(pay) / 1e6:.0f} MB per step > L2",
                       "launch": launch_mode, "eager_ms_per_step": eager_ms / args.steps,
                       "parallelism": f"replicas x{world}"},
            "roofline": roofline, "e2e": e2e, "gpu_launches": launches, "clocks": clk.summary(),
            "chain_of_single_launches": chain,
            "kernel_ms": {k: {"launches": v[0], "us_each": v[1] / v[0] * 1e3} for k, v in prof.items()},
            "grouped_same_x": grouped, "sweep": sweep, "other_configs": other, "decode_tokens_per_s": decode}
    if isinstance(decode.get("llama7b"), dict) and "tokens_per_s" in decode["llama7b"]:
        d7 = decode["llama7b"]
        line["tp_decode"] = {"model": "llama7b-shaped, batch 16, context 1024", "tp": d7["tp"],
                             "tokens_per_s": d7["tokens_per_s"], "ms_per_step": d7["ms_per_step"],
                             "exchange": d7.get("partial_sums", "none (one rank)")}
    if rank == 0:
        if not args.no_cpu and world == 1:
            line["cpu_baseline"] = cpu_baseline(pay)
        elif world > 1:
            line["cpu_baseline"] = None
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
