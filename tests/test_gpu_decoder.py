"""Decoder-layer driver on the GPU against the CPU restatement of the reference's
run_transformer_decode (oracle/decoder_oracle.c), with every linear decoded by the oracle
from the same archive. Tolerance on logits: 2e-2 max-abs, as the task states (observed
differences are orders of magnitude smaller). No reference test covers this code, so
parity here is against the restatement only."""
import os

import numpy as np
import pytest

import cortexsdr_b200 as cs
from tests import synth

pytestmark = pytest.mark.gpu
LOGIT_TOL = 2e-2

CFG = dict(n_layers=2, hidden=128, q_heads=4, kv_heads=2, head_dim=32, inter=256, vocab=300)


def _build_model(tmp_path_factory, oracle, tag, raw_formats=None, CFG=CFG, k=3, shared_dicts=False, **atoms):
    path = str(tmp_path_factory.mktemp("dec") / f"{tag}.sdr")
    raw_formats = raw_formats or {}
    synth.decoder_archive(path, **CFG, k=k, seed=7, raw=raw_formats, shared_dicts=shared_dicts, **atoms)
    ld = cs.SDRModelLoader(path, index_only=True)
    shapes = {"token_embd.weight": (CFG["vocab"], CFG["hidden"]), "output.weight": (CFG["vocab"], CFG["hidden"])}
    dictionaries = {}

    def dense(n):
        if n not in raw_formats:
            payload = ld.loadCompressedBytesByName(n)
            if bytes(payload[:4]) == b"HSDC":
                # codes only: the dictionary is the resource segment the header's data_format names
                dname = ld.findSegmentHeader(n).data_format.split("@", 1)[1]
                if dname not in dictionaries:
                    from oracle.bindings import SharedDict
                    dictionaries[dname] = SharedDict(*synth.read_dictionary_record(ld.loadSegmentByName(dname)))
                return oracle.hsdc_decompress(payload, dictionaries[dname])
            return oracle.decompress(payload)
        data = ld.loadSegmentByName(n)                       # stored raw: widen like the reference does
        fmt = raw_formats[n]
        # widened as the reference's inference side does it: ggml's element order for block formats
        w = (data.view(np.float32) if fmt == "f32" else
             oracle.dequantize_inference(fmt, data) if fmt.startswith("q") else oracle.dequantize(fmt, data))
        if n in shapes:
            return w.reshape(shapes[n])
        r, c = {"attn_q": (CFG["q_heads"] * CFG["head_dim"], CFG["hidden"]),
                "attn_k": (CFG["kv_heads"] * CFG["head_dim"], CFG["hidden"]),
                "attn_v": (CFG["kv_heads"] * CFG["head_dim"], CFG["hidden"]),
                "attn_output": (CFG["hidden"], CFG["q_heads"] * CFG["head_dim"]),
                "ffn_gate": (CFG["inter"], CFG["hidden"]), "ffn_up": (CFG["inter"], CFG["hidden"]),
                "ffn_down": (CFG["hidden"], CFG["inter"])}[n.split(".")[2]]
        return w.reshape(r, c)
    raw = lambda n: ld.loadSegmentByName(n).view(np.float32)
    blocks = []
    for i in range(CFG["n_layers"]):
        p = f"blk.{i}."
        blocks.append(dict(attn_norm=raw(p + "attn_norm.weight"), wq=dense(p + "attn_q.weight"),
                           wk=dense(p + "attn_k.weight"), wv=dense(p + "attn_v.weight"),
                           wo=dense(p + "attn_output.weight"), ffn_norm=raw(p + "ffn_norm.weight"),
                           w_gate=dense(p + "ffn_gate.weight"), w_up=dense(p + "ffn_up.weight"),
                           w_down=dense(p + "ffn_down.weight")))
    weights = dict(tok=dense("token_embd.weight"), blocks=blocks, out_norm=raw("output_norm.weight"),
                   head=dense("output.weight"))
    return path, weights


@pytest.fixture(scope="module")
def model(tmp_path_factory, oracle):
    return _build_model(tmp_path_factory, oracle, "tiny", n_atoms=32, kv_atoms=16)


@pytest.fixture(scope="module")
def model_shared(tmp_path_factory, oracle):
    return _build_model(tmp_path_factory, oracle, "shared", shared_dicts=True, n_atoms=32, kv_atoms=16)


@pytest.fixture(scope="module")
def model_tc(tmp_path_factory, oracle):
    """Dictionaries of 128 atoms: steps of eight tokens or more take the tensor-core projection
    and the block loop that hands activations on as bf16 planes."""
    return _build_model(tmp_path_factory, oracle, "tc", n_atoms=128, kv_atoms=128)


@pytest.fixture(scope="module")
def model_raw(tmp_path_factory, oracle):
    """Some tensors stored uncompressed in a source dtype, as a converter leaves protected ones:
    the embedding as f16, the head as q8_0, one block's down projection as bf16, another's
    query projection as plain f32, and three k-quant tensors (q4_k, q5_k, q6_k), which the
    reference's inference side reads in ggml's element order."""
    return _build_model(tmp_path_factory, oracle, "raw", n_atoms=32, kv_atoms=16,
                        raw_formats={"token_embd.weight": "f16", "output.weight": "q8_0",
                                     "blk.0.ffn_down.weight": "bf16", "blk.1.attn_q.weight": "f32",
                                     "blk.1.ffn_up.weight": "q4_k", "blk.0.attn_output.weight": "q6_k",
                                     "blk.1.ffn_gate.weight": "q5_k"})


def oracle_forward(oracle, weights, tokens, eps=1e-6, theta=1e6, CFG=CFG):
    cfg = dict(CFG, eps=eps, theta=theta)
    return oracle.decoder_forward(cfg, weights["tok"], weights["blocks"], weights["out_norm"], weights["head"], tokens)


def make_decoder(path, ctx, CFG=CFG, max_seq=64, **kw):
    ld = cs.SDRModelLoader(path, ctx)
    return cs.Decoder(ld, **CFG, max_seq=max_seq, rms_eps=1e-6, rope_theta=1e6, **kw)


def test_prefill_matches_oracle(ctx, oracle, model):
    path, weights = model
    tokens = np.random.default_rng(0).integers(0, CFG["vocab"], 12)
    hid, logits = oracle_forward(oracle, weights, tokens)
    dec = make_decoder(path, ctx)
    g_logits, g_hid = dec.forward(tokens, want_hidden=True)
    assert np.abs(g_hid - hid).max() < 1e-3
    assert np.abs(g_logits - logits).max() < LOGIT_TOL
    assert int(g_logits.argmax()) == int(logits.argmax())


def test_stored_raw_source_dtypes_are_widened_on_the_device(ctx, oracle, model_raw):
    path, weights = model_raw
    tokens = np.random.default_rng(5).integers(0, CFG["vocab"], 10)
    hid, logits = oracle_forward(oracle, weights, tokens)
    dec = make_decoder(path, ctx)
    g_logits, g_hid = dec.forward(tokens, want_hidden=True)
    assert np.abs(g_hid - hid).max() < 1e-3
    assert np.abs(g_logits - logits).max() < LOGIT_TOL
    assert int(g_logits.argmax()) == int(logits.argmax())
    nxt, lg = dec.step([int(g_logits.argmax())], want_logits=True)
    _, want = oracle_forward(oracle, weights, np.append(tokens, int(g_logits.argmax())))
    assert np.abs(lg[0] - want).max() < LOGIT_TOL and int(nxt[0]) == int(want.argmax())


def test_shared_dictionaries_inside_the_archive(ctx, oracle, model_shared):
    """An .sdr whose seven block roles each share one dictionary over all blocks: the dictionary a
    resource segment (stored raw, data_format "hsdr_dict", one .hsda dictionary record), every
    block's tensor a codes-only "HSDC" payload whose data_format names it. The reference has this
    only as a separate container (.hsda; ai_compression_cli.cpp:727-733 names the missing archive
    section). Prefill, steps and a product by name against the oracle's external-dictionary
    decode (decompressWithExternalDictionary, HierarchicalSDRStrategy.cpp:1804-1828)."""
    path, weights = model_shared
    ld = cs.SDRModelLoader(path, ctx)
    hdr = ld.findSegmentHeader("blk.1.ffn_up.weight")
    assert hdr.data_format == "hsdc@hsdr.shared_dict/ffn_up" and hdr.compression_strategy_id == 5
    assert ld.findSegmentHeader("hsdr.shared_dict/ffn_up").data_format == "hsdr_dict"
    # a product by name goes through the shared dictionary
    x = np.random.default_rng(3).normal(0, 1, (CFG["hidden"], 2)).astype(np.float32)
    y = ld.matmulHSDR("blk.1.ffn_up.weight", x, 2)
    want = weights["blocks"][1]["w_up"].astype(np.float64) @ x
    assert np.abs(y - want).max() / np.abs(want).max() < 1e-4
    tokens = np.random.default_rng(4).integers(0, CFG["vocab"], 11)
    _, logits = oracle_forward(oracle, weights, tokens)
    dec = cs.Decoder(ld, **CFG, max_seq=64, rms_eps=1e-6, rope_theta=1e6)
    got, _ = dec.forward(tokens)
    assert np.abs(got - logits).max() < LOGIT_TOL and int(got.argmax()) == int(logits.argmax())
    seq, nxt = list(tokens), int(got.argmax())
    for _ in range(2):
        seq.append(nxt)
        _, want_l = oracle_forward(oracle, weights, np.array(seq))
        got_next, got_l = dec.step([nxt], want_logits=True)
        assert np.abs(got_l[0] - want_l).max() < LOGIT_TOL and int(got_next[0]) == int(want_l.argmax())
        nxt = int(got_next[0])
    # the blocks hold two images per role and ONE dictionary: resident bytes count it once
    per_role = {"attn_q": CFG["hidden"], "attn_k": CFG["hidden"], "attn_v": CFG["hidden"],
                "attn_output": CFG["q_heads"] * CFG["head_dim"], "ffn_gate": CFG["hidden"], "ffn_up": CFG["hidden"],
                "ffn_down": CFG["inter"]}
    atoms = {r: (16 if r in ("attn_k", "attn_v") else 32) for r in per_role}
    dict_bytes = sum(atoms[r] * c * 4 for r, c in per_role.items())
    own = 2 * 32 * CFG["hidden"] * 4                      # embedding and head keep dictionaries of their own
    resident = ld.resident_bytes()
    assert dict_bytes + own < resident < 2 * dict_bytes + own
    dec.close()
    ld.close()


def test_kv_cache_equals_recompute(ctx, oracle, model):
    path, weights = model
    tokens = np.random.default_rng(1).integers(0, CFG["vocab"], 12)
    dec = make_decoder(path, ctx)
    one_shot, _ = dec.forward(tokens)
    dec.reset()
    dec.forward(tokens[:8], want_logits=False)
    chunked, _ = dec.forward(tokens[8:])
    assert np.abs(one_shot - chunked).max() < 1e-4
    # greedy decode three tokens; the oracle recomputes the whole sequence each step, as the reference does
    seq = list(tokens)
    nxt = int(chunked.argmax())
    for _ in range(3):
        seq.append(nxt)
        _, want = oracle_forward(oracle, weights, np.array(seq))
        got_next, got = dec.step([nxt], want_logits=True)
        assert np.abs(got[0] - want).max() < LOGIT_TOL
        assert int(got_next[0]) == int(want.argmax())
        nxt = int(got_next[0])


def test_folded_glue_equals_separate_kernels(oracle, model, monkeypatch):
    """A short step runs its normalisations, residual additions and SwiGLU inside the one-launch
    GEMVs (six launches per block); CSDR_DECODER_FOLD=0 keeps them as kernels of their own (nine).
    Both against the oracle, and against each other, for one, three and five tokens per pass."""
    path, weights = model
    rng = np.random.default_rng(21)
    prompt = rng.integers(0, CFG["vocab"], 7)
    results = {}
    for fold in ("1", "0"):
        monkeypatch.setenv("CSDR_DECODER_FOLD", fold)
        c = cs.Context(0)
        dec = make_decoder(path, c, max_batch=3)
        launches0 = c.launch_count
        lg5, _ = dec.forward(prompt[:5])                     # five tokens: token tile of 8
        n5 = c.launch_count - launches0
        lg1, _ = dec.forward(prompt[5:6])                    # one token
        lg3 = []
        dec.forward(prompt[:3], seq=1, want_logits=False)    # three tokens: token tile of 4
        dec.forward(prompt[:2], seq=2, want_logits=False)
        nxt, step = dec.step([int(prompt[6]), 11, 12], want_logits=True)
        results[fold] = (lg5, lg1, step, n5)
        dec.close()
        c.close()
    _, want5 = oracle_forward(oracle, weights, prompt[:5])
    _, want6 = oracle_forward(oracle, weights, prompt[:6])
    _, want7 = oracle_forward(oracle, weights, prompt[:7])
    for fold in ("1", "0"):
        lg5, lg1, step, _ = results[fold]
        assert np.abs(lg5 - want5).max() < LOGIT_TOL, fold
        assert np.abs(lg1 - want6).max() < LOGIT_TOL, fold
        assert np.abs(step[0] - want7).max() < LOGIT_TOL, fold
    assert np.abs(results["1"][2] - results["0"][2]).max() < 1e-4
    # per block: 9 launches apart, 6 folded
    assert results["0"][3] - results["1"][3] == 3 * CFG["n_layers"]


def test_batched_step_sequences_are_independent(ctx, oracle, model):
    path, weights = model
    rng = np.random.default_rng(2)
    prompts = [rng.integers(0, CFG["vocab"], n) for n in (5, 9, 3)]
    dec = make_decoder(path, ctx, max_batch=3)
    for s, p in enumerate(prompts):
        dec.forward(p, seq=s, want_logits=False)
    new = rng.integers(0, CFG["vocab"], 3)
    nxt, logits = dec.step(new, want_logits=True)
    for s, p in enumerate(prompts):
        _, want = oracle_forward(oracle, weights, np.append(p, new[s]))
        assert np.abs(logits[s] - want).max() < LOGIT_TOL
        assert int(nxt[s]) == int(want.argmax())


def test_tensor_core_block_loop_matches_oracle(ctx, oracle, model_tc):
    path, weights = model_tc
    rng = np.random.default_rng(3)
    tokens = rng.integers(0, CFG["vocab"], 21)
    hid, logits = oracle_forward(oracle, weights, tokens)
    dec = make_decoder(path, ctx, max_batch=9)
    g_logits, g_hid = dec.forward(tokens, want_hidden=True)          # 21 tokens: wide gather
    assert np.abs(g_hid - hid).max() < 1e-3
    assert np.abs(g_logits - logits).max() < LOGIT_TOL
    assert int(g_logits.argmax()) == int(logits.argmax())
    # nine sequences stepping together: one token tile, grouped gather, residual on the gather
    dec.reset()
    prompts = [rng.integers(0, CFG["vocab"], n) for n in (5, 9, 3, 1, 7, 2, 11, 4, 6)]
    for s_, p_ in enumerate(prompts):
        dec.forward(p_, seq=s_, want_logits=False)
    new = rng.integers(0, CFG["vocab"], 9)
    nxt, lg = dec.step(new, want_logits=True)
    for s_, p_ in enumerate(prompts):
        _, want = oracle_forward(oracle, weights, np.append(p_, new[s_]))
        assert np.abs(lg[s_] - want).max() < LOGIT_TOL
        assert int(nxt[s_]) == int(want.argmax())
    # a second step reads the cache rows the first one filed
    nxt2, lg2 = dec.step(nxt, want_logits=True)
    for s_, p_ in enumerate(prompts):
        _, want = oracle_forward(oracle, weights, np.concatenate([p_, [new[s_]], [nxt[s_]]]))
        assert np.abs(lg2[s_] - want).max() < LOGIT_TOL
        assert int(nxt2[s_]) == int(want.argmax())


def test_selection_policy_matches_the_reference_rule(ctx, oracle, model):
    """Steps under select_best_from_logits: what the device picks equals the oracle's pick on the
    same logits with the same history, for two sequences with different histories; turning the
    policy off gives plain argmax again."""
    path, _ = model
    rng = np.random.default_rng(6)
    dec = make_decoder(path, ctx, max_batch=2)
    dec.selection_policy(True, temperature=0.7)
    prompts = [rng.integers(0, CFG["vocab"], 6), rng.integers(0, CFG["vocab"], 4)]
    history = [[], []]
    cur = []
    for s_, p_ in enumerate(prompts):
        lg, _ = dec.forward(p_, seq=s_)
        first = oracle.select_best_from_logits(lg, history[s_], 0.7)
        history[s_].append(first)
        dec.note_generated([first], seq=s_)
        cur.append(first)
    repeats = 0
    for _ in range(12):
        nxt, lg = dec.step(cur, want_logits=True)
        for s_ in range(2):
            want = oracle.select_best_from_logits(lg[s_], history[s_], 0.7)
            assert int(nxt[s_]) == want
            repeats += int(np.argmax(lg[s_])) != want          # the penalty changed the pick
            history[s_].append(want)
        cur = [int(t) for t in nxt]
    assert repeats > 0                                          # a 300-token random model does repeat itself
    dec.selection_policy(False)
    nxt, lg = dec.step(cur, want_logits=True)
    assert [int(t) for t in nxt] == [int(np.argmax(lg[0])), int(np.argmax(lg[1]))]
    dec.reset()
    with pytest.raises(ValueError):
        dec.note_generated([1], seq=5)


def test_decoder_limits_and_errors(ctx, model):
    path, _ = model
    dec = make_decoder(path, ctx)
    with pytest.raises(ValueError, match="vocabulary"):
        dec.forward([CFG["vocab"]])
    with pytest.raises(ValueError, match="capacity"):
        dec.forward(np.zeros(65, np.int32))
    ld = cs.SDRModelLoader(path, ctx)
    with pytest.raises(cs.CompressionError, match="does not match the config"):
        cs.Decoder(ld, **dict(CFG, hidden=64), max_seq=8)
    with pytest.raises(RuntimeError, match="not found|not in archive"):
        cs.Decoder(ld, **dict(CFG, n_layers=3), max_seq=8)


def test_exchange_needs_tensor_parallel_ranks(ctx, model):
    """A single-rank decoder has no exchange region: export and import say so instead of
    handing out a handle nobody could use."""
    import ctypes as C
    path, _ = model
    dec = make_decoder(path, ctx)
    buf = C.create_string_buffer(64)
    lib = ctx._lib
    assert lib.csdr_decoder_exchange_export(dec._h, buf) == cs._lib.ERR_UNSUPPORTED
    assert lib.csdr_decoder_exchange_import(dec._h, buf.raw, 1) == cs._lib.ERR_UNSUPPORTED
    assert lib.csdr_decoder_exchange_import(dec._h, buf.raw, 2) == cs._lib.ERR_INVALID_ARG
    assert b"exchange" in lib.csdr_last_error() or b"handle" in lib.csdr_last_error()


# ---- the two decoder configurations at their real WIDTHS (depth reduced) ----
# Width selects the kernel variants: the 14 : 2 grouped heads of 64 and the 151 936-row head of
# the 0.5B shape; the 32 heads of 128, the 11 008-wide MLP and the 16-token step of the 7B shape.
QWEN_W = dict(n_layers=2, hidden=896, q_heads=14, kv_heads=2, head_dim=64, inter=4864, vocab=151936)
LLAMA_W = dict(n_layers=1, hidden=4096, q_heads=32, kv_heads=32, head_dim=128, inter=11008, vocab=32000)


@pytest.fixture(scope="module")
def model_qwen_width(tmp_path_factory, oracle):
    return _build_model(tmp_path_factory, oracle, "qwenw", CFG=QWEN_W, k=8, n_atoms=512, kv_atoms=128)


@pytest.fixture(scope="module")
def model_llama_width(tmp_path_factory, oracle):
    return _build_model(tmp_path_factory, oracle, "llamaw", CFG=LLAMA_W, k=8, n_atoms=512)


_ORACLE_MEMO = {}


def oracle_forward_memo(oracle, weights, tokens, CFG):
    """The oracle's logits for a token sequence, kept so that the fp32- and bf16-cache runs of a
    test share one CPU recompute."""
    key = (id(weights), np.asarray(tokens, np.int64).tobytes())
    if key not in _ORACLE_MEMO:
        _ORACLE_MEMO[key] = oracle_forward(oracle, weights, tokens, CFG=CFG)
    return _ORACLE_MEMO[key]


# The 16-bit KV cache OPTIONS (rows rounded on entry, scores and sums fp32). fp16 (10 mantissa bits)
# meets the fp32 cache's bar of 2e-2; bf16 (7 bits) does not at the 7B widths (observed 2.4e-2) and
# has a bar of its own, 5e-2. The default stays fp32, the reference's arithmetic.
KV_TOL = {"f32": LOGIT_TOL, "f16": LOGIT_TOL, "bf16": 5e-2}


def same_pick(got, want, tol):
    """Equal argmax; at the bf16 cache's wider bar, unless the oracle's two best logits are closer
    than that bar allows to tell."""
    if int(got.argmax()) == int(want.argmax()):
        return True
    top2 = np.partition(want, -2)[-2:]
    return tol > LOGIT_TOL and float(top2[1] - top2[0]) < 2 * tol


@pytest.mark.parametrize("kv_dtype", ["f32", "f16", "bf16"])
def test_qwen_width_prefill_and_greedy_steps(ctx, oracle, model_qwen_width, kv_dtype):
    """Hidden 896, 14 query / 2 kv heads of 64, SwiGLU 4864, vocabulary 151 936, eps 1e-6, k/v
    dictionaries of 128 atoms; two blocks. A 64-token prompt (tensor-core block loop), then
    three greedy steps at batch 1 (fused GEMV path), each against the oracle's whole-sequence
    recompute."""
    path, weights = model_qwen_width
    tokens = np.random.default_rng(7).integers(0, QWEN_W["vocab"], 64)
    _, logits = oracle_forward_memo(oracle, weights, tokens, CFG=QWEN_W)
    dec = make_decoder(path, ctx, CFG=QWEN_W, max_seq=80, kv_dtype=kv_dtype)
    g_logits, _ = dec.forward(tokens)
    assert np.isfinite(g_logits).all()
    tol = KV_TOL[kv_dtype]
    assert np.abs(g_logits - logits).max() < tol
    assert same_pick(g_logits, logits, tol)
    seq, nxt = list(tokens), int(logits.argmax())
    for _ in range(3):
        seq.append(nxt)
        _, want = oracle_forward_memo(oracle, weights, np.array(seq), CFG=QWEN_W)
        got_next, got = dec.step([nxt], want_logits=True)
        assert np.abs(got[0] - want).max() < tol
        assert same_pick(got[0], want, tol) and int(got_next[0]) == int(got[0].argmax())
        nxt = int(want.argmax())
    dec.close()


def test_llama_width_batch11_step(ctx, oracle, model_llama_width):
    """Eleven sequences step together: a 16-token tile with five empty columns through the
    tensor-core projection, the gathers (the next norm's first half riding on the output and
    down gathers, its sums added up by the projection behind them) and attention."""
    path, weights = model_llama_width
    rng = np.random.default_rng(18)
    lens = [4, 1, 9, 6, 2, 11, 3, 7, 5, 8, 10]
    prompts = [rng.integers(0, LLAMA_W["vocab"], n) for n in lens]
    dec = make_decoder(path, ctx, CFG=LLAMA_W, max_seq=32, max_batch=16)
    for s_, p_ in enumerate(prompts):
        dec.forward(p_, seq=s_, want_logits=False)
    new = rng.integers(0, LLAMA_W["vocab"], len(lens))
    nxt, lg = dec.step(new, want_logits=True)
    assert lg.shape[0] == len(lens) and np.isfinite(lg).all()
    for s_ in (0, 1, 5, 10):
        _, want = oracle_forward_memo(oracle, weights, np.append(prompts[s_], new[s_]), CFG=LLAMA_W)
        assert np.abs(lg[s_] - want).max() < 2e-2, s_
        assert same_pick(lg[s_], want, 2e-2) and int(nxt[s_]) == int(lg[s_].argmax()), s_
    dec.close()


@pytest.mark.parametrize("which", ["qwen", "llama"])
def test_step_rotary_fold_matches_separate_kernel(which, model_qwen_width, model_llama_width, monkeypatch):
    """A decode step with the rotary embedding and the cache write inside the attention launch
    gives the logits of the step that runs them as a kernel of their own, now and one step later
    (the later step reads the cache rows the earlier one filed): same arithmetic, same bits."""
    path, CFGW = (model_qwen_width[0], QWEN_W) if which == "qwen" else (model_llama_width[0], LLAMA_W)
    rng = np.random.default_rng(21)
    n_seq = 1 if which == "qwen" else 9
    prompts = [rng.integers(0, CFGW["vocab"], 3 + 2 * s_) for s_ in range(n_seq)]
    new = rng.integers(0, CFGW["vocab"], n_seq)
    got = {}
    for fold in ("1", "0"):
        monkeypatch.setenv("CSDR_ATTENTION_ROPE_FOLD", fold)
        c = cs.Context(0)
        dec = make_decoder(path, c, CFG=CFGW, max_seq=32, max_batch=16)
        for s_, p_ in enumerate(prompts):
            dec.forward(p_, seq=s_, want_logits=False)
        nxt, lg = dec.step(new, want_logits=True)
        nxt2, lg2 = dec.step(nxt, want_logits=True)
        got[fold] = (np.array(lg), np.array(lg2), np.array(nxt2))
        dec.close()
        c.close()
    assert np.isfinite(got["1"][0]).all()
    assert np.array_equal(got["1"][0], got["0"][0])
    assert np.array_equal(got["1"][1], got["0"][1])
    assert np.array_equal(got["1"][2], got["0"][2])


@pytest.mark.parametrize("kv_dtype", ["f32", "f16", "bf16"])
def test_llama_width_batch16_step(ctx, oracle, model_llama_width, kv_dtype):
    """Hidden 4096, 32 heads of 128, SwiGLU 11 008, vocabulary 32 000; one block. Sixteen
    sequences with real, different, prefilled contexts step together (the 16-token tile of the
    tensor-core projection, the grouped gathers, the batch-16 attention), then step again over
    the cache rows the first step filed."""
    path, weights = model_llama_width
    rng = np.random.default_rng(8)
    lens = [3, 9, 5, 12, 1, 7, 4, 10, 2, 8, 6, 11, 3, 5, 9, 7]
    prompts = [rng.integers(0, LLAMA_W["vocab"], n) for n in lens]
    dec = make_decoder(path, ctx, CFG=LLAMA_W, max_seq=32, max_batch=16, kv_dtype=kv_dtype)
    for s_, p_ in enumerate(prompts):
        dec.forward(p_, seq=s_, want_logits=False)
    new = rng.integers(0, LLAMA_W["vocab"], 16)
    nxt, lg = dec.step(new, want_logits=True)
    assert np.isfinite(lg).all()
    tol = KV_TOL[kv_dtype]
    for s_, p_ in enumerate(prompts):
        _, want = oracle_forward_memo(oracle, weights, np.append(p_, new[s_]), CFG=LLAMA_W)
        assert np.abs(lg[s_] - want).max() < tol, s_
        assert same_pick(lg[s_], want, tol) and int(nxt[s_]) == int(lg[s_].argmax()), s_
    nxt2, lg2 = dec.step(nxt, want_logits=True)
    for s_ in (0, 3, 15):
        _, want = oracle_forward_memo(oracle, weights, np.concatenate([prompts[s_], [new[s_]], [nxt[s_]]]), CFG=LLAMA_W)
        assert np.abs(lg2[s_] - want).max() < tol, s_
        assert same_pick(lg2[s_], want, tol) and int(nxt2[s_]) == int(lg2[s_].argmax()), s_
    dec.close()
