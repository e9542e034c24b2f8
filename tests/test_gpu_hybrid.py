"""Layered hybrid decoders on the GPU against the plain fp64 restatement (oracle/kinetar_plain.py): each mechanism alone,
prefill against token-by-token decoding, portions, unequal batches, reuse of pages and slots, keys at page and key-group
borders, the first tokens of a sequence, long decoding, other sizes, and greedy generation through LLM.generate."""
import copy

import numpy as np
import pytest
import torch

from oracle import kinetar_plain as plain
from tests.hybrid_helpers import (SMALL, TOL, Harness, attn_scan, delta, model_config, oracle_logits, rand_tokens, rel_err)

pytestmark = pytest.mark.gpu


def _run(config, tokens, dtype="float32", cuts=None, seed=0, low=8, weights=None, **kw):
    w = weights if weights is not None else plain.random_weights(config, seed, low)
    hz = Harness(config, w, dtype=dtype, low=low, **kw)
    try:
        got = hz.feed("a", tokens, cuts)
    finally:
        hz.close()
    return got, oracle_logits(config, w, tokens)


# ---- each mechanism alone ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["attention", "scan", "delta", "ff_only_delta"])
def test_mechanism_alone(which, dtype):
    if which == "attention":
        layer = attn_scan(right_scale=0.0)
    elif which == "scan":
        layer = attn_scan(left_scale=0.0)
    elif which == "delta":
        layer = delta(ff=0)
    else:
        layer = delta()
    if which in ("attention", "scan"):
        layer["mlp"] = None
    cfg = model_config([layer])
    toks = rand_tokens(45, cfg["vocab"], 3)
    got, want = _run(cfg, toks, dtype)
    assert rel_err(got, want) < TOL[dtype]


# ---- prefill == decode, portions -------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prefill_equals_token_by_token(dtype):
    toks = rand_tokens(70, SMALL["vocab"], 5)
    whole, want = _run(SMALL, toks, dtype)
    single, _ = _run(SMALL, toks, dtype, cuts=[1])
    assert rel_err(whole, want) < TOL[dtype]
    assert rel_err(single, want) < TOL[dtype]
    assert rel_err(single, whole) < TOL[dtype]


@pytest.mark.parametrize("cuts", [[2], [3, 2, 7, 1, 16, 5], [17, 2, 2, 31], [33, 1]])
def test_portions(cuts):
    toks = rand_tokens(90, SMALL["vocab"], 7)
    got, want = _run(SMALL, toks, "float32", cuts=cuts)
    assert rel_err(got, want) < TOL["float32"]


def test_step_larger_than_the_runner_capacity_is_cut():
    toks = rand_tokens(100, SMALL["vocab"], 8)
    got, want = _run(SMALL, toks, "float32", max_step_tokens=32)
    assert rel_err(got, want) < TOL["float32"]


# ---- batches of unequal requests, reuse of pages and slots ------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_batches_and_reuse(dtype):
    w = plain.random_weights(SMALL, 11)
    V = SMALL["vocab"]
    reqs = {"a": rand_tokens(50, V, 1), "b": rand_tokens(7, V, 2), "c": rand_tokens(33, V, 3), "d": rand_tokens(1, V, 4),
            "e": rand_tokens(41, V, 5), "f": rand_tokens(20, V, 6)}
    ref = {k: oracle_logits(SMALL, w, v) for k, v in reqs.items()}
    hz = Harness(SMALL, w, dtype=dtype, page_size=16, num_pages=9, slots=3)          # a, c, e cannot be live together
    got = {k: [] for k in reqs}
    at = {k: 0 for k in reqs}

    def step(parts):
        ent = []
        for k, n in parts:
            n = min(n, len(reqs[k]) - at[k])
            ent.append((k, reqs[k][at[k]:at[k] + n], range(n)))
        out = hz.step(ent)
        o = 0
        for k, t, _ in ent:
            got[k].append(out[o:o + len(t)])
            o += len(t)
            at[k] += len(t)
            if at[k] == len(reqs[k]):
                hz.end(k)
    try:
        step([("a", 20), ("b", 3), ("d", 1)])           # d ends: its slot and page are free again
        step([("a", 1), ("b", 2), ("c", 9)])
        step([("c", 24), ("a", 1), ("b", 2)])           # c and b end
        step([("a", 12), ("e", 2)])
        step([("e", 17), ("a", 1), ("f", 5)])
        while at["a"] < 50 or at["e"] < 41 or at["f"] < 20:
            step([(k, 1 if k != "f" else 4) for k in ("a", "e", "f") if at[k] < len(reqs[k])])
        assert len(hz.sched.block_manager.free_block_ids) == 9 and len(hz.sched.state_manager.free_slots) == 3
    finally:
        hz.close()
    for k in reqs:
        assert rel_err(np.concatenate(got[k], 0), ref[k]) < TOL[dtype], k


def test_slot_and_pages_used_again_start_from_the_empty_state():
    w = plain.random_weights(SMALL, 12)
    V = SMALL["vocab"]
    hz = Harness(SMALL, w, "float32", page_size=16, num_pages=4, slots=1)
    try:
        for i in range(3):
            toks = rand_tokens(40 + i, V, 20 + i)
            got = hz.feed("x", toks, cuts=[13, 1])
            hz.end("x")
            assert rel_err(got, oracle_logits(SMALL, w, toks)) < TOL["float32"]
    finally:
        hz.close()


# ---- a key that must be found: far back, at page borders, at key-group borders ------------------------------------------------
def _needle_model():
    """One attention layer whose query and key projections are equal and whose convolutions pass the current token
    through: a query scores highest against the key of the same token id, so one marked token far back carries the
    answer.  The scan side and the feed-forward are off."""
    layer = attn_scan(heads=2, kv_heads=1, dim=16, conv=2, coef=0.0, every=1, scale=2.0, left_scale=1.0, right_scale=0.0)
    layer["mlp"] = None
    cfg = model_config([layer], width=32, vocab=64, emb_scale=8.0)
    w = plain.random_weights(cfg, 31)
    g = torch.Generator().manual_seed(32)
    p = torch.randn(16, 32, generator=g) * 0.5
    w["l0.mix.left.q"] = torch.cat([p, p]).to(torch.bfloat16)
    w["l0.mix.left.k"] = p.to(torch.bfloat16)
    for n, rows in (("q", 32), ("k", 16)):
        c = torch.zeros(rows, 2)
        c[:, 1] = 1.0
        w[f"l0.mix.left.{n}.conv"] = c.to(torch.bfloat16)
    w["l0.mix.left.sink"] = torch.tensor([-1.0, 0.5]).to(torch.bfloat16)
    w["l0.norm1"] = torch.zeros(32).to(torch.bfloat16)
    return cfg, w


@pytest.mark.parametrize("needle_at", [0, 1, 15, 16, 31, 32, 47, 48, 63, 64])
@pytest.mark.parametrize("decode", [False, True])
def test_marked_key_far_back_is_found(needle_at, decode):
    cfg, w = _needle_model()
    n = 150
    toks = [2 + (i % 50) for i in range(n)]
    toks[needle_at] = 60
    toks[-1] = 60                                        # the last query asks for the marked key
    want = oracle_logits(cfg, w, toks)
    without = list(toks)
    without[needle_at] = 2 + (needle_at % 50)
    # the marked key decides the answer: without it the oracle's last row moves a lot
    assert rel_err(oracle_logits(cfg, w, without)[-1], want[-1]) > 0.1
    hz = Harness(cfg, w, "float32", page_size=16, num_pages=12, slots=1)
    try:
        got = hz.feed("n", toks, cuts=([n - 20, 1] if decode else [n]))
    finally:
        hz.close()
    assert rel_err(got[-1], want[-1]) < TOL["float32"]
    assert rel_err(got, want) < TOL["float32"]


def _needle_model_wide(dim, heads, kv_heads):
    """The marked-key model at key sizes the tensor-core attention serves (bf16 build)."""
    layer = attn_scan(heads=heads, kv_heads=kv_heads, dim=dim, conv=2, coef=0.0, every=1, scale=12.0 / (dim * 7.84), left_scale=1.0,
                      right_scale=0.0)       # a matching key scores about 12
    layer["mlp"] = None
    cfg = model_config([layer], width=64, vocab=64, emb_scale=40.0)      # the token outweighs the position
    w = plain.random_weights(cfg, 33)
    g = torch.Generator().manual_seed(34)
    p = torch.randn(dim, 64, generator=g) * 0.35
    w["l0.mix.left.q"] = torch.cat([p] * heads).to(torch.bfloat16)
    w["l0.mix.left.k"] = torch.cat([p] * kv_heads).to(torch.bfloat16)
    for n, rows in (("q", heads * dim), ("k", kv_heads * dim)):
        c = torch.zeros(rows, 2)
        c[:, 1] = 1.0
        if n == "k":
            c[:, 0], c[:, 1] = 1.0, 0.0   # a key (= value) is the token BEFORE it: the last query matches the key right
                                          # after the marked token and not its own
        w[f"l0.mix.left.{n}.conv"] = c.to(torch.bfloat16)
    w["l0.norm1"] = torch.zeros(64).to(torch.bfloat16)
    w["l0.mix.left.o"] = (w["l0.mix.left.o"].float() * 30.0).to(torch.bfloat16)   # as large as the embedding in the stream
    w["l0.mix.left.sink"] = torch.full((heads,), -2.0).to(torch.bfloat16)
    return cfg, w


@pytest.mark.parametrize("dim,heads,kv_heads", [(64, 4, 2), (32, 8, 1), (128, 2, 2)])
@pytest.mark.parametrize("needle_at", [0, 62, 63, 254, 255, 299])      # marked keys at 1, 63, 64, 255, 256, 300
@pytest.mark.parametrize("decode", [False, True])
def test_marked_key_tensor_core_attention(dim, heads, kv_heads, needle_at, decode):
    cfg, w = _needle_model_wide(dim, heads, kv_heads)
    n = 330
    toks = [2 + (i % 50) for i in range(n)]
    toks[needle_at] = 60
    toks[-1] = 60
    want = oracle_logits(cfg, w, toks)
    without = list(toks)
    without[needle_at] = 2 + (needle_at % 50)
    assert rel_err(oracle_logits(cfg, w, without)[-1], want[-1]) > 0.3
    hz = Harness(cfg, w, "bfloat16", page_size=16, num_pages=24, slots=1)
    try:
        got = hz.feed("n", toks, cuts=([n - 40, 1] if decode else [100, 230]))
    finally:
        hz.close()
    assert rel_err(got[-1], want[-1]) < 2e-2
    assert rel_err(got, want) < 3e-2


@pytest.mark.parametrize("dim,heads,kv_heads", [(64, 4, 2), (32, 16, 2), (128, 4, 1)])
def test_tensor_core_attention_in_a_model(dim, heads, kv_heads):
    cfg = model_config([attn_scan(heads=heads, kv_heads=kv_heads, dim=dim, every=50), delta(),
                        attn_scan(heads=heads, kv_heads=kv_heads, dim=dim, every=64)], width=64)
    w = plain.random_weights(cfg, 90)
    V = cfg["vocab"]
    reqs = {"a": rand_tokens(300, V, 91), "b": rand_tokens(70, V, 92), "c": rand_tokens(3, V, 93)}
    ref = {k: oracle_logits(cfg, w, v) for k, v in reqs.items()}
    hz = Harness(cfg, w, "bfloat16", page_size=16, num_pages=30, slots=3)
    try:
        o1 = hz.step([("a", reqs["a"][:259], range(259)), ("b", reqs["b"][:5], range(5))])
        o2 = hz.step([("a", reqs["a"][259:260], [0]), ("b", reqs["b"][5:70], range(65)), ("c", reqs["c"], range(3))])
        o3 = hz.step([("a", reqs["a"][260:], range(40))])
    finally:
        hz.close()
    a = np.concatenate([o1[:259], o2[:1], o3], 0)
    bb = np.concatenate([o1[259:], o2[1:66]], 0)
    assert rel_err(a, ref["a"]) < TOL["bfloat16"]
    assert rel_err(bb, ref["b"]) < TOL["bfloat16"]
    assert rel_err(o2[66:], ref["c"]) < TOL["bfloat16"]


@pytest.mark.parametrize("sink", [-20.0, 0.0, 8.0])
def test_sink_takes_its_share(sink):
    cfg, w = _needle_model()
    cfg["layers"][0]["mixer"]["left"]["scale"] = 0.05          # scores of a few units, so that a sink of 8 outweighs them
    w["l0.mix.left.sink"] = torch.tensor([sink, sink]).to(torch.bfloat16)
    toks = rand_tokens(40, 64, 9)
    want = oracle_logits(cfg, w, toks)
    if sink == 8.0:                                      # the sink matters: leaving it out changes the answer
        w2 = dict(w)
        w2["l0.mix.left.sink"] = torch.tensor([-30.0, -30.0]).to(torch.bfloat16)
        assert rel_err(oracle_logits(cfg, w2, toks), want) > 0.05
    hz = Harness(cfg, w, "float32", page_size=16, num_pages=4, slots=1)
    try:
        got = hz.feed("s", toks, cuts=[25, 1])
    finally:
        hz.close()
    assert rel_err(got, want) < TOL["float32"]


def test_query_temperature_steps_inside_prompt_and_decoding():
    layer = attn_scan(coef=1.5, every=7, right_scale=0.0)
    cfg = model_config([layer])
    toks = rand_tokens(40, cfg["vocab"], 13)
    got, want = _run(cfg, toks, "float32", cuts=[10, 1])
    flat = copy.deepcopy(cfg)
    flat["layers"][0]["mixer"]["left"]["q_temp"]["coef"] = 0.0
    w = plain.random_weights(cfg, 0)
    assert rel_err(oracle_logits(flat, w, toks)[6:], want[6:]) > 1e-3          # the temperature is visible from p = 6 on
    assert rel_err(got, want) < TOL["float32"]


# ---- the first tokens, long decoding, other sizes --------------------------------------------------------------------------------
@pytest.mark.parametrize("n", [1, 2, 3, 5])
def test_first_tokens(n):
    toks = rand_tokens(n, SMALL["vocab"], 40 + n)
    got, want = _run(SMALL, toks, "float32")
    assert rel_err(got, want) < TOL["float32"]
    single, _ = _run(SMALL, toks, "float32", cuts=[1])
    assert rel_err(single, want) < TOL["float32"]


def test_long_decoding():
    toks = rand_tokens(260, SMALL["vocab"], 50)
    got, want = _run(SMALL, toks, "float32", cuts=[4, 1], num_pages=20)
    assert rel_err(got, want) < TOL["float32"]
    got16, _ = _run(SMALL, toks, "bfloat16", cuts=[4, 1], num_pages=20)
    assert rel_err(got16, want) < TOL["bfloat16"]


OTHER = [
    # one key head, taps of 1, a state of one, rank one, heads == kv_heads == 1 on the delta side, sizes that are not powers of two
    model_config([attn_scan(heads=3, kv_heads=1, dim=24, conv=1, inner=20, state=1, dt_rank=1, sconv=1),
                  delta(heads=1, kv_heads=1, dim=12, vdim=20, conv=1)], width=40, vocab=50),
    # wide state (lanes hold several entries), key size above a warp, many heads sharing one key head
    model_config([delta(heads=6, kv_heads=2, dim=40, vdim=40, conv=5),
                  attn_scan(heads=8, kv_heads=2, dim=48, conv=5, inner=70, state=150, dt_rank=9, sconv=6, every=1)],
                 width=72, vocab=130, emb_scale=1.0, logit_scale=1.0, eps=1e-6),
    # a delta-rule key size beyond what a thread keeps in registers (the state lives in shared memory), width not a multiple of 8
    model_config([delta(heads=2, kv_heads=1, dim=136, vdim=24, conv=2), attn_scan(heads=2, kv_heads=1, dim=40)], width=44, vocab=61),
]


@pytest.mark.parametrize("idx", range(len(OTHER)))
@pytest.mark.parametrize("low", [1, 11])
def test_other_sizes(idx, low):
    cfg = OTHER[idx]
    toks = rand_tokens(60, cfg["vocab"], 60 + idx)
    got, want = _run(cfg, toks, "float32", cuts=[21, 3, 1], low=low, page_size=32, num_pages=4)
    assert rel_err(got, want) < TOL["float32"]


# ---- greedy generation through the engine's own entry point ------------------------------------------------------------------------
def test_greedy_generation_through_llm_generate():
    from jacobiforcing_b200 import LLM, SamplingParams
    from jacobiforcing_b200.hybrid_config import HybridConfig
    w = plain.random_weights(SMALL, 70)
    hc = HybridConfig.from_dict(SMALL, {k: tuple(v.shape) for k, v in w.items()})
    llm = LLM(None, hf_config=hc, state_dict=w, dtype="float32", kvcache_block_size=16, num_kvcache_blocks=16, max_num_seqs=2,
              max_model_len=128, max_num_batched_tokens=24)
    V = SMALL["vocab"]
    prompts = [rand_tokens(30, V, 71), rand_tokens(5, V, 72), rand_tokens(17, V, 73)]      # three requests, two slots,
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True), use_tqdm=False)
    llm.exit()                                                                               # prompts cut at 24 tokens
    for prompt, out in zip(prompts, outs):
        ids = out["token_ids"]
        assert len(ids) == 10
        seq = list(prompt)
        for tok in ids:
            lg = oracle_logits(SMALL, w, seq)[-1]
            top = np.argsort(lg)[::-1]
            assert tok == top[0] or (lg[top[0]] - lg[tok]) < 1e-3 * (lg.max() - lg.min()), "not the oracle's greedy token"
            seq.append(tok)


def test_generate_command_line_and_trace_replay_on_a_checkpoint_directory(tmp_path):
    """A checkpoint directory (config.json + model.safetensors) through the registry: the generate command line gives the
    oracle's greedy tokens, and bin/trace_run writes the oracle's logits for a replayed trace."""
    import json
    import os
    import subprocess
    import sys
    from tests.test_hybrid_host import _write_checkpoint
    w = plain.random_weights(SMALL, 75, low=6)
    _write_checkpoint(tmp_path, SMALL, w)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    prompt = rand_tokens(21, SMALL["vocab"], 76)
    out = subprocess.run([sys.executable, "-m", "jacobiforcing_b200.generate", "--model", str(tmp_path), "--prompt-ids",
                          ",".join(map(str, prompt)), "--max-tokens", "6", "--dtype", "float32", "--page-size", "16",
                          "--max-model-len", "64", "--max-num-batched-tokens", "64"], cwd=root, capture_output=True, text=True)
    assert out.returncode == 0, out.stderr[-2000:]
    ids = json.loads(out.stdout.strip().splitlines()[-1])["token_ids"]
    seq = list(prompt)
    for tok in ids:
        lg = oracle_logits(SMALL, w, seq)[-1]
        assert tok == int(np.argmax(lg)) or lg.max() - lg[tok] < 1e-3 * (lg.max() - lg.min())
        seq.append(tok)
    # trace replay: two requests, portions beside single tokens, one ends and its slot is used again
    a, b = rand_tokens(30, SMALL["vocab"], 77), rand_tokens(9, SMALL["vocab"], 78)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:17], "want": [0, 16]}, {"id": "b", "tokens": b[:2], "want": [1]}], "end": []},
             {"step": 1, "entries": [{"id": "b", "tokens": b[2:], "want": [6]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": a[17:18], "want": [0]}, {"id": "c", "tokens": b, "want": [8]}], "end": ["c"]},
             {"step": 3, "entries": [{"id": "a", "tokens": a[18:], "want": []}], "end": ["a"]}]
    outdir = tmp_path / "out"
    r = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", str(tmp_path), "--dtype", "float32", "--out",
                        str(outdir), "--max-tokens", "128", "--page-size", "16"], input="\n".join(json.dumps(x) for x in steps) + "\n",
                       cwd=root, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [ln for ln in r.stdout.splitlines() if ln.startswith("done")] == ["done 0", "done 1", "done 2", "done 3"]
    la, lb = oracle_logits(SMALL, w, a), oracle_logits(SMALL, w, b)
    V = SMALL["vocab"]
    g0 = np.fromfile(outdir / "0.f32", dtype="<f4").reshape(-1, V)
    g1 = np.fromfile(outdir / "1.f32", dtype="<f4").reshape(-1, V)
    g2 = np.fromfile(outdir / "2.f32", dtype="<f4").reshape(-1, V)
    assert not (outdir / "3.f32").exists()
    assert rel_err(g0, np.stack([la[0], la[16], lb[1]])) < TOL["float32"]
    assert rel_err(g1, lb[8:9]) < TOL["float32"]
    assert rel_err(g2, np.stack([la[17], lb[8]])) < TOL["float32"]


def test_sampling_at_a_temperature_follows_the_distribution():
    from tests.hybrid_helpers import Harness as H
    cfg = model_config([delta(ff=0)], width=32, vocab=12)
    w = plain.random_weights(cfg, 80)
    hz = H(cfg, w, "float32")
    try:
        toks = rand_tokens(6, 12, 81)
        lg = oracle_logits(cfg, w, toks)[-1] / 0.8
        p = np.exp(lg - lg.max())
        p /= p.sum()
        counts = np.zeros(12)
        rt = hz.runner.rt
        for i in range(600):
            r = rt.step([(toks, 0, 0, [0])], [5], want_logits=False, sample=True, temperature=[0.8], seed=1000 + i)
            counts[int(r["sampled"][0])] += 1
        chi2 = float((((counts - 600 * p) ** 2) / (600 * p + 1e-9))[600 * p > 5].sum())
        assert chi2 < 40.0
    finally:
        hz.close()
