"""Famepel on the GPU against the plain fp64 restatement (oracle/famepel_plain.py): each mechanism alone, prefill against
token-by-token decoding, portions, unequal batches, reuse of pages and slots, a marked key far back and at page, key-tile
and key-split borders, the sink, the rotation far from the start, the first tokens of a sequence, long decoding, other
sizes, and greedy generation through LLM.generate, the generate command line and the trace replay."""
import copy

import numpy as np
import pytest
import torch

from oracle import famepel_plain as plain
from tests.famepel_helpers import (SMALL, TOL, Harness, close, glr, latent, model_config, moe, needle_model, needle_tokens,
                                   oracle_logits, rand_tokens, rel_err, run, ssd)

pytestmark = pytest.mark.gpu


# ---- each mechanism alone ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["ssd", "latent", "borrowed", "glr", "experts"])
def test_mechanism_alone(which, dtype):
    layers = {"ssd": [ssd(mlp=None)], "latent": [latent(mlp=None)], "borrowed": [latent(mlp=None), latent(kv_from=0, heads=3, mlp=None)],
              "glr": [glr(mlp=None)], "experts": [glr(heads=1, dim=4, vdim=4)]}[which]
    cfg = model_config(layers)
    toks = rand_tokens(45, cfg["vocab"], 3)
    got, want = run(cfg, toks, dtype)
    assert close(got, want, dtype)


@pytest.mark.parametrize("kw", [dict(experts=8, top=3, count=4, keep=2), dict(experts=5, top=1, count=1, keep=1),
                                dict(experts=6, top=2, count=6, keep=3), dict(experts=9, top=4, count=3, keep=3),
                                dict(experts=40, top=2, count=5, keep=1, ff=9)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_router_shapes(kw, dtype):
    """Groups of two, one group, groups of one expert (a group is worth its single score), every group kept, more experts
    than a warp, an expert size that the tensor-core product does not take; many tokens so that the expert-sorted path
    runs, few so that the per-pair path runs."""
    cfg = model_config([glr(heads=1, dim=4, vdim=4, mlp=moe(**kw)), ssd(heads=2, vdim=4, state=3, groups=1, norm_groups=1, mlp=moe(**kw))])
    toks = rand_tokens(80, cfg["vocab"], 4)
    got, want = run(cfg, toks, dtype, cuts=[60, 1, 7, 1])
    assert close(got, want, dtype)


# ---- prefill == decode, portions -------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prefill_equals_token_by_token(dtype):
    toks = rand_tokens(70, SMALL["vocab"], 5)
    whole, want = run(SMALL, toks, dtype)
    single, _ = run(SMALL, toks, dtype, cuts=[1])
    assert close(whole, want, dtype)
    assert close(single, want, dtype)
    if dtype == "float32":
        assert close(single, whole)


@pytest.mark.parametrize("cuts", [[2], [3, 2, 7, 1, 16, 5], [17, 2, 2, 31], [33, 1]])
def test_portions(cuts):
    toks = rand_tokens(90, SMALL["vocab"], 7)
    got, want = run(SMALL, toks, "float32", cuts=cuts)
    assert close(got, want)


def test_step_larger_than_the_runner_capacity_is_cut():
    toks = rand_tokens(100, SMALL["vocab"], 8)
    got, want = run(SMALL, toks, "float32", max_step_tokens=32)
    assert close(got, want)


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
        assert close(np.concatenate(got[k], 0), ref[k], dtype), k


def test_slot_and_pages_used_again_start_from_the_empty_state():
    w = plain.random_weights(SMALL, 12)
    V = SMALL["vocab"]
    hz = Harness(SMALL, w, "float32", page_size=16, num_pages=4, slots=1)
    try:
        for i in range(3):
            toks = rand_tokens(40 + i, V, 20 + i)
            got = hz.feed("x", toks, cuts=[13, 1])
            hz.end("x")
            assert close(got, oracle_logits(SMALL, w, toks))
    finally:
        hz.close()


# ---- a key that must be found: far back, at page borders, at key-tile and key-split borders -----------------------------------
@pytest.mark.parametrize("needle_at", [0, 1, 15, 16, 31, 32, 47, 48, 63, 64, 140])
@pytest.mark.parametrize("decode", [False, True])
def test_marked_key_far_back_is_found(needle_at, decode):
    cfg, w = needle_model()
    n = 150
    toks, without = needle_tokens(n, needle_at)
    want = oracle_logits(cfg, w, toks)
    assert rel_err(oracle_logits(cfg, w, without)[-1], want[-1]) > 0.3      # the marked key decides the answer
    hz = Harness(cfg, w, "float32", page_size=16, num_pages=12, slots=1)
    try:
        got = hz.feed("n", toks, cuts=([n - 20, 1] if decode else [n]))
    finally:
        hz.close()
    assert rel_err(got[-1], want[-1]) < TOL["float32"]
    assert rel_err(got, want) < TOL["float32"]


@pytest.mark.parametrize("sizes", [dict(), dict(rank=48, rot_dim=16, dim=16, heads=4, vdim=24, width=64),
                                   dict(rank=96, rot_dim=32, dim=24, heads=8, vdim=16, width=64),
                                   dict(rank=40, rot_dim=8, dim=16, heads=3, vdim=24, width=64),
                                   dict(rank=200, rot_dim=24, dim=16, heads=5, vdim=24, width=64),
                                   dict(rank=512, rot_dim=64, dim=32, heads=16, vdim=16, width=64),
                                   dict(rank=36, rot_dim=6, dim=16, heads=2, vdim=24, width=64)])
@pytest.mark.parametrize("needle_at", [0, 62, 63, 64, 255, 256, 300])
@pytest.mark.parametrize("decode", [False, True])
def test_marked_key_bfloat16_attention(sizes, needle_at, decode):
    """Cache rows of 32, 64 and 128 elements take the narrow tensor-core attention (64-key tiles, key splits of 256); rows
    of 48 (three heads), 224 (five heads) and 576 elements the wide one; rows of 42 elements the warp-per-row kernel."""
    cfg, w = needle_model(**sizes)
    n = 330
    toks, without = needle_tokens(n, needle_at)
    want = oracle_logits(cfg, w, toks)
    assert rel_err(oracle_logits(cfg, w, without)[-1], want[-1]) > 0.3
    hz = Harness(cfg, w, "bfloat16", page_size=16, num_pages=24, slots=1)
    try:
        got = hz.feed("n", toks, cuts=([n - 40, 1] if decode else [100, 230]))
    finally:
        hz.close()
    assert rel_err(got[-1], want[-1]) < 4e-2
    assert rel_err(got, want) < 0.15        # the other rows: random scores of +-20 under a sharp softmax magnify the rounding


@pytest.mark.parametrize("sink", [-20.0, 0.0, 8.0])
def test_sink_takes_its_share(sink):
    cfg, w = needle_model(scale=0.05)                       # scores of a few units, so that a sink of 8 outweighs them
    w["l0.mix.sink"] = torch.tensor([sink, sink]).to(torch.bfloat16)
    toks = rand_tokens(40, 64, 9)
    want = oracle_logits(cfg, w, toks)
    if sink == 8.0:                                      # the sink matters: leaving it out changes the answer
        w2 = dict(w)
        w2["l0.mix.sink"] = torch.tensor([-30.0, -30.0]).to(torch.bfloat16)
        assert rel_err(oracle_logits(cfg, w2, toks), want) > 0.05
    for dtype in ("float32", "bfloat16"):
        hz = Harness(cfg, w, dtype, page_size=16, num_pages=4, slots=1)
        try:
            got = hz.feed("s", toks, cuts=[25, 1])
        finally:
            hz.close()
        assert rel_err(got, want) < TOL[dtype]


@pytest.mark.parametrize("scaling", [None, {"factor": 8.0, "original": 64, "fast": 8.0, "slow": 1.0}])
@pytest.mark.parametrize("dims", [12, 6])
def test_rotation_decides_far_from_the_start(scaling, dims):
    """The rotated part carries the score (its projections are eight times louder than the rest), positions run to 400, in
    a prompt and in decoding; a plain rotation and an interpolated one; a rotation over half of the rotated part."""
    cfg = model_config([latent(mlp=None, base=50.0, dims=dims, scaling=scaling, scale=0.4)])
    w = plain.random_weights(cfg, 21)
    uq = w["l0.mix.uq"].float().view(4, 20, -1)
    uq[:, 8:] *= 8.0
    w["l0.mix.uq"] = uq.reshape(80, -1).to(torch.bfloat16)
    toks = rand_tokens(400, cfg["vocab"], 22)
    want = oracle_logits(cfg, w, toks)
    flat = copy.deepcopy(cfg)
    flat["layers"][0]["mixer"]["rot"]["base"] = 50.5
    assert rel_err(oracle_logits(flat, w, toks)[300:], want[300:]) > 0.02        # a frequency 1 % off shows
    got, _ = run(cfg, toks, "float32", cuts=[370, 1], weights=w, page_size=32, num_pages=13)
    assert rel_err(got, want) < TOL["float32"]


# ---- the first tokens, long decoding, other sizes --------------------------------------------------------------------------------
@pytest.mark.parametrize("n", [1, 2, 3, 5])
def test_first_tokens(n):
    toks = rand_tokens(n, SMALL["vocab"], 40 + n)
    got, want = run(SMALL, toks, "float32")
    assert close(got, want)
    single, _ = run(SMALL, toks, "float32", cuts=[1])
    assert close(single, want)


def test_long_decoding():
    toks = rand_tokens(260, SMALL["vocab"], 50)
    got, want = run(SMALL, toks, "float32", cuts=[4, 1], num_pages=20)
    assert close(got, want)
    got16, _ = run(SMALL, toks, "bfloat16", cuts=[4, 1], num_pages=20)
    assert close(got16, want, "bfloat16")


OTHER = [
    # everything equal to one where it can be: one head, one group, one state, one tap, one norm part, one expert
    model_config([ssd(heads=1, vdim=8, state=1, groups=1, conv=1, norm_groups=1, mlp=moe(experts=1, top=1, count=1, keep=1, ff=8)),
                  latent(heads=1, dim=4, rot_dim=2, vdim=4, kv_rank=6, q_rank=3, mlp=None),
                  glr(heads=1, dim=1, vdim=1, mlp=None)], width=24, vocab=50),
    # groups == heads, norm parts == channels per part of one, a wide state (lanes hold several entries), many taps,
    # a key size above a warp on the gated recurrence, an odd head count in attention, no rotated part at all
    model_config([ssd(heads=6, vdim=7, state=300, groups=6, conv=6, norm_groups=42),
                  glr(heads=2, dim=40, vdim=70),
                  latent(heads=5, dim=12, rot_dim=0, vdim=9, kv_rank=33, q_rank=17, scaling=None),
                  latent(heads=7, dim=6, rot_dim=0, vdim=5, kv_rank=33, q_rank=8, scaling=None, kv_from=2)],
                 width=72, vocab=130, emb_scale=1.0, eps=1e-6),
    # head sizes beyond what a thread keeps in registers (the state lives in shared memory), width not a multiple of 8,
    # a cache row wider than the tensor-core attention serves, borrowed twice
    model_config([glr(heads=2, dim=136, vdim=24), latent(heads=2, dim=20, rot_dim=24, vdim=40, kv_rank=200, q_rank=50),
                  ssd(heads=3, vdim=40, state=33, groups=3, conv=2, norm_groups=2), latent(heads=4, dim=8, rot_dim=24, vdim=10,
                                                                                          kv_rank=200, q_rank=12, kv_from=1),
                  latent(heads=1, dim=8, rot_dim=24, vdim=10, kv_rank=200, q_rank=12, kv_from=1, dims=10)], width=44, vocab=61),
]


@pytest.mark.parametrize("idx", range(len(OTHER)))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_other_sizes(idx, dtype):
    cfg = OTHER[idx]
    toks = rand_tokens(60, cfg["vocab"], 60 + idx)
    got, want = run(cfg, toks, dtype, cuts=[21, 3, 1], page_size=32, num_pages=4)
    assert close(got, want, dtype)


# ---- greedy generation through the engine's own entry points ------------------------------------------------------------------------
def _greedy_ok(cfg, w, prompt, ids):
    seq = list(prompt)
    for tok in ids:
        lg = oracle_logits(cfg, w, seq)[-1]
        assert tok == int(np.argmax(lg)) or lg.max() - lg[tok] < 1e-3 * (lg.max() - lg.min()), "not the oracle's greedy token"
        seq.append(tok)


def test_greedy_generation_through_llm_generate():
    from jacobiforcing_b200 import LLM, SamplingParams
    from jacobiforcing_b200.hybrid_config import HybridConfig
    w = plain.random_weights(SMALL, 70)
    hc = HybridConfig.from_dict(SMALL)
    llm = LLM(None, hf_config=hc, state_dict=w, dtype="float32", kvcache_block_size=16, num_kvcache_blocks=16, max_num_seqs=2,
              max_model_len=128, max_num_batched_tokens=24)
    V = SMALL["vocab"]
    prompts = [rand_tokens(30, V, 71), rand_tokens(5, V, 72), rand_tokens(17, V, 73)]      # three requests, two slots,
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True), use_tqdm=False)
    llm.exit()                                                                               # prompts cut at 24 tokens
    for prompt, out in zip(prompts, outs):
        assert len(out["token_ids"]) == 8
        _greedy_ok(SMALL, w, prompt, out["token_ids"])


def test_generate_command_line_and_trace_replay_on_a_checkpoint_directory(tmp_path):
    import json
    import os
    import subprocess
    import sys
    from tests.test_hybrid_host import _write_checkpoint
    w = plain.random_weights(SMALL, 75)
    _write_checkpoint(tmp_path, SMALL, w)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    prompt = rand_tokens(21, SMALL["vocab"], 76)
    out = subprocess.run([sys.executable, "-m", "jacobiforcing_b200.generate", "--model", str(tmp_path), "--prompt-ids",
                          ",".join(map(str, prompt)), "--max-tokens", "6", "--dtype", "float32", "--page-size", "16",
                          "--max-model-len", "64", "--max-num-batched-tokens", "64"], cwd=root, capture_output=True, text=True)
    assert out.returncode == 0, out.stderr[-2000:]
    _greedy_ok(SMALL, w, prompt, json.loads(out.stdout.strip().splitlines()[-1])["token_ids"])
    # trace replay: two requests, portions beside single tokens, one ends and its slot and pages are used again
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
