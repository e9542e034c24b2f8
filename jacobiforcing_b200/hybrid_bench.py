"""Throughput of the layered hybrid decoder (Kinetar) beside the Qwen2 engine at equal width / depth / feed-forward size:
prefill tokens/s, decode tokens/s, device time per kernel group of the hybrid decoder with its distance from the
roofline (tensor peak for prefill products, HBM bandwidth for decode).  Random weights, synthetic tokens.  Used by
`bench.py --compare-hybrid`."""
from __future__ import annotations

import time
from typing import Dict, List

import numpy as np

SIZES = {
    "w1024": dict(width=1024, layers=4, ff=4096, heads=8, kv_heads=2, dim=128, vocab=32000),
    "w2048": dict(width=2048, layers=4, ff=8192, heads=16, kv_heads=4, dim=128, vocab=32000),
    "w4096": dict(width=4096, layers=2, ff=14336, heads=32, kv_heads=8, dim=128, vocab=32000),
}


def hybrid_description(sz: dict) -> dict:
    W = sz["width"]
    par = {"type": "parallel",
           "mixer": {"left": {"conv": 4, "dim": sz["dim"], "heads": sz["heads"], "kv_heads": sz["kv_heads"],
                              "q_temp": {"coef": 0.5, "every": 1024}, "scale": sz["dim"] ** -0.5, "vdim": sz["dim"]},
                     "left_scale": 0.7,
                     "right": {"conv": 4, "dt_rank": W // 16, "inner": 2 * W, "state": 16}, "right_scale": 0.7},
           "mlp": {"ff": sz["ff"], "kind": "dense"}}
    dl = {"type": "channel_delta",
          "mixer": {"conv": 4, "dim": 128, "heads": W // 128, "kv_heads": max(1, W // 256), "vdim": 128},
          "mlp": {"ff": sz["ff"], "kind": "dense"}}
    layers = [par if i % 2 == 0 else dl for i in range(sz["layers"])]
    return {"architecture": "Kinetar", "embedding": {"scale": 1.0}, "layers": layers, "logit_scale": 1.0,
            "norm": {"eps": 1e-6}, "vocab": sz["vocab"], "width": W}


def hybrid_weights(desc: dict, seed: int, low: int = 64) -> Dict[str, np.ndarray]:
    rng = np.random.default_rng(seed)
    W, V = desc["width"], desc["vocab"]

    def lin(n, k):
        return (rng.standard_normal((n, k), dtype=np.float32) / np.sqrt(k)).astype(np.float32)

    def vec(n, s=0.1, b=0.0):
        return (rng.standard_normal(n, dtype=np.float32) * s + b).astype(np.float32)
    w = {"embed": lin(V, W) * 4.0, "final.norm": vec(W), "head": lin(V, W)}
    for i, lc in enumerate(desc["layers"]):
        p, m = f"l{i}.", lc["mixer"]
        w[p + "norm1"] = vec(W)
        if lc["type"] == "parallel":
            a, s = m["left"], m["right"]
            nq, nk, I, N, R = a["heads"] * a["dim"], a["kv_heads"] * a["dim"], s["inner"], s["state"], s["dt_rank"]
            L, Rt = p + "mix.left.", p + "mix.right."
            w.update({L + "q": lin(nq, W), L + "k": lin(nk, W), L + "q.conv": vec((nq, a["conv"]), 0.5),
                      L + "k.conv": vec((nk, a["conv"]), 0.5), L + "sink": vec(a["heads"], 1.0), L + "g": lin(nq, W),
                      L + "o": lin(W, nq), Rt + "in": lin(2 * I, W), Rt + "conv": vec((I, s["conv"]), 0.5),
                      Rt + "conv.b": vec(I), Rt + "x": lin(R + 2 * N, I), Rt + "dt": lin(I, R), Rt + "dt.b": vec(I, 0.5, -1.0),
                      Rt + "A_log": np.log(rng.uniform(0.2, 3.0, (I, N))).astype(np.float32), Rt + "D": vec(I, 0.3, 1.0),
                      Rt + "o": lin(W, I)})
        else:
            nq, nv = m["kv_heads"] * m["dim"], m["heads"] * m["vdim"]
            M = p + "mix."
            w.update({M + "q": lin(nq, W), M + "k": lin(nq, W), M + "v": lin(nv, W), M + "q.conv": vec((nq, m["conv"]), 0.5),
                      M + "k.conv": vec((nq, m["conv"]), 0.5), M + "v.conv": vec((nv, m["conv"]), 0.5),
                      M + "b": lin(m["heads"], W), M + "A_log": np.log(rng.uniform(0.1, 1.5, m["heads"])).astype(np.float32),
                      M + "norm": vec(m["vdim"], 0.2, 1.0), M + "a1": lin(low, W), M + "a2": lin(m["heads"] * m["dim"], low),
                      M + "dt_bias": vec(m["heads"] * m["dim"], 0.5, -1.0), M + "g1": lin(low, W), M + "g2": lin(nv, low),
                      M + "o": lin(W, nv)})
        w[p + "mlp.up"] = lin(lc["mlp"]["ff"], W)
        w[p + "mlp.down"] = lin(W, lc["mlp"]["ff"])
    return w


def _hybrid_costs(desc: dict, hc) -> dict:
    """Multiply-add FLOPs per token and weight bytes per kernel group (bf16 weights)."""
    W = desc["width"]
    per = {"gemm_in": 0, "gemm_out": 0, "small_gemm": 0}
    for s in hc.layers:
        if s.mixer == 0:
            n_in = s.a_heads * s.a_dim + s.a_kv_heads * s.a_dim + s.a_heads * s.a_vdim + 2 * s.s_inner + s.ff
            k_out = s.a_heads * s.a_vdim + s.s_inner + s.ff
            small = (s.s_dt_rank + 2 * s.s_state) * s.s_inner + s.s_inner * s.s_dt_rank
        else:
            nq, nv = s.d_kv_heads * s.d_dim, s.d_heads * s.d_vdim
            n_in = 2 * nq + nv + s.d_heads + s.d_low_a + s.d_low_g + s.ff
            k_out = nv + s.ff
            small = s.d_heads * s.d_dim * s.d_low_a + nv * s.d_low_g
        per["gemm_in"] += n_in * W
        per["gemm_out"] += k_out * W
        per["small_gemm"] += small
    per["head"] = desc["vocab"] * W
    return per


def run_hybrid(size: str, prompt: int, decode_steps: int, batches: List[int], peaks: dict, seed: int = 0) -> dict:
    from .hybrid_config import HybridConfig
    from .hybrid_runtime import HybridRuntime
    sz = SIZES[size]
    desc = hybrid_description(sz)
    w = hybrid_weights(desc, seed)
    hc = HybridConfig.from_dict(desc, {k: v.shape for k, v in w.items()})
    page = 256
    maxb = max(batches)
    pages_per = -(-(prompt + decode_steps + 1) // page)
    rt = HybridRuntime(hc, dtype="bfloat16", max_step_tokens=2048, max_step_entries=maxb, page_size=page,
                       num_pages=pages_per * maxb, max_pages_per_seq=pages_per, num_slots=maxb, max_want=maxb)
    rt.load_state_dict(w)
    del w
    rng = np.random.default_rng(seed + 1)
    toks = rng.integers(0, sz["vocab"], prompt + decode_steps + 1).tolist()
    costs = _hybrid_costs(desc, hc)
    out = {"size": size, "description": {k: sz[k] for k in sz}, "memory": rt.memory_info()}

    def prefill(slot):
        ms, at = 0.0, 0
        pages = list(range(slot * pages_per, (slot + 1) * pages_per))
        while at < prompt:
            n = min(2048, prompt - at)
            rt.step([(toks[at:at + n], at, slot, pages)], [n - 1] if at + n == prompt else [], want_logits=False, sample=True)
            ms += float(rt.lib.hy_last_step_ms(rt.h))
            at += n
        return ms
    for _ in range(3):
        prefill(0)
    rt.profile(True)
    t0 = time.perf_counter()
    runs = [prefill(0) for _ in range(3)]
    wall = (time.perf_counter() - t0) / 3
    prof = rt.profile_read()
    rt.profile(False)
    ms = float(np.median(runs))
    out["prefill"] = {"tokens": prompt, "device_ms": ms, "tokens_per_s": prompt / ms * 1e3, "e2e_tokens_per_s": prompt / wall,
                      "ms_by_group": {k: v / 3 for k, v in prof.items()}}
    tf = {}
    for g in ("gemm_in", "gemm_out"):
        t = prof[g] / 3 * 1e-3
        tf[g] = {"tflops": 2.0 * costs[g] * prompt / t / 1e12, "of_measured_bf16_peak": 2.0 * costs[g] * prompt / t / 1e12 / peaks["bf16_tflops"]}
    out["prefill"]["roofline"] = tf
    out["decode"] = {}
    for B in batches:
        for s in range(B):
            prefill(s)
        entries = lambda step: [([toks[prompt + step]], prompt + step, s, list(range(s * pages_per, (s + 1) * pages_per)))
                                for s in range(B)]
        for step in range(3):
            rt.step(entries(step), list(range(B)), want_logits=False, sample=True)
        rt.profile(True)
        ms = 0.0
        t0 = time.perf_counter()
        for step in range(3, decode_steps):
            rt.step(entries(step), list(range(B)), want_logits=False, sample=True)
            ms += float(rt.lib.hy_last_step_ms(rt.h))
        wall = time.perf_counter() - t0
        n = decode_steps - 3
        prof = rt.profile_read()
        rt.profile(False)
        roof = {}
        for g in ("gemm_in", "gemm_out", "head"):
            t = prof[g] / n * 1e-3
            roof[g] = {"gb_per_s": 2.0 * costs[g] / t / 1e9, "of_measured_hbm": 2.0 * costs[g] / t / 1e9 / peaks["hbm_gbs"]}
        wbytes = 2.0 * sum(costs.values())
        out["decode"][f"batch{B}"] = {"ms_per_step": ms / n, "tokens_per_s": B * n / ms * 1e3, "e2e_tokens_per_s": B * n / wall,
                                      "ms_by_group": {k: v / n for k, v in prof.items()}, "roofline": roof,
                                      "weights_over_time_of_measured_hbm": wbytes / (ms / n * 1e-3) / 1e9 / peaks["hbm_gbs"]}
    out["launches"] = rt.launches
    rt.close()
    return out


def run_qwen2(size: str, prompt: int, decode_steps: int, batches: List[int], peaks: dict, seed: int = 0) -> dict:
    """The closest existing model: Qwen2 of the same width / depth / feed-forward / heads through JacobiRuntime (prefill in
    chunks of 2048 rows; decoding = one row per request per forward)."""
    import torch
    from .runtime import JacobiRuntime, PAGE
    sz = SIZES[size]
    cfg = dict(hidden_size=sz["width"], num_hidden_layers=sz["layers"], num_attention_heads=sz["heads"],
               num_key_value_heads=sz["kv_heads"], head_dim=sz["dim"], intermediate_size=sz["ff"], vocab_size=sz["vocab"],
               tie_word_embeddings=False, rope_theta=1e6, max_position_embeddings=32768, rms_norm_eps=1e-6)
    maxb = max(batches)
    pages_per = -(-(prompt + decode_steps + 64) // PAGE)
    rt = JacobiRuntime(cfg, max_rows=2048, max_seqs=maxb, num_kv_pages=pages_per * maxb + 1, max_pages_per_seq=pages_per)
    import bench as _bench
    _bench.load_random_weights(rt, cfg, seed, "cuda")
    hd = cfg["head_dim"]
    inv = 1.0 / (cfg["rope_theta"] ** (torch.arange(0, hd, 2, dtype=torch.float32) / hd))
    ang = torch.arange(prompt + decode_steps + 64, dtype=torch.float32)[:, None] * inv[None, :]
    emb = torch.cat([ang, ang], -1)
    rt.set_rope_tables(emb.cos().numpy(), emb.sin().numpy())
    rng = np.random.default_rng(seed + 1)
    toks = rng.integers(0, sz["vocab"], prompt + decode_steps + 1).tolist()
    out = {"size": size}

    def prefill():
        s = rt.new_sequence()
        _, _, ms = rt.prefill(s, toks[:prompt], [])
        return s, ms
    for _ in range(3):
        s, _ = prefill()
        rt.release(s)
    runs = []
    t0 = time.perf_counter()
    for _ in range(3):
        s, ms = prefill()
        rt.release(s)
        runs.append(ms)
    wall = (time.perf_counter() - t0) / 3
    ms = float(np.median(runs))
    W, I, L = sz["width"], sz["ff"], sz["layers"]
    qkv = (sz["heads"] + 2 * sz["kv_heads"]) * sz["dim"]
    wparams = L * (qkv * W + sz["heads"] * sz["dim"] * W + 3 * W * I)
    out["prefill"] = {"tokens": prompt, "device_ms": ms, "tokens_per_s": prompt / ms * 1e3, "e2e_tokens_per_s": prompt / wall,
                      "layer_gemm_tflops_if_all_time_were_gemm": 2.0 * wparams * prompt / (ms * 1e-3) / 1e12}
    out["decode"] = {}
    for B in batches:
        seqs = [prefill()[0] for _ in range(B)]
        ms, n = 0.0, 0
        t0 = None
        for step in range(decode_steps):
            if step == 3:
                t0 = time.perf_counter()
            groups = [(k, 1, k, prompt + step) for k in range(B)]
            commits = [(k, k, prompt + step) for k in range(B)]
            for s in seqs:
                rt.ensure_capacity(s, prompt + step + 1)
            r = rt.forward([toks[prompt + step]] * B, groups, seqs, 0, B, commits)
            if step >= 3:
                ms += r["ms"]
                n += 1
        wall = time.perf_counter() - t0
        wbytes = 2.0 * (wparams + sz["vocab"] * W)
        out["decode"][f"batch{B}"] = {"ms_per_step": ms / n, "tokens_per_s": B * n / ms * 1e3, "e2e_tokens_per_s": B * n / wall,
                                      "weights_over_time_of_measured_hbm": wbytes / (ms / n * 1e-3) / 1e9 / peaks["hbm_gbs"]}
        for s in seqs:
            rt.release(s)
    out["launches"] = int(rt.launches)
    rt.close()
    return out
