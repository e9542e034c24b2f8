"""Shared pieces of the layered-hybrid-decoder tests: small configurations, random bf16 weights, a harness that drives
the engine's scheduler and step function the way a trace replay does, and the error measure against the plain oracle."""
from __future__ import annotations

import copy

import numpy as np
import torch

from oracle import kinetar_plain as plain


def attn_scan(heads=4, kv_heads=2, dim=16, conv=3, coef=0.4, every=5, scale=0.3, inner=40, state=12, dt_rank=3,
              sconv=2, left_scale=0.7, right_scale=1.1):
    return {"type": "parallel",
            "mixer": {"left": {"conv": conv, "dim": dim, "heads": heads, "kv_heads": kv_heads,
                               "q_temp": {"coef": coef, "every": every}, "scale": scale, "vdim": dim},
                      "left_scale": left_scale,
                      "right": {"conv": sconv, "dt_rank": dt_rank, "inner": inner, "state": state},
                      "right_scale": right_scale},
            "mlp": {"ff": 72, "kind": "dense"}}


def delta(heads=4, kv_heads=2, dim=8, vdim=24, conv=3, ff=72):
    return {"type": "channel_delta", "mixer": {"conv": conv, "dim": dim, "heads": heads, "kv_heads": kv_heads, "vdim": vdim},
            "mlp": ({"ff": ff, "kind": "dense"} if ff else None)}


def model_config(layers, width=48, vocab=80, emb_scale=6.0, logit_scale=0.7, eps=1e-5):
    return {"architecture": "Kinetar", "embedding": {"scale": emb_scale}, "layers": copy.deepcopy(layers),
            "logit_scale": logit_scale, "norm": {"eps": eps}, "vocab": vocab, "width": width}


SMALL = model_config([attn_scan(), delta(), attn_scan(heads=2, kv_heads=2, dim=32, conv=4, inner=24, state=5, dt_rank=2, sconv=4),
                      delta(heads=2, kv_heads=1, dim=16, vdim=8, conv=2, ff=0)])


def oracle_logits(config, weights, tokens, dtype=torch.float64):
    return plain.forward(config, weights, list(tokens), dtype=dtype).numpy()


def rel_err(got: np.ndarray, want: np.ndarray) -> float:
    """Root mean square of the centred difference over the centred reference, worst row."""
    got, want = np.atleast_2d(got).astype(np.float64), np.atleast_2d(want).astype(np.float64)
    d = got - want
    d = d - d.mean(1, keepdims=True)
    w = want - want.mean(1, keepdims=True)
    return float((np.sqrt((d ** 2).mean(1)) / np.sqrt((w ** 2).mean(1) + 1e-30)).max())


TOL = {"float32": 3e-4, "bfloat16": 6e-2}


class Harness:
    """Scheduler + runner wired as the engine wires them; requests are fed portion by portion."""

    def __init__(self, config, weights, dtype="float32", page_size=16, num_pages=24, slots=4, low=8, max_step_tokens=512):
        from jacobiforcing_b200.config import Config
        from jacobiforcing_b200.engine.hybrid_runner import HybridModelRunner
        from jacobiforcing_b200.engine.scheduler import Scheduler
        from jacobiforcing_b200.hybrid_config import HybridConfig
        shapes = {k: tuple(v.shape) for k, v in weights.items()}
        hc = HybridConfig.from_dict(config, shapes)
        self.cfg = Config(None, hf_config=hc, state_dict=weights, dtype=dtype, kvcache_block_size=page_size,
                          num_kvcache_blocks=num_pages, max_num_seqs=slots, num_state_slots=slots,
                          max_model_len=page_size * num_pages, max_num_batched_tokens=max_step_tokens)
        self.runner = HybridModelRunner(self.cfg, 0, [])
        self.sched = Scheduler(self.cfg)
        self.runner.block_manager = self.sched.block_manager
        self.live = {}

    def step(self, entries):
        """entries: [(id, tokens, want offsets)] -> logits [sum(want), vocab] in entry order."""
        from jacobiforcing_b200.engine.sequence import Sequence
        from jacobiforcing_b200.sampling_params import SamplingParams
        portions, want = [], []
        for rid, toks, w in entries:
            seq = self.live.get(rid)
            if seq is None:
                seq = Sequence(list(toks), SamplingParams(temperature=0.0))
                self.sched.admit(seq)
                self.live[rid] = seq
            else:
                seq.extend_tokens(list(toks))
            self.sched.reserve(seq, len(seq))
            portions.append((seq, len(toks)))
            want.append(list(w))
        out = self.runner.run_portions(portions, want)
        for seq, n in portions:
            seq.num_cached_tokens += n
        return out

    def end(self, rid):
        self.sched.release(self.live.pop(rid))

    def feed(self, rid, tokens, cuts=None):
        """All logits of one request fed alone in portions of the given sizes (the last size repeats)."""
        cuts = list(cuts or [len(tokens)])
        outs, at, i = [], 0, 0
        while at < len(tokens):
            n = min(cuts[min(i, len(cuts) - 1)], len(tokens) - at)
            outs.append(self.step([(rid, tokens[at:at + n], range(n))]))
            at += n
            i += 1
        return np.concatenate(outs, 0)

    def close(self):
        self.runner.exit()


def rand_tokens(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()
