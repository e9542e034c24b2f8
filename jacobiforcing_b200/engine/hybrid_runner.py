"""HybridModelRunner — the per-rank operator of layered hybrid decoders (attention layers over a paged cache, recurrent
layers over state slots).  Same place in the engine as ModelRunner (`call("run", ...)`), but the unit of work is a
*portion*: the next tokens of a live request, a slice of its prompt or one decoded token.  One step runs all portions of
a batch together through libjf_hybrid.so against the paged key cache (pages from the scheduler's BlockManager) and the
request's recurrent-state slot (StateSlotManager)."""
from __future__ import annotations

import random
from typing import List, Optional, Sequence as Seq, Tuple

import numpy as np

from ..config import Config
from ..hybrid_runtime import HybridRuntime
from .sequence import Sequence


class HybridModelRunner:
    def __init__(self, config: Config, rank: int = 0, event=None):
        if config.tensor_parallel_size != 1:
            raise NotImplementedError("layered hybrid decoders run on one GPU")
        self.config = config
        self.rank = rank
        hc = config.hf_config
        page = config.kvcache_block_size
        self.block_size = page
        self.max_pages_per_seq = -(-(config.max_model_len + 1) // page)
        if config.num_kvcache_blocks <= 0:
            config.num_kvcache_blocks = self._size_cache(hc, config)
        slots = getattr(config, "num_state_slots", 0) or min(config.max_num_seqs, 64)
        config.num_state_slots = slots
        self.max_step_tokens = int(min(config.max_num_batched_tokens, 8192))
        self.rt = HybridRuntime(hc, dtype=getattr(config, "dtype", "bfloat16"), device=config.device,
                                max_step_tokens=self.max_step_tokens, max_step_entries=max(slots, 1), page_size=page,
                                num_pages=config.num_kvcache_blocks, max_pages_per_seq=self.max_pages_per_seq,
                                num_slots=slots, max_want=self.max_step_tokens)
        if config.state_dict is not None:
            self.rt.load_state_dict(config.state_dict)
        else:
            self.rt.load_dir(config.model)
        self.kv_cache = ("device", config.num_kvcache_blocks)
        self.block_manager = None
        self._rng = random.Random(config.draft_seed)

    @staticmethod
    def _size_cache(hc, config: Config) -> int:
        """Pages for max_num_seqs requests of max_model_len tokens, capped by a share of the device memory."""
        per_page = sum(2 * s.cache_elems_per_token() for s in hc.layers) * config.kvcache_block_size
        want = config.max_num_seqs * (-(-config.max_model_len // config.kvcache_block_size) + 1)
        cap = int(64e9 * config.gpu_memory_utilization // max(per_page, 1))
        return int(max(4, min(want, cap, 65536)))

    def call(self, method_name, *args):
        return getattr(self, method_name)(*args)

    def exit(self):
        self.rt.close()

    # ---- the step function ----------------------------------------------------------------------------------------------
    def run_portions(self, portions: Seq[Tuple[Sequence, int]], want: Optional[Seq[Seq[int]]] = None,
                     want_layers: bool = False):
        """portions: (request, n) = feed the request's next n tokens (those after `num_cached_tokens`).
        want: None = sample one token after every portion that ends the request's known tokens (generation), else for every
        portion the offsets inside it whose logits are returned (scoring).  Steps that exceed the runner's token capacity
        are cut into sub-steps; nothing a request computes depends on the cut."""
        assert portions
        if want is not None:
            logits = self._forward(portions, want, want_layers=want_layers)
            return logits
        wanted = [[n - 1] if seq.num_cached_tokens + n == len(seq) else [] for seq, n in portions]
        temps = [float(seq.temperature) for (seq, n), w in zip(portions, wanted) if w]
        out = self._forward(portions, wanted, sample=True, temperature=temps)
        it = iter(out)
        return [int(next(it)) if w else None for w in wanted]

    def _forward(self, portions, want, *, sample=False, temperature=None, want_layers=False):
        cap = self.max_step_tokens
        results = []
        layers = []
        # sub-steps: walk the portions in order, cutting where the capacity runs out
        cursor = [(seq, seq.num_cached_tokens, n, list(w)) for (seq, n), w in zip(portions, want)]
        ti = 0
        while cursor:
            entries, wl, used, rest = [], [], 0, []
            for seq, pos0, n, w in cursor:
                room = cap - used
                take = min(n, room) if len(entries) < self.rt.max_step_entries else 0
                if take > 0:
                    toks = seq.token_ids[pos0:pos0 + take]
                    if seq.state_slot < 0:
                        raise RuntimeError("request without a state slot (admit it through the scheduler first)")
                    entries.append((toks, pos0, seq.state_slot, seq.block_table))
                    wl.extend(used + k for k in w if k < take)
                    used += take
                if take < n:
                    rest.append((seq, pos0 + take, n - take, [k - take for k in w if k >= take]))
            cursor = rest
            nw = len(wl)
            temp = None
            if sample and nw:
                temp = temperature[ti:ti + nw]
                ti += nw
            r = self.rt.step(entries, wl, want_logits=not sample, sample=sample, temperature=temp,
                             seed=self._rng.getrandbits(63), want_layers=want_layers)
            if nw:
                results.append(r["sampled"] if sample else r["logits"])
            if want_layers:
                layers.append(r["layers"])
        if want_layers:
            return (np.concatenate(results, 0) if results else None), layers
        if not results:
            return np.empty((0,), dtype=np.int32) if sample else np.empty((0, self.rt.vocab), dtype=np.float32)
        return np.concatenate(results, 0)

    # ---- ModelRunner-compatible entry: whole prompts, then one token per request ---------------------------------------
    def run(self, seqs: List[Sequence], is_prefill: bool):
        portions = [(s, len(s) - s.num_cached_tokens) for s in seqs]
        toks = self.run_portions(portions)
        for s, n in portions:
            s.num_cached_tokens += n
        return toks
