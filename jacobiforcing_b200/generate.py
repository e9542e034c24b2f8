"""Command line over `LLM.generate` for every registered model family:

    python -m jacobiforcing_b200.generate --model DIR --prompt-ids 5,17,3 [--prompt-ids ...] --max-tokens 32
                                          [--temperature 0.8] [--dtype bfloat16|float32] [--page-size 256]

Prompts are token ids (tokenizers are the caller's business unless the model directory carries one and --prompt is
used).  Prints one JSON line per prompt: {"prompt_ids": [...], "token_ids": [...], "text": "..."}.  The model class is
chosen by config.json through the model registry; layered hybrid decoders build their native library on first use."""
from __future__ import annotations

import argparse
import json
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m jacobiforcing_b200.generate")
    ap.add_argument("--model", required=True)
    ap.add_argument("--prompt-ids", action="append", default=[], help="comma-separated token ids; may be repeated")
    ap.add_argument("--prompt", action="append", default=[], help="text prompt (needs a tokenizer in the model directory)")
    ap.add_argument("--max-tokens", type=int, default=32)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--dtype", choices=("bfloat16", "float32"), default="bfloat16")
    ap.add_argument("--page-size", type=int, default=256)
    ap.add_argument("--max-model-len", type=int, default=4096)
    ap.add_argument("--max-num-seqs", type=int, default=8)
    ap.add_argument("--max-num-batched-tokens", type=int, default=4096)
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args(argv)
    prompts = [[int(x) for x in p.split(",") if x.strip()] for p in a.prompt_ids] + list(a.prompt)
    if not prompts:
        ap.error("give at least one --prompt-ids or --prompt")
    from . import LLM, SamplingParams
    llm = LLM(a.model, dtype=a.dtype, kvcache_block_size=a.page_size, max_model_len=a.max_model_len,
              max_num_seqs=a.max_num_seqs, max_num_batched_tokens=max(a.max_num_batched_tokens, a.max_model_len),
              draft_seed=a.seed)
    sp = SamplingParams(temperature=a.temperature, max_tokens=a.max_tokens, ignore_eos=llm.tokenizer is None)
    outs = llm.generate(prompts, sp, use_tqdm=False)
    llm.exit()
    for p, o in zip(prompts, outs):
        print(json.dumps({"prompt_ids": p if isinstance(p, list) else None, "token_ids": o["token_ids"], "text": o["text"]}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
