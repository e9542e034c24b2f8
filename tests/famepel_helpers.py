"""Shared pieces of the Famepel tests: small configurations (sizes chosen unequal on purpose: key, rotated and value
sizes differ, norm parts differ from groups, expert groups of several shapes), random bf16 weights from the plain oracle,
and the error measures.  The engine is driven through tests.hybrid_helpers.Harness (scheduler + runner)."""
from __future__ import annotations

import copy

import numpy as np
import torch

from oracle import famepel_plain as plain
from tests.hybrid_helpers import Harness, rand_tokens, rel_err  # noqa: F401  (re-exported)


def moe(experts=6, top=2, count=3, keep=2, ff=24, scale=1.3):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "scale": scale,
                                                           "groups": {"count": count, "keep": keep}}}


def ssd(heads=4, vdim=12, state=10, groups=2, conv=3, norm_groups=4, mlp="default"):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv,
                                        "norm_groups": norm_groups}, "mlp": moe() if mlp == "default" else mlp}


def latent(heads=4, dim=8, rot_dim=12, vdim=20, kv_rank=20, q_rank=28, scale=0.3, base=1000.0, dims=None, scaling="default",
           kv_from=None, mlp="default"):
    rot = {"base": base, "dims": rot_dim if dims is None else dims}
    if scaling == "default":
        scaling = {"factor": 3.0, "original": 48, "fast": 6.0, "slow": 1.5}
    if scaling:
        rot["scaling"] = scaling
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale,
         "rot": rot}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m, "mlp": moe() if mlp == "default" else mlp}


def glr(heads=3, dim=10, vdim=14, mlp="default"):
    return {"type": "hgrn2", "mixer": {"heads": heads, "dim": dim, "vdim": vdim}, "mlp": moe() if mlp == "default" else mlp}


def model_config(layers, width=40, vocab=70, emb_scale=5.0, eps=1e-5):
    return {"architecture": "Famepel", "embedding": {"scale": emb_scale}, "layers": copy.deepcopy(layers), "norm": {"eps": eps},
            "vocab": vocab, "width": width}


# every mixer, a borrowed latent, a layer without feed-forward, attention first
SMALL = model_config([latent(), ssd(), glr(mlp=None), latent(kv_from=0, heads=2, dim=16, vdim=6, q_rank=9,
                                                             mlp=moe(experts=4, top=1, count=1, keep=1)), ssd(groups=1, norm_groups=1)])


def oracle_logits(config, weights, tokens, dtype=torch.float64):
    return plain.forward(config, weights, list(tokens), dtype=dtype).numpy()


def row_errs(got: np.ndarray, want: np.ndarray) -> np.ndarray:
    """Per row: root mean square of the centred difference over the centred reference."""
    got, want = np.atleast_2d(got).astype(np.float64), np.atleast_2d(want).astype(np.float64)
    d = got - want
    d = d - d.mean(1, keepdims=True)
    w = want - want.mean(1, keepdims=True)
    return np.sqrt((d ** 2).mean(1)) / np.sqrt((w ** 2).mean(1) + 1e-30)


TOL = {"float32": 3e-4, "bfloat16": 6e-2}


def close(got, want, dtype="float32") -> bool:
    """float32: every row within the tolerance.  bfloat16: a token whose two best experts are nearly tied may choose the
    other one after rounding, and the recurrent layers carry that token's different result into the next few tokens; so
    a fifth of the rows may lie outside (typical rows are ten times below the tolerance)."""
    e = row_errs(got, want)
    if dtype == "float32":
        return bool(e.max() < TOL[dtype])
    return bool(np.mean(e < TOL[dtype]) >= 0.8 and np.median(e) < TOL[dtype] / 3)


def run(config, tokens, dtype="float32", cuts=None, seed=0, weights=None, **kw):
    w = weights if weights is not None else plain.random_weights(config, seed)
    hz = Harness(config, w, dtype=dtype, **kw)
    try:
        got = hz.feed("a", tokens, cuts)
    finally:
        hz.close()
    return got, oracle_logits(config, w, tokens)


def needle_model(rank=20, rot_dim=12, dim=8, heads=2, vdim=16, width=32, scale=3.0):
    """One latent-attention layer in which token 61 asks for token 60: the residual's first quarter is a token's key
    address, the second quarter its query address, the second half its content; the latent's first half carries the key
    address, its second half the content; queries are made from the query address with the key side's matrices, keys read
    only the address half of the latent and values only the content half.  Token 61's query address is token 60's key
    address, four times louder than the other tokens' addresses, so that among hundreds of keys the marked one takes
    nearly all the weight and its content decides the answer.  The rotated part is silent on the query side."""
    layer = latent(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=rank, q_rank=rank, scale=scale, mlp=None)
    cfg = model_config([layer], width=width, vocab=64, emb_scale=8.0)
    w = plain.random_weights(cfg, 31)
    g = torch.Generator().manual_seed(32)
    half, q4, ra = width // 2, width // 4, rank // 2
    m = torch.randn(ra, q4, generator=g) * 0.7
    dk = torch.zeros(rank + rot_dim, width)
    dk[:ra, :q4] = m
    dk[ra:rank, half:] = torch.randn(rank - ra, half, generator=g) * 0.5
    dk[rank:] = torch.randn(rot_dim, width, generator=g) * 0.3
    dq = torch.zeros(rank, width)
    dq[:ra, q4:half] = m
    dq[ra:, half:] = dk[ra:rank, half:]
    uk = torch.zeros(heads * dim, rank)
    uk[:, :ra] = torch.randn(heads * dim, ra, generator=g) / ra ** 0.5
    uv = torch.zeros(heads * vdim, rank)
    uv[:, ra:] = torch.randn(heads * vdim, rank - ra, generator=g) / ra ** 0.5
    uq = torch.zeros(heads * (dim + rot_dim), rank)
    for h in range(heads):
        uq[h * (dim + rot_dim):h * (dim + rot_dim) + dim] = uk[h * dim:(h + 1) * dim]
    e = w["embed"].float()
    e[60, :q4] *= 4.0
    e[61, q4:half] = e[60, :q4]
    new = {"dq": dq, "dkv": dk, "dq.norm": torch.ones(rank), "dkv.norm": torch.ones(rank), "uk": uk, "uv": uv, "uq": uq,
           "sink": torch.tensor(([-1.0, 0.5] * heads)[:heads]), "o": w["l0.mix.o"].float() * 4.0}
    for k, v in new.items():
        w["l0.mix." + k] = v.to(torch.bfloat16)
    w["embed"] = e.to(torch.bfloat16)
    w["l0.norm1"], w["l0.norm1.b"] = torch.ones(width).to(torch.bfloat16), torch.zeros(width).to(torch.bfloat16)
    w["l0.norm1.alpha"] = torch.tensor(0.25).to(torch.bfloat16)
    return cfg, w


def needle_tokens(n, needle_at):
    """(tokens with the marked token and the asking token, the same without the marked token)."""
    toks = [2 + (i % 50) for i in range(n)]
    without = list(toks)
    toks[needle_at] = 60
    toks[-1] = without[-1] = 61
    return toks, without
