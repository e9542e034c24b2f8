"""Host-side pieces of the Famepel design (no GPU): configuration reader and registry, closed forms of the plain oracle's
mechanisms (the oracle is the yardstick of the GPU tests, so it is checked against hand-derived values here)."""
import json
import math

import pytest
import torch

from oracle import famepel_plain as plain
from tests.famepel_helpers import SMALL, glr, latent, model_config, moe, ssd
from tests.test_hybrid_host import _write_checkpoint


def test_config_reader_and_registry(tmp_path):
    from jacobiforcing_b200.hybrid_config import (BLOCK_SANDWICH, FF_NONE, FF_ROUTED, MIX_GLR, MIX_LATENT, MIX_SSD, NORM_TANH,
                                                  POS_NONE, HybridConfig)
    from jacobiforcing_b200.registry import architecture_of, resolve
    w = plain.random_weights(SMALL, 0)
    _write_checkpoint(tmp_path, SMALL, {k: (v if v.dim() else v.reshape(())) for k, v in w.items()})
    assert architecture_of(str(tmp_path)) == "Famepel"
    fam = resolve(str(tmp_path))
    assert fam.name == "hybrid" and fam.native_config
    hc = fam.load_config(str(tmp_path))
    assert isinstance(hc, HybridConfig) and hc.is_hybrid
    assert (hc.norm_kind, hc.block_kind, hc.pos_kind, hc.logit_scale) == (NORM_TANH, BLOCK_SANDWICH, POS_NONE, 1.0)
    assert [s.mixer for s in hc.layers] == [MIX_LATENT, MIX_SSD, MIX_GLR, MIX_LATENT, MIX_SSD]
    a, b = hc.layers[0], hc.layers[3]
    assert (a.l_heads, a.l_dim, a.l_rot_dim, a.l_vdim, a.l_kv_rank, a.l_q_rank, a.l_kv_from) == (4, 8, 12, 20, 20, 28, -1)
    assert (a.r_dims, a.r_base, a.r_factor, a.r_original, a.r_fast, a.r_slow) == (12, 1000.0, 3.0, 48.0, 6.0, 1.5)
    assert b.l_kv_from == 0 and b.l_heads == 2 and b.x_experts == 4 and b.x_top == 1 and b.x_groups == 1
    assert a.cache_elems_per_token() == 32 and b.cache_elems_per_token() == 0 and hc.layers[1].cache_elems_per_token() == 0
    m = hc.layers[1]
    assert (m.m_heads, m.m_vdim, m.m_state, m.m_groups, m.m_conv, m.m_norm_groups) == (4, 12, 10, 2, 3, 4)
    assert (m.ff_kind, m.ff, m.x_experts, m.x_top, m.x_groups, m.x_keep) == (FF_ROUTED, 24, 6, 2, 3, 2) and abs(m.x_scale - 1.3) < 1e-7
    assert hc.layers[2].ff_kind == FF_NONE and (hc.layers[2].g_heads, hc.layers[2].g_dim, hc.layers[2].g_vdim) == (3, 10, 14)
    from jacobiforcing_b200.config import Config
    c = Config(str(tmp_path), kvcache_block_size=64, num_kvcache_blocks=8, max_num_batched_tokens=128)
    assert c.hf_config.architecture == "Famepel"


@pytest.mark.parametrize("bad", ["kv_from_later", "kv_from_borrower", "kv_rank", "groups", "top", "keep", "norm_groups", "rot_dims", "type",
                                 "ff_kind"])
def test_config_reader_refuses(bad):
    from jacobiforcing_b200.hybrid_config import HybridConfig
    layers = [latent(), latent(kv_from=0), ssd()]
    if bad == "kv_from_later":
        layers[0]["mixer"]["kv_from"] = 1
    elif bad == "kv_from_borrower":
        layers.append(latent(kv_from=1))
    elif bad == "kv_rank":
        layers[1]["mixer"]["kv_rank"] = 24
    elif bad == "groups":
        layers[2]["mixer"]["groups"] = 3
    elif bad == "top":
        layers[2]["mlp"] = moe(experts=6, top=5, count=3, keep=2)
    elif bad == "keep":
        layers[2]["mlp"] = moe(experts=6, top=1, count=3, keep=4)
    elif bad == "norm_groups":
        layers[2]["mixer"]["norm_groups"] = 5
    elif bad == "rot_dims":
        layers[0]["mixer"]["rot"]["dims"] = 14
    elif bad == "type":
        layers[2]["type"] = "mystery"
    elif bad == "ff_kind":
        layers[2]["mlp"]["kind"] = "dense"
    with pytest.raises((ValueError, NotImplementedError)):
        HybridConfig.from_dict(model_config(layers))


def test_rotation_tables_closed_forms():
    pos = torch.tensor([0, 1, 7])
    cos, sin = plain.rotary_tables({"base": 100.0, "dims": 4}, pos)
    f = torch.tensor([1.0, 100.0 ** -0.5], dtype=torch.float64)
    assert torch.allclose(cos, torch.cos(pos[:, None] * f)) and torch.allclose(sin, torch.sin(pos[:, None] * f))
    # interpolation: base 10000 over 8 dims, original 64: pair i turns 64 f_i / 2 pi times
    rot = {"base": 10000.0, "dims": 8, "scaling": {"factor": 4.0, "original": 64, "fast": 4.0, "slow": 0.5}}
    cos, sin = plain.rotary_tables(rot, torch.tensor([3]))
    mag = 0.1 * math.log(4.0) + 1.0
    # dim(4 turns) = 8 ln(64 / 8 pi) / (2 ln 1e4) = 0.406 -> lo 0 ; dim(0.5) = 8 ln(64 / pi) / (2 ln 1e4) = 1.309 -> hi 2
    ramp = [0.0, 0.5, 1.0, 1.0]
    for i in range(4):
        fi = 10000.0 ** (-2.0 * i / 8)
        fe = fi / 4.0 * ramp[i] + fi * (1 - ramp[i])
        assert abs(float(cos[0, i]) - mag * math.cos(3 * fe)) < 1e-12 and abs(float(sin[0, i]) - mag * math.sin(3 * fe)) < 1e-12
    v = torch.tensor([[1.0, 2.0, 3.0, 4.0, 5.0]], dtype=torch.float64)
    c, s = torch.tensor([[0.0, 1.0]], dtype=torch.float64), torch.tensor([[1.0, 0.0]], dtype=torch.float64)
    assert plain.rotate_pairs(v, c, s).tolist() == [[-2.0, 1.0, 3.0, 4.0, 5.0]]       # a quarter turn, identity, untouched tail


def test_route_by_hand():
    r = {"experts": 6, "top": 2, "scale": 2.0, "groups": {"count": 3, "keep": 2}}
    # logits are the router rows dotted with h = e0: column 0 of the router
    logits = torch.tensor([2.0, -1.0, 1.5, 1.4, 0.0, 1.9], dtype=torch.float64)
    router = torch.zeros(6, 3, dtype=torch.float64)
    router[:, 0] = logits
    idx, w = plain.route(torch.tensor([[1.0, 0.0, 0.0]], dtype=torch.float64), router, r)
    s = torch.sigmoid(logits)
    # group sums: {0,1}: s0 + s1 = 1.150, {2,3}: 1.620, {4,5}: 1.370 -> groups 1 and 2 are kept, expert 0 (the best) is not
    assert sorted(idx[0].tolist()) == [2, 5]
    tot = float(s[2] + s[5])
    got = dict(zip(idx[0].tolist(), w[0].tolist()))
    assert abs(got[5] - 2.0 * float(s[5]) / tot) < 1e-12 and abs(got[2] - 2.0 * float(s[2]) / tot) < 1e-12
    # groups of one expert: a group is worth its only score
    r1 = {"experts": 6, "top": 2, "scale": 1.0, "groups": {"count": 6, "keep": 3}}
    idx, _ = plain.route(torch.tensor([[1.0, 0.0, 0.0]], dtype=torch.float64), router, r1)
    assert sorted(idx[0].tolist()) == [0, 5]


def test_recurrences_closed_forms():
    # gated linear recurrence with a constant gate f and a constant value v: S_t = (1 - f^(t+1)) v per row
    c = {"heads": 1, "dim": 2, "vdim": 3}
    W = 4
    p = {"q": torch.zeros(2, W), "f": torch.zeros(2, W), "f.b": torch.zeros(2), "lower": torch.tensor([0.2, 0.6]),
         "v": torch.zeros(3, W), "norm": torch.ones(3), "o": torch.eye(W, 3)}
    p = {k: v.double() for k, v in p.items()}
    p["v"][:, 0] = torch.tensor([1.0, 2.0, 3.0])
    p["q"][:, 1] = 50.0                                     # silu(50) = 50: q = (50, 50)
    h = torch.zeros(5, W, dtype=torch.float64)
    h[:, 0] = 1.0
    h[:, 1] = 1.0
    out = plain.gated_linear_mixer(h, p, c, 0.0)
    f = torch.tensor([0.2 + 0.8 * 0.5, 0.6 + 0.4 * 0.5], dtype=torch.float64)
    for t in range(5):
        o = 50.0 * ((1 - f ** (t + 1)).sum()) * torch.tensor([1.0, 2.0, 3.0], dtype=torch.float64)
        want = o / torch.sqrt((o * o).mean())
        assert torch.allclose(out[t, :3], want, atol=1e-9)
    # state-space recurrence, one head, one state, no convolution memory (one tap of weight 1): geometric sum
    c = {"heads": 1, "vdim": 1, "state": 1, "groups": 1, "conv": 1, "norm_groups": 1}
    inp = torch.zeros(1 + 1 + 1 + 1 + 1, W, dtype=torch.float64)       # rows: z, x, B, C, dt
    big = 30.0
    inp[0, 0], inp[1, 0], inp[2, 0], inp[3, 0], inp[4, 0] = big, big, big, big, 0.0
    p = {"in": inp, "conv": torch.ones(3, 1).double(), "conv.b": torch.zeros(3).double(), "dt_bias": torch.tensor([0.0]).double(),
         "A_log": torch.tensor([math.log(0.5)]).double(), "D": torch.tensor([0.25]).double(), "norm": torch.ones(1).double(),
         "o": torch.ones(W, 1).double()}
    h = torch.zeros(4, W, dtype=torch.float64)
    h[:, 0] = 1.0
    # x = B = C = silu(30) ~ 30, dt = softplus(0) = ln 2, decay = exp(-0.5 ln 2); eps = 0: the norm leaves the sign only
    out = plain.ssd_mixer(h, p, c, 0.0)
    assert torch.allclose(out[:, 0], torch.ones(4, dtype=torch.float64))
    u = plain.silu(torch.tensor(big, dtype=torch.float64))
    dt, dec = math.log(2.0), math.exp(-0.5 * math.log(2.0))
    S, ys = 0.0, []
    for t in range(4):
        S = dec * S + dt * float(u) * float(u)
        ys.append(S * float(u) + 0.25 * float(u))
    p["norm"] = torch.tensor([1.0]).double()
    raw = plain.ssd_mixer(h, p, c, 1e30)                     # a huge eps makes the norm a known factor: y / sqrt(eps)
    for t in range(4):
        assert abs(float(raw[t, 0]) * 1e15 - ys[t] * float(u)) < 1e-6 * ys[t] * float(u)


def test_sink_and_borrowed_latent_in_the_oracle():
    cfg = model_config([latent(mlp=None), latent(kv_from=0, mlp=None)])
    w = plain.random_weights(cfg, 3)
    toks = list(range(1, 12))
    base = plain.forward(cfg, w, toks)
    # one token: the softmax over one key and the sink gives the value times 1 / (1 + exp(sink - score))
    one = plain.forward(cfg, w, toks[:1])
    assert torch.allclose(one[0], base[0])
    w2 = dict(w)
    w2["l0.mix.sink"] = torch.full_like(w["l0.mix.sink"], 30.0)           # a huge sink silences layer 0's attention
    silenced = plain.forward(cfg, w2, toks, want_layers=True)[1][0]
    x0 = w["embed"].double()[torch.tensor(toks)] * cfg["embedding"]["scale"]
    post = plain.tanh_norm(torch.zeros_like(x0), {k: v.double() for k, v in w.items()}, "l0.norm1b") * w["l0.ls1"].double()
    assert torch.allclose(silenced, x0 + post, atol=1e-9)
    # the borrower reads layer 0's latent: changing layer 0's down-projection changes layer 1's attention input too
    assert not torch.allclose(base, plain.forward(cfg, {**w, "l0.mix.dkv": w["l0.mix.dkv"] * 0.5}, toks))
