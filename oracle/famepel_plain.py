"""Plain, slow restatement of the Famepel design: a decoder whose layers are norm - mixer - norm and norm - feed-forward -
norm around one residual stream, with element-wise tanh norms, per-channel layer scales, three kinds of mixer (a scalar
-decay state-space recurrence, attention over a shared low-rank latent with a rotated key part and a sink, a gated linear
recurrence whose forget gate is also its input gate) and a routed mixture of small gated feed-forward experts.

One function per mechanism, whole sequences only, plain torch on the CPU: every token of a sequence from position 0, no
cache, no state hand-over, no batching.  It shares no code with the product path; tests compare the engine (portions,
decoding through cache and state, mixed batches) with it.

Notation: T tokens, W width, weights are [out, in] and applied as x @ w.T; `p` maps a mixer's tensor leaf name ("in",
"conv.b", "dq.norm", ...) to its tensor, `c` is the mixer's block of the configuration.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

DT = torch.float64


# ---- elementary pieces -------------------------------------------------------------------------------------------
def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def tanh_norm(x: torch.Tensor, w: Dict[str, torch.Tensor], name: str) -> torch.Tensor:
    """Element-wise norm without statistics: tanh(alpha x) w + b."""
    return torch.tanh(w[name + ".alpha"] * x) * w[name] + w[name + ".b"]


def short_conv(u: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal depthwise convolution over time.  u [T, C], w [C, taps]; the last tap multiplies the current token,
    inputs before the sequence's start are zero."""
    T, C = u.shape
    taps = w.shape[1]
    y = torch.zeros_like(u)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                y[t] += w[:, j] * u[s]
    if bias is not None:
        y = y + bias
    return y


# ---- rotary positions with frequency interpolation ---------------------------------------------------------------------
def rotary_tables(rot: dict, positions: torch.Tensor, dtype=DT):
    """cos, sin [T, dims / 2] of a rotation over `dims` dimensions.  With a "scaling" block the frequencies below a ramp
    are divided by `factor` (long wavelengths are interpolated, short ones kept) and both tables are multiplied by
    0.1 ln(factor) + 1."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=dtype)
    f = torch.pow(torch.tensor(base, dtype=dtype), -2.0 * i / dims)
    mag = 1.0
    sc = rot.get("scaling")
    if sc:
        factor, orig = float(sc["factor"]), float(sc["original"])

        def turn_dim(turns):
            return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
        lo = max(math.floor(turn_dim(float(sc["fast"]))), 0)
        hi = min(math.ceil(turn_dim(float(sc["slow"]))), dims - 1)
        ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        f = f / factor * ramp + f * (1.0 - ramp)
        mag = 0.1 * math.log(factor) + 1.0
    ang = positions.to(dtype)[:, None] * f[None, :]
    return torch.cos(ang) * mag, torch.sin(ang) * mag


def rotate_pairs(v: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """v [T, ..., n]: dimension 2i is paired with 2i + 1 over the first 2 * cos.shape[1] dimensions; the rest pass."""
    r = 2 * cos.shape[1]
    shape = [v.shape[0]] + [1] * (v.dim() - 2) + [cos.shape[1]]
    c, s = cos.view(shape), sin.view(shape)
    a, b = v[..., 0:r:2], v[..., 1:r:2]
    out = v.clone()
    out[..., 0:r:2] = a * c - b * s
    out[..., 1:r:2] = b * c + a * s
    return out


# ---- state-space recurrence with one decay per head ------------------------------------------------------------------------
def ssd_mixer(h: torch.Tensor, p: Dict[str, torch.Tensor], c: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, P, N, G = c["heads"], c["vdim"], c["state"], c["groups"]
    inner = H * P
    u = h @ p["in"].T
    z, xbc, dt = u[:, :inner], u[:, inner:2 * inner + 2 * G * N], u[:, 2 * inner + 2 * G * N:]
    xbc = silu(short_conv(xbc, p["conv"], p["conv.b"]))
    x = xbc[:, :inner].view(T, H, P)
    B = xbc[:, inner:inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    dt = softplus(dt + p["dt_bias"])                                     # [T, H]
    rate = torch.exp(p["A_log"])
    y = torch.zeros(T, H, P, dtype=h.dtype)
    for hh in range(H):
        g = hh // (H // G)
        S = torch.zeros(N, P, dtype=h.dtype)
        for t in range(T):
            S = torch.exp(-rate[hh] * dt[t, hh]) * S + dt[t, hh] * torch.outer(B[t, g], x[t, hh])
            y[t, hh] = S.T @ C[t, g] + p["D"][hh] * x[t, hh]
    y = y.reshape(T, inner) * silu(z)
    parts = c["norm_groups"]
    y = unit_rms(y.view(T, parts, inner // parts), eps).reshape(T, inner) * p["norm"]
    return y @ p["o"].T


# ---- attention over a shared latent ---------------------------------------------------------------------------------------
def latent_kv(h: torch.Tensor, p: Dict[str, torch.Tensor], c: dict, eps: float):
    """What a layer with its own down-projection leaves for itself and for layers that borrow from it: the normed latent
    [T, kv_rank] and the rotated key part [T, rot_dim] shared by all heads."""
    T = h.shape[0]
    r = c["kv_rank"]
    d = h @ p["dkv"].T
    lat = unit_rms(d[:, :r], eps) * p["dkv.norm"]
    cos, sin = rotary_tables(c["rot"], torch.arange(T), h.dtype)
    return lat, rotate_pairs(d[:, r:], cos, sin)


def latent_attention(h: torch.Tensor, p: Dict[str, torch.Tensor], c: dict, eps: float, kv) -> torch.Tensor:
    T = h.shape[0]
    H, dn, dr, dv = c["heads"], c["dim"], c["rot_dim"], c["vdim"]
    lat, k_rot = kv
    cq = unit_rms(h @ p["dq"].T, eps) * p["dq.norm"]
    q = (cq @ p["uq"].T).view(T, H, dn + dr)
    cos, sin = rotary_tables(c["rot"], torch.arange(T), h.dtype)
    q_rot = rotate_pairs(q[..., dn:], cos, sin)
    k = (lat @ p["uk"].T).view(T, H, dn)
    v = (lat @ p["uv"].T).view(T, H, dv)
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    hidden = torch.ones(T, T).triu(1).bool()
    for hh in range(H):
        s = (q[:, hh, :dn] @ k[:, hh].T + q_rot[:, hh] @ k_rot.T) * c["scale"]
        s = s.masked_fill(hidden, float("-inf"))
        m = torch.maximum(s.max(-1).values, p["sink"][hh])
        e = torch.exp(s - m[:, None])
        den = e.sum(-1) + torch.exp(p["sink"][hh] - m)                   # the sink: a logit without key or value
        out[:, hh] = (e / den[:, None]) @ v[:, hh]
    return out.reshape(T, H * dv) @ p["o"].T


# ---- gated linear recurrence -------------------------------------------------------------------------------------------------
def gated_linear_mixer(h: torch.Tensor, p: Dict[str, torch.Tensor], c: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, d, dv = c["heads"], c["dim"], c["vdim"]
    q = silu(h @ p["q"].T).view(T, H, d)
    v = (h @ p["v"].T).view(T, H, dv)
    low = p["lower"]
    f = (low + (1.0 - low) * torch.sigmoid(h @ p["f"].T + p["f.b"])).view(T, H, d)
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for hh in range(H):
        S = torch.zeros(d, dv, dtype=h.dtype)
        for t in range(T):
            S = f[t, hh][:, None] * S + torch.outer(1.0 - f[t, hh], v[t, hh])
            out[t, hh] = S.T @ q[t, hh]
    out = unit_rms(out, eps) * p["norm"]
    return out.reshape(T, H * dv) @ p["o"].T


# ---- routed feed-forward --------------------------------------------------------------------------------------------------------
def route(h: torch.Tensor, router: torch.Tensor, r: dict):
    """(chosen experts [T, top], their weights [T, top])."""
    E, top = int(r["experts"]), int(r["top"])
    count, keep = int(r["groups"]["count"]), int(r["groups"]["keep"])
    s = torch.sigmoid(h @ router.T)                                      # [T, E]
    T = s.shape[0]
    per = E // count
    grp = s.view(T, count, per)
    gscore = grp.topk(min(2, per), dim=-1).values.sum(-1)                # a group is worth its two best experts
    kept = gscore.topk(keep, dim=-1).indices                             # [T, keep]
    allowed = torch.zeros(T, count, dtype=torch.bool)
    allowed.scatter_(1, kept, True)
    masked = torch.where(allowed[:, :, None].expand(T, count, per).reshape(T, E), s, torch.full_like(s, -1.0))
    idx = masked.topk(top, dim=-1).indices
    w = s.gather(1, idx)
    w = w / (w.sum(-1, keepdim=True) + 1e-20) * float(r["scale"])
    return idx, w


def routed_ff(h: torch.Tensor, p: Dict[str, torch.Tensor], c: dict) -> torch.Tensor:
    idx, w = route(h, p["router"], c["router"])
    out = torch.zeros(h.shape[0], p["e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for j in range(idx.shape[1]):
            e = int(idx[t, j])
            a = silu(p[f"e{e}.gate"] @ h[t]) * (p[f"e{e}.up"] @ h[t])
            out[t] += w[t, j] * (p[f"e{e}.down"] @ a)
    return out


# ---- the model -------------------------------------------------------------------------------------------------------------
def _sub(w, prefix):
    return {k[len(prefix):]: v for k, v in w.items() if k.startswith(prefix)}


def forward(config: dict, weights: Dict[str, torch.Tensor], tokens: List[int], dtype=DT, want_layers: bool = False):
    """Logits [T, vocab] of one sequence (and the residual stream after every layer when asked)."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = config["norm"]["eps"]
    x = w["embed"][torch.tensor(tokens)] * config["embedding"]["scale"]
    layers, latents = [], {}
    for i, lc in enumerate(config["layers"]):
        pre = f"l{i}."
        mc = lc["mixer"]
        h = tanh_norm(x, w, pre + "norm1")
        mix = _sub(w, pre + "mix.")
        if lc["type"] == "mamba2":
            m = ssd_mixer(h, mix, mc, eps)
        elif lc["type"] == "latent_attention":
            if mc.get("kv_from") is None:
                latents[i] = latent_kv(h, mix, mc, eps)
                kv = latents[i]
            else:
                kv = latents[int(mc["kv_from"])]
            m = latent_attention(h, mix, mc, eps, kv)
        elif lc["type"] == "hgrn2":
            m = gated_linear_mixer(h, mix, mc, eps)
        else:
            raise ValueError(lc["type"])
        x = x + tanh_norm(m, w, pre + "norm1b") * w[pre + "ls1"]
        if lc.get("mlp") is not None:
            assert lc["mlp"]["kind"] == "moe"
            h = tanh_norm(x, w, pre + "norm2")
            x = x + tanh_norm(routed_ff(h, _sub(w, pre + "mlp."), lc["mlp"]), w, pre + "norm2b") * w[pre + "ls2"]
        layers.append(x.clone())
    logits = tanh_norm(x, w, "final.norm") @ w["head"].T
    return (logits, torch.stack(layers)) if want_layers else logits


# ---- random models for tests -------------------------------------------------------------------------------------------------
def tensor_shapes(config: dict) -> Dict[str, tuple]:
    W, V = config["width"], config["vocab"]
    s = {"embed": (V, W), "head": (V, W)}

    def norm(name):
        s[name], s[name + ".b"], s[name + ".alpha"] = (W,), (W,), ()
    norm("final.norm")
    for i, lc in enumerate(config["layers"]):
        pre, m, M = f"l{i}.", lc["mixer"], f"l{i}.mix."
        for n in ("norm1", "norm1b"):
            norm(pre + n)
        s[pre + "ls1"] = (W,)
        if lc["type"] == "mamba2":
            inner, gn = m["heads"] * m["vdim"], m["groups"] * m["state"]
            s.update({M + "in": (2 * inner + 2 * gn + m["heads"], W), M + "conv": (inner + 2 * gn, m["conv"]),
                      M + "conv.b": (inner + 2 * gn,), M + "dt_bias": (m["heads"],), M + "A_log": (m["heads"],),
                      M + "D": (m["heads"],), M + "norm": (inner,), M + "o": (W, inner)})
        elif lc["type"] == "latent_attention":
            H = m["heads"]
            s.update({M + "dq": (m["q_rank"], W), M + "dq.norm": (m["q_rank"],),
                      M + "uq": (H * (m["dim"] + m["rot_dim"]), m["q_rank"]), M + "uk": (H * m["dim"], m["kv_rank"]),
                      M + "uv": (H * m["vdim"], m["kv_rank"]), M + "sink": (H,), M + "o": (W, H * m["vdim"])})
            if m.get("kv_from") is None:
                s.update({M + "dkv": (m["kv_rank"] + m["rot_dim"], W), M + "dkv.norm": (m["kv_rank"],)})
        elif lc["type"] == "hgrn2":
            H = m["heads"]
            s.update({M + "q": (H * m["dim"], W), M + "f": (H * m["dim"], W), M + "f.b": (H * m["dim"],),
                      M + "lower": (H * m["dim"],), M + "v": (H * m["vdim"], W), M + "norm": (m["vdim"],),
                      M + "o": (W, H * m["vdim"])})
        else:
            raise ValueError(lc["type"])
        if lc.get("mlp") is not None:
            for n in ("norm2", "norm2b"):
                norm(pre + n)
            s[pre + "ls2"] = (W,)
            ff, E = lc["mlp"]["expert"]["ff"], lc["mlp"]["router"]["experts"]
            s[pre + "mlp.router"] = (E, W)
            for e in range(E):
                s.update({f"{pre}mlp.e{e}.gate": (ff, W), f"{pre}mlp.e{e}.up": (ff, W), f"{pre}mlp.e{e}.down": (W, ff)})
    return s


def random_weights(config: dict, seed: int = 0) -> Dict[str, torch.Tensor]:
    """bfloat16 weights with magnitudes that keep every branch alive: tanh norms away from both the linear and the
    saturated range, decays neither 0 nor 1, sinks that take a visible share, routers with spread-out scores."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(config).items():
        leaf = name.split(".", 1)[1] if name[0] == "l" and name[1].isdigit() else name
        if leaf.endswith(".alpha"):
            t = torch.rand(shape, generator=g) * 0.6 + 0.5
        elif leaf in ("ls1", "ls2"):
            t = torch.rand(shape, generator=g) * 0.6 + 0.5
        elif leaf.endswith("norm.b") or leaf.endswith("norm1.b") or leaf.endswith("norm2.b") or leaf.endswith("b.b"):
            t = torch.randn(shape, generator=g) * 0.1
        elif leaf == "embed":
            t = torch.randn(shape, generator=g) * 0.08
        elif leaf == "mlp.router":
            t = torch.randn(shape, generator=g) * 2.0 / math.sqrt(shape[1])
        elif len(shape) == 2 and not leaf.endswith("conv"):
            t = torch.randn(shape, generator=g) / math.sqrt(shape[1])
        elif leaf.endswith("conv"):
            t = torch.randn(shape, generator=g) * 0.5
        elif leaf.endswith("A_log"):
            t = torch.log(torch.rand(shape, generator=g) * 2.0 + 0.2)
        elif leaf.endswith("sink"):
            t = torch.randn(shape, generator=g) * 1.5
        elif leaf.endswith("dt_bias"):
            t = torch.randn(shape, generator=g) * 0.7 - 1.0
        elif leaf.endswith("mix.D"):
            t = torch.randn(shape, generator=g) * 0.5 + 1.0
        elif leaf.endswith("lower"):
            t = torch.rand(shape, generator=g) * 0.9
        elif leaf.endswith("f.b") or leaf.endswith("conv.b"):
            t = torch.randn(shape, generator=g) * 0.3
        else:                                   # norm weights: mixer norms, latent norms, tanh norms
            t = torch.rand(shape, generator=g) + 0.5
        out[name] = t.to(torch.bfloat16)
    return out
