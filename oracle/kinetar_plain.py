"""Plain, slow restatement of the Kinetar design (layered hybrid decoder: softmax attention with a sink beside a
selective scan, gated delta rule layers, squared-ReLU feed-forward), one function per mechanism, whole sequences only.

It shares no code with the product path: plain torch on the CPU, every token of a sequence from position 0, no cache,
no state hand-over, no batching.  Tests compare the engine (chunked prefill, decoding through the cache, mixed batches)
with it.  `dtype` is torch.float64 for tests that want an exact yardstick, torch.float32 otherwise.

Notation: T tokens, W width, weights are [out, in] and applied as x @ w.T.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

DT = torch.float64


# ---- elementary pieces -------------------------------------------------------------------------------------------
def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_one_plus(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """RMS norm whose stored weight is an offset from one."""
    return unit_rms(x, eps) * (1.0 + w)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def sinusoid(positions: torch.Tensor, width: int, dtype=DT) -> torch.Tensor:
    """[T, width]: even entries sin(p f_i), odd entries cos(p f_i), f_i = 10000^(-2i / width)."""
    half = (width + 1) // 2
    i = torch.arange(half, dtype=dtype)
    f = torch.pow(torch.tensor(10000.0, dtype=dtype), -2.0 * i / width)
    ang = positions.to(dtype)[:, None] * f[None, :]
    out = torch.zeros(len(positions), 2 * half, dtype=dtype)
    out[:, 0::2] = torch.sin(ang)
    out[:, 1::2] = torch.cos(ang)
    return out[:, :width]


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


# ---- attention with a sink, values = keys -----------------------------------------------------------------------------
def sink_attention(h: torch.Tensor, p: Dict[str, torch.Tensor], c: dict) -> torch.Tensor:
    """Causal softmax attention whose values are its keys.  p: q, k, q.conv, k.conv, sink, g, o."""
    T = h.shape[0]
    H, G, d = c["heads"], c["kv_heads"], c["dim"]
    assert c["vdim"] == d, "values are the keys: the value size equals the key size"
    q = short_conv(h @ p["q"].T, p["q.conv"])
    k = short_conv(h @ p["k"].T, p["k.conv"])
    pos = torch.arange(T, dtype=h.dtype)
    temp = 1.0 + c["q_temp"]["coef"] * torch.log(torch.floor((pos + 1) / c["q_temp"]["every"]) + 1.0)
    q = (q * temp[:, None]).view(T, H, d)
    k = k.view(T, G, d)
    out = torch.zeros(T, H, d, dtype=h.dtype)
    for hh in range(H):
        kk = k[:, hh // (H // G)]
        s = (q[:, hh] @ kk.T) * c["scale"]
        s = s.masked_fill(torch.ones(T, T).triu(1).bool(), float("-inf"))
        m = torch.maximum(s.max(-1).values, p["sink"][hh])
        e = torch.exp(s - m[:, None])
        den = e.sum(-1) + torch.exp(p["sink"][hh] - m)
        out[:, hh] = (e / den[:, None]) @ kk
    out = out.reshape(T, H * d) * torch.sigmoid(h @ p["g"].T)
    return out @ p["o"].T


# ---- selective scan ------------------------------------------------------------------------------------------------------
def selective_scan(h: torch.Tensor, p: Dict[str, torch.Tensor], c: dict) -> torch.Tensor:
    """p: in, conv, conv.b, x, dt, dt.b, A_log, D, o."""
    T = h.shape[0]
    inner, N, R = c["inner"], c["state"], c["dt_rank"]
    xz = h @ p["in"].T
    x, z = xz[:, :inner], xz[:, inner:]
    x = silu(short_conv(x, p["conv"], p["conv.b"]))
    low = x @ p["x"].T
    dt = softplus(low[:, :R] @ p["dt"].T + p["dt.b"])
    B, Cm = low[:, R:R + N], low[:, R + N:R + 2 * N]
    A = -torch.exp(p["A_log"])
    S = torch.zeros(inner, N, dtype=h.dtype)
    y = torch.zeros(T, inner, dtype=h.dtype)
    for t in range(T):
        S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * B[t][None, :]
        y[t] = S @ Cm[t] + p["D"] * x[t]
    return (y * silu(z)) @ p["o"].T


def parallel_mixer(h, p, c):
    left = sink_attention(h, {k[5:]: v for k, v in p.items() if k.startswith("left.")}, c["left"])
    right = selective_scan(h, {k[6:]: v for k, v in p.items() if k.startswith("right.")}, c["right"])
    return c["left_scale"] * left + c["right_scale"] * right


# ---- gated delta rule with a decay per key channel ------------------------------------------------------------------------
def channel_delta(h: torch.Tensor, p: Dict[str, torch.Tensor], c: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, G, d, dv = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    q = silu(short_conv(h @ p["q"].T, p["q.conv"])).view(T, G, d)
    k = silu(short_conv(h @ p["k"].T, p["k.conv"])).view(T, G, d)
    v = silu(short_conv(h @ p["v"].T, p["v.conv"])).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ p["b"].T)                                             # [T, H]
    a = ((h @ p["a1"].T) @ p["a2"].T + p["dt_bias"]).view(T, H, d)
    decay = torch.exp(-torch.exp(p["A_log"])[None, :, None] * softplus(a))         # [T, H, d]
    gate = torch.sigmoid((h @ p["g1"].T) @ p["g2"].T).view(T, H, dv)
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for hh in range(H):
        g = hh // (H // G)
        S = torch.zeros(d, dv, dtype=h.dtype)
        for t in range(T):
            S = decay[t, hh][:, None] * S
            u = beta[t, hh] * (v[t, hh] - S.T @ k[t, g])
            S = S + torch.outer(k[t, g], u)
            out[t, hh] = S.T @ q[t, g]
    out = unit_rms(out, eps) * p["norm"] * gate
    return out.reshape(T, H * dv) @ p["o"].T


# ---- feed-forward -----------------------------------------------------------------------------------------------------------
def dense_ff(h, p, c):
    assert c["kind"] == "dense"
    return (torch.relu(h @ p["up"].T) ** 2) @ p["down"].T


# ---- the model -------------------------------------------------------------------------------------------------------------
def forward(config: dict, weights: Dict[str, torch.Tensor], tokens: List[int], dtype=DT, want_layers: bool = False):
    """Logits [T, vocab] of one sequence (and the residual stream after every layer when asked)."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    W = config["width"]
    eps = config["norm"]["eps"]
    T = len(tokens)
    x = w["embed"][torch.tensor(tokens)] * config["embedding"]["scale"]
    x = x + sinusoid(torch.arange(T), W, dtype)
    layers = []
    for i, lc in enumerate(config["layers"]):
        pre = f"l{i}."
        h = norm_one_plus(x, w[pre + "norm1"], eps)
        mix = {k[len(pre) + 4:]: v for k, v in w.items() if k.startswith(pre + "mix.")}
        if lc["type"] == "parallel":
            m = parallel_mixer(h, mix, lc["mixer"])
        elif lc["type"] == "channel_delta":
            m = channel_delta(h, mix, lc["mixer"], eps)
        else:
            raise ValueError(lc["type"])
        if lc.get("mlp") is not None:
            m = m + dense_ff(h, {k[len(pre) + 4:]: v for k, v in w.items() if k.startswith(pre + "mlp.")}, lc["mlp"])
        x = x + m
        layers.append(x.clone())
    logits = (norm_one_plus(x, w["final.norm"], eps) @ w["head"].T) * config["logit_scale"]
    return (logits, torch.stack(layers)) if want_layers else logits


# ---- random models for tests -------------------------------------------------------------------------------------------------
def tensor_shapes(config: dict, low: int = 8) -> Dict[str, tuple]:
    """Names and shapes; `low` is the inner size of the two-step decay / gate projections (a tensor shape, not a
    configuration key)."""
    W, V = config["width"], config["vocab"]
    s = {"embed": (V, W), "final.norm": (W,), "head": (V, W)}
    for i, lc in enumerate(config["layers"]):
        pre, m = f"l{i}.", lc["mixer"]
        s[pre + "norm1"] = (W,)
        if lc["type"] == "parallel":
            a, r = m["left"], m["right"]
            L, R = pre + "mix.left.", pre + "mix.right."
            s.update({L + "q": (a["heads"] * a["dim"], W), L + "k": (a["kv_heads"] * a["dim"], W),
                      L + "q.conv": (a["heads"] * a["dim"], a["conv"]), L + "k.conv": (a["kv_heads"] * a["dim"], a["conv"]),
                      L + "sink": (a["heads"],), L + "g": (a["heads"] * a["vdim"], W), L + "o": (W, a["heads"] * a["vdim"]),
                      R + "in": (2 * r["inner"], W), R + "conv": (r["inner"], r["conv"]), R + "conv.b": (r["inner"],),
                      R + "x": (r["dt_rank"] + 2 * r["state"], r["inner"]), R + "dt": (r["inner"], r["dt_rank"]),
                      R + "dt.b": (r["inner"],), R + "A_log": (r["inner"], r["state"]), R + "D": (r["inner"],),
                      R + "o": (W, r["inner"])})
        else:
            M = pre + "mix."
            s.update({M + "q": (m["kv_heads"] * m["dim"], W), M + "q.conv": (m["kv_heads"] * m["dim"], m["conv"]),
                      M + "k": (m["kv_heads"] * m["dim"], W), M + "k.conv": (m["kv_heads"] * m["dim"], m["conv"]),
                      M + "v": (m["heads"] * m["vdim"], W), M + "v.conv": (m["heads"] * m["vdim"], m["conv"]),
                      M + "b": (m["heads"], W), M + "A_log": (m["heads"],), M + "norm": (m["vdim"],),
                      M + "a1": (low, W), M + "a2": (m["heads"] * m["dim"], low), M + "dt_bias": (m["heads"] * m["dim"],),
                      M + "g1": (low, W), M + "g2": (m["heads"] * m["vdim"], low), M + "o": (W, m["heads"] * m["vdim"])})
        if lc.get("mlp") is not None:
            s[pre + "mlp.up"] = (lc["mlp"]["ff"], W)
            s[pre + "mlp.down"] = (W, lc["mlp"]["ff"])
    return s


def random_weights(config: dict, seed: int = 0, low: int = 8) -> Dict[str, torch.Tensor]:
    """bfloat16 weights with magnitudes that keep every branch alive (decays neither 0 nor 1, sinks that matter)."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(config, low).items():
        leaf = name.split(".", 1)[1] if name.startswith("l") else name
        if len(shape) == 2 and not leaf.endswith("conv") and not leaf.endswith("A_log"):
            t = torch.randn(shape, generator=g) / math.sqrt(shape[1])
            if name == "embed":
                t = torch.randn(shape, generator=g) * 0.08
        elif leaf.endswith("conv"):
            t = torch.randn(shape, generator=g) * 0.5
        elif leaf.endswith("right.A_log"):
            t = torch.log(torch.rand(shape, generator=g) * 3.0 + 0.2)
        elif leaf.endswith("A_log"):
            t = torch.log(torch.rand(shape, generator=g) * 1.5 + 0.1)
        elif leaf.endswith("sink"):
            t = torch.randn(shape, generator=g) * 1.5
        elif leaf.endswith("dt.b") or leaf.endswith("dt_bias"):
            t = torch.randn(shape, generator=g) * 0.7 - 1.0
        elif leaf.endswith("D"):
            t = torch.randn(shape, generator=g) * 0.5 + 1.0
        elif leaf == "mix.norm":
            t = torch.rand(shape, generator=g) + 0.5
        else:                                   # norm offsets, conv bias
            t = torch.randn(shape, generator=g) * 0.2
        out[name] = t.to(torch.bfloat16)
    return out
