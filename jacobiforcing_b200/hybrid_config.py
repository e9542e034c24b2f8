"""Configuration of layered hybrid decoders (architecture "Kinetar"): a list of layers over one residual stream, each a
mixer beside a feed-forward that share one norm.  Mixers: "parallel" (softmax attention with a sink whose values are its
keys, beside a selective scan) and "channel_delta" (gated delta rule with a decay per key channel).

Every size and every constant that can differ between models is read from config.json; sizes that only the tensors know
(the inner sizes of the two-step decay and gate projections) are read from the checkpoint's tensor shapes."""
from __future__ import annotations

import json
import os
import struct
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import numpy as np

MIX_ATTN_SCAN, MIX_DELTA = 0, 1
FF_NONE, FF_RELU2 = 0, 1
_ST_DTYPES = {"BF16": (0, 2), "F32": (1, 4), "F16": (2, 2), "I32": (3, 4)}


@dataclass
class LayerSpec:
    mixer: int
    # attention beside scan
    a_heads: int = 0
    a_kv_heads: int = 0
    a_dim: int = 0
    a_vdim: int = 0
    a_conv: int = 1
    a_qt_every: int = 1
    a_scale: float = 1.0
    a_qt_coef: float = 0.0
    s_inner: int = 0
    s_state: int = 0
    s_dt_rank: int = 0
    s_conv: int = 1
    left_scale: float = 1.0
    right_scale: float = 1.0
    # gated delta rule
    d_heads: int = 0
    d_kv_heads: int = 0
    d_dim: int = 0
    d_vdim: int = 0
    d_conv: int = 1
    d_low_a: int = 0
    d_low_g: int = 0
    ff_kind: int = FF_NONE
    ff: int = 0


@dataclass
class HybridConfig:
    architecture: str
    width: int
    vocab: int
    emb_scale: float
    logit_scale: float
    norm_eps: float
    layers: List[LayerSpec] = field(default_factory=list)
    # what the engine's configuration reads from a model description
    max_position_embeddings: int = 1 << 30          # positions enter through a sinusoid: no table to run out of
    is_hybrid: bool = True

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @classmethod
    def from_dict(cls, cfg: dict, shapes: Optional[Dict[str, Tuple[int, ...]]] = None) -> "HybridConfig":
        """cfg: the parsed config.json; shapes: tensor name -> shape (needed by channel_delta layers)."""
        layers = []
        for i, lc in enumerate(cfg["layers"]):
            m = lc["mixer"]
            kind = lc["type"]
            if kind == "parallel":
                a, s = m["left"], m["right"]
                qt = a.get("q_temp") or {"coef": 0.0, "every": 1}
                spec = LayerSpec(MIX_ATTN_SCAN, a_heads=int(a["heads"]), a_kv_heads=int(a["kv_heads"]), a_dim=int(a["dim"]),
                                 a_vdim=int(a["vdim"]), a_conv=int(a["conv"]), a_qt_every=int(qt["every"]),
                                 a_scale=float(a["scale"]), a_qt_coef=float(qt["coef"]), s_inner=int(s["inner"]),
                                 s_state=int(s["state"]), s_dt_rank=int(s["dt_rank"]), s_conv=int(s["conv"]),
                                 left_scale=float(m["left_scale"]), right_scale=float(m["right_scale"]))
            elif kind == "channel_delta":
                if shapes is None:
                    raise ValueError("channel_delta layers need the checkpoint's tensor shapes")
                spec = LayerSpec(MIX_DELTA, d_heads=int(m["heads"]), d_kv_heads=int(m["kv_heads"]), d_dim=int(m["dim"]),
                                 d_vdim=int(m["vdim"]), d_conv=int(m["conv"]),
                                 d_low_a=int(shapes[f"l{i}.mix.a1"][0]), d_low_g=int(shapes[f"l{i}.mix.g1"][0]))
            else:
                raise NotImplementedError(f"layer type {kind!r}")
            mlp = lc.get("mlp")
            if mlp is not None:
                if mlp.get("kind") != "dense":
                    raise NotImplementedError(f"feed-forward kind {mlp.get('kind')!r}")
                spec.ff_kind, spec.ff = FF_RELU2, int(mlp["ff"])
            layers.append(spec)
        return cls(architecture=cfg["architecture"], width=int(cfg["width"]), vocab=int(cfg["vocab"]),
                   emb_scale=float(cfg["embedding"]["scale"]), logit_scale=float(cfg["logit_scale"]),
                   norm_eps=float(cfg["norm"]["eps"]), layers=layers)

    @classmethod
    def from_dir(cls, path: str) -> "HybridConfig":
        with open(os.path.join(path, "config.json")) as f:
            cfg = json.load(f)
        shapes = {}
        for name in sorted(os.listdir(path)):
            if name.endswith(".safetensors"):
                shapes.update({k: tuple(v[1]) for k, v in read_safetensors_header(os.path.join(path, name))[0].items()})
        return cls.from_dict(cfg, shapes)


def read_safetensors_header(path: str):
    """({name: (dtype, shape, begin, end)}, offset of the data section).  The file is an 8-byte little-endian length, that
    many bytes of JSON, then the data."""
    with open(path, "rb") as f:
        n = struct.unpack("<Q", f.read(8))[0]
        hdr = json.loads(f.read(n))
    out = {k: (v["dtype"], v["shape"], v["data_offsets"][0], v["data_offsets"][1]) for k, v in hdr.items() if k != "__metadata__"}
    return out, 8 + n


def iter_safetensors(path: str):
    """(name, dtype code of the C ABI, shape, contiguous numpy byte view) for every tensor of one file."""
    hdr, base = read_safetensors_header(path)
    data = np.memmap(path, dtype=np.uint8, mode="r")
    for name, (dt, shape, b, e) in hdr.items():
        if dt not in _ST_DTYPES:
            raise ValueError(f"tensor {name}: dtype {dt} is not supported")
        yield name, _ST_DTYPES[dt][0], list(shape), np.ascontiguousarray(data[base + b:base + e])
