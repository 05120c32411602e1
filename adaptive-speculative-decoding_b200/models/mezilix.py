"""Mezilix family: configuration (read from a checkpoint's ``config.json``), tensor names, random initialisation and the
packing of a named state dict into the layouts ``asd_mezilix_set_layer`` expects (include/asd_b200.h).

A Mezilix model is a stack of parallel blocks: ONE scalar-gain RMS norm feeds both the mixer (after a token shift
towards the previous position) and the feed-forward, and both are added to the stream; after every layer the stream is
replaced by a learned average of the embedding output and all layer results so far.  The mixer is latent key/value
attention with a sliding window, the feed-forward a softmax-routed mixture of squared-ReLU experts, and the embedding
adds a row of a hashed (previous token, token) table.  The reference project has no model code of its own (its stages
are vLLM checkpoints, src/serving/real_model_pipeline.py:98-108); this family runs behind the same ``Stage`` seam."""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

ARCHITECTURE = "Mezilix"
MIXERS = ("latent_attention",)
NO_WINDOW = 1 << 30


@dataclass(frozen=True)
class MezilixLayer:
    heads: int
    dim: int            # unrotated query/key size per head
    rot_dim: int        # rotated query/key size per head (the key part is shared by the heads)
    vdim: int
    kv_rank: int        # latent size
    window: int         # position p attends p - window < j <= p
    rot_base: float
    rot_dims: int       # coordinates of the rotated part that rotate
    scale: float
    experts: int = 0    # 0: no feed-forward
    top: int = 0
    ff: int = 0

    @property
    def q_rows(self) -> int:
        return self.heads * (self.dim + self.rot_dim)

    @property
    def cache_row(self) -> int:
        return self.kv_rank + self.rot_dim


@dataclass(frozen=True)
class MezilixConfig:
    width: int
    vocab_size: int
    layers: List[MezilixLayer] = field(default_factory=list)
    eps: float = 1e-5
    buckets: int = 1
    mul_prev: int = 1
    mul_cur: int = 1
    name: str = "mezilix"

    architecture = ARCHITECTURE
    build_components = ("mezilix",)

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    @property
    def hidden_size(self) -> int:
        return self.width

    @classmethod
    def from_dict(cls, d: dict, name: str = "mezilix") -> "MezilixConfig":
        layers = []
        for i, e in enumerate(d["layers"]):
            if e.get("type") not in MIXERS:
                raise ValueError(f"layer {i}: unknown mixer type {e.get('type')!r} (have {MIXERS})")
            m, f = e["mixer"], e.get("mlp")
            rot = m.get("rot") or {}
            kw = {}
            if f is not None:
                if f.get("kind", "moe") != "moe":
                    raise ValueError(f"layer {i}: unknown feed-forward kind {f.get('kind')!r}")
                kw = dict(experts=int(f["router"]["experts"]), top=int(f["router"]["top"]), ff=int(f["expert"]["ff"]))
            layers.append(MezilixLayer(
                heads=int(m["heads"]), dim=int(m["dim"]), rot_dim=int(m["rot_dim"]), vdim=int(m["vdim"]),
                kv_rank=int(m["kv_rank"]), window=_window(m.get("mask")), rot_base=float(rot.get("base", 10000.0)),
                rot_dims=int(rot.get("dims", m["rot_dim"])), scale=float(m["scale"]), **kw))
        bg = d["embedding"]["bigram"]
        return cls(width=int(d["width"]), vocab_size=int(d["vocab"]), layers=layers, eps=float(d["norm"]["eps"]),
                   buckets=int(bg["buckets"]), mul_prev=int(bg["mul_prev"]), mul_cur=int(bg["mul_cur"]), name=name)

    def to_dict(self) -> dict:
        """the ``config.json`` form (inverse of ``from_dict``)"""
        out = []
        for l in self.layers:
            e = {"type": "latent_attention",
                 "mixer": {"heads": l.heads, "dim": l.dim, "rot_dim": l.rot_dim, "vdim": l.vdim, "kv_rank": l.kv_rank,
                           "mask": {"size": l.window}, "rot": {"base": l.rot_base, "dims": l.rot_dims}, "scale": l.scale},
                 "mlp": None}
            if l.experts:
                e["mlp"] = {"kind": "moe", "router": {"experts": l.experts, "top": l.top}, "expert": {"ff": l.ff}}
            out.append(e)
        return {"architecture": ARCHITECTURE, "width": self.width, "vocab": self.vocab_size, "norm": {"eps": self.eps},
                "embedding": {"bigram": {"buckets": self.buckets, "mul_prev": self.mul_prev, "mul_cur": self.mul_cur}},
                "layers": out}

    @property
    def params(self) -> int:
        D, n = self.width, 2 * self.vocab_size * self.width + (self.buckets + 1) * self.width + 1
        for i, l in enumerate(self.layers):
            n += 1 + D + (i + 2) + (l.q_rows + l.cache_row) * D + l.kv_rank
            n += l.heads * (l.dim + l.vdim) * l.kv_rank + D * l.heads * l.vdim
            n += l.experts * (D + 2 * l.ff * D)
        return n

    def streamed_bytes(self, elem: int = 2) -> int:
        """weight bytes one decode step of ONE token reads: every dense matrix, `top` experts per layer, the head"""
        D, n = self.width, self.vocab_size * self.width
        for l in self.layers:
            n += (l.q_rows + l.cache_row) * D + l.heads * (l.dim + l.vdim) * l.kv_rank + D * l.heads * l.vdim
            n += l.experts * D + l.top * 2 * l.ff * D
        return n * elem

    def kv_bytes_per_token(self, elem: int = 2) -> int:
        return sum(l.cache_row for l in self.layers) * elem


def _window(mask) -> int:
    """a layer without a mask entry attends to everything before it"""
    size = (mask or {}).get("size")
    return NO_WINDOW if size is None else int(size)


def tiny_config(**kw) -> MezilixConfig:
    """two small layers with unequal sizes (tests, smoke runs)"""
    layers = [MezilixLayer(heads=2, dim=16, rot_dim=8, vdim=24, kv_rank=32, window=12, rot_base=1000.0, rot_dims=8,
                           scale=0.2, experts=4, top=2, ff=40),
              MezilixLayer(heads=3, dim=8, rot_dim=16, vdim=8, kv_rank=40, window=7, rot_base=500.0, rot_dims=16,
                           scale=0.25)]
    base = dict(width=64, vocab_size=96, layers=layers, eps=1e-5, buckets=53, mul_prev=31, mul_cur=7, name="tiny")
    base.update(kw)
    return MezilixConfig(**base)


def sized_config(width: int, n_layers: int, heads: int, vocab: int = 32768, dim: int = 128, rot_dim: int = 64,
                 kv_rank: int = 512, window: int = 4096, experts: int = 8, top: int = 2, ff: Optional[int] = None,
                 name: str = "mezilix-sized") -> MezilixConfig:
    """layers of a realistic size for throughput measurements (random weights)"""
    ff = ff if ff is not None else 2 * width
    l = MezilixLayer(heads=heads, dim=dim, rot_dim=rot_dim, vdim=dim, kv_rank=kv_rank, window=window, rot_base=10000.0,
                     rot_dims=rot_dim, scale=1.0 / math.sqrt(dim + rot_dim), experts=experts, top=top, ff=ff)
    return MezilixConfig(width=width, vocab_size=vocab, layers=[l] * n_layers, buckets=65521, mul_prev=1000003,
                         mul_cur=31, name=name)


def tensor_shapes(cfg: MezilixConfig) -> Dict[str, tuple]:
    """every tensor of a checkpoint, by name"""
    D, V = cfg.width, cfg.vocab_size
    s = {"embed": (V, D), "bigram": (cfg.buckets + 1, D), "final.norm": (), "head": (V, D)}
    for i, l in enumerate(cfg.layers):
        p = f"l{i}."
        s.update({p + "norm1": (), p + "shift": (D,), p + "dwa": (i + 2,), p + "mix.q": (l.q_rows, D),
                  p + "mix.dkv": (l.cache_row, D), p + "mix.dkv.norm": (l.kv_rank,),
                  p + "mix.uk": (l.heads * l.dim, l.kv_rank), p + "mix.uv": (l.heads * l.vdim, l.kv_rank),
                  p + "mix.o": (D, l.heads * l.vdim)})
        if l.experts:
            s[p + "mlp.router"] = (l.experts, D)
            for e in range(l.experts):
                s[p + f"mlp.e{e}.up"] = (l.ff, D)
                s[p + f"mlp.e{e}.down"] = (D, l.ff)
    return s


def random_weights(cfg: MezilixConfig, seed: int, device="cpu", dtype=torch.bfloat16) -> Dict[str, torch.Tensor]:
    """Named state dict with variance-preserving random matrices, gains near 1, shift weights in [0, 1) and depth
    coefficients that sum to about 1 (throughput runs and smoke tests; nothing trained)."""
    g = torch.Generator(device=device).manual_seed(seed)
    n = max(1, cfg.num_hidden_layers)
    w = {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.rsplit(".", 1)[-1]
        if name.endswith("dkv.norm") or leaf in ("norm1", "norm"):
            t = 1.0 + 0.1 * torch.randn(shape, generator=g, device=device)
        elif leaf == "shift":
            t = torch.rand(shape, generator=g, device=device)
        elif leaf == "dwa":
            t = torch.softmax(torch.randn(shape, generator=g, device=device), 0)
        elif leaf in ("embed", "bigram"):
            t = torch.randn(shape, generator=g, device=device)
        else:
            std = 1.0 / math.sqrt(shape[-1])
            if leaf in ("o", "down"):
                std /= math.sqrt(n)
            t = torch.randn(shape, generator=g, device=device) * std
        w[name] = t.to(dtype)
    return w


def pack_layer(w: Dict[str, torch.Tensor], cfg: MezilixConfig, i: int, device, dtype) -> Dict[str, Optional[torch.Tensor]]:
    """checkpoint names -> engine layout of layer i: the query and latent projections stacked into one matrix, the key
    up-projection transposed per head, the experts stacked into [experts, ff, width] / [experts, width, ff]"""
    l, p = cfg.layers[i], f"l{i}."
    dev = lambda t: t.to(device=device, dtype=dtype).contiguous()
    want = tensor_shapes(cfg)
    for k in want:
        if k.startswith(p):
            if k not in w:
                raise KeyError(f"checkpoint lacks tensor {k}")
            if tuple(w[k].shape) != tuple(want[k]):
                raise ValueError(f"tensor {k} has shape {tuple(w[k].shape)}, the configuration says {tuple(want[k])}")
    out = {"gain": dev(w[p + "norm1"].reshape(1)), "shift": dev(w[p + "shift"]), "coeff": dev(w[p + "dwa"]),
           "wqd": dev(torch.cat([w[p + "mix.q"], w[p + "mix.dkv"]], 0)), "latent_gain": dev(w[p + "mix.dkv.norm"]),
           # per head [kv_rank, dim]: the query is carried into latent space as a product with rows of this matrix
           "wuk": dev(w[p + "mix.uk"].reshape(l.heads, l.dim, l.kv_rank).transpose(1, 2)),
           "wuv": dev(w[p + "mix.uv"]), "wo": dev(w[p + "mix.o"]),
           "router": None, "w_up": None, "w_down": None}
    if l.experts:
        out["router"] = dev(w[p + "mlp.router"])
        out["w_up"] = dev(torch.stack([w[p + f"mlp.e{e}.up"] for e in range(l.experts)], 0))
        out["w_down"] = dev(torch.stack([w[p + f"mlp.e{e}.down"] for e in range(l.experts)], 0))
    return out


def load_config_dir(path: str) -> MezilixConfig:
    with open(os.path.join(path, "config.json")) as f:
        return MezilixConfig.from_dict(json.load(f), name=os.path.basename(os.path.normpath(path)) or "mezilix")
