"""Rivetar family: configuration (read from a checkpoint's ``config.json``), tensor names, random initialisation and
the packing of a named state dict into the buffers ``asd_rivetar_set_tensor`` expects (include/asd_b200.h).

A Rivetar model is a stack of sandwich-normed layers, x <- x + norm_b(f(norm(x))) for the mixer and then for the
feed-forward, every norm an RMS norm whose stored weight is the deviation from one.  Each layer names ONE of three
mixers: latent key/value attention whose queries also pass through a normed latent; gated linear attention, a
recurrence with a [key, value] state per head and a decay per key channel; grouped-query softmax attention over a
sliding window plus kept first positions, with a learned sink in the denominator and values that are rotated by their
own position and turned back by the query's.  The feed-forward is a two-matrix layer with a normalised cubic
polynomial as activation (or absent).  A span of layers may run several times in a row with the same weights; every
pass has its own cache and state and starts from a learned mix of the stream and the embedding output plus a learned
vector per pass.  The logits are squashed by a scaled tanh.  The reference project has no model code of its own (its
stages are vLLM checkpoints, src/serving/real_model_pipeline.py:98-108); this family runs behind the same ``Stage`` seam."""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch

ARCHITECTURE = "Rivetar"
MIXERS = ("latent_attention", "gla", "attention")
MIXER_CODE = {m: i for i, m in enumerate(MIXERS)}
LAYOUTS = ("interleaved", "halves")
NO_WINDOW = 1 << 30


@dataclass(frozen=True)
class RivetarLayer:
    type: str
    heads: int
    dim: int                 # query/key size per head (latent attention: the unrotated part)
    vdim: int
    kv_heads: int = 0        # attention: key/value heads
    rot_dim: int = 0         # latent attention: rotated query/key size per head (the key part is shared by the heads)
    kv_rank: int = 0         # latent attention: size of the cached latent
    q_rank: int = 0          # latent attention: size of the query latent
    decay_rank: int = 0      # gla: inner size of the two-matrix decay projection (a tensor's shape, not a config key)
    tau: float = 1.0         # gla: the decay is sigmoid(z)^(1 / tau)
    rot_base: float = 10000.0
    rot_dims: int = 0        # leading coordinates of a head's query/key (of the rotated part) that rotate
    rot_layout: str = "interleaved"
    window: int = NO_WINDOW  # position i sees j <= i with i - j < window ...
    keep_first: int = 0      # ... or j < keep_first
    scale: float = 1.0
    ff: int = 0              # 0: no feed-forward

    @property
    def cache_row(self) -> int:
        """cached elements per position (paged); the gla state is per sequence, not per position"""
        if self.type == "latent_attention":
            return self.kv_rank + self.rot_dim
        if self.type == "attention":
            return self.kv_heads * (self.dim + self.vdim)
        return 0

    @property
    def state_elems(self) -> int:
        return self.heads * self.dim * self.vdim if self.type == "gla" else 0


@dataclass(frozen=True)
class RivetarConfig:
    width: int
    vocab_size: int
    layers: List[RivetarLayer] = field(default_factory=list)
    eps: float = 1e-5
    embed_scale: float = 1.0
    logit_softcap: float = 0.0          # 0: logits are not squashed
    loop: Optional[Tuple[int, int, int]] = None     # (start, stop, times): layers start .. stop - 1 run `times` times
    name: str = "rivetar"

    architecture = ARCHITECTURE
    build_components = ("rivetar",)

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    @property
    def hidden_size(self) -> int:
        return self.width

    def runs(self) -> List[Tuple[int, int]]:
        """(layer, pass) of every layer execution in order; pass is -1 outside the repeated span"""
        n = len(self.layers)
        if self.loop is None:
            return [(i, -1) for i in range(n)]
        a, b, times = self.loop
        out = [(i, -1) for i in range(a)]
        for t in range(times):
            out += [(i, t) for i in range(a, b)]
        return out + [(i, -1) for i in range(b, n)]

    @classmethod
    def from_dict(cls, d: dict, name: str = "rivetar") -> "RivetarConfig":
        layers = []
        for i, e in enumerate(d["layers"]):
            t = e.get("type")
            if t not in MIXERS:
                raise ValueError(f"layer {i}: unknown mixer type {t!r} (have {MIXERS})")
            m, f = e["mixer"], e.get("mlp")
            rot, mask = m.get("rot") or {}, m.get("mask") or {}
            layout = rot.get("layout", "interleaved")
            if layout not in LAYOUTS:
                raise ValueError(f"layer {i}: unknown rotation layout {layout!r} (have {LAYOUTS})")
            if f is not None and f.get("kind", "dense") != "dense":
                raise ValueError(f"layer {i}: unknown feed-forward kind {f.get('kind')!r}")
            kw = dict(type=t, heads=int(m["heads"]), dim=int(m["dim"]), vdim=int(m["vdim"]),
                      rot_base=float(rot.get("base", 10000.0)), rot_layout=layout,
                      window=NO_WINDOW if mask.get("size") is None else int(mask["size"]),
                      keep_first=int(mask.get("keep_first", 0)), ff=int(f["ff"]) if f is not None else 0)
            if t == "latent_attention":
                kw.update(rot_dim=int(m["rot_dim"]), kv_rank=int(m["kv_rank"]), q_rank=int(m["q_rank"]),
                          rot_dims=int(rot.get("dims", m["rot_dim"])), scale=float(m["scale"]))
            elif t == "gla":
                kw.update(tau=float(m["tau"]), decay_rank=int(m.get("decay_rank", 0)))
            else:
                kw.update(kv_heads=int(m.get("kv_heads", m["heads"])), rot_dims=int(rot.get("dims", 0)),
                          scale=float(m["scale"]))
            layers.append(RivetarLayer(**kw))
        lp = d.get("loop")
        loop = None
        if lp:
            loop = (int(lp["start"]), int(lp["stop"]), int(lp["times"]))
            if not (0 <= loop[0] < loop[1] <= len(layers)) or loop[2] < 1:
                raise ValueError(f"loop {lp!r} does not fit {len(layers)} layers")
        return cls(width=int(d["width"]), vocab_size=int(d["vocab"]), layers=layers, eps=float(d["norm"]["eps"]),
                   embed_scale=float((d.get("embedding") or {}).get("scale", 1.0)),
                   logit_softcap=float(d.get("logit_softcap") or 0.0), loop=loop, name=name)

    def to_dict(self) -> dict:
        """the ``config.json`` form (inverse of ``from_dict``)"""
        out = []
        for l in self.layers:
            mask = None if l.window >= NO_WINDOW else {"size": l.window, "keep_first": l.keep_first}
            rot = {"base": l.rot_base, "dims": l.rot_dims}
            if l.rot_layout != "interleaved":
                rot["layout"] = l.rot_layout
            if l.type == "latent_attention":
                m = {"heads": l.heads, "dim": l.dim, "rot_dim": l.rot_dim, "vdim": l.vdim, "kv_rank": l.kv_rank,
                     "q_rank": l.q_rank, "rot": rot, "scale": l.scale}
            elif l.type == "gla":
                m = {"heads": l.heads, "dim": l.dim, "vdim": l.vdim, "tau": l.tau}
            else:
                m = {"heads": l.heads, "kv_heads": l.kv_heads, "dim": l.dim, "vdim": l.vdim, "rot": rot, "scale": l.scale}
            if mask is not None and l.type != "gla":
                m["mask"] = mask
            out.append({"type": l.type, "mixer": m, "mlp": {"kind": "dense", "ff": l.ff} if l.ff else None})
        d = {"architecture": ARCHITECTURE, "width": self.width, "vocab": self.vocab_size, "norm": {"eps": self.eps},
             "embedding": {"scale": self.embed_scale}, "layers": out}
        if self.logit_softcap:
            d["logit_softcap"] = self.logit_softcap
        if self.loop is not None:
            d["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        return d

    def with_shapes(self, shapes: Dict[str, tuple]) -> "RivetarConfig":
        """sizes that only a tensor's shape gives (the inner size of the gla decay projection)"""
        layers = []
        for i, l in enumerate(self.layers):
            k = f"l{i}.mix.a1"
            if l.type == "gla" and k in shapes:
                l = RivetarLayer(**{**l.__dict__, "decay_rank": int(shapes[k][0])})
            layers.append(l)
        return RivetarConfig(**{**self.__dict__, "layers": layers})

    @property
    def params(self) -> int:
        return sum(math.prod(s) for s in tensor_shapes(self).values())

    def streamed_bytes(self, elem: int = 2) -> int:
        """weight bytes one decode step of ONE token reads: every matrix once per execution of its layer, the head"""
        shapes = tensor_shapes(self)
        n = self.vocab_size * self.width
        for i, t in self.runs():
            n += sum(math.prod(s) for k, s in shapes.items() if k.startswith(f"l{i}.") and len(s) == 2)
            if t >= 0 and i == self.loop[0]:
                n += 2 * self.width * self.width
        return n * elem

    def kv_bytes_per_token(self, elem: int = 2) -> int:
        return sum(self.layers[i].cache_row for i, _ in self.runs()) * elem


def tensor_shapes(cfg: RivetarConfig) -> Dict[str, tuple]:
    """every tensor of a checkpoint, by name"""
    D, V = cfg.width, cfg.vocab_size
    s = {"embed": (V, D), "final.norm": (D,), "head": (V, D)}
    if cfg.loop is not None:
        s["loop.in"] = (D, 2 * D)
        s["loop.step"] = (cfg.loop[2], D)
    for i, l in enumerate(cfg.layers):
        p = f"l{i}."
        s[p + "norm1"] = s[p + "norm1b"] = (D,)
        if l.type == "latent_attention":
            s.update({p + "mix.dq": (l.q_rank, D), p + "mix.dq.norm": (l.q_rank,),
                      p + "mix.uq": (l.heads * (l.dim + l.rot_dim), l.q_rank),
                      p + "mix.dkv": (l.kv_rank + l.rot_dim, D), p + "mix.dkv.norm": (l.kv_rank,),
                      p + "mix.uk": (l.heads * l.dim, l.kv_rank), p + "mix.uv": (l.heads * l.vdim, l.kv_rank),
                      p + "mix.o": (D, l.heads * l.vdim)})
        elif l.type == "gla":
            s.update({p + "mix.q": (l.heads * l.dim, D), p + "mix.k": (l.heads * l.dim, D),
                      p + "mix.v": (l.heads * l.vdim, D), p + "mix.g": (l.heads * l.vdim, D),
                      p + "mix.o": (D, l.heads * l.vdim), p + "mix.norm": (l.vdim,),
                      p + "mix.a1": (l.decay_rank, D), p + "mix.a2": (l.heads * l.dim, l.decay_rank),
                      p + "mix.a2.b": (l.heads * l.dim,)})
        else:
            s.update({p + "mix.q": (l.heads * l.dim, D), p + "mix.k": (l.kv_heads * l.dim, D),
                      p + "mix.v": (l.kv_heads * l.vdim, D), p + "mix.sink": (l.heads,),
                      p + "mix.o": (D, l.heads * l.vdim)})
        if l.ff:
            s.update({p + "norm2": (D,), p + "norm2b": (D,), p + "mlp.up": (l.ff, D), p + "mlp.down": (D, l.ff),
                      p + "mlp.act": (4,)})
    return s


def tiny_config(**kw) -> RivetarConfig:
    """one small layer of every mixer, unequal sizes, a repeated span (tests, smoke runs)"""
    layers = [
        RivetarLayer(type="gla", heads=2, dim=24, vdim=16, decay_rank=8, tau=8.0, ff=48),
        RivetarLayer(type="attention", heads=4, kv_heads=2, dim=16, vdim=24, rot_base=1000.0, rot_dims=8, window=9,
                     keep_first=3, scale=0.25),
        RivetarLayer(type="latent_attention", heads=3, dim=16, vdim=8, rot_dim=8, kv_rank=24, q_rank=40, rot_base=500.0,
                     rot_dims=8, scale=0.2, ff=56),
    ]
    base = dict(width=64, vocab_size=96, layers=layers, eps=1e-5, embed_scale=4.0, logit_softcap=20.0, loop=(0, 2, 2),
                name="tiny")
    base.update(kw)
    return RivetarConfig(**base)


def sized_config(width: int, n_layers: int, heads: int, vocab: int = 32768, dim: int = 128, window: int = 1024,
                 keep_first: int = 4, ff: Optional[int] = None, loop: Optional[Tuple[int, int, int]] = None,
                 name: str = "rivetar-sized") -> RivetarConfig:
    """layers of a realistic size for throughput measurements (random weights): the three mixers in turn"""
    ff = ff if ff is not None else 4 * width
    lat = RivetarLayer(type="latent_attention", heads=heads, dim=dim, vdim=dim, rot_dim=dim // 2, kv_rank=512,
                       q_rank=max(256, width // 2), rot_dims=dim // 2, scale=1.0 / math.sqrt(dim + dim // 2), ff=ff)
    gla = RivetarLayer(type="gla", heads=heads, dim=dim, vdim=dim, decay_rank=32, tau=8.0, ff=ff)
    att = RivetarLayer(type="attention", heads=heads, kv_heads=max(1, heads // 4), dim=dim, vdim=dim, rot_dims=dim,
                       window=window, keep_first=keep_first, scale=1.0 / math.sqrt(dim), ff=ff)
    return RivetarConfig(width=width, vocab_size=vocab, layers=[(lat, gla, att)[i % 3] for i in range(n_layers)],
                         embed_scale=math.sqrt(width), logit_softcap=30.0, loop=loop, name=name)


def random_weights(cfg: RivetarConfig, seed: int, device="cpu", dtype=torch.bfloat16) -> Dict[str, torch.Tensor]:
    """Named state dict with variance-preserving random matrices, norm offsets near zero, decay biases that keep the
    state alive for tens of tokens (throughput runs and smoke tests; nothing trained)."""
    g = torch.Generator(device=device).manual_seed(seed)
    w = {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.rsplit(".", 1)[-1]
        rnd = lambda: torch.randn(shape, generator=g, device=device)
        if leaf in ("norm1", "norm1b", "norm2", "norm2b") or name == "final.norm":
            t = 0.1 * rnd()
        elif name.endswith("dq.norm") or name.endswith("dkv.norm") or name.endswith("mix.norm"):
            t = 1.0 + 0.1 * rnd()
        elif leaf == "sink":
            t = rnd()
        elif leaf == "b":
            t = 2.0 + rnd()
        elif leaf == "act":
            t = torch.tensor([0.7, 0.4, -0.3, 0.05], device=device) + 0.1 * rnd()
        elif leaf == "step":
            t = 0.3 * rnd()
        elif leaf == "embed":
            t = rnd() / cfg.embed_scale
        else:
            t = rnd() / math.sqrt(shape[-1])
        w[name] = t.to(dtype)
    return w


def pack(w: Dict[str, torch.Tensor], cfg: RivetarConfig, device, dtype) -> Dict[Tuple[int, str], torch.Tensor]:
    """checkpoint names -> engine buffers keyed (layer or -1, engine tensor name).  Matrices that read the same input
    are stacked into one ([dq | dkv], [q | k | v | g | a1], [q | k | v]); the key up-projection is transposed per head
    (the query is carried into latent space through it); matrices take the engine's element type, everything that
    enters 32-bit arithmetic directly (norm weights, sinks, decay projection, activation coefficients) stays fp32."""
    want = tensor_shapes(cfg)
    for k, shape in want.items():
        if k not in w:
            raise KeyError(f"checkpoint lacks tensor {k}")
        if tuple(w[k].shape) != tuple(shape):
            raise ValueError(f"tensor {k} has shape {tuple(w[k].shape)}, the configuration says {tuple(shape)}")
    mat = lambda t: t.to(device=device, dtype=dtype).contiguous()
    vec = lambda t: t.to(device=device, dtype=torch.float32).contiguous()
    out = {(-1, "embed"): mat(w["embed"]), (-1, "final_norm"): vec(w["final.norm"]), (-1, "head"): mat(w["head"])}
    if cfg.loop is not None:
        out[(-1, "loop_in")] = mat(w["loop.in"])
        out[(-1, "loop_step")] = vec(w["loop.step"])
    for i, l in enumerate(cfg.layers):
        p = f"l{i}."
        out[(i, "norm1")], out[(i, "norm1b")] = vec(w[p + "norm1"]), vec(w[p + "norm1b"])
        if l.type == "latent_attention":
            out[(i, "w_in")] = mat(torch.cat([w[p + "mix.dq"], w[p + "mix.dkv"]], 0))
            out[(i, "q_norm")], out[(i, "kv_norm")] = vec(w[p + "mix.dq.norm"]), vec(w[p + "mix.dkv.norm"])
            out[(i, "w_uq")] = mat(w[p + "mix.uq"])
            out[(i, "w_uk")] = mat(w[p + "mix.uk"].reshape(l.heads, l.dim, l.kv_rank).transpose(1, 2))
            out[(i, "w_uv")] = mat(w[p + "mix.uv"])
        elif l.type == "gla":
            out[(i, "w_in")] = mat(torch.cat([w[p + x] for x in ("mix.q", "mix.k", "mix.v", "mix.g", "mix.a1")], 0))
            out[(i, "w_decay")], out[(i, "b_decay")] = vec(w[p + "mix.a2"]), vec(w[p + "mix.a2.b"])
            out[(i, "out_norm")] = vec(w[p + "mix.norm"])
        else:
            out[(i, "w_in")] = mat(torch.cat([w[p + x] for x in ("mix.q", "mix.k", "mix.v")], 0))
            out[(i, "sink")] = vec(w[p + "mix.sink"])
        out[(i, "w_o")] = mat(w[p + "mix.o"])
        if l.ff:
            out[(i, "norm2")], out[(i, "norm2b")] = vec(w[p + "norm2"]), vec(w[p + "norm2b"])
            out[(i, "w_up")], out[(i, "w_down")] = mat(w[p + "mlp.up"]), mat(w[p + "mlp.down"])
            out[(i, "act")] = vec(w[p + "mlp.act"])
    return out


def load_config_dir(path: str) -> RivetarConfig:
    with open(os.path.join(path, "config.json")) as f:
        return RivetarConfig.from_dict(json.load(f), name=os.path.basename(os.path.normpath(path)) or "rivetar")
