"""Plain, slow restatement of the Rivetar decoder in PyTorch on the CPU: one function per mechanism, whole sequences
at a time, explicit loops over positions where a mechanism is a recurrence or a mask, no cache, no batching.
Test infrastructure only: the product package never imports it and it imports nothing of the product.

Notation: T tokens, D model width, H heads, G key/value heads, dk query/key size per head, dv value size, R latent
size, F feed-forward width.  ``w`` maps tensor names to [out, in] matrices (or vectors); ``cfg`` is the dictionary
form of a checkpoint's ``config.json``."""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


# ------------------------------------------------------------------------------------------------ norms, activations
def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis"""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def plain_norm(x, weight, eps):
    return unit_rms(x, eps) * weight


def offset_norm(x, weight, eps):
    """RMS norm whose stored weight is the deviation from one"""
    return unit_rms(x, eps) * (1.0 + weight)


def polynorm(z, coeff, eps):
    """a N(z) + b N(z^2) + c N(z^3) + e with N = division by the root mean square over the feed-forward axis"""
    a, b, c, e = [coeff[i] for i in range(4)]
    return a * unit_rms(z, eps) + b * unit_rms(z * z, eps) + c * unit_rms(z * z * z, eps) + e


def dense_ff(h, w: Dict[str, torch.Tensor], eps: float):
    return polynorm(h @ w["up"].T, w["act"], eps) @ w["down"].T


# ------------------------------------------------------------------------------------------------ rotations
def pair_angles(positions, pairs: int, base: float, span: int):
    """angle of pair i at position p: p * base^(-2 i / span); [T, pairs] in fp64"""
    i = torch.arange(pairs, dtype=torch.float64)
    return positions.to(torch.float64)[:, None] * (base ** (-2.0 * i / span))[None]


def rotate_pairs(x, positions, dims: int, base: float, layout: str = "interleaved", sign: float = 1.0):
    """Turns the first ``dims`` coordinates of the last axis of x [T, ..., d] by the position's angles; the rest pass.
    interleaved: coordinate 2i pairs with 2i + 1; halves: i with i + dims / 2."""
    half = dims // 2
    a = sign * pair_angles(positions, half, base, dims)
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    cos, sin = a.cos().to(x.dtype).reshape(shape), a.sin().to(x.dtype).reshape(shape)
    out = x.clone()
    if layout == "interleaved":
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = u * cos - v * sin
        out[..., 1:dims:2] = v * cos + u * sin
    else:
        u, v = x[..., :half], x[..., half:dims]
        out[..., :half] = u * cos - v * sin
        out[..., half:dims] = v * cos + u * sin
    return out


# ------------------------------------------------------------------------------------------------ masks
def visible(i: int, j: int, size: Optional[int], keep_first: int) -> bool:
    """may position i look at position j?  causal; inside the window of ``size`` positions or among the kept first ones"""
    if j > i:
        return False
    if size is None:
        return True
    return i - j < size or j < keep_first


def visibility(positions, mask: Optional[dict]) -> torch.Tensor:
    """[T, T] booleans: may the row's position look at the column's?"""
    mask = mask or {}
    pos = [int(p) for p in positions]
    return torch.tensor([[visible(i, j, mask.get("size"), mask.get("keep_first", 0)) for j in pos] for i in pos])


# ------------------------------------------------------------------------------------------------ mixers
def latent_attention(h, positions, w: Dict[str, torch.Tensor], m: dict, eps: float):
    """Queries through a normed latent; keys and values rebuilt per head from a shared normed latent plus one rotated
    key part common to the heads; causal softmax attention."""
    T = h.shape[0]
    H, dn, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    rot = m["rot"]
    layout = rot.get("layout", "interleaved")
    cq = plain_norm(h @ w["dq"].T, w["dq.norm"], eps)
    q = (cq @ w["uq"].T).reshape(T, H, dn + dr)
    q_plain, q_rot = q[..., :dn], rotate_pairs(q[..., dn:], positions, rot["dims"], rot["base"], layout)
    ckr = h @ w["dkv"].T
    c = plain_norm(ckr[:, :R], w["dkv.norm"], eps)
    k_rot = rotate_pairs(ckr[:, R:], positions, rot["dims"], rot["base"], layout)          # [T, dr], all heads
    k_plain = (c @ w["uk"].T).reshape(T, H, dn)
    v = (c @ w["uv"].T).reshape(T, H, dv)
    see = visibility(positions, m.get("mask"))                                             # [T, T]
    s = (torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihd,jd->hij", q_rot, k_rot)) * m["scale"]
    p = torch.softmax(s.masked_fill(~see[None], -math.inf), -1)
    out = torch.einsum("hij,jhd->ihd", p, v)
    return out.reshape(T, H * dv) @ w["o"].T


def gated_linear_attention(h, w: Dict[str, torch.Tensor], m: dict, eps: float, state=None):
    """Per head a [dk, dv] state S: S <- diag(alpha_t) S + k_t v_t^T, o_t = S^T q_t, with a decay per key channel
    alpha = sigmoid(z)^(1 / tau).  Returns (output [T, D], final state [H, dk, dv])."""
    T = h.shape[0]
    H, dk, dv, tau = m["heads"], m["dim"], m["vdim"], float(m["tau"])
    q = (h @ w["q"].T).reshape(T, H, dk) * dk ** -0.5
    k = (h @ w["k"].T).reshape(T, H, dk)
    v = (h @ w["v"].T).reshape(T, H, dv)
    z = (h @ w["a1"].T) @ w["a2"].T + w["a2.b"]
    alpha = torch.sigmoid(z).pow(1.0 / tau).reshape(T, H, dk)
    S = torch.zeros(H, dk, dv, dtype=h.dtype) if state is None else state.clone()
    o = torch.zeros(T, H, dv, dtype=h.dtype)
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S, q[t])
    o = plain_norm(o, w["norm"], eps).reshape(T, H * dv)
    g = h @ w["g"].T
    return (o * (g * torch.sigmoid(g))) @ w["o"].T, S


def windowed_attention(h, positions, w: Dict[str, torch.Tensor], m: dict):
    """Grouped-query softmax attention over a sliding window plus kept first positions, with a learned sink in the
    denominator and values that are rotated by their own position and turned back by the query's."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    rot = m["rot"]
    layout = rot.get("layout", "interleaved")
    q = rotate_pairs((h @ w["q"].T).reshape(T, H, dk), positions, rot["dims"], rot["base"], layout)
    k = rotate_pairs((h @ w["k"].T).reshape(T, G, dk), positions, rot["dims"], rot["base"], layout)
    v = rotate_pairs((h @ w["v"].T).reshape(T, G, dv), positions, dv, rot["base"], layout)
    see = visibility(positions, m.get("mask"))
    kv_of = torch.arange(H) // (H // G)                                                    # query head -> key/value head
    s = torch.einsum("ihd,jhd->hij", q, k[:, kv_of]) * m["scale"]
    s = s.masked_fill(~see[None], -math.inf)
    # the sink is one more column of scores that carries no value
    full = torch.cat([s, w["sink"].to(h.dtype)[:, None, None].expand(H, T, 1)], -1)
    p = torch.softmax(full, -1)[..., :T]
    out = torch.einsum("hij,jhd->ihd", p, v[:, kv_of])
    out = rotate_pairs(out, positions, dv, rot["base"], layout, sign=-1.0)
    return out.reshape(T, H * dv) @ w["o"].T


# ------------------------------------------------------------------------------------------------ the model
def sub(w: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v for k, v in w.items() if k.startswith(prefix)}


def layer_runs(cfg: dict) -> List[tuple]:
    """(layer index, pass number or None, first of its pass) for every layer execution in order"""
    n, loop = len(cfg["layers"]), cfg.get("loop")
    if not loop:
        return [(i, None, False) for i in range(n)]
    runs = [(i, None, False) for i in range(loop["start"])]
    for t in range(loop["times"]):
        runs += [(i, t, i == loop["start"]) for i in range(loop["start"], loop["stop"])]
    return runs + [(i, None, False) for i in range(loop["stop"], n)]


def layer(x, positions, w: Dict[str, torch.Tensor], entry: dict, eps: float):
    h = offset_norm(x, w["norm1"], eps)
    mw = sub(w, "mix.")
    if entry["type"] == "latent_attention":
        y = latent_attention(h, positions, mw, entry["mixer"], eps)
    elif entry["type"] == "gla":
        y, _ = gated_linear_attention(h, mw, entry["mixer"], eps)
    elif entry["type"] == "attention":
        y = windowed_attention(h, positions, mw, entry["mixer"])
    else:
        raise ValueError(entry["type"])
    x = x + offset_norm(y, w["norm1b"], eps)
    if entry.get("mlp") is not None:
        x = x + offset_norm(dense_ff(offset_norm(x, w["norm2"], eps), sub(w, "mlp."), eps), w["norm2b"], eps)
    return x


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float64):
    """tokens of ONE sequence from position 0 -> (logits [T, V], residual stream after every layer run [runs, T, D])"""
    w = {k: v.to(dtype) for k, v in w.items()}
    eps = float(cfg["norm"]["eps"])
    T = len(tokens)
    positions = torch.arange(T)
    x0 = w["embed"][torch.tensor(tokens, dtype=torch.long)] * float(cfg["embedding"]["scale"])
    x, streams = x0, []
    for i, t, first in layer_runs(cfg):
        if first:
            x = torch.cat([x, x0], -1) @ w["loop.in"].T + w["loop.step"][t]
        x = layer(x, positions, sub(w, f"l{i}."), cfg["layers"][i], eps)
        streams.append(x)
    logits = offset_norm(x, w["final.norm"], eps) @ w["head"].T
    cap = cfg.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return logits, torch.stack(streams, 0) if streams else torch.zeros(0, T, cfg["width"], dtype=dtype)


# ------------------------------------------------------------------------------------------------ random models
def tensor_shapes(cfg: dict) -> Dict[str, tuple]:
    D, V = cfg["width"], cfg["vocab"]
    s = {"embed": (V, D), "final.norm": (D,), "head": (V, D)}
    if cfg.get("loop"):
        s["loop.in"] = (D, 2 * D)
        s["loop.step"] = (cfg["loop"]["times"], D)
    for i, e in enumerate(cfg["layers"]):
        p, m = f"l{i}.", e["mixer"]
        s[p + "norm1"] = s[p + "norm1b"] = (D,)
        if e["type"] == "latent_attention":
            H = m["heads"]
            s.update({p + "mix.dq": (m["q_rank"], D), p + "mix.dq.norm": (m["q_rank"],),
                      p + "mix.uq": (H * (m["dim"] + m["rot_dim"]), m["q_rank"]),
                      p + "mix.dkv": (m["kv_rank"] + m["rot_dim"], D), p + "mix.dkv.norm": (m["kv_rank"],),
                      p + "mix.uk": (H * m["dim"], m["kv_rank"]), p + "mix.uv": (H * m["vdim"], m["kv_rank"]),
                      p + "mix.o": (D, H * m["vdim"])})
        elif e["type"] == "gla":
            H = m["heads"]
            low = m.get("decay_rank", 8)
            s.update({p + "mix.q": (H * m["dim"], D), p + "mix.k": (H * m["dim"], D), p + "mix.v": (H * m["vdim"], D),
                      p + "mix.g": (H * m["vdim"], D), p + "mix.o": (D, H * m["vdim"]), p + "mix.norm": (m["vdim"],),
                      p + "mix.a1": (low, D), p + "mix.a2": (H * m["dim"], low), p + "mix.a2.b": (H * m["dim"],)})
        else:
            s.update({p + "mix.q": (m["heads"] * m["dim"], D), p + "mix.k": (m["kv_heads"] * m["dim"], D),
                      p + "mix.v": (m["kv_heads"] * m["vdim"], D), p + "mix.sink": (m["heads"],),
                      p + "mix.o": (D, m["heads"] * m["vdim"])})
        if e.get("mlp") is not None:
            F = e["mlp"]["ff"]
            s.update({p + "norm2": (D,), p + "norm2b": (D,), p + "mlp.up": (F, D), p + "mlp.down": (D, F),
                      p + "mlp.act": (4,)})
    return s


def random_model(cfg: dict, seed: int, scale: float = 1.0) -> Dict[str, torch.Tensor]:
    """weights whose every mechanism matters in the logits: matrices of unit-variance outputs, norm offsets around
    zero, sinks and decay biases of order one, activation coefficients of mixed sign"""
    g = torch.Generator().manual_seed(seed)
    w = {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.rsplit(".", 1)[-1]
        if leaf in ("norm1", "norm1b", "norm2", "norm2b") or name == "final.norm":
            t = 0.2 * torch.randn(shape, generator=g)
        elif name.endswith("dq.norm") or name.endswith("dkv.norm") or name.endswith("mix.norm"):
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif leaf == "sink":
            t = torch.randn(shape, generator=g)
        elif leaf == "b":
            t = 2.0 + torch.randn(shape, generator=g)
        elif leaf == "act":
            t = torch.tensor([0.7, 0.4, -0.3, 0.05]) + 0.1 * torch.randn(shape, generator=g)
        elif leaf == "step":
            t = 0.5 * torch.randn(shape, generator=g)
        elif leaf == "embed":
            t = torch.randn(shape, generator=g) / float(cfg["embedding"]["scale"])
        else:
            t = torch.randn(shape, generator=g) * (scale / math.sqrt(shape[-1]))
        w[name] = t.to(torch.bfloat16)          # what a checkpoint stores
    return w
