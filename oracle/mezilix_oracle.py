"""Plain, slow restatement of the Mezilix decoder in PyTorch on the CPU: one function per mechanism, whole
sequences at a time, every key and value written out per head (no latent-space shortcut, no cache, no batching).
Test infrastructure only: the product package never imports it and it imports nothing of the product.

Notation: T tokens, D model width, H heads, dn / dr unrotated / rotated query-key sizes, dv value size, R latent
size, E experts, F expert width.  ``w`` maps tensor names to 2-D [out, in] matrices (or vectors / scalars)."""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis"""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def scalar_rms_norm(x, g, eps):
    """RMS norm whose gain is ONE number for all coordinates"""
    return unit_rms(x, eps) * g.reshape(())


def bigram_embed(tokens: List[int], embed, bigram, buckets: int, mul_prev: int, mul_cur: int,
                 prev_token: Optional[int] = None):
    """embed[t] + bigram[(prev * mul_prev + t * mul_cur) mod buckets]; a sequence's first token takes the table's
    last row (index ``buckets``)"""
    rows = []
    prev = prev_token
    for t in tokens:
        rows.append(buckets if prev is None else (prev * mul_prev + t * mul_cur) % buckets)
        prev = t
    idx = torch.tensor(tokens, dtype=torch.long)
    return embed[idx] + bigram[torch.tensor(rows, dtype=torch.long)]


def token_shift(h, mu, h_before=None):
    """h_t + (h_{t-1} - h_t) * mu with the UNSHIFTED h of the previous token (zeros before the first token)"""
    first = torch.zeros_like(h[:1]) if h_before is None else h_before.reshape(1, -1)
    prev = torch.cat([first, h[:-1]], 0)
    return h + (prev - h) * mu


def rotate_half_rope(x, positions, dims: int, base: float):
    """Rotates the first ``dims`` coordinates of the last axis: coordinate i pairs with i + dims/2, angle
    p * base^(-2 i / dims).  x [T, ..., d]; positions [T]."""
    half = dims // 2
    i = torch.arange(half, dtype=torch.float64)
    f = base ** (-2.0 * i / dims)
    a = positions.to(torch.float64)[:, None] * f[None]                      # [T, half]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    cos, sin = a.cos().to(x.dtype).reshape(shape), a.sin().to(x.dtype).reshape(shape)
    u, v, rest = x[..., :half], x[..., half:dims], x[..., dims:]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, rest], -1)


def latent_attention(h, positions, w: Dict[str, torch.Tensor], m: dict, eps: float):
    """Queries per head [dn unrotated | dr rotated]; keys and values rebuilt per head from a shared latent (RMS-normed,
    plain weight) plus ONE rotated key part shared by the heads; banded causal softmax attention."""
    H, dn, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    T = h.shape[0]
    q = (h @ w["q"].T).reshape(T, H, dn + dr)
    dkv = h @ w["dkv"].T
    c = unit_rms(dkv[:, :R], eps) * w["dkv.norm"]
    k_rot = rotate_half_rope(dkv[:, R:R + dr], positions, m["rot"]["dims"], m["rot"]["base"])       # [T, dr]
    q_rot = rotate_half_rope(q[..., dn:], positions, m["rot"]["dims"], m["rot"]["base"])            # [T, H, dr]
    k_n = (c @ w["uk"].T).reshape(T, H, dn)
    v = (c @ w["uv"].T).reshape(T, H, dv)
    s = torch.einsum("ihd,jhd->hij", q[..., :dn], k_n) + torch.einsum("ihd,jd->hij", q_rot, k_rot)
    s = s * m["scale"]
    gap = positions[:, None] - positions[None, :]
    seen = (gap >= 0) & (gap < m["mask"]["size"])
    s = s.masked_fill(~seen[None], float("-inf"))
    p = torch.softmax(s, -1)
    o = torch.einsum("hij,jhd->ihd", p, v).reshape(T, H * dv)
    return o @ w["o"].T


def squared_relu_experts(h, w: Dict[str, torch.Tensor], f: dict):
    """softmax router over ALL experts, the ``top`` largest scores kept as they are (no renormalisation),
    expert = down(relu(up x)^2)"""
    E, top = f["router"]["experts"], f["router"]["top"]
    s = torch.softmax(h.float() @ w["router"].float().T, -1).to(h.dtype)
    val, idx = torch.topk(s, top, dim=-1)
    out = torch.zeros(h.shape[0], w["e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for j in range(top):
            e = int(idx[t, j])
            a = torch.relu(w[f"e{e}.up"] @ h[t]) ** 2
            out[t] += val[t, j] * (w[f"e{e}.down"] @ a)
    return out


def depth_average(streams: List[torch.Tensor], coeff):
    """sum_j coeff[j] * streams[j] over the embedding output and every layer result so far"""
    return sum(coeff[j] * streams[j] for j in range(len(streams)))


def sub(w: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v for k, v in w.items() if k.startswith(prefix)}


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float64):
    """Whole sequence from position 0.  Returns (logits [T, V], streams [layers, T, D]: what leaves each layer)."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}
    eps = cfg["norm"]["eps"]
    bg = cfg["embedding"]["bigram"]
    T = len(tokens)
    pos = torch.arange(T)
    x = bigram_embed(tokens, w["embed"], w["bigram"], bg["buckets"], bg["mul_prev"], bg["mul_cur"])
    results, leaving = [x], []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = scalar_rms_norm(x, w[p + "norm1"], eps)
        if layer["type"] != "latent_attention":
            raise ValueError(layer["type"])
        y = latent_attention(token_shift(h, w[p + "shift"]), pos, sub(w, p + "mix."), layer["mixer"], eps)
        if layer.get("mlp") is not None:
            y = y + squared_relu_experts(h, sub(w, p + "mlp."), layer["mlp"])
        results.append(x + y)
        x = depth_average(results, w[p + "dwa"])
        leaving.append(x)
    logits = scalar_rms_norm(x, w["final.norm"], eps) @ w["head"].T
    return logits, (torch.stack(leaving) if leaving else x.new_zeros(0, T, x.shape[-1]))


def random_model(cfg: dict, seed: int, scale: float = 1.0) -> Dict[str, torch.Tensor]:
    """bf16-representable random weights for a config (tests make their own small models with this)"""
    g = torch.Generator().manual_seed(seed)
    D, V = cfg["width"], cfg["vocab"]

    def rn(*shape, std=1.0, mean=0.0):
        return (torch.randn(tuple(shape), generator=g) * std + mean).to(torch.bfloat16)

    w = {"embed": rn(V, D), "bigram": rn(cfg["embedding"]["bigram"]["buckets"] + 1, D, std=0.5)}
    n = len(cfg["layers"])
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        H, dn, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
        w[p + "norm1"] = rn(mean=1.0, std=0.1)
        w[p + "shift"] = (torch.rand(D, generator=g)).to(torch.bfloat16)
        w[p + "dwa"] = (torch.softmax(torch.randn(i + 2, generator=g), 0) * 1.2).to(torch.bfloat16)
        w[p + "mix.q"] = rn(H * (dn + dr), D, std=scale / math.sqrt(D))
        w[p + "mix.dkv"] = rn(R + dr, D, std=scale / math.sqrt(D))
        w[p + "mix.dkv.norm"] = rn(R, mean=1.0, std=0.2)
        w[p + "mix.uk"] = rn(H * dn, R, std=scale / math.sqrt(R))
        w[p + "mix.uv"] = rn(H * dv, R, std=scale / math.sqrt(R))
        w[p + "mix.o"] = rn(D, H * dv, std=1.0 / math.sqrt(H * dv * n))
        f = layer.get("mlp")
        if f is not None:
            E, F = f["router"]["experts"], f["expert"]["ff"]
            w[p + "mlp.router"] = rn(E, D, std=1.0)
            for e in range(E):
                w[p + f"mlp.e{e}.up"] = rn(F, D, std=1.0 / math.sqrt(D))
                w[p + f"mlp.e{e}.down"] = rn(D, F, std=1.0 / math.sqrt(F * n))
    w["final.norm"] = rn(mean=1.0, std=0.1)
    w["head"] = rn(V, D, std=1.0 / math.sqrt(D))
    return w
