"""A plain, slow implementation of the Fipavik decoder, for tests only: whole sequences, no cache, float64,
one function per mechanism, and no code shared with the library under test (it reads config.json's keys and
looks tensors up by name on its own).

The design in this file's notation (T tokens, width D, ``r`` the config's ``residual_mult``):

* a layer is one layer norm (mean and variance, weight and bias) whose output ``h`` feeds the mixer and the
  feed-forward side by side: ``x' = x + r (mixer(h) + ff(h))``; a layer may have no feed-forward.
* mixer "attention": grouped queries; per-head RMS norm of queries and keys with one weight vector of the head's
  size; rotation of the first ``rot.dims`` elements of every head by halves; ``scores = (q . k) scale`` inside the
  query's own chunk of ``mask.size`` positions (chunks counted from position 0); a learned sink per head in the
  softmax's denominator; values of layers that say ``v_mix`` are blended with the values of the first such
  layer, ``v' = (1 - lam) v + lam v_first`` (the first one keeps its own).
* mixer "latent_attention": keys and values of all heads come from one latent vector ``c`` per token (RMS-normed)
  through ``W_uk`` and ``W_uv``; beside it one rotated key part shared by all heads; queries are, head by head,
  an unrotated part that meets ``W_uk c`` and a rotated part that meets the shared key part; sliding window of
  ``mask.size`` positions; the same sink.
* feed-forward: a router (float, with bias) picks the ``top`` experts of largest logit, weights them by a softmax
  over the picked logits, and adds a shared expert; every expert is ``W_down (silu(W_gate h) * W_up h)``.
* final layer norm, logits against the embedding table.
"""
from __future__ import annotations

import math
from typing import Dict, Optional, Sequence

import torch

F64 = torch.float64


# ---- mechanisms ---------------------------------------------------------------------------------

def linear(x, w):
    return x.to(F64) @ w.to(F64).t()


def layer_norm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, eps: float) -> torch.Tensor:
    x = x.to(F64)
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * weight.to(F64) + bias.to(F64)


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    x = x.to(F64)
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * weight.to(F64)


def rotate_halves(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x: [T, heads, d]; the first ``dims`` elements of every head are rotated, element i with element i + dims/2,
    by the angle ``position * base^(-2i/dims)``; the rest pass."""
    half = dims // 2
    i = torch.arange(half, dtype=F64)
    ang = positions.to(F64)[:, None] * (float(base) ** (-2.0 * i / dims))[None, :]          # [T, half]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    x = x.to(F64)
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def chunk_mask(t: int, size: int) -> torch.Tensor:
    """[t, t] bool: query i sees key j <= i of its own chunk (i // size == j // size)."""
    i = torch.arange(t)[:, None]
    j = torch.arange(t)[None, :]
    return (j <= i) & (i // size == j // size)


def window_mask(t: int, size: int) -> torch.Tensor:
    """[t, t] bool: query i sees key j when 0 <= i - j < size."""
    i = torch.arange(t)[:, None]
    j = torch.arange(t)[None, :]
    return (j <= i) & (i - j < size)


def sink_softmax(scores: torch.Tensor, visible: torch.Tensor, sink: torch.Tensor) -> torch.Tensor:
    """scores, visible: [T, keys]; sink: a number.  p_j = e^{s_j} / (e^{sink} + sum_visible e^{s_j})."""
    s = scores.to(F64).masked_fill(~visible, -math.inf)
    sink = sink.to(F64)
    m = torch.maximum(s.max(-1, keepdim=True).values, sink)
    e = torch.exp(s - m)
    return e / (torch.exp(sink - m) + e.sum(-1, keepdim=True))


def attention_values(h, w, p, *, kv_heads: int, vdim: int) -> torch.Tensor:
    """The unblended values of an "attention" mixer: [T, kv_heads, vdim]."""
    return linear(h, w[p + "v"]).view(h.shape[0], kv_heads, vdim)


def chunked_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, mx: dict, eps: float,
                      v_first: Optional[torch.Tensor]) -> torch.Tensor:
    """h: [T, D] -> [T, D]; ``p`` is the prefix of the mixer's tensors; ``v_first``: the values to blend with
    (None: this layer keeps its own)."""
    t = h.shape[0]
    heads, kv_heads, dim, vdim = int(mx["heads"]), int(mx["kv_heads"]), int(mx["dim"]), int(mx["vdim"])
    pos = torch.arange(t)
    q = rms_norm(linear(h, w[p + "q"]).view(t, heads, dim), w[p + "q.norm"], eps)
    k = rms_norm(linear(h, w[p + "k"]).view(t, kv_heads, dim), w[p + "k.norm"], eps)
    q = rotate_halves(q, pos, int(mx["rot"]["dims"]), float(mx["rot"]["base"]))
    k = rotate_halves(k, pos, int(mx["rot"]["dims"]), float(mx["rot"]["base"]))
    v = attention_values(h, w, p, kv_heads=kv_heads, vdim=vdim)
    if v_first is not None:
        lam = w[p + "vmix"].to(F64)
        v = (1.0 - lam) * v + lam * v_first
    vis = chunk_mask(t, int(mx["mask"]["size"]))
    group = heads // kv_heads
    out = torch.zeros(t, heads, vdim, dtype=F64)
    for hh in range(heads):
        g = hh // group
        s = (q[:, hh] @ k[:, g].t()) * float(mx["scale"])
        out[:, hh] = sink_softmax(s, vis, w[p + "sink"][hh]) @ v[:, g]
    return linear(out.reshape(t, heads * vdim), w[p + "o"])


def latent_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, mx: dict, eps: float) -> torch.Tensor:
    t = h.shape[0]
    heads, dim, rdim, vdim, rank = int(mx["heads"]), int(mx["dim"]), int(mx["rot_dim"]), int(mx["vdim"]), int(mx["kv_rank"])
    pos = torch.arange(t)
    base = float(mx["rot"]["base"])
    q = linear(h, w[p + "q"]).view(t, heads, dim + rdim)
    q_plain, q_rot = q[..., :dim], rotate_halves(q[..., dim:], pos, rdim, base)
    down = linear(h, w[p + "dkv"])
    c = rms_norm(down[:, :rank], w[p + "dkv.norm"], eps)                                    # [T, rank]
    k_rot = rotate_halves(down[:, None, rank:], pos, rdim, base)[:, 0]                      # [T, rdim], one for all heads
    k_plain = linear(c, w[p + "uk"]).view(t, heads, dim)
    v = linear(c, w[p + "uv"]).view(t, heads, vdim)
    vis = window_mask(t, int(mx["mask"]["size"]))
    out = torch.zeros(t, heads, vdim, dtype=F64)
    for hh in range(heads):
        s = (q_plain[:, hh] @ k_plain[:, hh].t() + q_rot[:, hh] @ k_rot.t()) * float(mx["scale"])
        out[:, hh] = sink_softmax(s, vis, w[p + "sink"][hh]) @ v[:, hh]
    return linear(out.reshape(t, heads * vdim), w[p + "o"])


def expert(h, w, p):
    g = linear(h, w[p + "gate"])
    return linear(g * torch.sigmoid(g) * linear(h, w[p + "up"]), w[p + "down"])


def route(h, w, p, top: int):
    """(chosen experts [T, top], their weights [T, top], by how much the last chosen logit beats the best one left
    out [T]; infinite where every expert is chosen)."""
    z = linear(h, w[p + "router"]) + w[p + "router.b"].to(F64)
    val, idx = torch.topk(z, top, dim=-1)
    if top < z.shape[-1]:
        margin = val[:, -1] - torch.topk(z, top + 1, dim=-1).values[:, -1]
    else:
        margin = torch.full((z.shape[0],), math.inf, dtype=F64)
    return idx, torch.softmax(val, dim=-1), margin


def moe(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, ml: dict, margins: Optional[list] = None) -> torch.Tensor:
    n_exp, top = int(ml["router"]["experts"]), int(ml["router"]["top"])
    idx, wt, margin = route(h, w, p, top)
    if margins is not None:
        margins.append(margin)
    out = torch.zeros(h.shape[0], w[p + "e0.down"].shape[0], dtype=F64)
    for e in range(n_exp):
        hit = idx == e                                      # [T, top]
        rows = hit.any(-1)
        if rows.any():
            out[rows] += (wt * hit).sum(-1)[rows, None] * expert(h[rows], w, f"{p}e{e}.")
    if ml.get("shared"):
        out = out + expert(h, w, p + "shared.")
    return out


# ---- the model ------------------------------------------------------------------------------------

def forward(weights: Dict[str, torch.Tensor], cfg: dict, tokens: Sequence[int], trace: Optional[list] = None,
            margins: Optional[list] = None) -> torch.Tensor:
    """float64 logits [T, vocab] of one whole sequence.  ``trace`` (a list) receives the residual after every layer,
    ``margins`` every router's margins (see ``route``)."""
    w = weights
    eps = float(cfg["norm"]["eps"])
    r = float(cfg["residual_mult"])
    x = w["embed"].to(F64)[torch.as_tensor(list(tokens), dtype=torch.long)]
    v_first = None
    for li, layer in enumerate(cfg["layers"]):
        p = f"l{li}."
        mx = layer["mixer"]
        h = layer_norm(x, w[p + "norm1"], w[p + "norm1.b"], eps)
        if layer["type"] == "attention":
            blend = bool(mx.get("v_mix"))
            y = chunked_attention(h, w, p + "mix.", mx, eps, v_first if blend else None)
            if blend and v_first is None:
                v_first = attention_values(h, w, p + "mix.", kv_heads=int(mx["kv_heads"]), vdim=int(mx["vdim"]))
        elif layer["type"] == "latent_attention":
            y = latent_attention(h, w, p + "mix.", mx, eps)
        else:
            raise ValueError(f"layer type {layer['type']!r}")
        if layer.get("mlp"):
            y = y + moe(h, w, p + "mlp.", layer["mlp"], margins)
        x = x + r * y
        if trace is not None:
            trace.append(x.clone())
    return linear(layer_norm(x, w["final.norm"], w["final.norm.b"], eps), w["embed"])
