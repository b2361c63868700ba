"""A plain, slow implementation of the Karitar decoder, for tests only: whole sequences, no cache, float64,
one function per mechanism, and no code shared with the library under test (it reads config.json's keys and
looks tensors up by name on its own).

The design in this file's notation (T tokens, width D):

* residual as ``S`` streams (hyper-connections): every stream starts as the embedding; a sublayer f with read
  weights a[S], write weights b[S] and a stream-mixing matrix M[S, S] (indexed [from, to]) does
  ``u = sum_s a_s X_s;  y = f(rmsnorm(u));  X'_t = sum_s M[s, t] X_s + b_t y``; the model's output norm sees
  ``sum_s X_s``.
* attention: biased q/k/v projections; one RMS norm over the whole q row (all heads together) and one over
  the whole k row, each with a weight vector of the row's size; no position encoding; scores
  ``(q . k) * scale`` over the last ``window`` keys (own included); weights ``exp(s_j) / (1 + sum_j exp(s_j))``
  (a sink of score 0 that carries no value); every head's output times ``sigmoid(W_g h)`` (one number per
  head, from the mixer's input); output projection.  Keys and values may have different sizes per head.
* feed-forward: ``W_down relu(W_up h)^2``; a layer may have none.
* a run of layers may be repeated several times with the same weights before the rest follow.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import torch

F64 = torch.float64


# ---- mechanisms ---------------------------------------------------------------------------------

def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    x = x.to(F64)
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * weight.to(F64)


def linear(x, w, b=None):
    y = x.to(F64) @ w.to(F64).t()
    return y if b is None else y + b.to(F64)


def sink_softmax(scores: torch.Tensor, visible: torch.Tensor) -> torch.Tensor:
    """scores, visible: [..., keys].  p_j = e^{s_j} / (1 + sum_visible e^{s_j}); 0 where not visible."""
    s = scores.to(F64).masked_fill(~visible, -math.inf)
    m = torch.clamp(s.max(-1, keepdim=True).values, min=0.0)          # the sink's score 0 takes part in the maximum
    e = torch.exp(s - m)
    return e / (torch.exp(-m) + e.sum(-1, keepdim=True))


def window_mask(t: int, window: int) -> torch.Tensor:
    """[t, t] bool: query i sees key j when 0 <= i - j < window (window 0: every earlier key and itself)."""
    i = torch.arange(t)[:, None]
    j = torch.arange(t)[None, :]
    ok = j <= i
    if window > 0:
        ok = ok & (i - j < window)
    return ok


def gated_sink_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, *, heads: int, kv_heads: int, dim: int,
                         vdim: int, scale: float, window: int, eps: float) -> torch.Tensor:
    """h: [T, D] -> [T, D]; ``p`` is the prefix of the mixer's tensors ('l3.mix.')."""
    t = h.shape[0]
    q = linear(h, w[p + "q"], w[p + "q.b"])
    k = linear(h, w[p + "k"], w[p + "k.b"])
    v = linear(h, w[p + "v"], w[p + "v.b"])
    q = rms_norm(q, w[p + "q.norm"], eps).view(t, heads, dim)
    k = rms_norm(k, w[p + "k.norm"], eps).view(t, kv_heads, dim)
    v = v.view(t, kv_heads, vdim)
    gate = torch.sigmoid(linear(h, w[p + "g"]))                      # [T, heads]
    group = heads // kv_heads
    vis = window_mask(t, window)
    out = torch.zeros(t, heads, vdim, dtype=F64)
    for hh in range(heads):
        g = hh // group
        s = (q[:, hh] @ k[:, g].t()) * scale
        out[:, hh] = sink_softmax(s, vis) @ v[:, g]
    out = out * gate[:, :, None]
    return linear(out.reshape(t, heads * vdim), w[p + "o"])


def relu2_mlp(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    z = torch.relu(linear(h, w[p + "up"]))
    return linear(z * z, w[p + "down"])


def hyper_sublayer(streams: torch.Tensor, w: Dict[str, torch.Tensor], p: str, f) -> torch.Tensor:
    """streams: [S, T, D]; ``p`` the prefix of the connection's tensors ('l3.hc1.'); f maps the read-out u to y."""
    a, b, m = w[p + "in"].to(F64), w[p + "out"].to(F64), w[p + "mix"].to(F64)
    u = torch.einsum("s,std->td", a, streams)
    y = f(u)
    return torch.einsum("sr,std->rtd", m, streams) + b[:, None, None] * y[None]


def run_order(cfg: dict) -> List[int]:
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    start, stop, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    return list(range(start)) + list(range(start, stop)) * times + list(range(stop, n))


# ---- the model ------------------------------------------------------------------------------------

def forward(weights: Dict[str, torch.Tensor], cfg: dict, tokens: Sequence[int], trace: Optional[list] = None) -> torch.Tensor:
    """float64 logits [T, vocab] of one whole sequence.  ``trace`` (a list) receives the sum of the streams
    after every layer run."""
    w = weights
    eps = float(cfg["norm"]["eps"])
    n_streams = int(cfg.get("streams") or 0)
    x = w["embed"].to(F64)[torch.as_tensor(list(tokens), dtype=torch.long)]
    streams = x[None].repeat(max(1, n_streams), 1, 1)
    for li in run_order(cfg):
        layer = cfg["layers"][li]
        if layer["type"] != "attention":
            raise ValueError(f"layer type {layer['type']!r}")
        mx = layer["mixer"]
        mask = mx.get("mask") or {}
        p = f"l{li}."

        def mixer(u, p=p, mx=mx, mask=mask):
            return gated_sink_attention(rms_norm(u, w[p + "norm1"], eps), w, p + "mix.", heads=int(mx["heads"]),
                                        kv_heads=int(mx["kv_heads"]), dim=int(mx["dim"]), vdim=int(mx["vdim"]),
                                        scale=float(mx["scale"]), window=int(mask.get("size") or 0), eps=eps)

        def ff(u, p=p):
            return relu2_mlp(rms_norm(u, w[p + "norm2"], eps), w, p + "mlp.")

        subs = [("hc1.", mixer)] + ([("hc2.", ff)] if layer.get("mlp") else [])
        for hc, f in subs:
            if n_streams:
                streams = hyper_sublayer(streams, w, p + hc, f)
            else:
                streams = streams + f(streams[0])[None]
        if trace is not None:
            trace.append(streams.sum(0).clone())
    x = streams.sum(0)
    return linear(rms_norm(x, w["final.norm"], eps), w["head"])
