"""A residual kept as several streams (hyper-connections).

Instead of one residual ``x`` there are S streams ``X_1 .. X_S`` (float32 ``[S, N, hidden]``) that all start as the
embedding.  A sublayer f reads a weighted sum of the streams and writes its output back into every stream while the
streams are mixed among themselves:

    u = sum_s read[s] X_s;   y = f(norm(u));   X_t <- sum_s mix[s, t] X_s + write[t] y   (all t at once)

and what follows the last layer sees ``sum_s X_s``.  With S = 1, read = write = mix = 1 this is the ordinary
residual add.  The three weight sets belong to the sublayer; here the read weights live with the norm that reads
(``HyperRmsNorm``) and the write and mix weights with a ``StreamWrite`` part that the block attaches to the
sublayer's ``Branch``: the next norm, whichever block it is in, then applies the write, reads with its own weights
and normalises in ONE kernel (``ops.hc_add_rmsnorm``), as ``RmsNorm`` does for the single residual.  The streams
and every sum over them are float32.
"""
from __future__ import annotations

from typing import Optional

import torch

from .base import Block, Branch, Norm, Part, TensorDecl, register_part


def _f32(t: torch.Tensor, env) -> torch.Tensor:
    """A small weight vector in float32 on the part's device (the kernel reads these as float32 whatever the
    checkpoint stored)."""
    if t.dtype == torch.float32:
        return t.contiguous()
    if t.is_cuda and hasattr(env.ops, "cast"):
        out = torch.empty(t.shape, dtype=torch.float32, device=t.device)
        env.ops.cast(t.contiguous(), out)
        return out
    return t.to(torch.float32).contiguous()


class StreamWrite(Part):
    """How a sublayer's output enters the streams.  params: streams.  Tensors: ``mix`` [S, S] indexed [from, to],
    ``out`` [S]."""

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        self.streams = int(params["streams"])
        self.mix = self.out = None

    def tensors(self):
        return {"mix": TensorDecl((self.streams, self.streams), "stream_mix"),
                "out": TensorDecl((self.streams,), "stream_gain")}

    def bind(self, tensors):
        self.mix, self.out = _f32(tensors["mix"], self.env), _f32(tensors["out"], self.env)


class HyperRmsNorm(Norm):
    """RMSNorm of a read-out of the streams, fused with the pending branch's write.  params: size, eps, streams,
    read ("weights": a tensor ``in`` [S]; "sum": the plain sum of the streams, no tensor)."""

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.streams = int(params["streams"])
        self.read_kind = params.get("read", "weights")
        if self.read_kind not in ("weights", "sum"):
            raise ValueError(f"hyper_rmsnorm: read '{self.read_kind}' is not known (weights, sum)")
        if self.eps <= 0:
            raise ValueError("RMSNorm eps must be positive")
        limit = getattr(env.ops, "hc_max_streams", None)
        if self.streams < 1 or (limit is not None and env.device.type == "cuda" and self.streams > limit()):
            raise ValueError(f"hyper_rmsnorm: {self.streams} streams; the kernel takes 1 to {limit() if limit else '?'}")
        self.weight: Optional[torch.Tensor] = None
        self.read: Optional[torch.Tensor] = None

    def tensors(self):
        t = {"weight": TensorDecl((self.size,), "norm")}
        if self.read_kind == "weights":
            t["in"] = TensorDecl((self.streams,), "stream_gain")
        return t

    def bind(self, tensors):
        self.weight = tensors["weight"]
        if self.read_kind == "weights":
            self.read = _f32(tensors["in"], self.env)

    def forward(self, residual, branch: Optional[Branch], ctx, rows=None):
        if residual.dim() != 3 or residual.shape[0] != self.streams:
            raise ValueError(f"hyper_rmsnorm: the residual has shape {tuple(residual.shape)}, expected {self.streams} streams")
        m = residual.shape[1] if rows is None else rows.numel()
        out = ctx.buffer("norm.out", (m, self.size))
        mix = write = data = None
        if branch is not None and (branch.more or branch.scale != 1.0):
            raise ValueError("hyper_rmsnorm: the pending branch carries several sublayers' outputs or a scale")
        if branch is not None:
            if not isinstance(branch.write, StreamWrite) or branch.write.streams != self.streams:
                raise ValueError("hyper_rmsnorm: the pending branch carries no write weights for these streams")
            data, mix, write = branch.data, branch.write.mix, branch.write.out
        ctx.ops.hc_add_rmsnorm(residual, data, mix, write, self.read, self.weight, self.eps, out, rows)
        return out


class HyperPreNormBlock(Block):
    """Pre-norm sublayers over a residual of several streams.  roles: norm1, mixer, write1 and, where the layer has a
    feed-forward, norm2, ffn, write2 (the norms are ``hyper_rmsnorm`` parts, the writes ``stream_write`` parts).  The
    block hands its last sublayer's branch on with the write weights attached; the next block's first norm (or the
    model's final norm) applies it."""

    ROLES = {"norm1": "norm", "mixer": "mixer", "write1": "connection",
             "norm2": "norm", "ffn": "ffn", "write2": "connection"}

    def __init__(self, params, prefix, env, parts):
        super().__init__(params, prefix, env, parts)
        for role in ("norm1", "mixer", "write1"):
            if role not in parts:
                raise ValueError(f"hyper_prenorm: no part for the role '{role}'")
        if ("ffn" in parts) != ("norm2" in parts) or ("ffn" in parts) != ("write2" in parts):
            raise ValueError("hyper_prenorm: norm2, ffn and write2 come together or not at all")

    def forward(self, residual, pending: Optional[Branch], ctx, cache) -> Optional[Branch]:
        p = self.parts
        a = p["mixer"].forward(p["norm1"].forward(residual, pending, ctx), ctx, cache)
        a.write = p["write1"]
        if "ffn" not in p:
            return a
        f = p["ffn"].forward(p["norm2"].forward(residual, a, ctx), ctx)
        f.write = p["write2"]
        return f


register_part("connection", "stream_write", StreamWrite)
register_part("norm", "hyper_rmsnorm", HyperRmsNorm)
register_part("block", "hyper_prenorm", HyperPreNormBlock)
