"""Attention whose keys and values of all heads come from one small latent vector per token.

Per token the mixer's input ``h`` gives

* queries ``q = W_q h``, head by head ``[dim unrotated | rot_dim rotated]``;
* ``W_dkv h`` = ``[kv_rank | rot_dim]``: the first part, RMS-normed with a weight, is the latent ``c``; the second,
  rotated by the token's position, is one key part that every head shares;
* per head ``k_h = [W_uk,h c | shared rotated part]`` and ``v_h = W_uv,h c``.

Only ``c`` and the rotated key part are kept per position.  The products with ``W_uk`` and ``W_uv`` are moved to the
query's side (they are linear): ``q_h . W_uk,h c = (W_uk,h^T q_h) . c`` and ``sum_j p_j W_uv,h c_j = W_uv,h sum_j p_j c_j``.
So attention runs over ONE key/value head whose keys are ``[c | rotated part]`` (``kv_rank + rot_dim`` elements) and
whose values are ``c``, with queries ``[W_uk,h^T q_h,unrotated | q_h,rotated]``, in the same kernels, cache pages and
rings as every other attention; the score's scale, the mask (sliding window or chunks) and a learned sink per head are
parameters.  The cache holds one row per position: the key's pages are read as the values too (a value head as long as a
key head, so that the tensor-core kernels take it), and the per-head product with ``W_uv`` reads the first ``kv_rank``
elements of what attention returns; the rest (the weighted rotated parts) is never looked at.  One kernel (``ops.latent_prep``) adds the input product's partial sums, norms
the latent, rotates and writes queries, keys and values; ``ops.head_linear`` is the per-head product on either side.
Norm statistics, angles, scores and softmax weights are float32 whatever the compute type.
"""
from __future__ import annotations

import torch

from ..kernels.linear import linear
from .base import Branch, KvNeed, Mixer, TensorDecl, as_f32, register_part

_Q, _DKV, _UK, _UV, _O = "q_proj.weight", "kv_down_proj.weight", "k_up_proj.weight", "v_up_proj.weight", "o_proj.weight"


class LatentAttention(Mixer):
    """params: hidden_size, num_heads, head_dim (unrotated elements of a query/key head), rot_dim (rotated elements),
    value_dim, kv_rank, norm_eps (of the latent's norm), window (0 = all keys), mask ("window" or "chunk"),
    softmax_scale, sink (None or "learned": a tensor ``sink`` [num_heads]), position (name of a rotary encoding over
    ``rot_dim`` elements)."""

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        p = params
        self.hidden = int(p["hidden_size"])
        self.nh = int(p["num_heads"])
        self.dim = int(p["head_dim"])
        self.rdim = int(p["rot_dim"])
        self.vdim = int(p["value_dim"])
        self.rank = int(p["kv_rank"])
        for what, v in (("num_heads", self.nh), ("head_dim", self.dim), ("value_dim", self.vdim), ("kv_rank", self.rank)):
            if v <= 0:
                raise ValueError(f"latent_attention: {what} must be positive, got {v}")
        if self.rdim < 0 or self.rdim % 2:
            raise ValueError(f"latent_attention: rot_dim {self.rdim} must be even and not negative")
        self.kd = self.rank + self.rdim                      # elements of a cached key
        limit = getattr(env.ops, "ATTN_MAX_HEAD_DIM", None)
        if limit is not None and self.kd > limit:
            raise ValueError(f"latent_attention: kv_rank + rot_dim = {self.kd}; the attention kernels take keys of up to {limit}")
        self.eps = float(p["norm_eps"])
        self.window = int(p.get("window", 0) or 0)
        self.mask = p.get("mask", "window")
        if self.mask not in ("window", "chunk"):
            raise ValueError(f"latent_attention: mask '{self.mask}' is not known (window, chunk)")
        self.scale = float(p["softmax_scale"])
        if not self.scale > 0:
            raise ValueError("latent_attention: the score scale must be positive")
        self.sink_kind = p.get("sink")
        if self.sink_kind not in (None, "learned"):
            raise ValueError(f"latent_attention: sink '{self.sink_kind}' is not known (None, 'learned')")
        enc = p.get("position")
        self.encoding = env.encodings[enc] if enc is not None else None
        if (self.encoding is None) != (self.rdim == 0):
            raise ValueError("latent_attention: rotated elements and a position encoding come together")
        self.w_in = self.w_o = self.w_absorb = self.w_uv = self.c_norm_w = self.sinks = self.form = None

    def tensors(self):
        t = {_Q: TensorDecl((self.nh * (self.dim + self.rdim), self.hidden)),
             _DKV: TensorDecl((self.rank + self.rdim, self.hidden)),
             "kv_norm.weight": TensorDecl((self.rank,), "norm"),
             _UK: TensorDecl((self.nh * self.dim, self.rank)),
             _UV: TensorDecl((self.nh * self.vdim, self.rank)),
             _O: TensorDecl((self.hidden, self.nh * self.vdim))}
        if self.sink_kind == "learned":
            t["sink"] = TensorDecl((self.nh,), "bias")
        return t

    def bind(self, tensors):
        ws = [tensors[_Q], tensors[_DKV]]
        if ws[0].dtype != ws[1].dtype:
            raise ValueError(f"{self.prefix}: the input projections are stored with different types")
        self.w_in = torch.cat(ws, dim=0).contiguous()
        # [head][rank][dim]: the key up-projection as it meets the query
        self.w_absorb = tensors[_UK].view(self.nh, self.dim, self.rank).transpose(1, 2).contiguous()
        self.w_uv = tensors[_UV].view(self.nh, self.vdim, self.rank).contiguous()
        self.w_o = tensors[_O]
        self.c_norm_w = tensors["kv_norm.weight"]
        if self.sink_kind == "learned":
            self.sinks = as_f32(tensors["sink"], self.env)
        self.form = self.env.ops.AttentionForm(sinks=self.sinks, chunked=self.mask == "chunk")

    def cache_need(self):
        return KvNeed(1, self.kd, self.window, values_in_keys=True)

    def forward(self, x, ctx, cache) -> Branch:
        ops = ctx.ops
        n = x.shape[0]
        rot = self.encoding.rotation() if self.encoding is not None else None
        rows = linear(ctx, x, self.w_in, "lattn.in", torch.float32)
        q_plain = ctx.buffer("lattn.q_plain", (n, self.nh, self.dim))
        q = ctx.buffer("lattn.q", (n, self.nh, self.kd))
        common = dict(n_heads=self.nh, head_dim=self.dim, rot_dim=self.rdim, kv_rank=self.rank, c_norm_w=self.c_norm_w,
                      norm_eps=self.eps, cos=rot.cos if rot else None, sin=rot.sin if rot else None,
                      positions=ctx.positions, q_plain_out=q_plain, q_out=q)
        pages = dict(k_pages=cache.k_pages, page_table=cache.page_table,
                     ring_pages=cache.ring_pages, seq_of_token=ctx.seq_of_token, slots=ctx.slots)
        mixed = ctx.buffer("lattn.mixed", (n, self.nh, self.kd))            # per head sum_j p_j [c_j | rotated part]
        if ctx.decode:
            ops.latent_prep(rows, **common, **pages)
            ops.head_linear(q_plain, self.w_absorb, q[:, :, :self.rank])
            plan = ops.attn_decode_plan(q.dtype, ctx.n_seqs, self.nh, 1, self.kd, ctx.max_len_after, self.form)
            scratch = ctx.buffer("attn.scratch", (max(1, plan.scratch_floats),), torch.float32)
            counters = None
            if plan.n_counters:
                counters = ctx.buffer("attn.counters", (plan.n_counters,), torch.int32, zero=True)
            ops.attn_decode(q, cache.k_pages, cache.v_pages, cache.page_table, cache.ring_pages, ctx.slots,
                            ctx.len_before, mixed.view(n, self.nh * self.kd), scratch, scale=self.scale,
                            window=self.window, plan=plan, counters=counters, form=self.form)
        else:
            write_now = self.window == 0
            k_new = ctx.buffer("lattn.k_new", (n, 1, self.kd))
            if write_now:
                ops.latent_prep(rows, **common, k_new=k_new, **pages)
            else:
                ops.latent_prep(rows, **common, k_new=k_new)
            ops.head_linear(q_plain, self.w_absorb, q[:, :, :self.rank])
            tq = ops.prefill_tile_queries(q.dtype, self.kd, self.form)
            ops.attn_prefill(q, k_new, k_new, cache.k_pages, cache.v_pages, cache.page_table, cache.ring_pages,
                             ctx.query_tiles(tq), ctx.cu_tokens, ctx.len_before, ctx.slots,
                             mixed.view(n, self.nh * self.kd), scale=self.scale, window=self.window,
                             tile_queries=tq, form=self.form)
            if not write_now:
                ops.kv_write(k_new, k_new, cache.k_pages, cache.v_pages, cache.page_table, cache.ring_pages,
                             ctx.positions, ctx.seq_of_token, ctx.slots, ctx.cu_tokens, ctx.len_before)
        out = ctx.buffer("lattn.out", (n, self.nh, self.vdim))
        ops.head_linear(mixed[:, :, :self.rank], self.w_uv, out)
        return Branch(linear(ctx, out.view(n, self.nh * self.vdim), self.w_o, "lattn.proj", torch.float32))


register_part("mixer", "latent_attention", LatentAttention)
