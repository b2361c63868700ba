"""Grouped-query attention with a sink in the softmax, a gate per head and norms over whole projections.

Beside ``parts/attention.py`` (rotary positions, per-head norms): a mixer for designs whose attention

* adds biases inside the q, k and v projections and then, optionally, normalises the WHOLE query row and the whole
  key row (all heads together, RMS norm with a weight vector of the row's size) instead of every head by itself;
* may keep value heads of another size than the key heads (``value_dim``);
* uses a score scale and a window of its own (the last ``window`` keys, the query's own included; 0 = all);
* may put a sink into the softmax, a score that joins the denominator and carries no value:
  ``p_j = exp(s_j) / (exp(sink) + sum_j exp(s_j))``;
* may multiply every head's output by ``sigmoid(w_g . h)``, one number per (token, head) from the mixer's own
  input, before the output projection;
* applies no position encoding (``position`` names one or is None; none is implemented here yet).

One product gives q, k, v and the gates' arguments; one kernel (``ops.qkv_row_prep``) adds partial sums and biases,
applies the two norms and writes queries, keys, values (into the step's packed buffers and/or the cache pages) and
the gates; the attention kernel applies sink and gate in its epilogue.  Norm statistics, scores, softmax weights
and gates are float32 whatever the compute type.
"""
from __future__ import annotations

import math

import torch

from ..kernels.linear import linear
from .base import Branch, KvNeed, Mixer, TensorDecl, register_part

# the part's own names for its tensors; a spec's ``tensor_names`` maps them to a checkpoint's
_Q, _K, _V, _O, _G = "q_proj.weight", "k_proj.weight", "v_proj.weight", "o_proj.weight", "gate_proj.weight"


class GatedSinkAttention(Mixer):
    """params: hidden_size, num_heads, num_kv_heads, head_dim, value_dim (None = head_dim), qkv_bias,
    qk_norm (None or "row"), qk_norm_eps, window (0 = all keys), softmax_scale (None = 1/sqrt(head_dim)),
    sink (None, or the sink's score), head_gate (bool), position (must be None)."""

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        p = params
        self.hidden = int(p["hidden_size"])
        self.nh = int(p["num_heads"])
        self.nkv = int(p["num_kv_heads"])
        self.hd = int(p["head_dim"])
        self.vd = int(p.get("value_dim") or self.hd)
        if self.nkv <= 0 or self.nh % self.nkv:
            raise ValueError(f"{self.nh} heads are not a multiple of {self.nkv} key/value heads")
        limit = getattr(env.ops, "ATTN_MAX_HEAD_DIM", None)
        for what, d in (("head_dim", self.hd), ("value_dim", self.vd)):
            if d <= 0 or (limit is not None and d > limit):
                raise ValueError(f"{what} {d}: the attention kernels take head sizes from 1 to {limit}")
        self.qkv_bias = bool(p.get("qkv_bias", False))
        self.qk_norm = p.get("qk_norm")
        if self.qk_norm not in (None, "row"):
            raise ValueError(f"gated_sink_attention: qk_norm '{self.qk_norm}' is not known (None, 'row')")
        self.qk_norm_eps = float(p.get("qk_norm_eps", 1e-6))
        self.window = int(p.get("window", 0) or 0)
        if self.window < 0:
            raise ValueError("gated_sink_attention: the window must not be negative")
        scale = p.get("softmax_scale")
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.hd)
        if not self.scale > 0:
            raise ValueError("gated_sink_attention: the score scale must be positive")
        sink = p.get("sink")
        self.sink = None if sink is None else float(sink)
        self.head_gate = bool(p.get("head_gate", False))
        if p.get("position") is not None:
            raise ValueError("gated_sink_attention applies no position encoding")
        make_form = getattr(env.ops, "AttentionForm", None)
        self.form = make_form(value_dim=self.vd, sink=self.sink, gated=self.head_gate) if make_form else None
        self.w_in = self.w_o = self.bias = self.q_norm_w = self.k_norm_w = None

    # ---- tensors -------------------------------------------------------------------------
    def tensors(self):
        q, k, v = self.nh * self.hd, self.nkv * self.hd, self.nkv * self.vd
        t = {_Q: TensorDecl((q, self.hidden)), _K: TensorDecl((k, self.hidden)), _V: TensorDecl((v, self.hidden)),
             _O: TensorDecl((self.hidden, self.nh * self.vd))}
        if self.qkv_bias:
            t["q_proj.bias"] = TensorDecl((q,), "bias")
            t["k_proj.bias"] = TensorDecl((k,), "bias")
            t["v_proj.bias"] = TensorDecl((v,), "bias")
        if self.qk_norm == "row":
            t["q_norm.weight"] = TensorDecl((q,), "norm")
            t["k_norm.weight"] = TensorDecl((k,), "norm")
        if self.head_gate:
            t[_G] = TensorDecl((self.nh, self.hidden))
        return t

    def bind(self, tensors):
        ws = [tensors[_Q], tensors[_K], tensors[_V]] + ([tensors[_G]] if self.head_gate else [])
        if len({w.dtype for w in ws}) != 1:
            raise ValueError(f"{self.prefix}: the input projections are stored with different types")
        self.w_in = torch.cat(ws, dim=0).contiguous()
        self.w_o = tensors[_O]
        if self.qkv_bias:
            self.bias = torch.cat([tensors["q_proj.bias"], tensors["k_proj.bias"], tensors["v_proj.bias"]], dim=0).contiguous()
        if self.qk_norm == "row":
            self.q_norm_w, self.k_norm_w = tensors["q_norm.weight"], tensors["k_norm.weight"]
            if self.bias is not None and self.bias.dtype != self.q_norm_w.dtype:
                self.bias = self.bias.to(self.q_norm_w.dtype)

    def cache_need(self):
        return KvNeed(self.nkv, self.hd, self.window, 0 if self.vd == self.hd else self.vd)

    # ---- one step ------------------------------------------------------------------------
    def forward(self, x, ctx, cache) -> Branch:
        ops = ctx.ops
        n = x.shape[0]
        form = self.form
        rows = linear(ctx, x, self.w_in, "gattn.in", torch.float32)
        q = ctx.buffer("gattn.q", (n, self.nh, self.hd))
        gate = ctx.buffer("gattn.gate", (n, self.nh), torch.float32) if self.head_gate else None
        out = ctx.buffer("gattn.out", (n, self.nh * self.vd))
        common = dict(n_heads=self.nh, n_kv_heads=self.nkv, head_dim=self.hd, value_dim=self.vd, bias=self.bias,
                      q_norm_w=self.q_norm_w, k_norm_w=self.k_norm_w, norm_eps=self.qk_norm_eps,
                      positions=ctx.positions, q_out=q, gate_out=gate)
        pages = dict(k_pages=cache.k_pages, v_pages=cache.v_pages, page_table=cache.page_table,
                     ring_pages=cache.ring_pages, seq_of_token=ctx.seq_of_token, slots=ctx.slots)
        if ctx.decode:
            ops.qkv_row_prep(rows, **common, **pages)
            plan = ops.attn_decode_plan(q.dtype, ctx.n_seqs, self.nh, self.nkv, self.hd, ctx.max_len_after, form)
            scratch = ctx.buffer("attn.scratch", (max(1, plan.scratch_floats),), torch.float32)
            counters = None
            if plan.n_counters:
                counters = ctx.buffer("attn.counters", (plan.n_counters,), torch.int32, zero=True)
            ops.attn_decode(q, cache.k_pages, cache.v_pages, cache.page_table, cache.ring_pages, ctx.slots,
                            ctx.len_before, out, scratch, scale=self.scale, window=self.window, plan=plan,
                            counters=counters, form=form, gate=gate)
        else:
            # as in parts/attention.py: a group that keeps every key takes the step's keys into its pages at once;
            # a ring waits until the attention has read the old keys that the new ones overwrite
            write_now = self.window == 0
            k_new = ctx.buffer("gattn.k_new", (n, self.nkv, self.hd))
            v_new = ctx.buffer("gattn.v_new", (n, self.nkv, self.vd))
            if write_now:
                ops.qkv_row_prep(rows, **common, k_new=k_new, v_new=v_new, **pages)
            else:
                ops.qkv_row_prep(rows, **common, k_new=k_new, v_new=v_new)
            tq = ops.prefill_tile_queries(q.dtype, self.hd, form)
            ops.attn_prefill(q, k_new, v_new, cache.k_pages, cache.v_pages, cache.page_table, cache.ring_pages,
                             ctx.query_tiles(tq), ctx.cu_tokens, ctx.len_before, ctx.slots, out,
                             scale=self.scale, window=self.window, tile_queries=tq, form=form, gate=gate)
            if not write_now:
                ops.kv_write(k_new, v_new, cache.k_pages, cache.v_pages, cache.page_table, cache.ring_pages,
                             ctx.positions, ctx.seq_of_token, ctx.slots, ctx.cu_tokens, ctx.len_before)
        return Branch(linear(ctx, out, self.w_o, "gattn.proj", torch.float32))


register_part("mixer", "gated_sink_attention", GatedSinkAttention)
