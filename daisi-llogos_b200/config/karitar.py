"""Typed configuration of the Karitar decoder and its model builder.

Karitar's config.json is nested and carries no ``architectures`` list but one name under ``architecture``:

    {"architecture": "Karitar", "vocab": V, "width": D, "norm": {"eps": e}, "streams": S,
     "layers": [{"type": "attention",
                 "mixer": {"heads": H, "kv_heads": G, "dim": dq, "vdim": dv, "scale": c, "mask": {"size": W}},
                 "mlp": {"kind": "dense", "ff": F} | null}, ...],
     "loop": {"start": a, "stop": b, "times": n}}

Every layer names its own sizes, so layers may differ in heads, head sizes, window and feed-forward (or have no
feed-forward).  ``loop`` runs layers a .. b-1 n times in a row with the same weights, every pass with a cache of its
own, before the rest follow.  ``streams`` is the number of residual streams (hyper-connections, parts/hyper.py);
without the key the residual is the ordinary single one.  What the design fixes and no file says: pre-norm sublayers
with RMS norm; attention without position encoding, with biases in q/k/v, RMS norms over the whole q and k rows, a sink
of score 0 in the softmax and a sigmoid gate per head (parts/gated_attention.py); a feed-forward of up, squared relu,
down; an untied output head.  Tensor names: ``embed``, ``l<i>.norm1``, ``l<i>.mix.{q,k,v,o,g}``, ``l<i>.mix.{q,k,v}.b``,
``l<i>.mix.{q,k}.norm``, ``l<i>.mlp.{up,down}``, ``l<i>.hc<1|2>.{in,out,mix}``, ``final.norm``, ``head``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .dense import ConfigError, _need

NAME = "Karitar"


@dataclass(frozen=True)
class KaritarAttention:
    heads: int
    kv_heads: int
    dim: int             # elements of a query / key head
    vdim: int            # elements of a value head
    scale: float         # multiplies q . k
    window: int          # 0: every earlier key; W: the last W keys, the query's own included


@dataclass(frozen=True)
class KaritarMlp:
    kind: str            # "dense"
    ff: int


@dataclass(frozen=True)
class KaritarLayer:
    type: str            # "attention"
    mixer: KaritarAttention
    mlp: Optional[KaritarMlp]


@dataclass(frozen=True)
class KaritarConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    streams: int                               # 0: one ordinary residual
    layers: Tuple[KaritarLayer, ...]
    loop: Optional[Tuple[int, int, int]]       # (start, stop, times)

    def run_order(self) -> Tuple[int, ...]:
        """Layer indices in the order they run."""
        n = len(self.layers)
        if self.loop is None:
            return tuple(range(n))
        start, stop, times = self.loop
        return tuple(range(start)) + tuple(range(start, stop)) * times + tuple(range(stop, n))

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "KaritarConfig":
        vocab = _positive(d, "vocab")
        width = _positive(d, "width")
        norm = _obj(d, "norm")
        eps = _need(norm, "eps", float)
        if eps <= 0:
            raise ConfigError(f"config.json: norm.eps must be positive, got {eps}")
        streams = _need(d, "streams", int, default=0, required=False)
        if streams < 0:
            raise ConfigError(f"config.json: key 'streams' must not be negative, got {streams}")
        raw_layers = d.get("layers")
        if not isinstance(raw_layers, (list, tuple)) or not raw_layers:
            raise ConfigError("config.json: missing key 'layers' (a non-empty list of layers)")
        layers = tuple(_layer(i, raw) for i, raw in enumerate(raw_layers))
        loop = None
        if d.get("loop") is not None:
            lo = _obj(d, "loop")
            start, stop, times = _need(lo, "start", int), _need(lo, "stop", int), _need(lo, "times", int)
            if not (0 <= start <= stop <= len(layers)) or times < 1:
                raise ConfigError(f"config.json: loop start {start}, stop {stop}, times {times} does not fit "
                                  f"{len(layers)} layers (0 <= start <= stop <= layers, times >= 1)")
            loop = (start, stop, times)
        return cls(architecture=str(d.get("architecture", NAME)), vocab=vocab, width=width, norm_eps=eps,
                   streams=streams, layers=layers, loop=loop)


def _obj(d: Mapping[str, Any], key: str) -> Mapping[str, Any]:
    v = d.get(key)
    if not isinstance(v, Mapping):
        raise ConfigError(f"config.json: key '{key}' must be an object")
    return v


def _positive(d: Mapping[str, Any], key: str, where: str = "") -> int:
    try:
        v = _need(d, key, int)
    except ConfigError as e:
        raise ConfigError(str(e).replace(f"'{key}'", f"'{where}{key}'")) from None
    if v <= 0:
        raise ConfigError(f"config.json: key '{where}{key}' must be positive, got {v}")
    return v


def _layer(i: int, raw: Any) -> KaritarLayer:
    where = f"layers[{i}]."
    if not isinstance(raw, Mapping):
        raise ConfigError(f"config.json: layers[{i}] must be an object")
    kind = raw.get("type")
    if kind != "attention":
        raise ConfigError(f"config.json: {where}type = {kind!r} is not supported (known: 'attention')")
    if not isinstance(raw.get("mixer"), Mapping):
        raise ConfigError(f"config.json: {where}mixer must be an object")
    m = raw["mixer"]
    mw = where + "mixer."
    heads, kv_heads = _positive(m, "heads", mw), _positive(m, "kv_heads", mw)
    if heads % kv_heads:
        raise ConfigError(f"config.json: {mw}heads {heads} is not a multiple of {mw}kv_heads {kv_heads}")
    dim, vdim = _positive(m, "dim", mw), _positive(m, "vdim", mw)
    try:
        scale = _need(m, "scale", float)
    except ConfigError as e:
        raise ConfigError(str(e).replace("'scale'", f"'{mw}scale'")) from None
    if not scale > 0:
        raise ConfigError(f"config.json: {mw}scale must be positive, got {scale}")
    window = 0
    if m.get("mask") is not None:
        if not isinstance(m["mask"], Mapping):
            raise ConfigError(f"config.json: {mw}mask must be an object or null")
        if m["mask"].get("size") is not None:
            window = _positive(m["mask"], "size", mw + "mask.")
    mlp = None
    if raw.get("mlp") is not None:
        if not isinstance(raw["mlp"], Mapping):
            raise ConfigError(f"config.json: {where}mlp must be an object or null")
        mk = raw["mlp"].get("kind")
        if mk != "dense":
            raise ConfigError(f"config.json: {where}mlp.kind = {mk!r} is not supported (known: 'dense')")
        mlp = KaritarMlp("dense", _positive(raw["mlp"], "ff", where + "mlp."))
    return KaritarLayer("attention", KaritarAttention(heads, kv_heads, dim, vdim, scale, window), mlp)


SINK_SCORE = 0.0          # the softmax's denominator has one more term, exp(0)
MLP_ACTIVATION = "relu2"  # the square of relu


def karitar_spec(cfg: KaritarConfig) -> ModelSpec:
    """Parts and run order of a Karitar model (see the module's text for what the design fixes)."""
    s = cfg.streams
    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = layer.mixer
        mixer = PartSpec("gated_sink_attention", {
            "hidden_size": cfg.width, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim,
            "value_dim": m.vdim, "qkv_bias": True, "qk_norm": "row", "qk_norm_eps": cfg.norm_eps,
            "window": m.window, "softmax_scale": m.scale, "sink": SINK_SCORE, "head_gate": True, "position": None,
            "tensor_names": {"q_proj.weight": "q", "k_proj.weight": "k", "v_proj.weight": "v", "o_proj.weight": "o",
                             "gate_proj.weight": "g", "q_proj.bias": "q.b", "k_proj.bias": "k.b", "v_proj.bias": "v.b",
                             "q_norm.weight": "q.norm", "k_norm.weight": "k.norm"},
        }, p + "mix.")
        parts = {"norm1": _norm(cfg, p, "norm1", "hc1.in"), "mixer": mixer}
        if s:
            parts["write1"] = PartSpec("stream_write", {"streams": s}, p + "hc1.")
        if layer.mlp is not None:
            parts["norm2"] = _norm(cfg, p, "norm2", "hc2.in")
            parts["ffn"] = PartSpec("dense_mlp", {
                "hidden_size": cfg.width, "intermediate_size": layer.mlp.ff, "activation": MLP_ACTIVATION,
                "tensor_names": {"up_proj.weight": "up", "down_proj.weight": "down"},
            }, p + "mlp.")
            if s:
                parts["write2"] = PartSpec("stream_write", {"streams": s}, p + "hc2.")
        layers.append(LayerSpec("hyper_prenorm" if s else "prenorm", parts))
    if s:
        final = PartSpec("hyper_rmsnorm", {"size": cfg.width, "eps": cfg.norm_eps, "streams": s, "read": "sum",
                                           "tensor_names": {"weight": "final.norm"}}, "")
    else:
        final = PartSpec("rmsnorm", {"size": cfg.width, "eps": cfg.norm_eps, "tensor_names": {"weight": "final.norm"}}, "")
    spec = ModelSpec(
        hidden_size=cfg.width,
        vocab_size=cfg.vocab,
        max_positions=None,                       # no position encoding: the cache's size is the only limit
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "streams": s,
                                               "tensor_names": {"weight": "embed"}}, ""),
        encodings={},
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in cfg.run_order()),
        final_norm=final,
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "tied_to": None,
                                      "tensor_names": {"weight": "head"}}, ""),
    )
    spec.validate()
    return spec


def _norm(cfg: KaritarConfig, prefix: str, name: str, read_name: str) -> PartSpec:
    if cfg.streams:
        return PartSpec("hyper_rmsnorm", {"size": cfg.width, "eps": cfg.norm_eps, "streams": cfg.streams, "read": "weights",
                                          "tensor_names": {"weight": name, "in": read_name}}, prefix)
    return PartSpec("rmsnorm", {"size": cfg.width, "eps": cfg.norm_eps, "tensor_names": {"weight": name}}, prefix)
