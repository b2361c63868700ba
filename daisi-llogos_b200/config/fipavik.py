"""Typed configuration of the Fipavik decoder and its model builder.

Fipavik's config.json is nested and names its architecture under ``architecture``:

    {"architecture": "Fipavik", "vocab": V, "width": D, "norm": {"eps": e}, "residual_mult": r,
     "layers": [{"type": "attention",
                 "mixer": {"heads": H, "kv_heads": G, "dim": dq, "vdim": dv, "scale": c, "mask": {"size": C},
                           "rot": {"base": b, "dims": R}, "v_mix": true},
                 "mlp": {"kind": "moe", "router": {"experts": E, "top": K}, "expert": {"ff": F},
                         "shared": {"ff": Fs}} | null},
                {"type": "latent_attention",
                 "mixer": {"heads": H, "dim": dq, "rot_dim": dr, "vdim": dv, "kv_rank": L, "scale": c,
                           "mask": {"size": W}, "rot": {"base": b, "dims": dr}},
                 "mlp": ...}, ...]}

Every layer names its own sizes and its kind of mixer, so the order of kinds and all sizes may differ from layer to
layer.  What the design fixes and no file says: a layer is ONE layer norm (weight and bias) whose output feeds mixer and
feed-forward side by side, both added to the residual times ``residual_mult`` (parts/block.py: ``parallel``); "attention"
is grouped-query attention with per-head RMS norms on queries and keys, rotation by halves of the first ``rot.dims``
elements, a mask by chunks of ``mask.size`` positions, a learned sink per head, and values blended with those of the
first layer that says ``v_mix`` (parts/attention.py); "latent_attention" keeps one latent vector and one rotated key part
per position, under a sliding window of ``mask.size`` positions, with the same sink (parts/latent_attention.py); the
feed-forward is a mixture of gated silu experts with a biased float32 router, a softmax over the chosen logits and a
shared expert (parts/moe.py); a final layer norm; the output head is the embedding table.  Tensor names: ``embed``,
``l<i>.norm1`` (+ ``.b``), ``l<i>.mix.{q,k,v,o,sink,vmix}``, ``l<i>.mix.{q,k}.norm``, ``l<i>.mix.{dkv,uk,uv}``,
``l<i>.mix.dkv.norm``, ``l<i>.mlp.router`` (+ ``.b``), ``l<i>.mlp.e<j>.{gate,up,down}``, ``l<i>.mlp.shared.{gate,up,down}``,
``final.norm`` (+ ``.b``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple, Union

from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .dense import ConfigError, _need
from .karitar import _obj, _positive

NAME = "Fipavik"

# what the design fixes
ATTENTION_MASK = "chunk"            # "attention" layers: a query sees the keys of its own chunk
LATENT_MASK = "window"              # "latent_attention" layers: the last mask.size keys
VALUE_GROUP = "v_mix"               # all layers that blend their values form one group


@dataclass(frozen=True)
class Rotation:
    base: float
    dims: int


@dataclass(frozen=True)
class FipavikAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    mask_size: int        # 0: every earlier key
    rot: Optional[Rotation]
    v_mix: bool


@dataclass(frozen=True)
class FipavikLatentAttention:
    heads: int
    dim: int              # unrotated elements of a query / key head
    rot_dim: int          # rotated elements
    vdim: int
    kv_rank: int
    scale: float
    mask_size: int
    rot: Optional[Rotation]


@dataclass(frozen=True)
class FipavikMoe:
    experts: int
    top: int
    ff: int
    shared_ff: int        # 0: no shared expert


@dataclass(frozen=True)
class FipavikLayer:
    type: str             # "attention" | "latent_attention"
    mixer: Union[FipavikAttention, FipavikLatentAttention]
    mlp: Optional[FipavikMoe]


@dataclass(frozen=True)
class FipavikConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    residual_mult: float
    layers: Tuple[FipavikLayer, ...]

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "FipavikConfig":
        vocab = _positive(d, "vocab")
        width = _positive(d, "width")
        eps = _need(_obj(d, "norm"), "eps", float)
        if eps <= 0:
            raise ConfigError(f"config.json: norm.eps must be positive, got {eps}")
        mult = _need(d, "residual_mult", float)
        raw_layers = d.get("layers")
        if not isinstance(raw_layers, (list, tuple)) or not raw_layers:
            raise ConfigError("config.json: missing key 'layers' (a non-empty list of layers)")
        layers = tuple(_layer(i, raw) for i, raw in enumerate(raw_layers))
        shapes = {(l.mixer.kv_heads, l.mixer.vdim) for l in layers if l.type == "attention" and l.mixer.v_mix}
        if len(shapes) > 1:
            raise ConfigError(f"config.json: layers with mixer.v_mix blend their values with the first such layer's, "
                              f"so their kv_heads and vdim must agree; found {sorted(shapes)}")
        return cls(architecture=str(d.get("architecture", NAME)), vocab=vocab, width=width, norm_eps=eps,
                   residual_mult=mult, layers=layers)


def _float(d: Mapping[str, Any], key: str, where: str) -> float:
    try:
        return _need(d, key, float)
    except ConfigError as e:
        raise ConfigError(str(e).replace(f"'{key}'", f"'{where}{key}'")) from None


def _mask_size(m: Mapping[str, Any], where: str) -> int:
    mask = m.get("mask")
    if mask is None:
        return 0
    if not isinstance(mask, Mapping):
        raise ConfigError(f"config.json: {where}mask must be an object or null")
    return 0 if mask.get("size") is None else _positive(mask, "size", where + "mask.")


def _rotation(m: Mapping[str, Any], where: str, most: int, what: str) -> Optional[Rotation]:
    rot = m.get("rot")
    if rot is None:
        return None
    if not isinstance(rot, Mapping):
        raise ConfigError(f"config.json: {where}rot must be an object or null")
    base = _float(rot, "base", where + "rot.")
    dims = _positive(rot, "dims", where + "rot.")
    if not base > 0:
        raise ConfigError(f"config.json: {where}rot.base must be positive, got {base}")
    if dims % 2 or dims > most:
        raise ConfigError(f"config.json: {where}rot.dims {dims} must be even and at most {what} {most}")
    return Rotation(base, dims)


def _layer(i: int, raw: Any) -> FipavikLayer:
    where = f"layers[{i}]."
    if not isinstance(raw, Mapping):
        raise ConfigError(f"config.json: layers[{i}] must be an object")
    kind = raw.get("type")
    if kind not in ("attention", "latent_attention"):
        raise ConfigError(f"config.json: {where}type = {kind!r} is not supported (known: 'attention', 'latent_attention')")
    if not isinstance(raw.get("mixer"), Mapping):
        raise ConfigError(f"config.json: {where}mixer must be an object")
    m, mw = raw["mixer"], where + "mixer."
    heads = _positive(m, "heads", mw)
    dim, vdim = _positive(m, "dim", mw), _positive(m, "vdim", mw)
    scale = _float(m, "scale", mw)
    if not scale > 0:
        raise ConfigError(f"config.json: {mw}scale must be positive, got {scale}")
    size = _mask_size(m, mw)
    if kind == "attention":
        kv_heads = _positive(m, "kv_heads", mw)
        if heads % kv_heads:
            raise ConfigError(f"config.json: {mw}heads {heads} is not a multiple of {mw}kv_heads {kv_heads}")
        mixer = FipavikAttention(heads, kv_heads, dim, vdim, scale, size, _rotation(m, mw, dim, "dim"), bool(m.get("v_mix", False)))
    else:
        rot_dim = _need(m, "rot_dim", int, default=0, required=False)
        if rot_dim < 0 or rot_dim % 2:
            raise ConfigError(f"config.json: {mw}rot_dim must be even and not negative, got {rot_dim}")
        rot = _rotation(m, mw, max(rot_dim, 0), "rot_dim") if rot_dim else None
        if rot_dim and rot is None:
            raise ConfigError(f"config.json: {mw}rot is missing although rot_dim is {rot_dim}")
        if rot is not None and rot.dims != rot_dim:
            raise ConfigError(f"config.json: {mw}rot.dims {rot.dims} must equal rot_dim {rot_dim}")
        mixer = FipavikLatentAttention(heads, dim, rot_dim, vdim, _positive(m, "kv_rank", mw), scale, size, rot)
    mlp = None
    if raw.get("mlp") is not None:
        ml, lw = raw["mlp"], where + "mlp."
        if not isinstance(ml, Mapping):
            raise ConfigError(f"config.json: {where}mlp must be an object or null")
        if ml.get("kind") != "moe":
            raise ConfigError(f"config.json: {lw}kind = {ml.get('kind')!r} is not supported (known: 'moe')")
        router = _obj(ml, "router")
        experts, top = _positive(router, "experts", lw + "router."), _positive(router, "top", lw + "router.")
        if top > experts:
            raise ConfigError(f"config.json: {lw}router.top {top} exceeds {lw}router.experts {experts}")
        ff = _positive(_obj(ml, "expert"), "ff", lw + "expert.")
        shared = 0
        if ml.get("shared") is not None:
            shared = _positive(_obj(ml, "shared"), "ff", lw + "shared.")
        mlp = FipavikMoe(experts, top, ff, shared)
    return FipavikLayer(kind, mixer, mlp)


def _encoding(encodings: Dict[str, PartSpec], rot: Optional[Rotation], head_dim: int) -> Optional[str]:
    """The name of the rotary tables for ``rot`` (layers with the same base and size share them)."""
    if rot is None:
        return None
    name = f"rot{rot.dims}@{rot.base!r}"
    if name not in encodings:
        encodings[name] = PartSpec("rotary", {"head_dim": max(head_dim, rot.dims), "rotary_dim": rot.dims, "theta": rot.base,
                                              "scaling": None, "pairing": "half"})
    return name


def fipavik_spec(cfg: FipavikConfig) -> ModelSpec:
    """Parts and run order of a Fipavik model (see the module's text for what the design fixes)."""
    norm = {"size": cfg.width, "eps": cfg.norm_eps}
    encodings: Dict[str, PartSpec] = {}
    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = layer.mixer
        if layer.type == "attention":
            mixer = PartSpec("attention", {
                "hidden_size": cfg.width, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim,
                "value_dim": m.vdim, "qkv_bias": False, "qk_norm": True, "qk_norm_eps": cfg.norm_eps,
                "window": m.mask_size, "mask": ATTENTION_MASK if m.mask_size else "window", "softmax_scale": m.scale,
                "sink": "learned", "value_blend": VALUE_GROUP if m.v_mix else None,
                "position": _encoding(encodings, m.rot, m.dim),
                "tensor_names": {"q_proj.weight": "q", "k_proj.weight": "k", "v_proj.weight": "v", "o_proj.weight": "o",
                                 "q_norm.weight": "q.norm", "k_norm.weight": "k.norm"},
            }, p + "mix.")
        else:
            mixer = PartSpec("latent_attention", {
                "hidden_size": cfg.width, "num_heads": m.heads, "head_dim": m.dim, "rot_dim": m.rot_dim,
                "value_dim": m.vdim, "kv_rank": m.kv_rank, "norm_eps": cfg.norm_eps, "window": m.mask_size,
                "mask": LATENT_MASK, "softmax_scale": m.scale, "sink": "learned",
                "position": _encoding(encodings, m.rot, m.rot_dim),
                "tensor_names": {"q_proj.weight": "q", "kv_down_proj.weight": "dkv", "kv_norm.weight": "dkv.norm",
                                 "k_up_proj.weight": "uk", "v_up_proj.weight": "uv", "o_proj.weight": "o"},
            }, p + "mix.")
        parts = {"norm1": PartSpec("layernorm", dict(norm, tensor_names={"weight": "norm1", "bias": "norm1.b"}), p),
                 "mixer": mixer}
        if layer.mlp is not None:
            ml = layer.mlp
            parts["ffn"] = PartSpec("moe", {
                "hidden_size": cfg.width, "num_experts": ml.experts, "top": ml.top, "expert_size": ml.ff,
                "shared_size": ml.shared_ff, "router_bias": True, "shared_prefix": "shared.",
                "shared_names": {"gate_proj.weight": "gate", "up_proj.weight": "up", "down_proj.weight": "down"},
                "tensor_names": {"router.weight": "router", "router.bias": "router.b",
                                 "experts.*.gate_proj.weight": "e*.gate", "experts.*.up_proj.weight": "e*.up",
                                 "experts.*.down_proj.weight": "e*.down"},
            }, p + "mlp.")
        layers.append(LayerSpec("parallel", parts, {"residual_scale": cfg.residual_mult}))
    spec = ModelSpec(
        hidden_size=cfg.width,
        vocab_size=cfg.vocab,
        max_positions=None,                       # the rotation has no limit of its own: the cache's size is the limit
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.width,
                                               "tensor_names": {"weight": "embed"}}, ""),
        encodings=encodings,
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in range(len(layers))),
        final_norm=PartSpec("layernorm", dict(norm, tensor_names={"weight": "final.norm", "bias": "final.norm.b"}), ""),
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "tied_to": "embed"}, ""),
    )
    spec.validate()
    return spec
