"""Small Fipavik configurations with random weights for the tests: written as a model folder (config.json and
model.safetensors under the design's tensor names) so that the library loads them as it loads any checkpoint."""
import json
import math
import os

import torch


def attention(heads, kv_heads, dim, vdim, chunk, rot_dims, base=10000.0, v_mix=False, scale=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": chunk},
         "rot": {"base": base, "dims": rot_dims}, "scale": float(scale if scale is not None else 1.0 / math.sqrt(dim))}
    if v_mix:
        m["v_mix"] = True
    return {"type": "attention", "mixer": m}


def latent(heads, dim, rot_dim, vdim, kv_rank, window, base=10000.0, scale=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "mask": {"size": window},
         "rot": {"base": base, "dims": rot_dim}, "scale": float(scale if scale is not None else 1.0 / math.sqrt(dim + rot_dim))}
    return {"type": "latent_attention", "mixer": m}


def moe(experts, top, ff, shared):
    m = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def layer(mixer, mlp):
    return dict(mixer, mlp=mlp)


def config(layers, *, vocab, width, mult, eps=1e-5):
    return {"architecture": "Fipavik", "vocab": vocab, "width": width, "norm": {"eps": eps}, "residual_mult": mult,
            "layers": layers}


# Every size differs between the configurations and from one layer to the next; none is a size of a published model.
CONFIGS = {
    # chunks and windows below, at and above a page; rotation over a part of the head and over all of it; a layer that
    # blends nothing; a layer without feed-forward; one expert per token, and no shared expert
    "mixed": config([
        layer(attention(6, 2, 16, 24, 37, 8, v_mix=True), moe(5, 2, 24, 40)),
        layer(latent(3, 16, 8, 20, 24, 50, base=5000.0), moe(4, 1, 32, 0)),
        layer(attention(6, 2, 16, 24, 64, 16, base=300.0, v_mix=True), None),
        layer(attention(4, 4, 24, 24, 5, 12), moe(8, 3, 16, 16)),
        layer(latent(2, 24, 16, 8, 16, 131), moe(5, 2, 24, 8)),
        layer(attention(3, 1, 16, 24, 130, 4, scale=0.4), moe(3, 2, 40, 24)),
    ], vocab=211, width=72, mult=0.7),
    # head sizes of the tensor-core attention kernels in bfloat16 (64: tcgen05 and TMA; 48: mma.sync), widths whose
    # products run on the tensor cores, the latent first
    "tensor": config([
        layer(latent(4, 32, 16, 32, 48, 70), moe(6, 2, 64, 96)),
        layer(attention(4, 2, 64, 64, 70, 32, v_mix=True), moe(6, 3, 48, 0)),
        layer(attention(6, 2, 48, 48, 100, 48), moe(4, 2, 64, 32)),
        layer(attention(2, 2, 64, 64, 128, 64, v_mix=True), None),
    ], vocab=300, width=128, mult=0.8),
    # sizes that fit no vector access and no tensor-core tile; a window and a chunk of one position (a query sees
    # itself alone); every expert chosen (top = experts); a residual factor of one
    "odd": config([
        layer(attention(3, 3, 20, 12, 1, 10), moe(3, 3, 10, 6)),
        layer(latent(5, 12, 4, 20, 20, 1), moe(2, 1, 14, 0)),
        layer(latent(1, 8, 6, 8, 10, 200), None),
        layer(attention(12, 1, 8, 8, 200, 2), moe(7, 4, 6, 10)),
    ], vocab=97, width=100, mult=1.0),
}


def random_weights(cfg, seed, *, steady_routing=False):
    """bfloat16-valued tensors by the design's names.  Spreads are chosen so that activations stay of order one.
    ``steady_routing``: the routers' biases lie far apart and their matrices are small, so that which experts a token
    gets hangs on the token only now and then and never on a close call (for comparisons in bfloat16, where the router's
    input is rounded)."""
    g = torch.Generator().manual_seed(seed)

    def normal(shape, std, mean=0.0):
        return (mean + std * torch.randn(shape, generator=g)).to(torch.bfloat16)

    d = cfg["width"]
    w = {"embed": normal((cfg["vocab"], d), 1.0), "final.norm": normal((d,), 0.1, 1.0), "final.norm.b": normal((d,), 0.1)}
    for i, lay in enumerate(cfg["layers"]):
        m, p = lay["mixer"], f"l{i}."
        w[p + "norm1"] = normal((d,), 0.1, 1.0)
        w[p + "norm1.b"] = normal((d,), 0.1)
        out_w = m["heads"] * m["vdim"]
        w[p + "mix.sink"] = normal((m["heads"],), 1.0)
        w[p + "mix.o"] = normal((d, out_w), out_w ** -0.5)
        if lay["type"] == "attention":
            w[p + "mix.q"] = normal((m["heads"] * m["dim"], d), d ** -0.5)
            w[p + "mix.k"] = normal((m["kv_heads"] * m["dim"], d), d ** -0.5)
            w[p + "mix.v"] = normal((m["kv_heads"] * m["vdim"], d), d ** -0.5)
            w[p + "mix.q.norm"] = normal((m["dim"],), 0.2, 1.5)
            w[p + "mix.k.norm"] = normal((m["dim"],), 0.2, 1.5)
            if m.get("v_mix"):
                w[p + "mix.vmix"] = (0.2 + 0.6 * torch.rand((), generator=g)).to(torch.bfloat16)
        else:
            r = m["kv_rank"]
            w[p + "mix.q"] = normal((m["heads"] * (m["dim"] + m["rot_dim"]), d), 1.5 * d ** -0.5)
            w[p + "mix.dkv"] = normal((r + m["rot_dim"], d), 1.5 * d ** -0.5)
            w[p + "mix.dkv.norm"] = normal((r,), 0.2, 1.2)
            w[p + "mix.uk"] = normal((m["heads"] * m["dim"], r), r ** -0.5)
            w[p + "mix.uv"] = normal((m["heads"] * m["vdim"], r), r ** -0.5)
        ml = lay.get("mlp")
        if ml:
            e_n, ff = ml["router"]["experts"], ml["expert"]["ff"]
            if steady_routing:
                w[p + "mlp.router"] = normal((e_n, d), 0.25 * d ** -0.5)
                w[p + "mlp.router.b"] = (1.5 * torch.randperm(e_n, generator=g).float()).to(torch.bfloat16)
            else:
                w[p + "mlp.router"] = normal((e_n, d), 2.0 * d ** -0.5)
                w[p + "mlp.router.b"] = normal((e_n,), 0.5)
            for e in range(e_n):
                w[p + f"mlp.e{e}.gate"] = normal((ff, d), 1.5 * d ** -0.5)
                w[p + f"mlp.e{e}.up"] = normal((ff, d), 1.5 * d ** -0.5)
                w[p + f"mlp.e{e}.down"] = normal((d, ff), ff ** -0.5)
            if ml.get("shared"):
                sf = ml["shared"]["ff"]
                w[p + "mlp.shared.gate"] = normal((sf, d), d ** -0.5)
                w[p + "mlp.shared.up"] = normal((sf, d), d ** -0.5)
                w[p + "mlp.shared.down"] = normal((d, sf), sf ** -0.5)
    return w


def write_model(llogos, folder, cfg, seed, weights=None, **kw):
    os.makedirs(folder, exist_ok=True)
    w = weights if weights is not None else random_weights(cfg, seed, **kw)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    llogos.weights.write_safetensors(os.path.join(folder, "model.safetensors"), w, {"format": "pt"})
    return w
