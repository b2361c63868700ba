"""Small Karitar configurations with random weights for the tests: written as a model folder (config.json and
model.safetensors under the design's tensor names) so that the library loads them as it loads any checkpoint."""
import json
import math
import os

import torch


def attention(heads, kv_heads, dim, vdim, window, scale=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
         "scale": float(scale if scale is not None else 1.0 / math.sqrt(dim))}
    if window is not None:
        m["mask"] = {"size": window}
    return m


def layer(mixer, ff):
    return {"type": "attention", "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def config(layers, *, vocab, width, streams, loop=None, eps=1e-5):
    cfg = {"architecture": "Karitar", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if streams is not None:
        cfg["streams"] = streams
    if loop is not None:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


# Every size differs between the configurations and from one layer to the next; none is a size of a published model.
CONFIGS = {
    # windows below, at and above a page; value heads smaller and larger than key heads; a layer without feed-forward
    "mixed": config([layer(attention(6, 2, 16, 24, 37), 88), layer(attention(4, 4, 24, 8, 64), None),
                     layer(attention(3, 1, 40, 40, 131), 56)], vocab=211, width=72, streams=3, loop=(0, 2, 2)),
    # one stream, every key visible, heads of 64 (the tcgen05 prompt kernel and the TMA decode kernel in bfloat16)
    "wide": config([layer(attention(4, 2, 64, 64, None), 160), layer(attention(2, 1, 64, 64, 70), 96)],
                   vocab=300, width=128, streams=1, loop=(1, 2, 3)),
    # no streams at all (the ordinary residual), no loop, heads of 48 and 32 (the mma.sync kernels in bfloat16)
    "plain_residual": config([layer(attention(4, 2, 48, 48, 20), 64), layer(attention(8, 8, 32, 32, 5), 120)],
                             vocab=190, width=96, streams=None),
    # sizes that fit no vector access and no tensor-core tile: a width that is no multiple of 8, three heads, heads of 20
    # and 12; twelve query heads on one key/value head; a window of one token (a position sees itself only); a loop
    # that runs once
    "odd": config([layer(attention(12, 1, 16, 16, 1), 50), layer(attention(3, 1, 20, 12, None), None),
                   layer(attention(5, 5, 8, 8, 200), 30)], vocab=97, width=100, streams=2, loop=(1, 3, 1)),
    # four streams, heads of 128, a loop over everything
    "four": config([layer(attention(2, 1, 128, 128, 100), 200)], vocab=150, width=80, streams=4, loop=(0, 1, 2)),
}


def random_weights(cfg, seed):
    """bfloat16-valued tensors by the design's names.  Spreads are chosen so that activations stay of order one."""
    g = torch.Generator().manual_seed(seed)

    def normal(shape, std, mean=0.0):
        return (mean + std * torch.randn(shape, generator=g)).to(torch.bfloat16)

    d, s = cfg["width"], cfg.get("streams") or 0
    w = {"embed": normal((cfg["vocab"], d), 1.0), "final.norm": normal((d,), 0.1, 1.0), "head": normal((cfg["vocab"], d), d ** -0.5)}
    for i, lay in enumerate(cfg["layers"]):
        m = lay["mixer"]
        q, k, v = m["heads"] * m["dim"], m["kv_heads"] * m["dim"], m["kv_heads"] * m["vdim"]
        p = f"l{i}."
        w[p + "norm1"] = normal((d,), 0.1, 1.0)
        for n, rows in (("q", q), ("k", k), ("v", v)):
            w[p + f"mix.{n}"] = normal((rows, d), d ** -0.5)
            w[p + f"mix.{n}.b"] = normal((rows,), 0.2)
        w[p + "mix.q.norm"] = normal((q,), 0.2, 1.5)
        w[p + "mix.k.norm"] = normal((k,), 0.2, 1.5)
        w[p + "mix.g"] = normal((m["heads"], d), d ** -0.5)
        w[p + "mix.o"] = normal((d, m["heads"] * m["vdim"]), (m["heads"] * m["vdim"]) ** -0.5)
        subs = ["hc1"]
        if lay["mlp"]:
            ff = lay["mlp"]["ff"]
            w[p + "norm2"] = normal((d,), 0.1, 1.0)
            w[p + "mlp.up"] = normal((ff, d), d ** -0.5)
            w[p + "mlp.down"] = normal((d, ff), ff ** -0.5)
            subs.append("hc2")
        for hc in subs if s else []:
            w[p + hc + ".in"] = normal((s,), 0.2, 1.0 / s)
            w[p + hc + ".out"] = normal((s,), 0.2, 1.0)
            w[p + hc + ".mix"] = (torch.eye(s) + 0.15 * torch.randn((s, s), generator=g)).to(torch.bfloat16)
    return w


def write_model(llogos, folder, cfg, seed, weights=None):
    os.makedirs(folder, exist_ok=True)
    w = weights if weights is not None else random_weights(cfg, seed)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    llogos.weights.write_safetensors(os.path.join(folder, "model.safetensors"), w, {"format": "pt"})
    return w
