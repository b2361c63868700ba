"""The Fipavik decoder without a GPU: its configuration reader and spec, the plain implementation's mechanisms against
closed forms, and the engine's host logic (packing, cache, rings, value lending, expert layout) over the CPU stand-ins
of the kernels against the plain implementation."""
import copy
import math

import pytest
import torch

import cpu_ops
import fipavik_models as FM
import fipavik_plain as FP


def test_reader_takes_every_size_from_the_file_and_names_the_key_of_an_error(llogos):
    cfg = llogos.config.registry.architecture_of(FM.CONFIGS["mixed"]).read_config(FM.CONFIGS["mixed"])
    assert (cfg.vocab, cfg.width, cfg.residual_mult, len(cfg.layers)) == (211, 72, 0.7, 6)
    a, l = cfg.layers[0].mixer, cfg.layers[1].mixer
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.mask_size, a.rot.dims, a.v_mix) == (6, 2, 16, 24, 37, 8, True)
    assert (l.heads, l.dim, l.rot_dim, l.vdim, l.kv_rank, l.mask_size, l.rot.base) == (3, 16, 8, 20, 24, 50, 5000.0)
    assert cfg.layers[2].mlp is None and cfg.layers[1].mlp.shared_ff == 0 and cfg.layers[3].mlp.top == 3
    ConfigError = llogos.config.ConfigError
    for path, value, word in ((("layers", 0, "mixer", "kv_heads"), 4, "kv_heads"), (("layers", 1, "mixer", "rot_dim"), 7, "rot_dim"),
                              (("layers", 0, "mlp", "router", "top"), 9, "top"), (("layers", 0, "type"), "conv", "type"),
                              (("residual_mult",), None, "residual_mult"), (("layers", 3, "mlp", "kind"), "dense", "kind"),
                              (("layers", 2, "mixer", "vdim"), 8, "v_mix"), (("layers", 0, "mixer", "rot", "dims"), 18, "rot.dims")):
        bad = copy.deepcopy(FM.CONFIGS["mixed"])
        node = bad
        for k in path[:-1]:
            node = node[k]
        node[path[-1]] = value
        with pytest.raises(ConfigError, match=word):
            llogos.config.registry.architecture_of(bad).read_config(bad)


def test_spec_names_parts_tensors_and_cache_units(llogos):
    cfg = FM.CONFIGS["mixed"]
    model = llogos.weights.build_model(cfg, dtype=torch.float32, device="cpu", ops=cpu_ops)
    names = set(model.tensor_decls())
    assert names == set(FM.random_weights(cfg, 0))
    assert model.tensor_decls()["l0.mix.vmix"].shape == () and model.tensor_decls()["l1.mix.uk"].shape == (3 * 16, 24)
    needs = model.cache_needs()
    KvNeed = llogos.parts.base.KvNeed
    assert needs[0] == KvNeed(2, 16, 37, 24) and needs[1] == KvNeed(1, 24 + 8, 50, values_in_keys=True) and needs[3] == KvNeed(4, 24, 5, 0)
    assert [type(b).__name__ for b in model.blocks] == ["ParallelBlock"] * 6
    assert model.spec.head.params["tied_to"] == "embed" and len(model.spec.encodings) == 6


def test_plain_mechanisms_against_closed_forms():
    # layer norm: zero mean, unit variance before weight and bias
    x = torch.tensor([[1.0, 2.0, 3.0, 6.0]])
    y = FP.layer_norm(x, torch.ones(4), torch.zeros(4), 0.0)
    assert abs(float(y.mean())) < 1e-12 and abs(float((y * y).mean()) - 1) < 1e-12
    assert torch.allclose(FP.layer_norm(x, 2 * torch.ones(4), torch.ones(4), 0.0), 2 * y + 1)
    # rotation: position 0 changes nothing; lengths are kept; only the first `dims` elements move
    v = torch.arange(12.0).view(1, 1, 12) + 1
    assert torch.allclose(FP.rotate_halves(v, torch.tensor([0]), 8, 100.0), v.double())
    r = FP.rotate_halves(v, torch.tensor([3]), 8, 100.0)
    assert torch.allclose(r[..., 8:], v[..., 8:].double()) and abs(float(r.norm() - v.double().norm())) < 1e-9
    f1 = 100.0 ** (-2 / 8)
    assert abs(float(r[0, 0, 1]) - (2 * math.cos(3 * f1) - 6 * math.sin(3 * f1))) < 1e-12      # element 1 pairs with element 5
    # masks
    c, wdw = FP.chunk_mask(7, 3), FP.window_mask(7, 3)
    assert c[5].tolist() == [False, False, False, True, True, True, False]
    assert c[3].tolist() == [False, False, False, True, False, False, False]
    assert wdw[5].tolist() == [False, False, False, True, True, True, False] and wdw[3].tolist()[:4] == [False, True, True, True]
    # sink: equal scores and a sink of the same score share the mass equally, the sink's share is lost
    p = FP.sink_softmax(torch.zeros(1, 3), torch.ones(1, 3, dtype=torch.bool), torch.tensor(0.0))
    assert torch.allclose(p, torch.full((1, 3), 0.25, dtype=torch.float64))
    p = FP.sink_softmax(torch.zeros(1, 3), torch.ones(1, 3, dtype=torch.bool), torch.tensor(-1e9))
    assert torch.allclose(p.sum(), torch.tensor(1.0, dtype=torch.float64))
    # routing: the chosen experts' weights are a softmax over the chosen logits alone
    w = {"r.router": torch.eye(4), "r.router.b": torch.tensor([0.0, 0.0, 0.0, 5.0])}
    idx, wt, margin = FP.route(torch.tensor([[1.0, 3.0, 2.0, -4.0]]), w, "r.", 2)
    assert idx.tolist() == [[1, 2]] and abs(float(wt[0, 0]) - 1 / (1 + math.exp(-1))) < 1e-12 and abs(float(margin) - 1) < 1e-12


@pytest.fixture(scope="module")
def small(llogos, tmp_path_factory):
    out = {}
    for i, name in enumerate(("mixed", "odd")):
        d = str(tmp_path_factory.mktemp("fipavik_" + name))
        w = FM.write_model(llogos, d, FM.CONFIGS[name], seed=11 + i)
        out[name] = (d, FM.CONFIGS[name], {k: v.float() for k, v in w.items()})
    return out


@pytest.mark.parametrize("name", ["mixed", "odd"])
def test_engine_host_logic_agrees_with_plain(llogos, small, name):
    d, cfg, w = small[name]
    model = llogos.weights.load_model(d, dtype=torch.float32, device="cpu", ops=cpu_ops)
    eng = llogos.engine.Engine(model, max_tokens=64 * 10, use_graphs=False)
    g = torch.Generator().manual_seed(0)
    seqs = [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in (1, 20, 75)]
    refs = [FP.forward(w, cfg, s) for s in seqs]
    tol = 2e-4
    for rnd in range(2):                                   # the second round uses slots and pages again
        slots = [eng.open() for _ in seqs]
        cut = [max(1, len(s) - 3 - 2 * i) for i, s in enumerate(seqs)]
        lg = eng.step([(sl, s[:c]) for sl, s, c in zip(slots, seqs, cut)])
        for i, c in enumerate(cut):
            assert float((lg[i].double() - refs[i][c - 1]).abs().max()) < tol
        live = [i for i in range(len(seqs)) if cut[i] < len(seqs[i])]
        for i in set(range(len(seqs))) - set(live):
            eng.close(slots[i])
        while live:
            lg = eng.step([(slots[i], [seqs[i][cut[i]]]) for i in live])
            for j, i in enumerate(live):
                assert float((lg[j].double() - refs[i][cut[i]]).abs().max()) < tol
                cut[i] += 1
            for i in [i for i in live if cut[i] == len(seqs[i])]:
                eng.close(slots[i])
            live = [i for i in live if cut[i] < len(seqs[i])]
        eng.cache.audit()
    # a prompt in portions of 2, 5 and the rest
    slot = eng.open()
    s, r = seqs[2], refs[2]
    got = [eng.step([(slot, s[a:b])], [list(range(b - a))]).clone() for a, b in ((0, 2), (2, 7), (7, len(s)))]
    assert float((torch.cat(got).double() - r).abs().max()) < tol
    eng.close(slot)


def test_other_norms_refuse_a_branch_of_several_sublayers(llogos):
    Branch = llogos.parts.base.Branch
    norm = llogos.parts.base.part_class("norm", "rmsnorm")({"size": 4, "eps": 1e-5}, "n.", None)
    with pytest.raises(ValueError, match="several sublayers"):
        norm.forward(torch.zeros(2, 4), Branch(torch.zeros(1, 2, 4), scale=0.5), None)


def test_cost_model_counts_chosen_experts_and_one_row_per_latent_position(llogos):
    import importlib
    measure = importlib.import_module("daisi-llogos_b200.measure")
    cfg = FM.CONFIGS["mixed"]
    model = llogos.weights.build_model(cfg, dtype=torch.bfloat16, device="cpu", ops=cpu_ops)
    costs = measure.model_costs(model)
    d = cfg["width"]
    stored = active = 0
    for lay in cfg["layers"]:
        m = lay["mixer"]
        if lay["type"] == "attention":
            n = d * (m["heads"] * m["dim"] + m["kv_heads"] * (m["dim"] + m["vdim"])) + d * m["heads"] * m["vdim"]
        else:
            n = d * (m["heads"] * (m["dim"] + m["rot_dim"]) + m["kv_rank"] + m["rot_dim"]) + m["kv_rank"] * m["heads"] * (m["dim"] + m["vdim"]) \
                + d * m["heads"] * m["vdim"]
        stored, active = stored + n, active + n
        ml = lay["mlp"]
        if ml:
            e_n, top, ff, sh = ml["router"]["experts"], ml["router"]["top"], ml["expert"]["ff"], (ml.get("shared") or {}).get("ff", 0)
            stored += e_n * d + e_n * 3 * d * ff + 3 * d * sh
            active += e_n * d + top * 3 * d * ff + 3 * d * sh
    assert costs.matrix_params == stored and costs.active_params == active
    assert costs.kv_units[0] == (2 * (16 + 24) * 2, 37) and costs.kv_units[1] == ((24 + 8) * 2, 50)
