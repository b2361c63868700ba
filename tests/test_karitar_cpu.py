"""Karitar without a GPU: the configuration reader, the model builder's tensor names and run order, the plain
implementation's own mechanisms against closed forms, and the engine's host logic over the CPU stand-ins."""
import copy
import importlib

import pytest
import torch

import cpu_ops
import karitar_models as KM
import karitar_plain as KP


@pytest.fixture(scope="module")
def small(llogos, tmp_path_factory):
    cfg = KM.config([KM.layer(KM.attention(4, 2, 8, 12, 9), 40), KM.layer(KM.attention(2, 2, 16, 16, None), None),
                     KM.layer(KM.attention(3, 1, 8, 8, 70), 24)], vocab=61, width=32, streams=3, loop=(1, 3, 2))
    d = str(tmp_path_factory.mktemp("karitar_small"))
    w = KM.write_model(llogos, d, cfg, seed=4)
    return d, cfg, {k: v.float() for k, v in w.items()}


def test_config_is_read_and_wrong_ones_are_named(llogos):
    cfg = KM.CONFIGS["mixed"]
    arch = llogos.config.architecture_of(cfg)
    c = arch.read_config(cfg)
    assert (c.vocab, c.width, c.streams, c.loop) == (211, 72, 3, (0, 2, 2))
    assert c.run_order() == (0, 1, 0, 1, 2)
    assert [l.mixer.window for l in c.layers] == [37, 64, 131] and c.layers[1].mlp is None
    assert c.layers[0].mixer.vdim == 24 and c.layers[2].mixer.kv_heads == 1
    for path, value, word in ((("layers", 0, "type"), "recurrent", "type"), (("layers", 1, "mixer", "heads"), 3, "multiple"),
                              (("layers", 2, "mlp", "kind"), "routed", "kind"), (("loop", "stop"), 9, "loop"),
                              (("norm", "eps"), 0.0, "eps"), (("layers", 0, "mixer", "scale"), -1.0, "scale"),
                              (("layers", 0, "mixer", "mask", "size"), 0, "mask.size"), (("width",), None, "width")):
        bad = copy.deepcopy(cfg)
        node = bad
        for key in path[:-1]:
            node = node[key]
        node[path[-1]] = value
        with pytest.raises(llogos.config.ConfigError, match=word):
            arch.read_config(bad)
    no_mask = copy.deepcopy(cfg)
    del no_mask["layers"][0]["mixer"]["mask"]
    assert arch.read_config(no_mask).layers[0].mixer.window == 0
    with pytest.raises(llogos.config.ConfigError, match="not registered"):
        llogos.config.architecture_of({"architecture": "Nonesuch"})


def test_tensor_names_and_run_order_of_the_built_model(llogos):
    cfg = KM.CONFIGS["mixed"]
    model = llogos.weights.build_model(cfg, dtype=torch.float32, device="cpu", ops=cpu_ops)
    want = {k: tuple(v.shape) for k, v in KM.random_weights(cfg, 0).items()}
    assert {k: tuple(d.shape) for k, d in model.tensor_decls().items()} == want
    assert [e.layer for e in model.spec.schedule] == [0, 1, 0, 1, 2]
    needs = model.cache_needs()
    assert len(needs) == 5 and needs[0] == needs[2] and needs[0] != needs[1]       # a cache per pass, grouped by geometry
    assert needs[0].value_dim == 24 and needs[4].value_dim == 0
    plain = copy.deepcopy(cfg)
    del plain["streams"]
    m2 = llogos.weights.build_model(plain, dtype=torch.float32, device="cpu", ops=cpu_ops)
    assert not any(".hc" in n for n in m2.tensor_decls())


def test_a_missing_tensor_is_reported_by_name(llogos, small, tmp_path):
    d, cfg, w = small
    short = {k: v.to(torch.bfloat16) for k, v in w.items() if k != "l1.hc1.mix"}
    KM.write_model(llogos, str(tmp_path / "m"), cfg, 0, weights=short)
    with pytest.raises(llogos.weights.WeightsError, match="l1.hc1.mix"):
        llogos.weights.load_model(str(tmp_path / "m"), dtype=torch.float32, device="cpu", ops=cpu_ops)


def test_plain_mechanisms_against_closed_forms():
    s = torch.tensor([[0.0, 0.0, 0.0]])
    p = KP.sink_softmax(s, torch.tensor([[True, True, False]]))
    assert torch.allclose(p, torch.tensor([[1 / 3, 1 / 3, 0.0]], dtype=torch.float64))      # the sink takes a third
    import math
    two = KP.sink_softmax(torch.tensor([[3.0, -3.0]]), torch.tensor([[True, True]]))
    total = 1 + math.exp(3.0) + math.exp(-3.0)
    assert abs(float(two[0, 0]) - math.exp(3.0) / total) < 1e-12 and abs(float(two.sum()) - (1 - 1 / total)) < 1e-12
    far = KP.sink_softmax(torch.tensor([[-800.0, 700.0]]), torch.tensor([[True, True]]))      # no overflow either way
    assert float(far[0, 1]) == 1.0 and float(far[0, 0]) == 0.0
    m = KP.window_mask(5, 2)
    assert m.tolist()[3] == [False, False, True, True, False] and KP.window_mask(3, 0).tolist()[2] == [True] * 3
    # one stream with unit weights is the ordinary residual
    x = torch.randn(1, 4, 6, dtype=torch.float64)
    w = {"c.in": torch.ones(1), "c.out": torch.ones(1), "c.mix": torch.ones(1, 1)}
    assert torch.allclose(KP.hyper_sublayer(x, w, "c.", lambda u: 2 * u), 3 * x)
    # the mix matrix is indexed [from, to]
    x = torch.stack([torch.ones(1, 2), 10 * torch.ones(1, 2)]).double()
    w = {"c.in": torch.zeros(2), "c.out": torch.zeros(2), "c.mix": torch.tensor([[0.0, 1.0], [0.0, 0.0]])}
    y = KP.hyper_sublayer(x, w, "c.", lambda u: u)
    assert float(y[0].abs().max()) == 0.0 and float(y[1].min()) == 1.0
    assert KP.run_order({"layers": [0] * 5, "loop": {"start": 1, "stop": 3, "times": 3}}) == [0, 1, 2, 1, 2, 1, 2, 3, 4]


def test_engine_host_logic_agrees_with_plain(llogos, small):
    d, cfg, w = small
    model = llogos.weights.load_model(d, dtype=torch.float32, device="cpu", ops=cpu_ops)
    eng = llogos.engine.Engine(model, max_tokens=64 * 10, use_graphs=False)
    g = torch.Generator().manual_seed(0)
    seqs = [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in (1, 20, 75)]
    refs = [KP.forward(w, cfg, s) for s in seqs]
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


def test_random_model_of_the_design_has_sane_stream_weights(llogos):
    cfg = KM.CONFIGS["four"]
    model = llogos.weights.build_model(cfg, dtype=torch.float32, device="cpu", ops=cpu_ops)
    t = llogos.weights.random_tensors(model.tensor_decls(), 3, norm_std=0.05, dtype=torch.float32)
    assert float((t["l0.hc1.mix"] - torch.eye(4)).abs().max()) < 0.5 and float((t["l0.hc2.out"] - 1).abs().max()) < 0.5


def test_trace_cost_model_counts_looped_layers_and_value_heads(llogos):
    measure = importlib.import_module("daisi-llogos_b200.measure")
    cfg = KM.CONFIGS["mixed"]
    model = llogos.weights.build_model(cfg, dtype=torch.bfloat16, device="cpu", ops=cpu_ops)
    costs = measure.model_costs(model)
    per_layer = []
    for lay in cfg["layers"]:
        m, d = lay["mixer"], cfg["width"]
        n = d * (m["heads"] * m["dim"] + m["kv_heads"] * (m["dim"] + m["vdim"]) + m["heads"]) + d * m["heads"] * m["vdim"]
        n += 2 * d * lay["mlp"]["ff"] if lay["mlp"] else 0
        per_layer.append(n)
    assert costs.matrix_params == 2 * (per_layer[0] + per_layer[1]) + per_layer[2]
    assert costs.head_params == cfg["vocab"] * cfg["width"]
    assert costs.kv_units[0] == (2 * (16 + 24) * 2, 37)
