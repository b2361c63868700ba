"""The Karitar decoder on the GPU against the plain implementation in karitar_plain.py, in float32 and bfloat16:
every mechanism's kernel alone; whole prompts; prompts against token-by-token decoding; prompts in portions down to two
tokens; batches of unequal requests against each alone, with slots and pages used again; keys at page borders and just
inside and outside every window, in prompts and in decoding; the first tokens; long decoding through a ring that goes
round several times; sizes that differ from layer to layer; greedy generation through the library's entry point."""
import math

import pytest
import torch

import karitar_models as KM
import karitar_plain as KP

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]
IDS = ["f32", "bf16"]

# float32: every logit within 1e-4 of the request's largest |logit|.  bfloat16: the root-mean-square error of a
# position's logits within 4e-2 of the logits' own root mean square, every logit within 8e-2 of the largest.
TOL = {torch.float32: (1e-4, 1e-4), torch.bfloat16: (4e-2, 8e-2)}


def close(got, ref, dtype, what=()):
    got = got.detach().to("cpu", torch.float64).reshape(ref.shape)
    rms_tol, max_tol = TOL[dtype]
    rms = float(((got - ref).pow(2).mean(-1).sqrt() / ref.pow(2).mean(-1).sqrt()).max())
    worst = float((got - ref).abs().max() / ref.abs().max())
    assert rms <= rms_tol and worst <= max_tol, (*what, "rms", rms, "max", worst)


@pytest.fixture(scope="module")
def models(llogos, tmp_path_factory):
    """name -> (folder, config, weights as float tensors)."""
    out = {}
    for i, (name, cfg) in enumerate(KM.CONFIGS.items()):
        d = str(tmp_path_factory.mktemp("karitar_" + name))
        w = KM.write_model(llogos, d, cfg, seed=40 + i)
        out[name] = (d, cfg, {k: v.float() for k, v in w.items()})
    return out


@pytest.fixture(scope="module")
def engines(llogos, models):
    kept = {}

    def get(name, dtype, graphs=True, max_tokens=64 * 40):
        key = (name, dtype, graphs, max_tokens)
        if key not in kept:
            model = llogos.weights.load_model(models[name][0], dtype=dtype, device="cuda:0")
            kept[key] = llogos.engine.Engine(model, max_tokens=max_tokens, use_graphs=graphs)
        return kept[key]
    return get


_refs = {}


def plain(models, name, tokens):
    key = (name, tuple(tokens))
    if key not in _refs:
        _, cfg, w = models[name]
        _refs[key] = KP.forward(w, cfg, tokens)
    return _refs[key]


def tokens_for(cfg, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()


# ---- mechanisms alone --------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("streams,hidden", [(1, 40), (2, 72), (3, 96), (4, 130), (8, 64), (8, 1024), (11, 64), (16, 48)])
def test_stream_norm_kernel(llogos, dtype, streams, hidden):
    from importlib import import_module
    ops = import_module("daisi-llogos_b200.kernels.ops")
    g = torch.Generator().manual_seed(streams * 100 + hidden)
    n, parts = 9, 3
    x = torch.randn((streams, n, hidden), generator=g)
    branch = torch.randn((parts, n, hidden), generator=g)
    mix = torch.eye(streams) + 0.3 * torch.randn((streams, streams), generator=g)
    write, read = torch.randn((streams,), generator=g), torch.randn((streams,), generator=g)
    weight = (1 + 0.2 * torch.randn((hidden,), generator=g)).to(dtype)
    eps = 3e-5
    w = {"c.in": read, "c.out": write, "c.mix": mix}
    tol = 2e-6 if dtype == torch.float32 else 1e-2
    # a pending branch is written into the streams, then the read-out is normalised
    want_streams = KP.hyper_sublayer(x.double(), w, "c.", lambda u: branch.double().sum(0))
    want = KP.rms_norm(torch.einsum("s,std->td", read.double(), want_streams), weight.float(), eps)
    dev = x.cuda().contiguous()
    out = torch.empty((n, hidden), dtype=dtype, device="cuda")
    ops.hc_add_rmsnorm(dev, branch.cuda(), mix.cuda(), write.cuda(), read.cuda(), weight.cuda(), eps, out)
    assert float((dev.cpu().double() - want_streams).abs().max()) < 1e-5
    assert float((out.cpu().double() - want).abs().max()) < tol * float(want.abs().max())
    # no branch, plain sum, chosen rows only: the streams stay as they are
    dev2 = x.cuda().contiguous()
    rows = torch.tensor([7, 0, 3], dtype=torch.int32, device="cuda")
    out2 = torch.empty((3, hidden), dtype=dtype, device="cuda")
    ops.hc_add_rmsnorm(dev2, None, None, None, None, weight.cuda(), eps, out2, rows)
    want2 = KP.rms_norm(x.double().sum(0)[[7, 0, 3]], weight.float(), eps)
    assert torch.equal(dev2.cpu(), x)
    assert float((out2.cpu().double() - want2).abs().max()) < tol * float(want2.abs().max())


@pytest.mark.parametrize("kind", ["relu2", "gelu_tanh", "silu", "relu"])
def test_activation_kernel(llogos, kind):
    from importlib import import_module
    ops = import_module("daisi-llogos_b200.kernels.ops")
    g = torch.Generator().manual_seed(3)
    x = 2 * torch.randn((2, 5, 77), generator=g)
    z = x.double().sum(0)
    want = {"relu2": torch.relu(z) ** 2, "relu": torch.relu(z), "silu": z / (1 + torch.exp(-z)),
            "gelu_tanh": 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))}[kind]
    out = torch.empty((5, 77), dtype=torch.float32, device="cuda")
    ops.act_rows(x.cuda(), out, kind)
    assert float((out.cpu().double() - want).abs().max()) < 2e-6 * float(want.abs().max())


def _paged(k, v, dtype):
    """Keys [T, nkv, hd] and values [T, nkv, vd] of ONE sequence as pages in scrambled order, with the page table."""
    t, nkv, hd = k.shape
    n_pages = (t + 63) // 64
    order = list(reversed(range(n_pages)))
    kp = torch.zeros((n_pages + 1, nkv, 64, hd), dtype=dtype)
    vp = torch.zeros((n_pages + 1, nkv, 64, v.shape[2]), dtype=dtype)
    for pos in range(t):
        kp[order[pos // 64], :, pos % 64] = k[pos].to(dtype)
        vp[order[pos // 64], :, pos % 64] = v[pos].to(dtype)
    table = torch.tensor([order], dtype=torch.int32)
    return kp.cuda(), vp.cuda(), table.cuda()


def _plain_attention(q, k, v, gate, scale, window, sink):
    """[T, nh, hd] x [T, nkv, hd] x [T, nkv, vd] -> [T, nh, vd], float64."""
    t, nh, _ = q.shape
    group = nh // k.shape[1]
    vis = KP.window_mask(t, window)
    out = torch.zeros((t, nh, v.shape[2]), dtype=torch.float64)
    for h in range(nh):
        s = (q[:, h].double() @ k[:, h // group].double().t()) * scale
        if sink:
            p = KP.sink_softmax(s, vis)
        else:
            p = torch.softmax(s.masked_fill(~vis, -math.inf), -1)
        out[:, h] = p @ v[:, h // group].double()
    return out * gate.double()[:, :, None] if gate is not None else out


# head sizes of every kernel family: tcgen05 / TMA (64, 128), mma.sync (48, 32), CUDA cores (40, and values of another size)
@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("nh,nkv,hd,vd,window", [(4, 2, 64, 64, 70), (2, 1, 128, 128, 0), (6, 2, 48, 48, 100), (4, 4, 32, 32, 33),
                                                 (3, 1, 40, 40, 64), (4, 2, 48, 16, 65), (2, 2, 16, 72, 0)])
def test_attention_kernels_with_sink_gate_and_standing_out_keys(llogos, dtype, nh, nkv, hd, vd, window):
    """One sequence of 300 tokens, a prompt step over all of it and a decode step for its last token.  In every head the
    key just inside the last queries' window and the key just outside it are made to stand out (a multiple of the query),
    so that a window that is one token off, or a sink that is left out, changes the output by far more than the bound;
    without a window the key that stands out lies hundreds of positions back."""
    from importlib import import_module
    ops = import_module("daisi-llogos_b200.kernels.ops")
    g = torch.Generator().manual_seed(nh * 1000 + hd + vd)
    t = 300
    q = torch.randn((t, nh, hd), generator=g)
    k = torch.randn((t, nkv, hd), generator=g)
    v = torch.randn((t, nkv, vd), generator=g)
    gate = torch.rand((t, nh), generator=g)
    scale = 0.7 / math.sqrt(hd)
    for qi in (t - 1, t - 2, 200):
        if window:
            marked = ((qi - window + 1, 1.0), (qi - window, 1.0), (0, -1.0))
        else:
            marked = ((t - qi + 1, 1.0),)          # no window: a key hundreds of positions back, one per marked query
        for pos, sign in marked:
            if 0 <= pos < qi:
                k[pos] = sign * 6.0 * q[qi, ::nh // nkv] / math.sqrt(hd)
    rnd = (lambda x: x.to(dtype).float())
    q, k, v = rnd(q), rnd(k), rnd(v)
    form = ops.AttentionForm(value_dim=vd, sink=0.0, gated=True)
    want = _plain_attention(q, k, v, gate, scale, window, sink=True)
    no_sink = _plain_attention(q, k, v, gate, scale, window, sink=False)
    assert float((want - no_sink).abs().max()) > 0.05          # the sink matters in this test
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    kp, vp, table = _paged(k, v, dtype)
    slots = torch.zeros(1, dtype=torch.int32, device="cuda")
    # prompt step: nothing in the cache before it
    tq = ops.prefill_tile_queries(dtype, hd, form)
    tiles = torch.tensor([[0, q0] for q0 in range(0, t, tq)], dtype=torch.int32, device="cuda")
    cu = torch.tensor([0, t], dtype=torch.int32, device="cuda")
    out = torch.empty((t, nh * vd), dtype=dtype, device="cuda")
    ops.attn_prefill(q.to(dtype).cuda(), k.to(dtype).cuda(), v.to(dtype).cuda(), kp, vp, table, table.shape[1], tiles, cu,
                     torch.zeros(1, dtype=torch.int32, device="cuda"), slots, out, scale=scale, window=window,
                     tile_queries=tq, form=form, gate=gate.cuda())
    err = float((out.cpu().double().view(t, nh, vd) - want).abs().max())
    assert err < tol * float(want.abs().max()), ("prompt", err)
    # a prompt step that continues a sequence: the first 171 keys come from the pages
    lb = 171
    tiles2 = torch.tensor([[0, q0] for q0 in range(0, t - lb, tq)], dtype=torch.int32, device="cuda")
    out2 = torch.empty((t - lb, nh * vd), dtype=dtype, device="cuda")
    ops.attn_prefill(q[lb:].to(dtype).cuda(), k[lb:].to(dtype).cuda(), v[lb:].to(dtype).cuda(), kp, vp, table, table.shape[1],
                     tiles2, torch.tensor([0, t - lb], dtype=torch.int32, device="cuda"),
                     torch.tensor([lb], dtype=torch.int32, device="cuda"), slots, out2, scale=scale, window=window,
                     tile_queries=tq, form=form, gate=gate[lb:].contiguous().cuda())
    err = float((out2.cpu().double().view(t - lb, nh, vd) - want[lb:]).abs().max())
    assert err < tol * float(want.abs().max()), ("continued prompt", err)
    # decode step of the last token
    plan = ops.attn_decode_plan(dtype, 1, nh, nkv, hd, 1024, form)
    scratch = torch.zeros(max(1, plan.scratch_floats), dtype=torch.float32, device="cuda")
    counters = torch.zeros(max(1, plan.n_counters), dtype=torch.int32, device="cuda")
    out3 = torch.empty((1, nh * vd), dtype=dtype, device="cuda")
    ops.attn_decode(q[t - 1:].to(dtype).cuda(), kp, vp, table, table.shape[1], slots,
                    torch.tensor([t - 1], dtype=torch.int32, device="cuda"), out3, scratch, scale=scale, window=window,
                    plan=plan, counters=counters, form=form, gate=gate[t - 1:].contiguous().cuda())
    err = float((out3.cpu().double().view(nh, vd) - want[t - 1]).abs().max())
    assert err < tol * float(want.abs().max()), ("decode", plan.kind, err)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_row_prep_kernel(llogos, dtype):
    from importlib import import_module
    ops = import_module("daisi-llogos_b200.kernels.ops")
    g = torch.Generator().manual_seed(8)
    n, nh, nkv, hd, vd = 7, 6, 2, 24, 40
    qw, kw, vw = nh * hd, nkv * hd, nkv * vd
    x = torch.randn((2, n, qw + kw + vw + nh), generator=g)
    bias = (0.3 * torch.randn((qw + kw + vw,), generator=g)).to(dtype)
    qn = (1 + 0.3 * torch.randn((qw,), generator=g)).to(dtype)
    kn = (1 + 0.3 * torch.randn((kw,), generator=g)).to(dtype)
    eps = 2e-5
    z = x.double().sum(0)
    z[:, :qw + kw + vw] += bias.double()
    want_q = KP.rms_norm(z[:, :qw], qn.float(), eps)
    want_k = KP.rms_norm(z[:, qw:qw + kw], kn.float(), eps)
    want_v, want_g = z[:, qw + kw:qw + kw + vw], torch.sigmoid(z[:, qw + kw + vw:])
    q = torch.empty((n, nh, hd), dtype=dtype, device="cuda")
    k_new = torch.empty((n, nkv, hd), dtype=dtype, device="cuda")
    v_new = torch.empty((n, nkv, vd), dtype=dtype, device="cuda")
    gate = torch.empty((n, nh), dtype=torch.float32, device="cuda")
    kp = torch.zeros((3, nkv, 64, hd), dtype=dtype, device="cuda")
    vp = torch.zeros((3, nkv, 64, vd), dtype=dtype, device="cuda")
    table = torch.tensor([[2, 0]], dtype=torch.int32, device="cuda")
    positions = torch.arange(60, 60 + n, dtype=torch.int32, device="cuda")      # across a page border
    ops.qkv_row_prep(x.cuda(), n_heads=nh, n_kv_heads=nkv, head_dim=hd, value_dim=vd, bias=bias.cuda(), q_norm_w=qn.cuda(),
                     k_norm_w=kn.cuda(), norm_eps=eps, positions=positions, q_out=q, gate_out=gate, k_new=k_new, v_new=v_new,
                     k_pages=kp, v_pages=vp, page_table=table, ring_pages=2,
                     seq_of_token=torch.zeros(n, dtype=torch.int32, device="cuda"), slots=torch.zeros(1, dtype=torch.int32, device="cuda"))
    tol = 2e-6 if dtype == torch.float32 else 8e-3
    for got, want in ((q, want_q), (k_new, want_k), (v_new, want_v), (gate, want_g)):
        assert float((got.cpu().double().reshape(want.shape) - want).abs().max()) < tol * float(want.abs().max())
    for i in range(n):
        pos = 60 + i
        page = [2, 0][pos // 64]
        assert torch.equal(kp[page, :, pos % 64], k_new[i]) and torch.equal(vp[page, :, pos % 64], v_new[i])


# ---- whole models ------------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("name", list(KM.CONFIGS))
def test_whole_prompt_and_first_tokens(engines, models, name, dtype):
    eng = engines(name, dtype)
    cfg = models[name][1]
    for n in (1, 2, 3, 190):
        toks = tokens_for(cfg, n, n)
        ref = plain(models, name, toks)
        slot = eng.open()
        lg = eng.step([(slot, toks)], [list(range(n))])
        close(lg, ref, dtype, (name, "whole", n))
        eng.close(slot)
    eng.cache.audit()


@pytest.mark.parametrize("graphs", [True, False], ids=["graph", "eager"])
@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("name", list(KM.CONFIGS))
def test_prompt_then_token_by_token(engines, models, name, dtype, graphs):
    """The decoded positions pass page borders (128, 192) and every window's edge; the first token alone too."""
    eng = engines(name, dtype, graphs)
    cfg = models[name][1]
    toks = tokens_for(cfg, 215, 7)
    ref = plain(models, name, toks)
    for cut in (1, 120):
        slot = eng.open()
        lg = eng.step([(slot, toks[:cut])])
        close(lg, ref[cut - 1:cut], dtype, (name, "prompt end", cut))
        got = [eng.step([(slot, [toks[p]])]).clone() for p in range(cut, len(toks) if cut > 1 else 40)]
        close(torch.cat(got), ref[cut:cut + len(got)], dtype, (name, "decoded from", cut))
        eng.close(slot)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("name", list(KM.CONFIGS))
def test_portions_of_several_sizes(engines, models, name, dtype):
    eng = engines(name, dtype)
    cfg = models[name][1]
    toks = tokens_for(cfg, 300, 9)
    ref = plain(models, name, toks)
    for sizes in ([2] * 20 + [3, 64, 65, 1, 1, 2, 124], [63, 1, 64, 2, 170], [129, 171]):
        assert sum(sizes) == len(toks)
        slot = eng.open()
        at, got = 0, []
        for s in sizes:
            got.append(eng.step([(slot, toks[at:at + s])], [list(range(s))]).clone())
            at += s
        close(torch.cat(got), ref, dtype, (name, "portions", sizes[:4]))
        eng.close(slot)
    eng.cache.audit()


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("name", list(KM.CONFIGS))
def test_unequal_batches_with_slots_and_pages_used_again(engines, models, name, dtype):
    eng = engines(name, dtype)
    cfg = models[name][1]
    seqs = [tokens_for(cfg, n, 20 + n) for n in (1, 66, 140, 259, 33)]
    refs = [plain(models, name, s) for s in seqs]
    for order in ([0, 1, 2, 3], [4, 3, 0], [2, 1, 4, 3, 0]):
        slots = {i: eng.open() for i in order}
        cut = {i: max(1, len(seqs[i]) - 4 - 9 * j) for j, i in enumerate(order)}
        lg = eng.step([(slots[i], seqs[i][:cut[i]]) for i in order])
        for j, i in enumerate(order):
            close(lg[j], refs[i][cut[i] - 1], dtype, (name, "batched prompt", i))
        live = [i for i in order if cut[i] < len(seqs[i])]
        for i in set(order) - set(live):
            eng.close(slots[i])
        while live:
            lg = eng.step([(slots[i], [seqs[i][cut[i]]]) for i in live])
            for j, i in enumerate(live):
                close(lg[j], refs[i][cut[i]], dtype, (name, "batched decode", i, cut[i]))
                cut[i] += 1
            for i in [i for i in live if cut[i] == len(seqs[i])]:
                eng.close(slots[i])
            live = [i for i in live if cut[i] < len(seqs[i])]
        eng.cache.audit()
    assert eng.cache.slots.free_count == eng.cache.slots.n_slots


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_long_decoding_round_the_ring(engines, models, dtype):
    """420 decoded tokens after a prompt of 30: the smallest window's ring of pages goes round several times."""
    name = "mixed"
    eng = engines(name, dtype)
    cfg = models[name][1]
    toks = tokens_for(cfg, 450, 5)
    ref = plain(models, name, toks)
    slot = eng.open()
    eng.step([(slot, toks[:30])], [[]])
    got = [eng.step([(slot, [toks[p]])]).clone() for p in range(30, len(toks))]
    close(torch.cat(got), ref[30:], dtype, ("long decoding",))
    eng.close(slot)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_a_key_that_stands_out_at_every_windows_edge(llogos, tmp_path, dtype):
    """One layer, one head group; the key projection is made so that token A's key matches token B's query strongly.
    Token A stands once just inside and once just outside the window of the B that asks for it, in a prompt and in
    decoding: the logits there differ widely between the two, and must follow the plain model in both."""
    window = 67
    cfg = KM.config([KM.layer(KM.attention(2, 1, 32, 32, window, scale=1.0), None)], vocab=50, width=48, streams=2)
    w = KM.random_weights(cfg, 77)
    a_tok, b_tok = 11, 12
    # Token b's embedding is token a's with its coordinates permuted, and the key matrix is the first head's query
    # matrix with its columns permuted the same way: a's key is then b's first-head query (before the norms, which
    # keep directions), while b's own key and a's value are unrelated to it.
    gen = torch.Generator().manual_seed(1)
    perm = torch.randperm(48, generator=gen)
    w["embed"][a_tok] = (2 * torch.randn(48, generator=gen)).to(torch.bfloat16)
    w["embed"][b_tok] = w["embed"][a_tok][perm]
    w["l0.mix.k"][:, perm] = w["l0.mix.q"][:32]
    w["l0.mix.k.b"][:] = w["l0.mix.q.b"][:32]
    w["l0.mix.k.norm"][:] = w["l0.mix.q.norm"][:32]
    d = str(tmp_path / "edge")
    KM.write_model(llogos, d, cfg, 0, weights=w)
    wf = {k: v.float() for k, v in w.items()}
    model = llogos.weights.load_model(d, dtype=dtype, device="cuda:0")
    eng = llogos.engine.Engine(model, max_tokens=64 * 8)
    g = torch.Generator().manual_seed(2)
    for a_at in (0, 61, 64):
        inside, outside = a_at + window - 1, a_at + window
        toks = torch.randint(13, 50, (outside + 3,), generator=g).tolist()
        toks[a_at] = a_tok
        for b_at in (inside, outside):
            t = list(toks)
            t[b_at] = b_tok
            ref = KP.forward(wf, cfg, t)
            for cut in (len(t), b_at):                 # b inside the prompt; b decoded alone
                slot = eng.open()
                lg = eng.step([(slot, t[:cut])], [[b_at] if b_at < cut else []])
                if b_at >= cut:
                    lg = eng.step([(slot, [t[b_at]])])
                close(lg, ref[b_at:b_at + 1], dtype, ("edge", a_at, b_at, cut))
                eng.close(slot)
        # and the two cases are far apart, so the test would see a window that is one token off
        t_in, t_out = list(toks), list(toks)
        t_in[inside], t_out[outside] = b_tok, b_tok
        r_in, r_out = KP.forward(wf, cfg, t_in)[inside], KP.forward(wf, cfg, t_out)[outside]
        assert float((r_in - r_out).abs().max()) > 0.15 * float(r_in.abs().max())


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_a_far_key_among_hundreds(llogos, tmp_path, dtype):
    """The same construction without a window: token a stands at position 2, token b 330 positions later (five pages on);
    b's logits with a there and with another token in a's place are far apart, in a prompt and decoded."""
    cfg = KM.config([KM.layer(KM.attention(2, 1, 32, 32, None, scale=2.0), None)], vocab=50, width=48, streams=2)
    w = KM.random_weights(cfg, 78)
    a_tok, b_tok = 11, 12
    gen = torch.Generator().manual_seed(3)
    perm = torch.randperm(48, generator=gen)
    w["embed"][a_tok] = (2 * torch.randn(48, generator=gen)).to(torch.bfloat16)
    w["embed"][b_tok] = w["embed"][a_tok][perm]
    w["l0.mix.k"][:, perm] = w["l0.mix.q"][:32]
    w["l0.mix.k.b"][:] = w["l0.mix.q.b"][:32]
    w["l0.mix.k.norm"][:] = w["l0.mix.q.norm"][:32]
    d = str(tmp_path / "far")
    KM.write_model(llogos, d, cfg, 0, weights=w)
    wf = {k: v.float() for k, v in w.items()}
    model = llogos.weights.load_model(d, dtype=dtype, device="cuda:0")
    eng = llogos.engine.Engine(model, max_tokens=64 * 8)
    toks = torch.randint(13, 50, (336,), generator=gen).tolist()
    b_at = 332
    toks[b_at] = b_tok
    with_a, without_a = list(toks), list(toks)
    with_a[2] = a_tok
    refs = [KP.forward(wf, cfg, t) for t in (with_a, without_a)]
    assert float((refs[0][b_at] - refs[1][b_at]).abs().max()) > 0.1 * float(refs[0][b_at].abs().max())
    for t, ref in zip((with_a, without_a), refs):
        for cut in (len(t), b_at):
            slot = eng.open()
            lg = eng.step([(slot, t[:cut])], [[b_at] if b_at < cut else []])
            if b_at >= cut:
                lg = eng.step([(slot, [t[b_at]])])
            close(lg, ref[b_at:b_at + 1], dtype, ("far key", cut))
            eng.close(slot)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_greedy_generation_through_the_entry_point(models, dtype):
    """``LlogosModel.generate`` (scheduler, sampler, run-ahead decoding) makes the plain model's best tokens."""
    import llogos_b200 as L
    name = "mixed"
    d, cfg, w = models[name]
    model = L.LlogosModel.load(d, dtype=dtype, max_context=256, max_batch=3)
    prompts = [tokens_for(cfg, n, 60 + n) for n in (5, 70, 23, 1)]
    out = model.generate(prompts, L.GenerationParams.greedy_params(12, stop_tokens=()))
    for p, made in zip(prompts, out.tokens):
        assert len(made) == 12
        toks = list(p)
        for tok in made:
            lg = KP.forward(w, cfg, toks)[-1]
            slack = 1e-4 if dtype == torch.float32 else 0.05
            assert float(lg[tok]) >= float(lg.max()) - slack * float(lg.abs().max()), (len(toks), tok)
            toks.append(tok)


@pytest.mark.parametrize("kind", ["relu2", "gelu_tanh"])
@pytest.mark.parametrize("n,o,k", [(5, 200, 96), (40, 333, 128), (300, 520, 192), (700, 130, 64)])
def test_product_with_the_activation_as_its_epilogue(llogos, kind, n, o, k):
    """Few rows (weights are the tensor cores' rows) and many (tokens are): act(x w^T) against the plain product."""
    from importlib import import_module
    ops = import_module("daisi-llogos_b200.kernels.ops")
    g = torch.Generator().manual_seed(n + o)
    x = torch.randn((n, k), generator=g).to(torch.bfloat16)
    w = (torch.randn((o, k), generator=g) / math.sqrt(k)).to(torch.bfloat16)
    z = x.double() @ w.double().t()
    want = torch.relu(z) ** 2 if kind == "relu2" else 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))
    out = torch.empty((n, o), dtype=torch.bfloat16, device="cuda")
    ops.gemm_tc_act(x.cuda(), w.cuda(), out, kind)
    assert float((out.cpu().double() - want).abs().max()) < 5e-3 * float(want.abs().max()), (n, o, k)
    assert ops.gemm_tc_status() == 0


def test_command_line_and_trace_replay_take_the_design(models, tmp_path):
    """``python -m llogos_b200`` generates and benchmarks a Karitar folder, and ``bin/trace_run`` replays steps on it
    (a prompt in two portions beside a second request, then decoding together), as they do for every model."""
    import json
    import os
    import subprocess
    import sys
    import numpy as np
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    d, cfg, w = models["wide"]
    env = dict(os.environ, PYTHONPATH=root)
    base = [sys.executable, "-m", "llogos_b200", "--model", d, "--dtype", "float32"]
    p = subprocess.run(base + ["--prompt-ids", "5,17,3", "-n", "6", "-t", "0", "--repeat-penalty", "1.0", "--max-context", "128"],
                       capture_output=True, text=True, env=env, cwd=root)
    assert p.returncode == 0, p.stderr
    made = [int(x) for x in p.stdout.split()]
    toks = [5, 17, 3]
    for tok in made:
        lg = KP.forward(w, cfg, toks)[-1]
        assert float(lg[tok]) >= float(lg.max()) - 1e-4 * float(lg.abs().max())
        toks.append(tok)
    p = subprocess.run(base + ["--bench", "--batch", "2", "--prompt-len", "20:40", "--context", "80", "--seed", "1"],
                       capture_output=True, text=True, env=env, cwd=root)
    assert p.returncode == 0 and "Decode step:" in p.stderr and "Prompt step:" in p.stderr, p.stderr
    a, b = tokens_for(cfg, 100, 1), tokens_for(cfg, 31, 2)
    ra, rb = plain(models, "wide", a), plain(models, "wide", b)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:70], "want": [0, 69]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[70:98], "want": [27]}, {"id": "b", "tokens": b[:30], "want": [29]}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": a[98:99], "want": [0]}, {"id": "b", "tokens": b[30:], "want": [0]}], "end": ["b"]},
             {"step": 3, "entries": [{"id": "a", "tokens": a[99:], "want": [0]}], "end": ["a"]}]
    out = tmp_path / "logits"
    p = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", d, "--dtype", "bfloat16", "--out", str(out), "--max-tokens", "200"],
                       input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, env=env, cwd=root)
    assert p.returncode == 0, p.stderr
    assert [l for l in p.stdout.split("\n") if l.startswith("done")] == ["done 0", "done 1", "done 2", "done 3"]
    want = [ra[[0, 69]], torch.stack([ra[97], rb[29]]), torch.stack([ra[98], rb[30]]), ra[99:100]]
    for i, ref in enumerate(want):
        got = torch.from_numpy(np.fromfile(str(out / f"{i}.f32"), dtype="<f4").reshape(-1, cfg["vocab"]))
        close(got, ref, torch.bfloat16, ("replayed step", i))
