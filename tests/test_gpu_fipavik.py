"""The Fipavik decoder on the GPU against the plain implementation in fipavik_plain.py, in float32 and bfloat16:
every mechanism's kernel alone; whole prompts; prompts against token-by-token decoding; prompts in portions down to two
tokens; batches of unequal requests against each alone, with slots and pages used again; keys at page borders and just
inside and outside every chunk and window, in prompts and in decoding; the first tokens; long decoding through rings that
go round several times; sizes that differ from layer to layer; greedy generation through the library's entry point."""
import math

import pytest
import torch

import fipavik_models as FM
import fipavik_plain as FP

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]
IDS = ["f32", "bf16"]

# float32: every logit within 1e-4 of the request's largest |logit|.  bfloat16: the root-mean-square error of a
# position's logits within 4e-2 of the logits' own root mean square, every logit within 8e-2 of the largest.
TOL = {torch.float32: (1e-4, 1e-4), torch.bfloat16: (4e-2, 8e-2)}


def ops_module():
    from importlib import import_module
    return import_module("daisi-llogos_b200.kernels.ops")


def close(got, ref, dtype, what=()):
    got = got.detach().to("cpu", torch.float64).reshape(ref.shape)
    rms_tol, max_tol = TOL[dtype]
    rms = float(((got - ref).pow(2).mean(-1).sqrt() / ref.pow(2).mean(-1).sqrt()).max())
    worst = float((got - ref).abs().max() / ref.abs().max())
    assert rms <= rms_tol and worst <= max_tol, (*what, "rms", rms, "max", worst)


@pytest.fixture(scope="module")
def models(llogos, tmp_path_factory):
    """(name, dtype) -> (folder, config, weights as float tensors).  The bfloat16 comparisons use routers that never
    decide by a close call (the router's input is rounded there); float32 takes routers that hang on every token."""
    out = {}
    for i, (name, cfg) in enumerate(FM.CONFIGS.items()):
        for dtype in DTYPES:
            d = str(tmp_path_factory.mktemp(f"fipavik_{name}_{IDS[DTYPES.index(dtype)]}"))
            w = FM.write_model(llogos, d, cfg, seed=70 + i, steady_routing=dtype == torch.bfloat16)
            out[name, dtype] = (d, cfg, {k: v.float() for k, v in w.items()})
    return out


@pytest.fixture(scope="module")
def engines(llogos, models):
    kept = {}

    def get(name, dtype, graphs=True, max_tokens=64 * 40):
        key = (name, dtype, graphs, max_tokens)
        if key not in kept:
            model = llogos.weights.load_model(models[name, dtype][0], dtype=dtype, device="cuda:0")
            kept[key] = llogos.engine.Engine(model, max_tokens=max_tokens, use_graphs=graphs)
        return kept[key]
    return get


_refs = {}


def plain(models, name, dtype, tokens):
    """The plain logits; in bfloat16 also a check that no router of this sequence decided by a close call."""
    key = (name, dtype, tuple(tokens))
    if key not in _refs:
        _, cfg, w = models[name, dtype]
        margins = []
        _refs[key] = FP.forward(w, cfg, tokens, margins=margins)
        if dtype == torch.bfloat16 and margins:
            assert float(torch.stack(margins).min()) > 0.05, "this test's sequence meets a close call in a router"
    return _refs[key]


def tokens_for(cfg, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()


# ---- mechanisms alone --------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("hidden,sets", [(40, (2, 1)), (72, (1,)), (130, (3, 2, 1)), (1024, (1, 4)), (4100, (2, 2))])
def test_layer_norm_kernel(llogos, dtype, hidden, sets):
    ops = ops_module()
    g = torch.Generator().manual_seed(hidden)
    n = 9
    x = 3 + 2 * torch.randn((n, hidden), generator=g)                   # a mean far from zero
    parts = [torch.randn((s, n, hidden), generator=g) for s in sets]
    weight = (1 + 0.2 * torch.randn((hidden,), generator=g)).to(dtype)
    bias = (0.3 * torch.randn((hidden,), generator=g)).to(dtype)
    eps, scale = 3e-5, 0.37
    want_res = x.double() + scale * sum(p.double().sum(0) for p in parts)
    want = FP.layer_norm(want_res, weight.float(), bias.float(), eps)
    tol = 3e-6 if dtype == torch.float32 else 1e-2
    dev = x.cuda()
    out = torch.empty((n, hidden), dtype=dtype, device="cuda")
    ops.add_layernorm(dev, [p.cuda() for p in parts], scale, weight.cuda(), bias.cuda(), eps, out)
    assert float((dev.cpu().double() - want_res).abs().max()) < 1e-5
    assert float((out.cpu().double() - want).abs().max()) < tol * float(want.abs().max())
    # nothing pending, chosen rows only: the residual stays as it is
    dev2 = x.cuda()
    rows = torch.tensor([7, 0, 3], dtype=torch.int32, device="cuda")
    out2 = torch.empty((3, hidden), dtype=dtype, device="cuda")
    ops.add_layernorm(dev2, (), 1.0, weight.cuda(), bias.cuda(), eps, out2, rows)
    want2 = FP.layer_norm(x.double()[[7, 0, 3]], weight.float(), bias.float(), eps)
    assert torch.equal(dev2.cpu(), x)
    assert float((out2.cpu().double() - want2).abs().max()) < tol * float(want2.abs().max())


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_head_preparation_with_values_of_their_own_size_and_blending(llogos, dtype):
    """Per-head norms with one weight for all heads, rotation of a part of the head, values of another size, lent out by
    one call and blended in by the next; writes across a page border."""
    ops = ops_module()
    g = torch.Generator().manual_seed(8)
    n, nh, nkv, hd, vd, rot = 7, 6, 2, 24, 40, 8
    width = (nh + nkv) * hd + nkv * vd
    x = torch.randn((2, n, width), generator=g)
    qn = (1 + 0.3 * torch.randn((hd,), generator=g)).to(dtype)
    kn = (1 + 0.3 * torch.randn((hd,), generator=g)).to(dtype)
    eps, base = 2e-5, 700.0
    pos = torch.arange(60, 60 + n)
    z = x.double().sum(0)
    want_q = FP.rotate_halves(FP.rms_norm(z[:, :nh * hd].view(n, nh, hd), qn.float(), eps), pos, rot, base)
    want_k = FP.rotate_halves(FP.rms_norm(z[:, nh * hd:(nh + nkv) * hd].view(n, nkv, hd), kn.float(), eps), pos, rot, base)
    want_v = z[:, (nh + nkv) * hd:].view(n, nkv, vd)
    i = torch.arange(rot // 2, dtype=torch.float64)
    ang = torch.arange(80, dtype=torch.float64)[:, None] * (base ** (-2 * i / rot))[None]
    cos, sin = torch.cos(ang).float().cuda(), torch.sin(ang).float().cuda()
    kp = torch.zeros((3, nkv, 64, hd), dtype=dtype, device="cuda")
    vp = torch.zeros((3, nkv, 64, vd), dtype=dtype, device="cuda")
    table = torch.tensor([[2, 0]], dtype=torch.int32, device="cuda")
    common = dict(n_heads=nh, n_kv_heads=nkv, head_dim=hd, q_norm_w=qn.cuda(), k_norm_w=kn.cuda(), norm_eps=eps, bias=None,
                  cos=cos, sin=sin, rotary_dim=rot, pairing=0, positions=pos.int().cuda(), value_dim=vd,
                  k_pages=kp, v_pages=vp, page_table=table, ring_pages=2,
                  seq_of_token=torch.zeros(n, dtype=torch.int32, device="cuda"), slots=torch.zeros(1, dtype=torch.int32, device="cuda"))
    q = torch.empty((n, nh, hd), dtype=dtype, device="cuda")
    k_new = torch.empty((n, nkv, hd), dtype=dtype, device="cuda")
    v_new = torch.empty((n, nkv, vd), dtype=dtype, device="cuda")
    lent = torch.empty((n, nkv, vd), dtype=torch.float32, device="cuda")
    ops.qk_prep(x.cuda(), **common, q_out=q, k_new=k_new, v_new=v_new, v_first_out=lent)
    tol = 3e-6 if dtype == torch.float32 else 8e-3
    for got, want in ((q, want_q), (k_new, want_k), (v_new, want_v)):
        assert float((got.cpu().double() - want).abs().max()) < tol * float(want.abs().max())
    assert float((lent.cpu().double() - want_v).abs().max()) < 3e-6 * float(want_v.abs().max())      # float32 whatever the type
    for j in range(n):
        p = 60 + j
        assert torch.equal(kp[[2, 0][p // 64], :, p % 64], k_new[j]) and torch.equal(vp[[2, 0][p // 64], :, p % 64], v_new[j])
    # the next layer blends its own values with the lent ones
    other = torch.randn((n, nkv, vd), generator=g)
    lam = torch.tensor([0.3], dtype=torch.float32)
    ops.qk_prep(x.cuda(), **common, q_out=q, k_new=k_new, v_new=v_new, v_first_in=other.cuda(), v_mix=lam.cuda())
    want_b = 0.7 * want_v + 0.3 * other.double()
    assert float((v_new.cpu().double() - want_b).abs().max()) < tol * float(want_b.abs().max())


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


def _plain_attention(q, k, v, scale, vis, sinks):
    t, nh, _ = q.shape
    group = nh // k.shape[1]
    out = torch.zeros((t, nh, v.shape[2]), dtype=torch.float64)
    for h in range(nh):
        s = (q[:, h].double() @ k[:, h // group].double().t()) * scale
        out[:, h] = FP.sink_softmax(s, vis, sinks[h]) @ v[:, h // group].double()
    return out


# head sizes of every kernel family: tcgen05 / TMA (64, 128), mma.sync (48, 32), CUDA cores (40, and values of another size)
@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("chunked", [True, False], ids=["chunk", "window"])
@pytest.mark.parametrize("nh,nkv,hd,vd,size", [(4, 2, 64, 64, 70), (2, 1, 128, 128, 64), (6, 2, 48, 48, 100), (4, 4, 32, 32, 33),
                                               (3, 1, 40, 40, 65), (4, 2, 48, 16, 63), (8, 1, 96, 64, 128)])
def test_attention_kernels_with_chunks_and_a_sink_per_head(llogos, dtype, chunked, nh, nkv, hd, vd, size):
    """One sequence of 300 tokens: a prompt step over all of it, a prompt step that continues it, and a decode step for
    its last token.  For a few queries the key just inside the mask and the key just outside it are made to stand out
    (a multiple of the query), so that a mask that is one position off changes the output by far more than the bound;
    the sinks differ widely from head to head, so that a sink left out or taken from another head shows too."""
    ops = ops_module()
    g = torch.Generator().manual_seed(nh * 1000 + hd + vd)
    t = 300
    q = torch.randn((t, nh, hd), generator=g)
    k = torch.randn((t, nkv, hd), generator=g)
    v = torch.randn((t, nkv, vd), generator=g)
    sinks = 3.0 * torch.randn((nh,), generator=g)
    scale = 0.7 / math.sqrt(hd)
    for qi in (t - 1, t - 2, 200, size, size - 1):
        first = (qi // size) * size if chunked else qi - size + 1       # the first position the query sees
        for pos in (first, first - 1):
            if 0 <= pos < qi:
                k[pos] = 6.0 * q[qi, ::nh // nkv] / math.sqrt(hd)
    rnd = (lambda x: x.to(dtype).float())
    q, k, v = rnd(q), rnd(k), rnd(v)
    vis = FP.chunk_mask(t, size) if chunked else FP.window_mask(t, size)
    want = _plain_attention(q, k, v, scale, vis, sinks)
    for wrong in (FP.chunk_mask(t, size) if not chunked else FP.window_mask(t, size),):
        assert float((want - _plain_attention(q, k, v, scale, wrong, sinks)).abs().max()) > 0.05     # the mask's kind matters here
    assert float((want - _plain_attention(q, k, v, scale, vis, sinks.flip(0))).abs().max()) > 0.05   # and whose sink it is
    form = ops.AttentionForm(value_dim=vd, sinks=sinks.cuda(), chunked=chunked)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    kp, vp, table = _paged(k, v, dtype)
    slots = torch.zeros(1, dtype=torch.int32, device="cuda")
    tq = ops.prefill_tile_queries(dtype, hd, form)
    for lb in (0, 171):                                  # nothing in the cache; the first 171 keys come from the pages
        tiles = torch.tensor([[0, q0] for q0 in range(0, t - lb, tq)], dtype=torch.int32, device="cuda")
        out = torch.empty((t - lb, nh * vd), dtype=dtype, device="cuda")
        ops.attn_prefill(q[lb:].to(dtype).cuda(), k[lb:].to(dtype).cuda(), v[lb:].to(dtype).cuda(), kp, vp, table, table.shape[1],
                         tiles, torch.tensor([0, t - lb], dtype=torch.int32, device="cuda"),
                         torch.tensor([lb], dtype=torch.int32, device="cuda"), slots, out, scale=scale, window=size,
                         tile_queries=tq, form=form)
        err = float((out.cpu().double().view(t - lb, nh, vd) - want[lb:]).abs().max())
        assert err < tol * float(want.abs().max()), ("prompt from", lb, err)
    for last in (t - 1, size, size - 1):                 # decode steps: the last token, the first of a chunk, the one before
        plan = ops.attn_decode_plan(dtype, 1, nh, nkv, hd, 1024, form)
        scratch = torch.zeros(max(1, plan.scratch_floats), dtype=torch.float32, device="cuda")
        counters = torch.zeros(max(1, plan.n_counters), dtype=torch.int32, device="cuda")
        out3 = torch.empty((1, nh * vd), dtype=dtype, device="cuda")
        ops.attn_decode(q[last:last + 1].to(dtype).cuda(), kp, vp, table, table.shape[1], slots,
                        torch.tensor([last], dtype=torch.int32, device="cuda"), out3, scratch, scale=scale, window=size,
                        plan=plan, counters=counters, form=form)
        err = float((out3.cpu().double().view(nh, vd) - want[last]).abs().max())
        assert err < tol * float(want.abs().max()), ("decode", plan.kind, last, err)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("nh,dim,rdim,rank", [(3, 16, 8, 24), (5, 40, 0, 33), (2, 8, 64, 100)])
def test_latent_preparation_and_per_head_products(llogos, dtype, nh, dim, rdim, rank):
    ops = ops_module()
    g = torch.Generator().manual_seed(nh + rank)
    n, eps, base = 70, 1e-5, 900.0
    width = nh * (dim + rdim) + rank + rdim
    x = torch.randn((3, n, width), generator=g)
    cw = (1 + 0.3 * torch.randn((rank,), generator=g)).to(dtype)
    pos = torch.arange(30, 30 + n)
    z = x.double().sum(0)
    qz = z[:, :nh * (dim + rdim)].view(n, nh, dim + rdim)
    want_c = FP.rms_norm(z[:, nh * (dim + rdim):nh * (dim + rdim) + rank], cw.float(), eps)
    cos = sin = None
    want_qr, want_kr = qz[..., dim:], z[:, nh * (dim + rdim) + rank:]
    if rdim:
        want_qr = FP.rotate_halves(qz[..., dim:], pos, rdim, base)
        want_kr = FP.rotate_halves(want_kr[:, None], pos, rdim, base)[:, 0]
        i = torch.arange(rdim // 2, dtype=torch.float64)
        ang = torch.arange(128, dtype=torch.float64)[:, None] * (base ** (-2 * i / rdim))[None]
        cos, sin = torch.cos(ang).float().cuda(), torch.sin(ang).float().cuda()
    kd = rank + rdim
    q_plain = torch.empty((n, nh, dim), dtype=dtype, device="cuda")
    q = torch.zeros((n, nh, kd), dtype=dtype, device="cuda")
    k_new = torch.empty((n, 1, kd), dtype=dtype, device="cuda")
    v_new = torch.empty((n, 1, rank), dtype=dtype, device="cuda")
    kp = torch.zeros((4, 1, 64, kd), dtype=dtype, device="cuda")
    vp = torch.zeros((4, 1, 64, rank), dtype=dtype, device="cuda")
    table = torch.tensor([[3, 1]], dtype=torch.int32, device="cuda")
    ops.latent_prep(x.cuda(), n_heads=nh, head_dim=dim, rot_dim=rdim, kv_rank=rank, c_norm_w=cw.cuda(), norm_eps=eps, cos=cos,
                    sin=sin, positions=pos.int().cuda(), q_plain_out=q_plain, q_out=q, k_new=k_new, v_new=v_new, k_pages=kp,
                    v_pages=vp, page_table=table, ring_pages=2, seq_of_token=torch.zeros(n, dtype=torch.int32, device="cuda"),
                    slots=torch.zeros(1, dtype=torch.int32, device="cuda"))
    tol = 3e-6 if dtype == torch.float32 else 8e-3
    want_k = torch.cat([want_c, want_kr], -1)
    for got, want in ((q_plain, qz[..., :dim]), (q[..., rank:], want_qr), (k_new[:, 0], want_k), (v_new[:, 0], want_c)):
        if want.numel():
            assert float((got.cpu().double() - want).abs().max()) < tol * float(want.abs().max())
    assert float(q[..., :rank].abs().max()) == 0.0                      # that part is the per-head product's to fill
    for j in range(n):
        p = 30 + j
        assert torch.equal(kp[[3, 1][p // 64], 0, p % 64], k_new[j, 0]) and torch.equal(vp[[3, 1][p // 64], 0, p % 64], v_new[j, 0])
    # per-head products into a part of wider rows, and out of one
    w = (torch.randn((nh, rank, dim), generator=g) / math.sqrt(dim)).to(dtype)
    ops.head_linear(q_plain, w.cuda(), q[:, :, :rank])
    want = torch.einsum("nha,hba->nhb", q_plain.cpu().double(), w.double())
    assert float((q[..., :rank].cpu().double() - want).abs().max()) < tol * float(want.abs().max())
    if rdim:
        assert float((q[..., rank:].cpu().double() - want_qr).abs().max()) < tol * float(want_qr.abs().max())   # untouched
    w2 = (torch.randn((nh, 7, rank), generator=g) / math.sqrt(rank)).to(dtype)
    y = torch.empty((n, nh, 7), dtype=dtype, device="cuda")
    ops.head_linear(q[:, :, :rank], w2.cuda(), y)
    want2 = torch.einsum("nha,hba->nhb", q[..., :rank].cpu().double(), w2.double())
    assert float((y.cpu().double() - want2).abs().max()) < tol * float(want2.abs().max())


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("n,hidden,n_exp,top,ff", [(1, 40, 3, 3, 10), (9, 72, 5, 2, 24), (300, 96, 16, 4, 40), (50, 100, 70, 1, 8),
                                                   (700, 192, 6, 2, 136)])
def test_expert_kernels(llogos, dtype, n, hidden, n_exp, top, ff):
    """Routing against the plain router; the layout's invariants; the grouped products and the weighted sum against the
    plain mixture given the same choices."""
    ops = ops_module()
    g = torch.Generator().manual_seed(n + n_exp)
    x = torch.randn((n, hidden), generator=g).to(dtype)
    w = {"m.router": 2 * torch.randn((n_exp, hidden), generator=g) / math.sqrt(hidden), "m.router.b": torch.randn((n_exp,), generator=g)}
    for e in range(n_exp):
        w[f"m.e{e}.gate"] = (torch.randn((ff, hidden), generator=g) / math.sqrt(hidden)).to(dtype).float()
        w[f"m.e{e}.up"] = (torch.randn((ff, hidden), generator=g) / math.sqrt(hidden)).to(dtype).float()
        w[f"m.e{e}.down"] = (torch.randn((hidden, ff), generator=g) / math.sqrt(ff)).to(dtype).float()
    idx, wt, margin = FP.route(x.float(), w, "m.", top)
    choice = torch.empty((n, top), dtype=torch.int32, device="cuda")
    weight = torch.empty((n, top), dtype=torch.float32, device="cuda")
    ops.moe_route(x.cuda(), w["m.router"].cuda(), w["m.router.b"].cuda(), choice, weight)
    sure = margin > 1e-4
    assert torch.equal(choice.cpu().long()[sure], idx[sure]), "the chosen experts, largest logit first"
    assert float((weight.cpu().double()[sure] - wt[sure]).abs().max()) < 1e-5
    # the same choice from logits that a product left as partial sums (here: the two halves of the sum over the width)
    half = hidden // 2
    parts = torch.stack([x.float()[:, :half] @ w["m.router"][:, :half].t(), x.float()[:, half:] @ w["m.router"][:, half:].t()])
    choice2 = torch.empty_like(choice)
    weight2 = torch.empty_like(weight)
    ops.moe_topk(parts.cuda().contiguous(), w["m.router.b"].cuda(), choice2, weight2)
    assert torch.equal(choice2.cpu().long()[sure], idx[sure])
    assert float((weight2.cpu().double()[sure] - wt[sure]).abs().max()) < 1e-5
    # the layout: every pair has a row of its own inside its expert's tiles
    cap = ops.moe_row_capacity(n * top, n_exp)
    row_of_pair = torch.empty((n * top,), dtype=torch.int32, device="cuda")
    token_of_row = torch.empty((cap,), dtype=torch.int32, device="cuda")
    tile_expert = torch.empty((cap // ops.MOE_TILE_ROWS,), dtype=torch.int32, device="cuda")
    ops.moe_plan(choice, n_exp, row_of_pair, token_of_row, tile_expert)
    rows, tok, tile = row_of_pair.cpu().long(), token_of_row.cpu().long(), tile_expert.cpu().long()
    assert len(set(rows.tolist())) == n * top
    flat = choice.cpu().long().reshape(-1)
    assert torch.equal(tile[rows // ops.MOE_TILE_ROWS], flat) and torch.equal(tok[rows], torch.arange(n * top) // top)
    assert int((tok >= 0).sum()) == n * top
    # the experts' two products and the weighted sum
    act = torch.empty((cap, ff), dtype=dtype, device="cuda")
    stack = lambda what: torch.stack([w[f"m.e{e}.{what}"] for e in range(n_exp)]).to(dtype).cuda()
    pad = -(-ff // 128) * 128
    gate_up = torch.zeros((n_exp, 2 * pad, hidden), dtype=dtype, device="cuda")       # the gated layout, expert by expert
    gate_up[:, :ff], gate_up[:, pad:pad + ff] = stack("gate"), stack("up")
    ops.moe_gated(x.cuda(), token_of_row, tile_expert, gate_up, act)
    y = torch.empty((cap, hidden), dtype=torch.float32, device="cuda")
    ops.moe_down(act, tile_expert, stack("down"), y)
    if dtype == torch.bfloat16 and hidden % 8 == 0 and ff % 8 == 0:
        # the same through the layout of 128-row tiles: gathered rows, grouped tcgen05 products
        cap2 = ops.moe_row_capacity(n * top, n_exp, ops.MOE_TC_TILE_ROWS)
        rop2 = torch.empty((n * top,), dtype=torch.int32, device="cuda")
        tor2 = torch.empty((cap2,), dtype=torch.int32, device="cuda")
        te2 = torch.empty((cap2 // ops.MOE_TC_TILE_ROWS,), dtype=torch.int32, device="cuda")
        ops.moe_plan(choice, n_exp, rop2, tor2, te2)
        rows2 = torch.empty((cap2, hidden), dtype=dtype, device="cuda")
        ops.moe_gather_rows(x.cuda(), tor2, rows2)
        act2 = torch.full((cap2, ff), 7.0, dtype=dtype, device="cuda")
        ops.moe_gated(rows2, None, te2, gate_up, act2)
        y2 = torch.full((cap2, hidden), 7.0, dtype=torch.float32, device="cuda")
        ops.moe_down(act2, te2, stack("down"), y2)
        assert ops.gemm_tc_status() == 0
        a1, a2 = act[row_of_pair.long()].float(), act2[rop2.long()].float()
        assert float((a1 - a2).abs().max()) <= 2e-2 * float(a1.abs().max())
        y1, y2r = y[row_of_pair.long()], y2[rop2.long()]
        assert float((y1 - y2r).abs().max()) <= 2e-2 * float(y1.abs().max())
        y, row_of_pair = y2, rop2                          # the weighted sum below then checks this path against the plain one
    shared = torch.randn((2, n, hidden), generator=g)
    out = torch.empty((n, hidden), dtype=torch.float32, device="cuda")
    ops.moe_combine(y, row_of_pair, weight, shared.cuda(), out)
    want = shared.double().sum(0)
    wc, cc = weight.cpu().double(), choice.cpu().long()
    for i in range(n):
        for j in range(top):
            want[i] += wc[i, j] * FP.expert(x[i:i + 1].float(), w, f"m.e{int(cc[i, j])}.")[0]
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert float((out.cpu().double() - want).abs().max()) < tol * float(want.abs().max())


# ---- whole models ------------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("name", list(FM.CONFIGS))
def test_whole_prompt_and_first_tokens(engines, models, name, dtype):
    eng = engines(name, dtype)
    cfg = models[name, dtype][1]
    for n in (1, 2, 3, 190):
        toks = tokens_for(cfg, n, n)
        ref = plain(models, name, dtype, toks)
        slot = eng.open()
        lg = eng.step([(slot, toks)], [list(range(n))])
        close(lg, ref, dtype, (name, "whole", n))
        eng.close(slot)
    eng.cache.audit()


def test_a_long_prompt_takes_the_experts_through_the_grouped_tensor_core_product(engines, models):
    """900 tokens in one step: enough (token, choice) pairs that the bfloat16 experts run on tiles of 128 rows; the same
    prompt in portions of 200 (small tiles) and token by token at its end give the same logits within the bound."""
    from importlib import import_module
    ops = import_module("daisi-llogos_b200.kernels.ops")
    name, dtype = "tensor", torch.bfloat16
    cfg = models[name, dtype][1]
    ml = cfg["layers"][0]["mlp"]
    assert ops.moe_tile_rows(dtype, 900 * ml["router"]["top"], ml["router"]["experts"], cfg["width"], ml["expert"]["ff"]) == ops.MOE_TC_TILE_ROWS
    eng = engines(name, dtype)
    toks = tokens_for(cfg, 900, 31)
    ref = plain(models, name, dtype, toks)
    want = list(range(0, 900, 7)) + [899]
    slot = eng.open()
    lg = eng.step([(slot, toks)], [want])
    close(lg, ref[want], dtype, ("long prompt",))
    eng.close(slot)
    assert ops.gemm_tc_status() == 0
    slot = eng.open()
    got = [eng.step([(slot, toks[a:a + 200])], [list(range(len(toks[a:a + 200])))]).clone() for a in range(0, 900, 200)]
    close(torch.cat(got), ref, dtype, ("long prompt in portions",))
    eng.close(slot)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_residual_after_every_layer(llogos, models, dtype):
    """The float32 residual stream after each layer, read from the engine by running models cut after 1, 2, ... layers
    (their final norm made the identity) is what the plain model's trace holds."""
    name = "mixed"
    d, cfg, w = models[name, dtype]
    toks = tokens_for(cfg, 50, 4)
    trace = []
    FP.forward(w, cfg, toks, trace=trace)
    import os
    for depth in (1, 2, 4, len(cfg["layers"])):
        cut = dict(cfg, layers=cfg["layers"][:depth])
        keep = {k: v for k, v in w.items() if not (k.startswith("l") and int(k[1:k.index(".")]) >= depth)}
        sub = os.path.join(d, f"cut{depth}")
        FM.write_model(llogos, sub, cut, 0, weights={k: v.to(torch.bfloat16) for k, v in keep.items()})
        model = llogos.weights.load_model(sub, dtype=dtype, device="cuda:0")
        eng = llogos.engine.Engine(model, max_tokens=256)
        slot = eng.open()
        lg = eng.step([(slot, toks)], [list(range(len(toks)))])
        ref = FP.linear(FP.layer_norm(trace[depth - 1], w["final.norm"], w["final.norm.b"], cfg["norm"]["eps"]), w["embed"])
        close(lg, ref, dtype, ("after layer", depth))
        eng.close(slot)


@pytest.mark.parametrize("graphs", [True, False], ids=["graph", "eager"])
@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("name", list(FM.CONFIGS))
def test_prompt_then_token_by_token(engines, models, name, dtype, graphs):
    """The decoded positions pass page borders (128, 192) and every chunk's and window's edge; the first token alone too."""
    eng = engines(name, dtype, graphs)
    cfg = models[name, dtype][1]
    toks = tokens_for(cfg, 215, 7)
    ref = plain(models, name, dtype, toks)
    for cut in (1, 120):
        slot = eng.open()
        lg = eng.step([(slot, toks[:cut])])
        close(lg, ref[cut - 1:cut], dtype, (name, "prompt end", cut))
        got = [eng.step([(slot, [toks[p]])]).clone() for p in range(cut, len(toks) if cut > 1 else 40)]
        close(torch.cat(got), ref[cut:cut + len(got)], dtype, (name, "decoded from", cut))
        eng.close(slot)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("name", list(FM.CONFIGS))
def test_portions_of_several_sizes(engines, models, name, dtype):
    eng = engines(name, dtype)
    cfg = models[name, dtype][1]
    toks = tokens_for(cfg, 300, 9)
    ref = plain(models, name, dtype, toks)
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
@pytest.mark.parametrize("name", list(FM.CONFIGS))
def test_unequal_batches_with_slots_and_pages_used_again(engines, models, name, dtype):
    eng = engines(name, dtype)
    cfg = models[name, dtype][1]
    seqs = [tokens_for(cfg, n, 20 + n) for n in (1, 66, 140, 259, 33)]
    refs = [plain(models, name, dtype, s) for s in seqs]
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


def _random_config(seed):
    """A configuration drawn from the seed: two to five layers of either kind in any order, sizes, masks, rotations, expert
    counts and the residual factor all drawn; layers that blend values agree in their values' shape, as they must."""
    g = torch.Generator().manual_seed(1000 + seed)
    pick = lambda xs: xs[int(torch.randint(0, len(xs), (1,), generator=g))]
    width = pick([40, 64, 72, 96, 136])
    kv_blend, vdim_blend = pick([1, 2, 3]), pick([8, 16, 24, 40])
    layers = []
    for _ in range(pick([2, 3, 4, 5])):
        mlp = None if pick([0, 0, 0, 1]) else FM.moe(pick([2, 3, 5, 9]), 1, pick([8, 24, 40]), pick([0, 16, 56]))
        if mlp:
            mlp["router"]["top"] = pick(list(range(1, mlp["router"]["experts"] + 1)))
        if pick([0, 1]):
            dim = pick([8, 16, 24, 32, 64])
            blend = bool(pick([0, 1]))
            kv = kv_blend if blend else pick([1, 2, 4])
            mix = FM.attention(kv * pick([1, 2, 3]), kv, dim, vdim_blend if blend else pick([8, dim, 48]), pick([1, 3, 17, 64, 65, 150]),
                               pick([d for d in (2, 4, 8, 16, 32, 64) if d <= dim]), base=pick([50.0, 10000.0, 3e6]), v_mix=blend,
                               scale=pick([0.05, 0.2, 0.5]))
        else:
            rot = pick([2, 4, 8, 16, 32])
            mix = FM.latent(pick([1, 2, 3, 5, 8]), pick([8, 16, 40]), rot, pick([8, 24, 32]), pick([8, 16, 30, 64, 112]),
                            pick([1, 2, 31, 64, 100, 160]), base=pick([50.0, 10000.0, 3e6]), scale=pick([0.05, 0.2, 0.5]))
        layers.append(FM.layer(mix, mlp))
    return FM.config(layers, vocab=pick([61, 128, 257]), width=width, mult=pick([0.25, 0.6, 1.0, 1.3]), eps=pick([1e-6, 1e-5, 1e-3]))


@pytest.mark.parametrize("seed", range(10))
def test_configurations_drawn_at_random(llogos, tmp_path, seed):
    """float32: a prompt whole, a batch of two unequal prompts decoded together for a dozen steps, against the plain model."""
    cfg = _random_config(seed)
    d = str(tmp_path / "m")
    w = {k: v.float() for k, v in FM.write_model(llogos, d, cfg, seed=seed).items()}
    model = llogos.weights.load_model(d, dtype=torch.float32, device="cuda:0")
    eng = llogos.engine.Engine(model, max_tokens=64 * 12)
    seqs = [tokens_for(cfg, n, seed * 7 + n) for n in (171, 40)]
    refs = [FP.forward(w, cfg, s) for s in seqs]
    slot = eng.open()
    close(eng.step([(slot, seqs[0])], [list(range(len(seqs[0])))]), refs[0], torch.float32, ("random", seed, "whole"))
    eng.close(slot)
    slots = [eng.open(), eng.open()]
    cut = [len(s) - 12 for s in seqs]
    lg = eng.step([(sl, s[:c]) for sl, s, c in zip(slots, seqs, cut)])
    for i in range(2):
        close(lg[i], refs[i][cut[i] - 1], torch.float32, ("random", seed, "prompt", i))
    for k in range(12):
        lg = eng.step([(sl, [s[c + k]]) for sl, s, c in zip(slots, seqs, cut)])
        for i in range(2):
            close(lg[i], refs[i][cut[i] + k], torch.float32, ("random", seed, "decode", i, k))
    for sl in slots:
        eng.close(sl)
    eng.cache.audit()


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_long_decoding_round_the_rings(engines, models, dtype):
    """420 decoded tokens after a prompt of 30: the smallest masks' rings of pages go round several times."""
    name = "mixed"
    eng = engines(name, dtype)
    cfg = models[name, dtype][1]
    toks = tokens_for(cfg, 450, 5)
    ref = plain(models, name, dtype, toks)
    slot = eng.open()
    eng.step([(slot, toks[:30])], [[]])
    got = [eng.step([(slot, [toks[p]])]).clone() for p in range(30, len(toks))]
    close(torch.cat(got), ref[30:], dtype, ("long decoding",))
    eng.close(slot)


def _edge_model(llogos, folder, kind, size):
    """One layer without feed-forward whose key projection is made so that token a's key matches token b's query
    strongly (b's embedding is a's with its coordinates permuted, the key matrix is the first head's query matrix with
    its columns permuted the same way; the per-head norms keep directions; no rotation, so that the match does not hang
    on the distance)."""
    if kind == "attention":
        lay = FM.layer(FM.attention(2, 1, 32, 24, size, 2, scale=1.0), None)
        lay["mixer"]["rot"]["base"] = 1e30                         # the one rotated pair turns by next to nothing
    else:
        lay = FM.layer(FM.latent(2, 32, 2, 24, 32, size, scale=1.0), None)
        lay["mixer"]["rot"]["base"] = 1e30
    cfg = FM.config([lay], vocab=50, width=48, mult=0.9)
    w = FM.random_weights(cfg, 77)
    a_tok, b_tok = 11, 12
    gen = torch.Generator().manual_seed(1)
    perm = torch.randperm(48, generator=gen)
    w["embed"][a_tok] = (2 * torch.randn(48, generator=gen)).to(torch.bfloat16)
    w["embed"][b_tok] = w["embed"][a_tok][perm]
    w["l0.norm1"][:] = 1.0
    w["l0.norm1.b"][:] = 0.0
    w["l0.mix.sink"][:] = -2.0
    w["l0.mix.o"] *= 4.0                                               # what the heads find weighs on the logits
    if kind == "attention":
        w["l0.mix.k"][:, perm] = w["l0.mix.q"][:32]
        w["l0.mix.k.norm"][:] = w["l0.mix.q.norm"]
    else:
        # the latent is the (normed) down projection; the first head's keys are W_uk c: make W_uk the identity there and
        # the down projection the first head's unrotated query rows, permuted
        w["l0.mix.dkv"][:32][:, perm] = w["l0.mix.q"][:32]
        w["l0.mix.dkv.norm"][:] = 1.0
        w["l0.mix.uk"][:32] = (3.0 * torch.eye(32)).to(torch.bfloat16)
    FM.write_model(llogos, folder, cfg, 0, weights=w)
    return cfg, {k: v.float() for k, v in w.items()}, a_tok, b_tok


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("kind", ["attention", "latent_attention"])
def test_a_key_that_stands_out_at_every_masks_edge(llogos, tmp_path, dtype, kind):
    """Token a stands once just inside and once just outside what the b that asks for it sees (the first position of
    b's chunk and the one before; the first of the last `size` positions and the one before), in a prompt and in decoding:
    the logits there differ widely between the two, and must follow the plain model in both."""
    size = 67
    d = str(tmp_path / "edge")
    cfg, wf, a_tok, b_tok = _edge_model(llogos, d, kind, size)
    model = llogos.weights.load_model(d, dtype=dtype, device="cuda:0")
    eng = llogos.engine.Engine(model, max_tokens=64 * 8)
    g = torch.Generator().manual_seed(2)
    cases = []                                          # (a's position, b's position that still sees it, one that does not)
    if kind == "attention":
        cases = [(size, 2 * size - 1, 2 * size), (2 * size, 2 * size + 1, 3 * size), (0, 64, size)]
    else:
        cases = [(0, size - 1, size), (61, 61 + size - 1, 61 + size), (64, 64 + size - 1, 64 + size)]
    for a_at, inside, outside in cases:
        toks = torch.randint(13, 50, (outside + 3,), generator=g).tolist()
        toks[a_at] = a_tok
        for b_at in (inside, outside):
            t = list(toks)
            t[b_at] = b_tok
            ref = FP.forward(wf, cfg, t)
            for cut in (len(t), b_at):                 # b inside the prompt; b decoded alone
                slot = eng.open()
                lg = eng.step([(slot, t[:cut])], [[b_at] if b_at < cut else []])
                if b_at >= cut:
                    lg = eng.step([(slot, [t[b_at]])])
                close(lg, ref[b_at:b_at + 1], dtype, ("edge", kind, a_at, b_at, cut))
                eng.close(slot)
        t_in, t_out = list(toks), list(toks)
        t_in[inside], t_out[outside] = b_tok, b_tok
        r_in, r_out = FP.forward(wf, cfg, t_in)[inside], FP.forward(wf, cfg, t_out)[outside]
        assert float((r_in - r_out).abs().max()) > 0.15 * float(r_in.abs().max())


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("kind", ["attention", "latent_attention"])
def test_a_far_key_among_hundreds(llogos, tmp_path, dtype, kind):
    """The same construction with a mask of 400 positions: token a stands at position 2, token b 330 positions later
    (five pages on); b's logits with a there and with another token in a's place are far apart, in a prompt and decoded."""
    d = str(tmp_path / "far")
    cfg, wf, a_tok, b_tok = _edge_model(llogos, d, kind, 400)
    model = llogos.weights.load_model(d, dtype=dtype, device="cuda:0")
    eng = llogos.engine.Engine(model, max_tokens=64 * 8)
    gen = torch.Generator().manual_seed(3)
    toks = torch.randint(13, 50, (336,), generator=gen).tolist()
    b_at = 332
    toks[b_at] = b_tok
    with_a, without_a = list(toks), list(toks)
    with_a[2] = a_tok
    refs = [FP.forward(wf, cfg, t) for t in (with_a, without_a)]
    assert float((refs[0][b_at] - refs[1][b_at]).abs().max()) > 0.1 * float(refs[0][b_at].abs().max())
    for t, ref in zip((with_a, without_a), refs):
        for cut in (len(t), b_at):
            slot = eng.open()
            lg = eng.step([(slot, t[:cut])], [[b_at] if b_at < cut else []])
            if b_at >= cut:
                lg = eng.step([(slot, [t[b_at]])])
            close(lg, ref[b_at:b_at + 1], dtype, ("far key", kind, cut))
            eng.close(slot)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_greedy_generation_through_the_entry_point(models, dtype):
    """``LlogosModel.generate`` (scheduler, sampler, run-ahead decoding) makes the plain model's best tokens."""
    import llogos_b200 as L
    name = "mixed"
    d, cfg, w = models[name, dtype]
    model = L.LlogosModel.load(d, dtype=dtype, max_context=256, max_batch=3)
    prompts = [tokens_for(cfg, n, 60 + n) for n in (5, 70, 23, 1)]
    out = model.generate(prompts, L.GenerationParams.greedy_params(12, stop_tokens=()))
    for p, made in zip(prompts, out.tokens):
        assert len(made) == 12
        toks = list(p)
        for tok in made:
            lg = FP.forward(w, cfg, toks)[-1]
            slack = 1e-4 if dtype == torch.float32 else 0.05
            assert float(lg[tok]) >= float(lg.max()) - slack * float(lg.abs().max()), (len(toks), tok)
            toks.append(tok)


def test_command_line_and_trace_replay_take_the_design(models, tmp_path):
    """``python -m llogos_b200`` generates and benchmarks a Fipavik folder, and ``bin/trace_run`` replays steps on it
    (a prompt in two portions beside a second request, then decoding together), as they do for every model."""
    import json
    import os
    import subprocess
    import sys
    import numpy as np
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    d, cfg, w = models["tensor", torch.float32]
    env = dict(os.environ, PYTHONPATH=root)
    base = [sys.executable, "-m", "llogos_b200", "--model", d, "--dtype", "float32"]
    p = subprocess.run(base + ["--prompt-ids", "5,17,3", "-n", "6", "-t", "0", "--repeat-penalty", "1.0", "--max-context", "128"],
                       capture_output=True, text=True, env=env, cwd=root)
    assert p.returncode == 0, p.stderr
    made = [int(x) for x in p.stdout.split()]
    toks = [5, 17, 3]
    for tok in made:
        lg = FP.forward(w, cfg, toks)[-1]
        assert float(lg[tok]) >= float(lg.max()) - 1e-4 * float(lg.abs().max())
        toks.append(tok)
    p = subprocess.run(base + ["--bench", "--batch", "2", "--prompt-len", "20:40", "--context", "80", "--seed", "1"],
                       capture_output=True, text=True, env=env, cwd=root)
    assert p.returncode == 0 and "Decode step:" in p.stderr and "Prompt step:" in p.stderr, p.stderr
    d, cfg, w = models["tensor", torch.bfloat16]
    a, b = tokens_for(cfg, 100, 1), tokens_for(cfg, 31, 2)
    ra, rb = plain(models, "tensor", torch.bfloat16, a), plain(models, "tensor", torch.bfloat16, b)
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
