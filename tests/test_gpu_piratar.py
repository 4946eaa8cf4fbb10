"""The Piratar decoder on the GPU against the plain implementation in piratar_plain.py, in float32 and bfloat16:
every mechanism's kernel alone; whole prompts; prompts against token-by-token decoding; prompts in portions down to two
tokens; batches of unequal requests against each alone, with slots, pages and state rows used again; a far key among
hundreds and across page borders; states written long ago in both recurrent mixers; the first tokens; long decoding; sizes
that differ from layer to layer; greedy generation through the library's entry point."""
import math

import pytest
import torch

import piratar_models as PM
import piratar_plain as PP

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]
IDS = ["f32", "bf16"]
F64 = torch.float64

# float32: every logit within 1e-4 of the request's largest |logit|.  bfloat16, relative to the root mean square of all
# compared logits: the root-mean-square error of every position within 1e-1 and of the positions on average within
# 3.5e-2, every logit within 1.5e-1 of the largest.  The models of one layer that are made to show a fault (TIGHT) stay
# within 2.5e-2 and 5e-2.
TOL = {torch.float32: (1e-4, 1e-4, 1e-4), torch.bfloat16: (1e-1, 3.5e-2, 1.5e-1)}
TIGHT = {torch.float32: (1e-4, 1e-4, 1e-4), torch.bfloat16: (2.5e-2, 2.5e-2, 5e-2)}
MARGIN = 0.01          # bfloat16: no router of a compared sequence decides by less than this (in score)


def ops_module():
    from importlib import import_module
    return import_module("daisi-llogos_b200.kernels.ops")


def close(got, ref, dtype, what=(), tol=TOL):
    got = got.detach().to("cpu", F64).reshape(ref.shape)
    rms_tol, mean_tol, max_tol = tol[dtype]
    per_position = (got - ref).pow(2).mean(-1).sqrt() / ref.pow(2).mean().sqrt()
    rms, mean = float(per_position.max()), float(per_position.mean())
    worst = float((got - ref).abs().max() / ref.abs().max())
    if per_position.numel() < 16:
        mean_tol = rms_tol
    assert rms <= rms_tol and mean <= mean_tol and worst <= max_tol, (*what, "rms", rms, "mean", mean, "max", worst)


def near(got, ref, tol, what=""):
    err = float((got.detach().to("cpu", F64) - ref.to(F64)).abs().max() / max(1.0, float(ref.abs().max())))
    assert err <= tol, (what, err)


@pytest.fixture(scope="module")
def models(llogos, tmp_path_factory):
    """(name, dtype) -> (folder, config, weights as float tensors); bfloat16 takes routers that read a code of the token
    (``steady_routing``), float32 routers that hang on everything."""
    out = {}
    for i, (name, cfg) in enumerate(PM.CONFIGS.items()):
        for dtype in DTYPES:
            d = str(tmp_path_factory.mktemp(f"piratar_{name}_{IDS[DTYPES.index(dtype)]}"))
            w = PM.write_model(llogos, d, cfg, seed=270 + i, steady_routing=dtype == torch.bfloat16)
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


_refs, _tokens, _pools = {}, {}, {}


def sequence(models, name, dtype, n, seed):
    """(tokens, plain logits) of a random sequence.  In bfloat16 the sequence is drawn again, without the tokens that met a
    close call in a router, until no router decides by less than ``MARGIN``."""
    key = (name, dtype, n, seed)
    if key in _tokens:
        return _tokens[key], _refs[key]
    _, cfg, w = models[name, dtype]
    pool = _pools.setdefault((name, dtype), list(range(cfg["vocab"])))
    for attempt in range(40):
        g = torch.Generator().manual_seed(seed * 1000 + attempt)
        toks = [pool[i] for i in torch.randint(0, len(pool), (n,), generator=g).tolist()]
        margins = []
        ref = PP.forward(w, cfg, toks, margins=margins)
        if dtype != torch.bfloat16 or not margins:
            break
        worst = torch.stack(margins).min(0).values
        if float(worst.min()) > MARGIN:
            break
        bad = {toks[i] for i in torch.nonzero(worst <= 1.5 * MARGIN).flatten().tolist()}
        pool[:] = [t for t in pool if t not in bad]
        assert len(pool) > 20, "too few tokens are left whose routing is steady"
    else:
        raise AssertionError("no sequence without a close call in a router was found")
    _tokens[key], _refs[key] = toks, ref
    return toks, ref


def layout(counts, before, slots):
    """Device tensors of a step's packed layout: (slots, cu_tokens, seq_of_token, len_before, positions)."""
    I = lambda xs: torch.tensor(list(xs), dtype=torch.int32, device="cuda")
    cu = [0]
    for c in counts:
        cu.append(cu[-1] + c)
    seq = [b for b, c in enumerate(counts) for _ in range(c)]
    pos = [p for lb, c in zip(before, counts) for p in range(lb, lb + c)]
    return I(slots), I(cu), I(seq), I(before), I(pos)


# ---- mechanisms alone --------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("hidden", [72, 90, 100, 1024, 4100])
def test_residual_add_of_normed_terms_and_two_norms_of_the_sum(dtype, hidden):
    ops = ops_module()
    g = torch.Generator().manual_seed(hidden)
    n = 9
    res = torch.randn(n, hidden, generator=g)
    t1, t2, t3 = (torch.randn(s, n, hidden, generator=g) for s in (2, 1, 3))
    w1, w3 = torch.randn(hidden, generator=g), torch.randn(hidden, generator=g)
    o1, o2 = 0.1 * torch.randn(hidden, generator=g), torch.randn(hidden, generator=g)
    want = res.double() + 0.5 * PP.norm_plain(t1.double().sum(0), w1, 1e-5) + t2.double().sum(0) - 2.0 * PP.norm_plain(t3.double().sum(0), w3, 1e-3)
    for rows in (None, [7, 0, 3]):
        idx = slice(None) if rows is None else rows
        m = n if rows is None else len(rows)
        dev = res.clone().cuda()
        a, b = torch.empty(m, hidden, dtype=dtype, device="cuda"), torch.empty(m, hidden, dtype=dtype, device="cuda")
        ops.multi_add_rmsnorm(dev, [(t1.cuda(), w1.cuda(), 1e-5, 0.5), (t2.cuda(), None, 0.0, 1.0), (t3.cuda(), w3.cuda(), 1e-3, -2.0)],
                              [(a, o1.cuda(), 1.0), (b, o2.cuda(), 0.0)], 1e-6,
                              None if rows is None else torch.tensor(rows, dtype=torch.int32, device="cuda"))
        tol = 1e-5 if dtype == torch.float32 else 1e-2
        near(dev[idx], want[idx], 1e-5, "sum")
        near(a, PP.norm_one_plus(want[idx], o1, 1e-6), tol, "first norm")
        near(b, PP.norm_plain(want[idx], o2, 1e-6), tol, "second norm")
        if rows is not None:
            rest = [i for i in range(n) if i not in rows]
            assert torch.equal(dev[rest].cpu(), res[rest])               # rows nobody asked for are left alone
    raw = torch.empty(n, hidden, dtype=dtype, device="cuda")
    dev = res.clone().cuda()
    ops.multi_add_rmsnorm(dev, [(t2.cuda(), None, 0.0, 1.0)], [(raw, None, 0.0)], 1e-6)
    near(raw, res.double() + t2.double().sum(0), 1e-6 if dtype == torch.float32 else 1e-2, "the sum as it is")


@pytest.mark.parametrize("table_dtype", DTYPES, ids=IDS)
def test_pair_embedding_carries_the_token_before_through_steps_and_slots(table_dtype):
    ops = ops_module()
    g = torch.Generator().manual_seed(1)
    vocab, hidden, buckets = 61, 40, 23
    cfg = {"embedding": {"scale": 3.0, "bigram": {"buckets": buckets, "mul_prev": 37, "mul_cur": 11}}}
    w = {"embed": torch.randn(vocab, hidden, generator=g).to(table_dtype), "bigram": torch.randn(buckets + 1, hidden, generator=g).to(table_dtype)}
    nw = 0.1 * torch.randn(hidden, generator=g)
    seqs = [torch.randint(0, vocab, (n,), generator=g).tolist() for n in (9, 1, 14)]
    refs = [PP.norm_one_plus(PP.embed(w, cfg, s), nw, 1e-5) for s in seqs]
    state = torch.full((6, 1), 7, dtype=torch.int32, device="cuda")       # what an earlier owner of the slots left
    slots, at = [4, 0, 2], [0, 0, 0]
    for counts in ([3, 1, 1], [1, 0, 2], [5, 0, 1], [0, 0, 10]):
        live = [b for b in range(3) if counts[b]]
        toks = [t for b in live for t in seqs[b][at[b]:at[b] + counts[b]]]
        sl, cu, seq, lb, pos = layout([counts[b] for b in live], [at[b] for b in live], [slots[b] for b in live])
        out = torch.empty(len(toks), hidden, device="cuda")
        ops.hash_embed(w["embed"].cuda(), 3.0, w["bigram"].cuda(), buckets, 37, 11, torch.tensor(toks, dtype=torch.int32, device="cuda"),
                       pos, seq, cu, sl, state, nw.cuda(), 1.0, 1e-5, out)
        o = 0
        for b in live:
            near(out[o:o + counts[b]], refs[b][at[b]:at[b] + counts[b]], 1e-5, ("pair embedding", b, at[b]))
            o += counts[b]
            at[b] += counts[b]
    assert [int(state[s]) for s in slots] == [seqs[0][-1], seqs[1][-1], seqs[2][-1]]


@pytest.mark.parametrize("taps", [1, 2, 4, 7])
def test_convolution_keeps_its_last_inputs_between_steps(taps):
    """Steps of one token, of fewer tokens than taps, and long ones; three sequences whose steps differ; a slot whose
    state an earlier sequence left."""
    ops = ops_module()
    g = torch.Generator().manual_seed(taps)
    c, lead = 37, 5
    seqs = [torch.randn(n, c, generator=g) for n in (40, 3, 21)]
    wt, ib, ob = torch.randn(c, taps, generator=g), torch.randn(c, generator=g), torch.randn(c, generator=g)
    refs = [PP.causal_conv(s + ib, wt, ob) for s in seqs]
    state = torch.randn(5, max(taps - 1, 1), c, generator=g)[:, :taps - 1].contiguous().cuda() if taps > 1 else None
    slots, at = [3, 1, 0], [0, 0, 0]
    if state is not None:
        state[slots] = 0                                         # the cache zeroes a slot's state when a sequence starts
    for counts in ([1, 1, 2], [2, 2, 1], [30, 0, 1], [1, 0, 9], [6, 0, 8]):
        live = [b for b in range(3) if counts[b]]
        x = torch.cat([seqs[b][at[b]:at[b] + counts[b]] for b in live])
        rows = torch.zeros(2, x.shape[0], lead + c + 3)
        rows[0, :, lead:lead + c] = 0.25 * x
        rows[1, :, lead:lead + c] = 0.75 * x
        sl, cu, seq, lb, _ = layout([counts[b] for b in live], [at[b] for b in live], [slots[b] for b in live])
        out = torch.empty(x.shape[0], c, device="cuda")
        out2 = torch.empty(x.shape[0], c, device="cuda", dtype=torch.bfloat16)
        ops.causal_conv(rows.cuda(), lead, wt.cuda(), state, sl, cu, seq, lb, out, in_bias=ib.cuda(), bias=ob.cuda(), out2=out2)
        o = 0
        for b in live:
            near(out[o:o + counts[b]], refs[b][at[b]:at[b] + counts[b]], 1e-5, ("convolution", taps, b, at[b]))
            near(out2[o:o + counts[b]], refs[b][at[b]:at[b] + counts[b]], 1e-2, ("convolution, rounded copy", taps, b))
            o += counts[b]
            at[b] += counts[b]


def _rglru_reference(y, u, gates, gate_bias, lam, scale, state):
    n, size = u.shape
    bw = gates.shape[2] // 2
    gg = gates.double() + gate_bias.double()
    r = torch.sigmoid(gg[:, :, :bw]).reshape(n, size)
    i = torch.sigmoid(gg[:, :, bw:]).reshape(n, size)
    a = torch.exp(-scale * r * torch.nn.functional.softplus(lam.double()))
    s, out = state.double().clone(), []
    for t in range(n):
        s = a[t] * s + torch.sqrt(1 - a[t] ** 2) * i[t] * u[t].double()
        out.append(s * PP.gelu_tanh(y[t].double()))
    return torch.stack(out), s


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("size,bw,counts", [(48, 16, (1, 5, 64)), (100, 100, (65, 1, 130, 2)), (256, 64, (300, 64)), (30, 6, (1, 1, 1))])
def test_rglru_scan_in_one_walk_and_in_pieces(dtype, size, bw, counts):
    ops = ops_module()
    g = torch.Generator().manual_seed(size)
    n, blocks = sum(counts), size // bw
    rows = torch.randn(2, n, size + 4, generator=g)
    yb, u = torch.randn(size, generator=g), torch.randn(n, size, generator=g)
    gates, gb = torch.randn(n, blocks, 2 * bw, generator=g), torch.randn(blocks, 2 * bw, generator=g)
    lam = torch.randn(size, generator=g) - 3.0
    state0 = torch.randn(len(counts) + 2, size, generator=g)
    slots = list(range(len(counts), 0, -1))
    sl, cu, _, _, _ = layout(counts, [0] * len(counts), slots)
    y = rows.sum(0)[:, 4:] + yb
    for pieces in (False, True):
        state = state0.clone().cuda()
        out = torch.empty(n, size, dtype=dtype, device="cuda")
        carry = torch.empty(len(counts), ops.mingru_pieces(max(counts)), 2, size, device="cuda") if pieces else None
        ops.rglru_scan(rows.cuda(), 4, yb.cuda(), u.cuda(), gates.cuda(), gb.cuda(), lam.cuda(), 8.0, state, sl, cu, out, carry)
        o = 0
        for b, c in enumerate(counts):
            want, last = _rglru_reference(y[o:o + c], u[o:o + c], gates[o:o + c], gb, lam, 8.0, state0[slots[b]])
            near(out[o:o + c], want, 2e-5 if dtype == torch.float32 else 1e-2, ("rglru", pieces, b))
            near(state[slots[b]], last, 2e-5, ("rglru state", pieces, b))
            o += c
        assert torch.equal(state[0].cpu(), state0[0])                      # a slot outside the step


def _retention_reference(q, k, v, gate, decay, eps, state):
    s, out = state.double().clone(), []
    for t in range(q.shape[0]):
        s = decay.double()[:, None, None] * s + k[t].double()[:, :, None] * v[t].double()[:, None, :]
        o = torch.einsum("hdv,hd->hv", s, q[t].double())
        out.append((PP.unit_rms(o, eps) * PP.silu(gate[t].double())).reshape(-1))
    return torch.stack(out), s


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("nh,dim,vdim,rot,counts", [(3, 16, 24, 8, (5, 1, 9)), (2, 32, 32, 32, (300, 1, 130)), (2, 64, 300, 0, (5, 2, 1)),
                                                    (5, 6, 6, 6, (129, 128)), (1, 128, 128, 64, (3, 140))])
def test_retention_in_one_walk_and_in_pieces(dtype, nh, dim, vdim, rot, counts):
    ops = ops_module()
    g = torch.Generator().manual_seed(dim + vdim)
    n, lead = sum(counts), 4
    width = lead + 2 * nh * dim + 2 * nh * vdim
    rows = torch.randn(2, n, width, generator=g)
    decay = torch.tensor([0.9, 1.0, 0.999, 0.5, 0.97][:nh])
    state0 = torch.randn(len(counts) + 1, nh, dim, vdim, generator=g)
    before = [7 * b for b in range(len(counts))]
    slots = list(range(len(counts) - 1, -1, -1))
    sl, cu, _, _, pos = layout(counts, before, slots)
    x = rows.sum(0)
    q = x[:, lead:lead + nh * dim].reshape(n, nh, dim)
    k = x[:, lead + nh * dim:lead + 2 * nh * dim].reshape(n, nh, dim)
    v = x[:, lead + 2 * nh * dim:lead + 2 * nh * dim + nh * vdim].reshape(n, nh, vdim)
    gate = x[:, lead + 2 * nh * dim + nh * vdim:].reshape(n, nh, vdim)
    cos = sin = None
    if rot:
        r = {"base": 100.0, "dims": rot}
        q, k = PP.rotate_halves(q, pos.cpu(), r), PP.rotate_halves(k, pos.cpu(), r)
        ang = torch.arange(512, dtype=F64)[:, None] * (100.0 ** (-2.0 * torch.arange(rot // 2, dtype=F64) / rot))[None, :]
        cos, sin = torch.cos(ang).float().cuda(), torch.sin(ang).float().cuda()
    k = k * dim ** -0.5
    for pieces in (False, True):
        state = state0.clone().cuda()
        out = torch.empty(n, nh * vdim, dtype=dtype, device="cuda")
        carry = torch.empty(len(counts), ops.retention_pieces(max(counts)), nh, dim, vdim, device="cuda") if pieces else None
        ops.retention(rows.cuda(), q_col=lead, k_col=lead + nh * dim, v_col=lead + 2 * nh * dim, g_col=lead + 2 * nh * dim + nh * vdim,
                      n_heads=nh, dim=dim, vdim=vdim, cos=cos, sin=sin, rotary_dim=rot, positions=pos, decay=decay.cuda(),
                      k_scale=dim ** -0.5, eps=1e-5, state=state, slots=sl, cu_tokens=cu, out=out, carry=carry)
        o = 0
        for b, c in enumerate(counts):
            want, last = _retention_reference(q[o:o + c], k[o:o + c], v[o:o + c], gate[o:o + c], decay, 1e-5, state0[slots[b]])
            near(out[o:o + c], want, 1e-4 if dtype == torch.float32 else 2e-2, ("retention", pieces, b))
            near(state[slots[b]], last, 1e-4, ("retention state", pieces, b))
            o += c
        assert torch.equal(state[len(counts)].cpu(), state0[len(counts)])


@pytest.mark.parametrize("n_exp,top,extra", [(8, 3, True), (9, 2, False), (6, 6, False), (40, 1, True), (12, 2, True)])
def test_routing_by_a_softmax_over_all_experts(n_exp, top, extra):
    """``moe_route`` (float32 router) and ``moe_topk`` (logits from a product's partial sums) against the plain rule."""
    ops = ops_module()
    g = torch.Generator().manual_seed(n_exp)
    n, hidden = 50, 40
    h = torch.randn(n, hidden, generator=g)
    wr = torch.randn(n_exp + (1 if extra else 0), hidden, generator=g) * 0.4
    idx, wt, _ = PP.route(h, {"router": wr[:n_exp]}, "", {"experts": n_exp, "top": top, "scale": 1.7})
    rule = ops.RouterRule("softmax_all", weight_scale=1.7, weight_sum_eps=1e-20)
    for way in ("route", "topk"):
        choice = torch.empty(n, top, dtype=torch.int32, device="cuda")
        weight = torch.empty(n, top, device="cuda")
        ex = torch.empty(n, device="cuda") if extra else None
        if way == "route":
            ops.moe_route(h.cuda(), wr.cuda(), None, choice, weight, rule, ex)
        else:
            z = h @ wr.t()
            parts = torch.stack([0.3 * z, 0.7 * z]).contiguous()
            ops.moe_topk(parts.cuda(), None, choice, weight, rule, ex)
        assert torch.equal(choice.cpu().long(), idx), way
        near(weight, wt, 1e-5, way)
        if extra:
            near(ex, torch.sigmoid(h.double() @ wr[n_exp].double()), 1e-5, way)


def test_per_block_products_leave_float32_sums_from_bfloat16_inputs():
    ops = ops_module()
    g = torch.Generator().manual_seed(0)
    for n, nh, k, o in ((70, 4, 64, 128), (9, 5, 6, 12), (300, 2, 80, 160)):
        x, w = torch.randn(n, nh, k, generator=g).bfloat16(), torch.randn(nh, o, k, generator=g).bfloat16()
        y = torch.empty(n, nh, o, device="cuda")
        ops.head_linear(x.cuda(), w.cuda(), y)
        near(y, torch.einsum("nha,hba->nhb", x.double(), w.double()), 1e-5, (n, nh, k, o))


# ---- whole models ------------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("name", list(PM.CONFIGS))
def test_whole_prompt_and_first_tokens(engines, models, name, dtype):
    eng = engines(name, dtype)
    for n in (1, 2, 3, 190):
        toks, ref = sequence(models, name, dtype, n, n)
        slot = eng.open()
        lg = eng.step([(slot, toks)], [list(range(n))])
        close(lg, ref, dtype, (name, "whole", n))
        eng.close(slot)
    eng.cache.audit()


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_residual_after_every_layer(llogos, models, dtype):
    """The residual stream after each layer, read from the engine by running models cut after 1, 2, ... layers, is what
    the plain model's trace holds."""
    import os
    name = "mixed"
    d, cfg, w = models[name, dtype]
    toks, _ = sequence(models, name, dtype, 50, 4)
    trace = []
    PP.forward(w, cfg, toks, trace=trace)
    assert len(trace) == len(cfg["layers"])
    side = cfg["token_side"]["dim"]
    for depth in range(1, len(cfg["layers"]) + 1):
        cut = dict(cfg, layers=cfg["layers"][:depth])
        keep = {k: v for k, v in w.items() if not (k.startswith("l") and k[1].isdigit() and int(k[1:k.index(".")]) >= depth)}
        keep["side.embed"] = keep["side.embed"][:, :side * depth]
        sub = os.path.join(d, f"cut{depth}")
        PM.write_model(llogos, sub, cut, 0, weights={k: v.to(torch.bfloat16) for k, v in keep.items()})
        model = llogos.weights.load_model(sub, dtype=dtype, device="cuda:0")
        eng = llogos.engine.Engine(model, max_tokens=256)
        slot = eng.open()
        lg = eng.step([(slot, toks)], [list(range(len(toks)))])
        close(lg, PP.linear(PP.norm_one_plus(trace[depth - 1], w["final.norm"], cfg["norm"]["eps"]), w["head"]), dtype, ("after layer", depth))
        eng.close(slot)


@pytest.mark.parametrize("graphs", [True, False], ids=["graph", "eager"])
@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("name", list(PM.CONFIGS))
def test_prompt_then_token_by_token(engines, models, name, dtype, graphs):
    """The decoded positions pass page borders (128, 192) and the pieces' borders of both scans; the first token alone too."""
    eng = engines(name, dtype, graphs)
    toks, ref = sequence(models, name, dtype, 215, 7)
    for cut in (1, 120):
        slot = eng.open()
        lg = eng.step([(slot, toks[:cut])])
        close(lg, ref[cut - 1:cut], dtype, (name, "prompt end", cut))
        got = [eng.step([(slot, [toks[p]])]).clone() for p in range(cut, len(toks) if cut > 1 else 40)]
        close(torch.cat(got), ref[cut:cut + len(got)], dtype, (name, "decoded from", cut))
        eng.close(slot)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("name", list(PM.CONFIGS))
def test_portions_of_several_sizes(engines, models, name, dtype):
    eng = engines(name, dtype)
    toks, ref = sequence(models, name, dtype, 300, 9)
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
@pytest.mark.parametrize("name", list(PM.CONFIGS))
def test_unequal_batches_with_slots_pages_and_states_used_again(engines, models, name, dtype):
    eng = engines(name, dtype)
    pairs = [sequence(models, name, dtype, n, 20 + n) for n in (1, 66, 140, 259, 33)]
    seqs, refs = [p[0] for p in pairs], [p[1] for p in pairs]
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
def test_long_decoding(engines, models, dtype):
    """420 decoded tokens after a prompt of 30: states and the token before are carried through every step, the keys
    grow over seven pages."""
    name = "mixed"
    eng = engines(name, dtype)
    toks, ref = sequence(models, name, dtype, 450, 5)
    slot = eng.open()
    eng.step([(slot, toks[:30])], [[]])
    got = [eng.step([(slot, [toks[p]])]).clone() for p in range(30, len(toks))]
    close(torch.cat(got), ref[30:], dtype, ("long decoding",))
    eng.close(slot)


def _random_config(seed):
    """A configuration drawn from the seed: two to five layers of both kinds in any order; sizes, taps, rotations, decays,
    the pair table, the per-token input, all drawn."""
    g = torch.Generator().manual_seed(3000 + seed)
    pick = lambda xs: xs[int(torch.randint(0, len(xs), (1,), generator=g))]
    width = pick([48, 64, 72, 96, 120])
    layers = []
    for _ in range(pick([2, 3, 4, 5])):
        kind = pick([0, 1, 2])
        if kind == 0:
            mlp = None
        elif kind == 1:
            mlp = PM.dense(pick([8, 24, 40, 100]))
        else:
            n_exp = pick([1, 2, 3, 6, 9])
            mlp = PM.moe(n_exp, pick(list(range(1, n_exp + 1))), pick([8, 24, 40]), pick([0, 16, 56]), scale=pick([None, 0.5, 2.5]))
        if pick([0, 1, 1]):
            kv = pick([1, 2, 3])
            dim = pick([8, 16, 24, 40, 64])
            rdim = pick([4, 8, 16, 32])
            le = PM.left(kv * pick([1, 2, 4]), kv, dim, pick([8, 16, 24, dim]), pick([0, 1, 2, 4, 6]), pick([0, 2, 4, dim]),
                         base=pick([50.0, 10000.0, 3e6]), scale=pick([0.05, 0.2, 0.5]))
            heads = pick([1, 2, 3, 5])
            ri = PM.right(heads, rdim, pick([4, 8, 20, rdim]), [pick([0.5, 0.9, 0.99, 0.999, 1.0]) for _ in range(heads)],
                          pick([0, 2, rdim]), base=pick([50.0, 10000.0]))
            mix = PM.parallel(le, ri)
        else:
            blocks = pick([1, 2, 4, 5])
            mix = PM.rglru(blocks * pick([2, 8, 16, 30]), blocks, pick([1, 2, 3, 4, 8]))
        layers.append(PM.layer(mix, mlp))
    return PM.config(layers, vocab=pick([61, 128, 257]), width=width, eps=pick([1e-6, 1e-5, 1e-3]), scale=pick([1.0, 7.0]),
                     bigram=pick([None, (pick([13, 101, 1000]), pick([1, 29, 1000003]), pick([1, 19]))]), side=pick([0, 4, 10]))


@pytest.mark.parametrize("seed", range(12))
def test_configurations_drawn_at_random(llogos, tmp_path, seed):
    """float32: a prompt whole, a batch of two unequal prompts decoded together for a dozen steps, against the plain model."""
    cfg = _random_config(seed)
    d = str(tmp_path / "m")
    w = {k: v.float() for k, v in PM.write_model(llogos, d, cfg, seed=seed).items()}
    model = llogos.weights.load_model(d, dtype=torch.float32, device="cuda:0")
    eng = llogos.engine.Engine(model, max_tokens=64 * 12)
    g = torch.Generator().manual_seed(seed)
    seqs = [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in (171, 40)]
    refs = [PP.forward(w, cfg, s) for s in seqs]
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


# ---- faults that random weights would hide ---------------------------------------------------------

A_TOK, B_TOK = 11, 12


def _ask(eng, t, b_at, cut):
    """Logits at ``b_at``: inside a prompt of ``cut`` tokens, or decoded alone after it."""
    slot = eng.open()
    lg = eng.step([(slot, t[:cut])], [[b_at] if b_at < cut else []])
    if b_at >= cut:
        lg = eng.step([(slot, [t[b_at]])])
    lg = lg.clone()
    eng.close(slot)
    return lg


def _one_side_model(llogos, folder, side):
    """One "parallel" layer without feed-forward, pair table or per-token input, made so that in the first head of
    ``side`` only tokens a and b write a key and ask with a query at all: the head's key and query matrices are ``e z^T``
    with z along a's normed embedding, b's embedding has the same share of z, and every other token's embedding is made orthogonal to z
    (the norms' weights are one, so the normed rows stay orthogonal).  ``e`` avoids the rotated elements and the
    convolutions pass the current token alone.  The other side's norm weight is small, so what ``side`` finds weighs on
    the logits."""
    le = PM.left(2, 1, 32, 24, 3, 4, scale=0.25)
    ri = PM.right(2, 32, 24, (1.0, 0.9), 4)
    cfg = PM.config([PM.layer(PM.parallel(le, ri), None)], vocab=50, width=48)
    w = PM.random_weights(cfg, 77)
    gen = torch.Generator().manual_seed(1)
    a = 2 * torch.randn(48, generator=gen)
    z = a / a.norm()
    emb = w["embed"].float()
    emb -= (emb @ z)[:, None] * z[None, :]
    r = torch.randn(48, generator=gen)
    r -= (r @ z) * z
    emb[A_TOK] = a
    emb[B_TOK] = a + r * (a.norm() / r.norm())                           # as much of z as a has, and values of its own
    w["embed"] = emb.to(torch.bfloat16)
    w["embed.norm"][:] = 0.0
    w["l0.norm1"][:] = 0.0
    e = torch.zeros(32)
    e[4:] = 28 ** -0.5
    p = f"l0.mix.{side}."
    w[p + "q"][:32] = (0.97 * e[:, None] * z[None, :]).to(torch.bfloat16)
    w[p + "k"][:32] = (0.97 * e[:, None] * z[None, :]).to(torch.bfloat16)
    for n in ("q", "k", "v"):
        w[f"l0.mix.left.{n}.conv"][:] = 0.0
        w[f"l0.mix.left.{n}.conv"][:, -1] = 1.0
    w["l0.mix.right.v"][24:] = 0.0                                       # the right side's second head stays silent
    w["l0.mix.left.out"][:] = 1.0 if side == "left" else 0.05
    w["l0.mix.right.out"][:] = 1.0 if side == "right" else 0.05
    PM.write_model(llogos, folder, cfg, 0, weights=w)
    return cfg, {k: v.float() for k, v in w.items()}


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("side", ["left", "right"])
def test_what_token_a_left_330_positions_back(llogos, tmp_path, dtype, side):
    """Token a stands at position 2, token b 330 positions (five pages, several pieces of the scan) later.  Left: a far key
    among hundreds in the softmax.  Right: a state entry written long ago under a decay of one.  b's logits with a there
    and with another token in a's place are far apart, in a prompt, in portions, decoded, and beside another request."""
    d = str(tmp_path / side)
    cfg, wf = _one_side_model(llogos, d, side)
    model = llogos.weights.load_model(d, dtype=dtype, device="cuda:0")
    eng = llogos.engine.Engine(model, max_tokens=64 * 16)
    gen = torch.Generator().manual_seed(3)
    toks = torch.randint(13, 50, (336,), generator=gen).tolist()
    b_at = 332
    toks[b_at] = B_TOK
    with_a, without_a = list(toks), list(toks)
    with_a[2] = A_TOK
    refs = [PP.forward(wf, cfg, t) for t in (with_a, without_a)]
    assert float((refs[0][b_at] - refs[1][b_at]).abs().max()) > 0.05 * float(refs[0][b_at].abs().max())
    for t, ref in zip((with_a, without_a), refs):
        for cut in (len(t), b_at, 3):
            slot = eng.open()
            lg = eng.step([(slot, t[:cut])], [[b_at] if b_at < cut else []])
            for p in range(cut, b_at + 1):
                lg = eng.step([(slot, [t[p]])])
            close(lg, ref[b_at:b_at + 1], dtype, (side, "a far back", cut), tol=TIGHT)
            eng.close(slot)
        slot = eng.open()
        for lo, hi in ((0, 2), (2, 4), (4, 70), (70, 199), (199, 330)):
            eng.step([(slot, t[lo:hi])], [[]])
        close(eng.step([(slot, t[330:])], [[b_at - 330]]), ref[b_at:b_at + 1], dtype, (side, "a far back, portions"), tol=TIGHT)
        eng.close(slot)
    slots = [eng.open(), eng.open()]
    eng.step([(slots[0], with_a[:200]), (slots[1], without_a[:90])], [[], []])
    eng.step([(slots[1], without_a[90:200])], [[]])
    for p in range(200, b_at):
        eng.step([(slots[0], [with_a[p]]), (slots[1], [without_a[p]])], [[], []])
    lg = eng.step([(slots[0], [with_a[b_at]]), (slots[1], [without_a[b_at]])])
    close(lg[0], refs[0][b_at], dtype, (side, "batched, with a"), tol=TIGHT)
    close(lg[1], refs[1][b_at], dtype, (side, "batched, without a"), tol=TIGHT)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_a_recurrent_state_written_long_ago(llogos, tmp_path, dtype):
    """An rglru layer whose first channels open their input gate for token a alone and decay by a thousandth a token: what
    a wrote at position 2 still decides the logits 330 tokens later, whole (the scan in pieces), in portions, one by one."""
    cfg = PM.config([PM.layer(PM.rglru(64, 1, 3), None)], vocab=50, width=48)
    w = PM.random_weights(cfg, 78)
    gen = torch.Generator().manual_seed(4)
    w["embed"][A_TOK] = (2 * torch.randn(48, generator=gen)).to(torch.bfloat16)
    w["l0.norm1"][:] = 0.0
    w["l0.mix.conv"][:] = 0.0
    w["l0.mix.conv"][:, -1] = 1.0                                      # u hangs on the current token alone
    w["l0.mix.conv.b"][:] = 0.0
    wf = {k: v.float() for k, v in w.items()}
    eps = cfg["norm"]["eps"]
    h = PP.norm_one_plus(PP.norm_one_plus(wf["embed"].double(), wf["embed.norm"], eps), wf["l0.norm1"], eps)
    u = PP.linear(h, wf["l0.mix.x"], wf["l0.mix.x.b"])                  # [vocab, 64]
    u_a = u[A_TOK]
    keep = 12
    w["l0.mix.ri"][0, :keep] = (40.0 * u_a / u_a.dot(u_a)).to(torch.bfloat16)
    w["l0.mix.ri.b"][0, :keep] = -20.0
    w["l0.mix.ra"][0, :keep] = 0.0
    w["l0.mix.ra.b"][0, :keep] = 0.0
    w["l0.mix.lam"][:keep] = -8.3                                      # a = exp(-8 * 1/2 * softplus(-8.3)) = 0.999
    w["l0.mix.o"][:, :keep] *= 30.0
    wf = {k: v.float() for k, v in w.items()}
    others = torch.sigmoid(u[13:50] @ wf["l0.mix.ri"][0, :keep].double().t() - 20.0)
    assert float(others.max()) < 0.05                                   # nobody but a opens those gates
    d = str(tmp_path / "state")
    PM.write_model(llogos, d, cfg, 0, weights=w)
    model = llogos.weights.load_model(d, dtype=dtype, device="cuda:0")
    eng = llogos.engine.Engine(model, max_tokens=64 * 16)
    toks = torch.randint(13, 50, (336,), generator=gen).tolist()
    b_at = 332
    with_a, without_a = list(toks), list(toks)
    with_a[2] = A_TOK
    refs = [PP.forward(wf, cfg, t) for t in (with_a, without_a)]
    assert float((refs[0][b_at] - refs[1][b_at]).abs().max()) > 0.1 * float(refs[0][b_at].abs().max())
    for t, ref in zip((with_a, without_a), refs):
        for cut in (len(t), b_at, 3):
            slot = eng.open()
            lg = eng.step([(slot, t[:cut])], [[b_at] if b_at < cut else []])
            for p in range(cut, b_at + 1):
                lg = eng.step([(slot, [t[p]])])
            close(lg, ref[b_at:b_at + 1], dtype, ("old state", cut), tol=TIGHT)
            eng.close(slot)
        slot = eng.open()
        for lo, hi in ((0, 2), (2, 4), (4, 70), (70, 199), (199, 330)):
            eng.step([(slot, t[lo:hi])], [[]])
        close(eng.step([(slot, t[330:])], [[b_at - 330]]), ref[b_at:b_at + 1], dtype, ("old state in portions",), tol=TIGHT)
        eng.close(slot)


# ---- the library's entry points ----------------------------------------------------------------------

@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_greedy_generation_through_the_entry_point(models, dtype):
    """``LlogosModel.generate`` (scheduler, sampler, run-ahead decoding) makes the plain model's best tokens."""
    import llogos_b200 as L
    name = "mixed"
    d, cfg, w = models[name, dtype]
    model = L.LlogosModel.load(d, dtype=dtype, max_context=256, max_batch=3)
    prompts = [sequence(models, name, dtype, n, 60 + n)[0] for n in (5, 70, 23, 1)]
    out = model.generate(prompts, L.GenerationParams.greedy_params(12, stop_tokens=()))
    for p, made in zip(prompts, out.tokens):
        assert len(made) == 12
        toks = list(p)
        for tok in made:
            lg = PP.forward(w, cfg, toks)[-1]
            slack = 1e-4 if dtype == torch.float32 else 0.05
            assert float(lg[tok]) >= float(lg.max()) - slack * float(lg.abs().max()), (len(toks), tok)
            toks.append(tok)


def test_command_line_and_trace_replay_take_the_design(models, tmp_path):
    """``python -m llogos_b200`` generates with a Piratar folder, and ``bin/trace_run`` replays steps on it (two requests
    started together, decoded together, the shorter one ending first, a third in portions), as they do for every model."""
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
        lg = PP.forward(w, cfg, toks)[-1]
        assert float(lg[tok]) >= float(lg.max()) - 1e-4 * float(lg.abs().max())
        toks.append(tok)
    d, cfg, w = models["tensor", torch.bfloat16]
    (a, ra), (b, rb) = sequence(models, "tensor", torch.bfloat16, 100, 1), sequence(models, "tensor", torch.bfloat16, 31, 2)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:98], "want": [0, 69, 97]}, {"id": "b", "tokens": b[:30], "want": [29]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[98:99], "want": [0]}, {"id": "b", "tokens": b[30:], "want": [0]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": a[99:], "want": [0]}], "end": ["a"]},
             {"step": 3, "entries": [{"id": "c", "tokens": b[:7], "want": []}], "end": []},
             {"step": 4, "entries": [{"id": "c", "tokens": b[7:30], "want": [22]}], "end": ["c"]}]
    out = tmp_path / "logits"
    p = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", d, "--dtype", "bfloat16", "--out", str(out), "--max-tokens", "200"],
                       input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, env=env, cwd=root)
    assert p.returncode == 0, p.stderr
    assert [l for l in p.stdout.split("\n") if l.startswith("done")] == [f"done {i}" for i in range(5)]
    want = {0: torch.stack([ra[0], ra[69], ra[97], rb[29]]), 1: torch.stack([ra[98], rb[30]]), 2: ra[99:100], 4: rb[29:30]}
    assert not (out / "3.f32").exists()
    for i, ref in want.items():
        got = torch.from_numpy(np.fromfile(str(out / f"{i}.f32"), dtype="<f4").reshape(-1, cfg["vocab"]))
        close(got, ref, torch.bfloat16, ("replayed step", i))
