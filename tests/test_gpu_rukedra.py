"""The Rukedra decoder on the GPU against the plain implementation in rukedra_plain.py, in float32 and bfloat16:
every mechanism's kernel alone; whole prompts; prompts against token-by-token decoding; prompts in portions down to two
tokens; batches of unequal requests against each alone, with slots, pages and state rows used again; keys at page borders
and just inside and outside the window, in prompts and in decoding; a far key and a state written long ago; the first
tokens; long decoding through rings that go round several times; sizes that differ from layer to layer; greedy generation
through the library's entry point."""
import math

import pytest
import torch

import rukedra_models as RM
import rukedra_plain as RP

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]
IDS = ["f32", "bf16"]

# float32: every logit within 1e-4 of the request's largest |logit|.  bfloat16, relative to the root mean square of all
# compared logits: the root-mean-square error of every position within 1e-1 and of the positions on average within
# 3.5e-2, every logit within 1.5e-1 of the largest (up to sixteen sublayers, each ending in a norm that brings its output,
# rounding error included, back to full size; a few positions of hundreds land several times above the average).  The
# models of one layer that are made to show a fault (TIGHT) stay within 2.5e-2 and 5e-2.
TOL = {torch.float32: (1e-4, 1e-4, 1e-4), torch.bfloat16: (1e-1, 3.5e-2, 1.5e-1)}
TIGHT = {torch.float32: (1e-4, 1e-4, 1e-4), torch.bfloat16: (2.5e-2, 2.5e-2, 5e-2)}
MARGIN = 0.02          # bfloat16: no router of a compared sequence decides by less than this (in score)


def ops_module():
    from importlib import import_module
    return import_module("daisi-llogos_b200.kernels.ops")


def close(got, ref, dtype, what=(), tol=TOL):
    got = got.detach().to("cpu", torch.float64).reshape(ref.shape)
    rms_tol, mean_tol, max_tol = tol[dtype]
    per_position = (got - ref).pow(2).mean(-1).sqrt() / ref.pow(2).mean().sqrt()
    rms, mean = float(per_position.max()), float(per_position.mean())
    worst = float((got - ref).abs().max() / ref.abs().max())
    if per_position.numel() < 16:           # an average of a few positions is no average: the per-position bound stands alone
        mean_tol = rms_tol
    assert rms <= rms_tol and mean <= mean_tol and worst <= max_tol, (*what, "rms", rms, "mean", mean, "max", worst)


@pytest.fixture(scope="module")
def models(llogos, tmp_path_factory):
    """(name, dtype) -> (folder, config, weights as float tensors).  The bfloat16 comparisons use routers that read a
    code of the token which no sublayer changes (``steady_routing``), so that rounding upstream does not move a choice;
    float32 takes routers that hang on everything."""
    out = {}
    for i, (name, cfg) in enumerate(RM.CONFIGS.items()):
        for dtype in DTYPES:
            d = str(tmp_path_factory.mktemp(f"rukedra_{name}_{IDS[DTYPES.index(dtype)]}"))
            w = RM.write_model(llogos, d, cfg, seed=170 + i, steady_routing=dtype == torch.bfloat16)
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
        ref = RP.forward(w, cfg, toks, margins=margins)
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


# ---- mechanisms alone --------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("hidden,groups,post_groups,sets", [(72, 3, 3, (2, 1)), (100, 1, 1, (1, 1)), (128, 4, 2, (3, 2)),
                                                            (1024, 64, 64, (1, 4)), (4100, 2, 5, (2, 2))])
def test_grouped_norm_with_gated_add(llogos, dtype, hidden, groups, post_groups, sets):
    ops = ops_module()
    g = torch.Generator().manual_seed(hidden)
    n = 9
    x = 2 * torch.randn((n, hidden), generator=g)
    x[:, :hidden // groups] *= 7.0                                         # groups of very different size: a norm over the whole row would show
    branch = torch.randn((sets[0], n, hidden), generator=g)
    gate = torch.randn((sets[1], n, hidden), generator=g)
    bias = torch.randn((hidden,), generator=g)
    weight = (1 + 0.2 * torch.randn((hidden,), generator=g)).to(dtype)
    post_w = (0.7 + 0.2 * torch.randn((hidden,), generator=g)).to(dtype)
    eps, post_eps = 3e-5, 2e-6
    y = branch.double().sum(0) * torch.sigmoid(gate.double().sum(0) + bias.double())
    want_res = x.double() + RP.group_rms_norm(y, post_w.float(), post_eps, post_groups)
    want = RP.group_rms_norm(want_res, weight.float(), eps, groups)
    tol = 3e-6 if dtype == torch.float32 else 1e-2
    dev = x.cuda()
    out = torch.empty((n, hidden), dtype=dtype, device="cuda")
    ops.gated_add_group_rmsnorm(dev, branch.cuda(), gate.cuda(), bias.cuda(), post_w.cuda(), post_groups, post_eps,
                                weight.cuda(), groups, eps, out)
    assert float((dev.cpu().double() - want_res).abs().max()) < 1e-5 * float(want_res.abs().max())
    assert float((out.cpu().double() - want).abs().max()) < tol * float(want.abs().max())
    # a branch added as it is (no gate, no norm of its own)
    dev = x.cuda()
    ops.gated_add_group_rmsnorm(dev, branch.cuda(), None, None, None, 1, eps, weight.cuda(), groups, eps, out)
    want1 = RP.group_rms_norm(x.double() + branch.double().sum(0), weight.float(), eps, groups)
    assert float((out.cpu().double() - want1).abs().max()) < tol * float(want1.abs().max())
    # nothing pending, chosen rows only: the residual stays as it is
    dev2 = x.cuda()
    rows = torch.tensor([7, 0, 3], dtype=torch.int32, device="cuda")
    out2 = torch.empty((3, hidden), dtype=dtype, device="cuda")
    ops.gated_add_group_rmsnorm(dev2, None, None, None, None, 1, eps, weight.cuda(), groups, eps, out2, rows)
    want2 = RP.group_rms_norm(x.double()[[7, 0, 3]], weight.float(), eps, groups)
    assert torch.equal(dev2.cpu(), x)
    assert float((out2.cpu().double() - want2).abs().max()) < tol * float(want2.abs().max())
    # a pending branch, chosen rows only: those rows' residual takes the branch
    dev3 = x.cuda()
    ops.gated_add_group_rmsnorm(dev3, branch.cuda(), gate.cuda(), bias.cuda(), post_w.cuda(), post_groups, post_eps,
                                weight.cuda(), groups, eps, out2, rows)
    assert float((out2.cpu().double() - want[[7, 0, 3]]).abs().max()) < tol * float(want.abs().max())
    assert float((dev3.cpu().double()[[7, 0, 3]] - want_res[[7, 0, 3]]).abs().max()) < 1e-5 * float(want_res.abs().max())


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("size,counts", [(40, (1, 5, 64)), (100, (65, 1, 130, 2)), (256, (300, 64)), (30, (1, 1, 1))])
def test_mingru_scan_in_one_walk_and_in_pieces(llogos, dtype, size, counts):
    """Sequences of unequal lengths from states that are not zero, token by token in one kernel and cut into pieces that
    are joined; lengths at, below and above a piece; the state left behind."""
    ops = ops_module()
    g = torch.Generator().manual_seed(size)
    n, b = sum(counts), len(counts)
    rows = torch.randn((2, n, 3 * size), generator=g)
    rows[:, :, :size] -= 0.6                                                # gates that keep much of the state
    bias = torch.randn((2 * size,), generator=g) * 0.5
    state0 = torch.randn((b + 3, size), generator=g)
    slots = torch.tensor([b + 2 - 2 * i if i < 2 else i for i in range(b)], dtype=torch.int32)     # not in order
    assert len(set(slots.tolist())) == b
    cu = torch.tensor([0] + list(torch.tensor(counts).cumsum(0)), dtype=torch.int32)
    z = torch.sigmoid(rows.double().sum(0)[:, :size] + bias[:size].double())
    c = RP.mingru_candidate(rows.double().sum(0)[:, size:2 * size] + bias[size:].double())
    gate = RP.silu(rows.double().sum(0)[:, 2 * size:])
    want = torch.zeros((n, size), dtype=torch.float64)
    want_state = state0.double().clone()
    for i in range(b):
        s = state0[int(slots[i])].double()
        for t in range(int(cu[i]), int(cu[i + 1])):
            s = (1 - z[t]) * s + z[t] * c[t]
            want[t] = s * gate[t]
        want_state[int(slots[i])] = s
    tol = 2e-5 if dtype == torch.float32 else 1e-2
    pieces = ops.mingru_pieces(max(counts))
    for carry in ([None] if pieces == 1 else [None, torch.empty((b, pieces, 2, size), dtype=torch.float32, device="cuda")]):
        state = state0.cuda()
        out = torch.empty((n, size), dtype=dtype, device="cuda")
        ops.mingru_scan(rows.cuda(), bias.cuda(), state, slots.cuda(), cu.cuda(), out, carry)
        assert float((out.cpu().double() - want).abs().max()) < tol * float(want.abs().max()), carry is None
        assert float((state.cpu().double() - want_state).abs().max()) < 2e-5 * float(want_state.abs().max()), carry is None


@pytest.mark.parametrize("n_exp,top,groups,keep,extra", [(8, 3, 4, 2, True), (9, 2, 3, 1, False), (16, 4, 4, 3, True), (6, 6, 1, 1, False),
                                                         (5, 1, 0, 0, True), (64, 8, 8, 4, False), (12, 4, 6, 2, True)])
def test_sigmoid_group_routing(llogos, n_exp, top, groups, keep, extra):
    """Both routing kernels (from the token's row; from a product's partial sums) against the plain rule: the chosen
    experts as a set, their weights, and the gate of the shared expert from one more row."""
    ops = ops_module()
    g = torch.Generator().manual_seed(n_exp * 10 + top)
    n, hidden = 37, 48
    x = torch.randn((n, hidden), generator=g)
    w_r = torch.randn((n_exp + (1 if extra else 0), hidden), generator=g) * 0.3
    router = {"experts": n_exp, "top": top, "scale": 1.7}
    if groups:
        router["groups"] = {"count": groups, "keep": keep}
    idx, wt, _ = RP.route(x, {"r.router": w_r[:n_exp]}, "r.", router)
    rule = ops.RouterRule("sigmoid", groups, keep, 2, 1.7, 1e-20)
    for way in ("route", "topk"):
        choice = torch.empty((n, top), dtype=torch.int32, device="cuda")
        weight = torch.empty((n, top), dtype=torch.float32, device="cuda")
        gate = torch.empty((n,), dtype=torch.float32, device="cuda") if extra else None
        if way == "route":
            ops.moe_route(x.cuda(), w_r.cuda(), None, choice, weight, rule=rule, extra_out=gate)
        else:
            z = x.double() @ w_r.double().t()
            parts = torch.stack([0.3 * z, 0.7 * z]).float()
            ops.moe_topk(parts.cuda(), None, choice, weight, rule=rule, extra_out=gate)
        got_i, got_w = choice.cpu().long(), weight.cpu().double()
        order = got_i.argsort(-1)
        want_order = idx.argsort(-1)
        assert torch.equal(got_i.gather(1, order), idx.gather(1, want_order)), way
        assert float((got_w.gather(1, order) - wt.gather(1, want_order)).abs().max()) < 1e-5, way
        assert bool((got_w[:, :-1] >= got_w[:, 1:] - 1e-7).all())            # largest first
        if extra:
            want_gate = torch.sigmoid(x.double() @ w_r[n_exp].double())
            assert float((gate.cpu().double() - want_gate).abs().max()) < 1e-5, way


def test_shared_expert_is_scaled_per_token_in_the_weighted_sum(llogos):
    ops = ops_module()
    g = torch.Generator().manual_seed(3)
    for hidden in (72, 100):
        n, top, cap = 11, 2, 64
        y = torch.randn((cap, hidden), generator=g)
        rows = torch.randperm(cap, generator=g)[:n * top].int()
        weight = torch.rand((n, top), generator=g)
        shared = torch.randn((2, n, hidden), generator=g)
        scale = torch.rand((n,), generator=g)
        out = torch.empty((n, hidden), dtype=torch.float32, device="cuda")
        ops.moe_combine(y.cuda(), rows.cuda(), weight.cuda(), shared.cuda(), out, shared_scale=scale.cuda())
        want = (weight.double()[:, :, None] * y.double()[rows.long()].view(n, top, hidden)).sum(1) + scale.double()[:, None] * shared.double().sum(0)
        assert float((out.cpu().double() - want).abs().max()) < 1e-5


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_latent_preparation_with_a_query_latent_and_neighbour_pairs(llogos, dtype):
    """One row of the input product holds the queries' latent, the keys' latent with the shared rotated part, and the
    gate's arguments: the first call norms both latents and writes the key across a page border, the second one makes the
    query heads from their own product; rotations pair neighbours, with stretched frequencies and a scaled amplitude."""
    ops = ops_module()
    g = torch.Generator().manual_seed(21)
    n, nh, dim, rdim, rank, q_rank, gate_w = 7, 3, 12, 6, 20, 10, 18
    rot = {"base": 300.0, "dims": rdim, "scaling": {"factor": 3.0, "original": 16, "fast": 2.0, "slow": 0.5}}
    width = q_rank + rank + rdim + gate_w
    rows = torch.randn((2, n, width), generator=g)
    cw = (1 + 0.3 * torch.randn((rank,), generator=g)).to(dtype)
    qw = (1 + 0.3 * torch.randn((q_rank,), generator=g)).to(dtype)
    eps = 2e-5
    pos = torch.arange(60, 60 + n)
    z = rows.double().sum(0)
    want_cq = RP.rms_norm(z[:, :q_rank], qw.float(), eps)
    want_c = RP.rms_norm(z[:, q_rank:q_rank + rank], cw.float(), eps)
    want_kr = RP.rotate_pairs(z[:, None, q_rank + rank:q_rank + rank + rdim], pos, rot)[:, 0]
    f, amp = RP.stretched_frequencies(rdim, rot["base"], rot["scaling"])
    ang = torch.arange(80, dtype=torch.float64)[:, None] * f[None]
    cos, sin = (amp * torch.cos(ang)).float().cuda(), (amp * torch.sin(ang)).float().cuda()
    kd = rank + rdim
    kp = torch.zeros((3, 1, 64, kd), dtype=dtype, device="cuda")
    table = torch.tensor([[2, 0]], dtype=torch.int32, device="cuda")
    common = dict(n_heads=nh, head_dim=dim, rot_dim=rdim, kv_rank=rank, c_norm_w=cw.cuda(), norm_eps=eps, cos=cos, sin=sin,
                  pairing=1, positions=pos.int().cuda())
    k_new = torch.empty((n, 1, kd), dtype=dtype, device="cuda")
    cq = torch.empty((n, q_rank), dtype=dtype, device="cuda")
    ops.latent_prep(rows.cuda(), **common, k_new=k_new, k_pages=kp, page_table=table, ring_pages=2,
                    seq_of_token=torch.zeros(n, dtype=torch.int32, device="cuda"), slots=torch.zeros(1, dtype=torch.int32, device="cuda"),
                    q_col=-1, kv_col=q_rank, cq_col=0, cq_norm_w=qw.cuda(), cq_out=cq)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    want_k = torch.cat([want_c, want_kr], -1)
    assert float((cq.cpu().double() - want_cq).abs().max()) < tol * float(want_cq.abs().max())
    assert float((k_new.cpu().double()[:, 0] - want_k).abs().max()) < tol * float(want_k.abs().max())
    stored = torch.cat([kp[2, 0, 60:64], kp[0, 0, 0:3]]).cpu().double()          # positions 60..63 in page 2, 64..66 in page 0
    assert torch.equal(stored, k_new.cpu().double()[:, 0])
    # the queries from a product of their own
    q_rows = torch.randn((1, n, nh * (dim + rdim)), generator=g)
    q_plain = torch.empty((n, nh, dim), dtype=dtype, device="cuda")
    q = torch.zeros((n, nh, kd), dtype=dtype, device="cuda")
    ops.latent_prep(q_rows.cuda(), **common, q_plain_out=q_plain, q_out=q, q_col=0, kv_col=-1)
    zq = q_rows.double()[0].view(n, nh, dim + rdim)
    want_qr = RP.rotate_pairs(zq[..., dim:], pos, rot)
    assert float((q_plain.cpu().double() - zq[..., :dim]).abs().max()) < tol * float(zq.abs().max())
    assert float((q.cpu().double()[..., rank:] - want_qr).abs().max()) < tol * float(want_qr.abs().max())
    # the gate on the concatenated heads, from the first product's last columns
    heads_out = torch.randn((n, gate_w), generator=g).to(dtype)
    dev = heads_out.cuda()
    ops.sigmoid_gate(dev, rows.cuda(), q_rank + rank + rdim)
    want_g = heads_out.double() * torch.sigmoid(z[:, q_rank + rank + rdim:])
    assert float((dev.cpu().double() - want_g).abs().max()) < tol * float(want_g.abs().max())


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_gelu_gated_products_and_the_cap(llogos, dtype):
    """The feed-forward's gating with the tanh form of gelu: from partial sums in the gated layout, and in bfloat16 as the
    epilogue of the tensor-core product with few and with many rows; the cap on logits."""
    ops = ops_module()
    lin = __import__("importlib").import_module("daisi-llogos_b200.kernels.linear")
    g = torch.Generator().manual_seed(5)
    for n, hidden, inter in ((5, 64, 40), (300, 128, 200)):
        x = torch.randn((n, hidden), generator=g).to(dtype)
        wg = (torch.randn((inter, hidden), generator=g) * hidden ** -0.5 * 2).to(dtype)
        wu = (torch.randn((inter, hidden), generator=g) * hidden ** -0.5).to(dtype)
        want = RP.gelu_tanh(RP.linear(x.float(), wg.float())) * RP.linear(x.float(), wu.float())
        layout = lin.gated_layout(wg, wu).cuda()
        tol = 1e-5 if dtype == torch.float32 else 1.5e-2
        gu = torch.empty((1, n, layout.shape[0]), dtype=dtype, device="cuda")
        ops.gemm_simt(x.cuda(), layout, gu[0])
        halves = torch.stack([0.25 * gu[0].float(), 0.75 * gu[0].float()])
        out = torch.empty((n, inter), dtype=dtype, device="cuda")
        ops.silu_mul(halves, out, activation="gelu_tanh")
        assert float((out.cpu().double() - want).abs().max()) < tol * float(want.abs().max())
        if dtype == torch.bfloat16:
            assert ops.gemm_tc_supported(x.cuda(), layout)
            out2 = torch.empty((1, n, inter), dtype=dtype, device="cuda")
            ops.gemm_tc(x.cuda(), layout, out2, gated_features=inter, gate_activation="gelu_tanh")
            assert ops.gemm_tc_status() == 0
            assert float((out2[0].cpu().double() - want).abs().max()) < tol * float(want.abs().max())
            out3 = torch.empty((1, n, inter), dtype=dtype, device="cuda")
            ops.gemm_tc(x.cuda(), layout, out3, gated_features=inter)                     # silu stays what it was
            want3 = RP.silu(RP.linear(x.float(), wg.float())) * RP.linear(x.float(), wu.float())
            assert float((out3[0].cpu().double() - want3).abs().max()) < tol * float(want3.abs().max())
    lg = (torch.randn((13, 97), generator=g) * 20).cuda()
    want = RP.soft_cap(lg.cpu().double(), 7.5)
    ops.tanh_cap(lg, 7.5)
    assert float((lg.cpu().double() - want).abs().max()) < 1e-5


# ---- whole models ------------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("name", list(RM.CONFIGS))
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
    """The residual stream after each layer run, read from the engine by running models cut after 1, 2, ... entries of the
    layer list, is what the plain model's trace holds (a layer that runs with another's tensors counts each time)."""
    import os
    name = "mixed"
    d, cfg, w = models[name, dtype]
    toks, _ = sequence(models, name, dtype, 50, 4)
    trace = []
    RP.forward(w, cfg, toks, trace=trace)
    assert len(trace) == len(cfg["layers"])
    for depth in (1, 2, 4, 7, len(cfg["layers"])):
        cut = dict(cfg, layers=cfg["layers"][:depth])
        keep = {k: v for k, v in w.items() if not (k.startswith("l") and int(k[1:k.index(".")]) >= depth)}
        sub = os.path.join(d, f"cut{depth}")
        RM.write_model(llogos, sub, cut, 0, weights={k: v.to(torch.bfloat16) for k, v in keep.items()})
        model = llogos.weights.load_model(sub, dtype=dtype, device="cuda:0")
        eng = llogos.engine.Engine(model, max_tokens=256)
        slot = eng.open()
        lg = eng.step([(slot, toks)], [list(range(len(toks)))])
        normed = RP.group_rms_norm(trace[depth - 1], w["final.norm"], cfg["norm"]["eps"], cfg["norm"]["groups"])
        close(lg, RP.soft_cap(RP.linear(normed, w["head"]), cfg.get("logit_softcap")), dtype, ("after layer", depth))
        eng.close(slot)


@pytest.mark.parametrize("graphs", [True, False], ids=["graph", "eager"])
@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("name", list(RM.CONFIGS))
def test_prompt_then_token_by_token(engines, models, name, dtype, graphs):
    """The decoded positions pass page borders (128, 192) and every window's edge; the first token alone too."""
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
@pytest.mark.parametrize("name", list(RM.CONFIGS))
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
@pytest.mark.parametrize("name", list(RM.CONFIGS))
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
def test_long_decoding_round_the_rings(engines, models, dtype):
    """420 decoded tokens after a prompt of 30: the windows' rings of pages go round several times, the recurrent states
    are carried through every step."""
    name = "mixed"
    eng = engines(name, dtype)
    toks, ref = sequence(models, name, dtype, 450, 5)
    slot = eng.open()
    eng.step([(slot, toks[:30])], [[]])
    got = [eng.step([(slot, [toks[p]])]).clone() for p in range(30, len(toks))]
    close(torch.cat(got), ref[30:], dtype, ("long decoding",))
    eng.close(slot)


def _random_config(seed):
    """A configuration drawn from the seed: two to six layers of the three kinds in any order, some run twice; sizes,
    windows, rotations, groups of the norm and of the experts, the cap, all drawn."""
    g = torch.Generator().manual_seed(2000 + seed)
    pick = lambda xs: xs[int(torch.randint(0, len(xs), (1,), generator=g))]
    width = pick([48, 64, 72, 96, 120])
    layers = []
    for _ in range(pick([2, 3, 4, 5])):
        kind = pick([0, 1, 2])
        if kind == 0:
            mlp = None
        elif kind == 1:
            mlp = RM.dense(pick([8, 24, 40, 100]))
        else:
            count = pick([1, 2, 3, 4])
            per = pick([1, 2, 3])
            keep = pick(list(range(1, count + 1)))
            grouped = pick([0, 1, 1])
            top = pick(list(range(1, (keep if grouped else count) * per + 1)))
            mlp = RM.moe(count * per, top, pick([8, 24, 40]), pick([0, 16, 56]), groups=(count, keep) if grouped else None,
                         scale=pick([None, 0.5, 2.5]))
        rot = pick([2, 4, 8, 16, 32])
        scaling = pick([None, (pick([2.0, 8.0, 40.0]), pick([16, 64, 4096]), pick([32.0, 4.0]), pick([1.0, 0.25]))])
        common = dict(base=pick([50.0, 10000.0, 3e6]), scaling=scaling, scale=pick([0.05, 0.2, 0.5]))
        which = pick([0, 1, 2])
        if which == 0:
            mix = RM.latent(pick([1, 2, 3, 5, 8]), pick([8, 16, 40]), rot, pick([8, 24, 32]), pick([8, 16, 30, 64, 112]),
                            pick([4, 16, 33, 96]), pick([1, 2, 31, 64, 100, 160]), **common)
        elif which == 1:
            mix = RM.latent2(pick([1, 2, 3, 5, 8]), pick([8, 16, 40]), rot, pick([8, 24, 32]), pick([8, 16, 30, 64, 112]), **common)
        else:
            mix = RM.mingru(pick([8, 30, 64, 136]))
        layers.append(RM.layer(mix, mlp))
    for _ in range(pick([0, 1, 2])):
        layers.insert(pick(list(range(1, len(layers) + 1))), None)
    # a layer run again stands after the layer it takes its tensors from
    out = []
    for lay in layers:
        out.append(lay if lay is not None else RM.again(out, pick([i for i, l in enumerate(out) if "weights_of" not in l])))
    return RM.config(out, vocab=pick([61, 128, 257]), width=width, groups=pick([g_ for g_ in (1, 2, 3, 4, 8) if width % g_ == 0]),
                     eps=pick([1e-6, 1e-5, 1e-3]), cap=pick([None, 5.0, 30.0]))


@pytest.mark.parametrize("seed", range(12))
def test_configurations_drawn_at_random(llogos, tmp_path, seed):
    """float32: a prompt whole, a batch of two unequal prompts decoded together for a dozen steps, against the plain model."""
    cfg = _random_config(seed)
    d = str(tmp_path / "m")
    w = {k: v.float() for k, v in RM.write_model(llogos, d, cfg, seed=seed).items()}
    model = llogos.weights.load_model(d, dtype=torch.float32, device="cuda:0")
    eng = llogos.engine.Engine(model, max_tokens=64 * 12)
    g = torch.Generator().manual_seed(seed)
    seqs = [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in (171, 40)]
    refs = [RP.forward(w, cfg, s) for s in seqs]
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
@pytest.mark.parametrize("kv_rank,rot_dim", [(272, 16), (320, 64)])
def test_latents_longer_than_the_tensor_core_kernels_take(llogos, tmp_path, dtype, kv_rank, rot_dim):
    """A cached row of kv_rank + rot_dim elements beyond 256: both attention mixers on the large form of the CUDA-core
    kernels, a prompt whole and the same prompt cut in two with its end decoded."""
    ls = [RM.layer(RM.latent(3, 24, rot_dim, 40, kv_rank, 56, 45, scaling=(4.0, 32, 16.0, 1.0)), RM.dense(48)),
          RM.layer(RM.latent2(2, 16, rot_dim, 24, kv_rank, base=700.0), None)]
    cfg = RM.config(ls, vocab=90, width=80, groups=5, cap=12.0)
    d = str(tmp_path / "m")
    w = {k: v.float() for k, v in RM.write_model(llogos, d, cfg, seed=kv_rank).items()}
    model = llogos.weights.load_model(d, dtype=dtype, device="cuda:0")
    eng = llogos.engine.Engine(model, max_tokens=64 * 8)
    g = torch.Generator().manual_seed(kv_rank)
    toks = torch.randint(0, cfg["vocab"], (150,), generator=g).tolist()
    ref = RP.forward(w, cfg, toks)
    slot = eng.open()
    close(eng.step([(slot, toks)], [list(range(150))]), ref, dtype, ("long latent", "whole"))
    eng.close(slot)
    slot = eng.open()
    eng.step([(slot, toks[:70])], [[]])
    close(eng.step([(slot, toks[70:140])], [list(range(70))]), ref[70:140], dtype, ("long latent", "second portion"))
    got = [eng.step([(slot, [toks[p]])]).clone() for p in range(140, 150)]
    close(torch.cat(got), ref[140:], dtype, ("long latent", "decoded"))
    eng.close(slot)
    eng.cache.audit()


# ---- faults that random weights would hide ---------------------------------------------------------

A_TOK, B_TOK = 11, 12


def _edge_model(llogos, folder, kind, size):
    """One attention layer without feed-forward, made so that token a's key matches token b's query strongly in the
    first head: b's embedding is a's with its elements permuted inside the norm's groups, the keys' down projection is
    the queries' first projection with its columns permuted the same way, and the matrices behind them are multiples of
    the identity.  ``kind``: "latent_attention" (a window of ``size``, queries through their bottleneck) or
    "latent_attention_2" (every earlier key)."""
    if kind == "latent_attention":
        lay = RM.layer(RM.latent(2, 32, 2, 24, 32, 32, size, scale=0.125), None)
    else:
        lay = RM.layer(RM.latent2(2, 32, 2, 24, 32, scale=0.125), None)
    cfg = RM.config([lay], vocab=50, width=48, groups=2, cap=20.0)
    w = RM.random_weights(cfg, 77)
    gen = torch.Generator().manual_seed(1)
    perm = torch.cat([torch.randperm(24, generator=gen), 24 + torch.randperm(24, generator=gen)])
    w["embed"][A_TOK] = (2 * torch.randn(48, generator=gen)).to(torch.bfloat16)
    w["embed"][B_TOK] = w["embed"][A_TOK][perm]
    w["l0.norm1"][:] = 1.0
    w["l0.mix.o"] *= 4.0                                               # what the heads find weighs on the logits
    w["l0.mix.dkv.norm"][:] = 1.0
    s = torch.tensor(1.75 if kind == "latent_attention" else 3.0, dtype=torch.bfloat16)     # a far key competes with hundreds
    w["l0.mix.uk"][:32] = s * torch.eye(32, dtype=torch.bfloat16)
    if kind == "latent_attention":
        w["l0.mix.dkv"][:32][:, perm] = w["l0.mix.dq"]
        w["l0.mix.dq.norm"][:] = 1.0
        w["l0.mix.uq"][:32] = s * torch.eye(32, dtype=torch.bfloat16)
    else:
        w["l0.mix.dkv"][:32][:, perm] = w["l0.mix.q"][:32]
    RM.write_model(llogos, folder, cfg, 0, weights=w)
    return cfg, {k: v.float() for k, v in w.items()}


def _ask(eng, t, b_at, cut):
    """Logits at ``b_at``: inside a prompt of ``cut`` tokens, or decoded alone after it."""
    slot = eng.open()
    lg = eng.step([(slot, t[:cut])], [[b_at] if b_at < cut else []])
    if b_at >= cut:
        lg = eng.step([(slot, [t[b_at]])])
    lg = lg.clone()
    eng.close(slot)
    return lg


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_a_key_that_stands_out_at_the_windows_edge(llogos, tmp_path, dtype):
    """Token a stands once just inside and once just outside what the b that asks for it sees (the first of the last
    `size` positions and the one before), at the sequence's start and across page borders, in a prompt and in decoding:
    the logits there differ widely between the two, and must follow the plain model in both."""
    size = 67
    d = str(tmp_path / "edge")
    cfg, wf = _edge_model(llogos, d, "latent_attention", size)
    model = llogos.weights.load_model(d, dtype=dtype, device="cuda:0")
    eng = llogos.engine.Engine(model, max_tokens=64 * 8)
    g = torch.Generator().manual_seed(2)
    for a_at in (0, 61, 64):
        inside, outside = a_at + size - 1, a_at + size
        toks = torch.randint(13, 50, (outside + 3,), generator=g).tolist()
        toks[a_at] = A_TOK
        at_b = {}
        for b_at in (inside, outside):
            t = list(toks)
            t[b_at] = B_TOK
            ref = RP.forward(wf, cfg, t)
            at_b[b_at] = ref[b_at]
            for cut in (len(t), b_at, b_at - 1):              # b inside the prompt; b decoded first; b decoded second
                if cut == b_at - 1:
                    slot = eng.open()
                    eng.step([(slot, t[:cut])], [[]])
                    eng.step([(slot, [t[cut]])])
                    lg = eng.step([(slot, [t[b_at]])]).clone()
                    eng.close(slot)
                else:
                    lg = _ask(eng, t, b_at, cut)
                close(lg, ref[b_at:b_at + 1], dtype, ("edge", a_at, b_at, cut), tol=TIGHT)
        assert float((at_b[inside] - at_b[outside]).abs().max()) > 0.15 * float(at_b[inside].abs().max())


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_a_far_key_among_hundreds(llogos, tmp_path, dtype):
    """The same construction in the mixer that sees every earlier key: token a stands at position 2, token b 330 positions
    later (five pages on); b's logits with a there and with another token in a's place are far apart, in a prompt, in
    portions and decoded."""
    d = str(tmp_path / "far")
    cfg, wf = _edge_model(llogos, d, "latent_attention_2", 0)
    model = llogos.weights.load_model(d, dtype=dtype, device="cuda:0")
    eng = llogos.engine.Engine(model, max_tokens=64 * 8)
    gen = torch.Generator().manual_seed(3)
    toks = torch.randint(13, 50, (336,), generator=gen).tolist()
    b_at = 332
    toks[b_at] = B_TOK
    with_a, without_a = list(toks), list(toks)
    with_a[2] = A_TOK
    refs = [RP.forward(wf, cfg, t) for t in (with_a, without_a)]
    assert float((refs[0][b_at] - refs[1][b_at]).abs().max()) > 0.1 * float(refs[0][b_at].abs().max())
    for t, ref in zip((with_a, without_a), refs):
        for cut in (len(t), b_at):
            close(_ask(eng, t, b_at, cut), ref[b_at:b_at + 1], dtype, ("far key", cut), tol=TIGHT)
        slot = eng.open()
        for lo in range(0, 320, 64):
            eng.step([(slot, t[lo:lo + 64])], [[]])
        close(eng.step([(slot, t[320:])], [[b_at - 320]]), ref[b_at:b_at + 1], dtype, ("far key in portions",), tol=TIGHT)
        eng.close(slot)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_a_state_written_long_ago(llogos, tmp_path, dtype):
    """A recurrent layer whose first channels open their gate for token a alone and keep what they hold otherwise: what
    a wrote at position 2 still decides the logits 330 tokens later, whether the tokens came whole (the scan in pieces),
    in portions, or one by one; a second request beside it keeps its own state."""
    cfg = RM.config([RM.layer(RM.mingru(40), None)], vocab=50, width=48, groups=2)
    w = RM.random_weights(cfg, 78)
    gen = torch.Generator().manual_seed(4)
    w["embed"][A_TOK] = (2 * torch.randn(48, generator=gen)).to(torch.bfloat16)
    w["l0.norm1"][:] = 1.0
    wf = {k: v.float() for k, v in w.items()}
    h_a = RP.group_rms_norm(wf["embed"][A_TOK][None], wf["l0.norm1"], cfg["norm"]["eps"], 2)[0]
    keep = 12                                                          # channels that hold on to what a wrote
    w["l0.mix.z"][:keep] = (3.0 * h_a / h_a.norm()).to(torch.bfloat16)
    w["l0.mix.z.b"][:keep] = -16.0
    w["l0.mix.x.b"][:keep] = 3.0
    w["l0.mix.o"][:, :keep] *= 4.0
    wf = {k: v.float() for k, v in w.items()}
    d = str(tmp_path / "state")
    RM.write_model(llogos, d, cfg, 0, weights=w)
    model = llogos.weights.load_model(d, dtype=dtype, device="cuda:0")
    eng = llogos.engine.Engine(model, max_tokens=64 * 16)
    toks = torch.randint(13, 50, (336,), generator=gen).tolist()
    b_at = 332
    with_a, without_a = list(toks), list(toks)
    with_a[2] = A_TOK
    refs = [RP.forward(wf, cfg, t) for t in (with_a, without_a)]
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
    # both side by side: each keeps its own state, through the prompt step and through decoding
    slots = [eng.open(), eng.open()]
    eng.step([(slots[0], with_a[:200]), (slots[1], without_a[:90])], [[], []])
    eng.step([(slots[1], without_a[90:200])], [[]])
    for p in range(200, b_at):
        eng.step([(slots[0], [with_a[p]]), (slots[1], [without_a[p]])], [[], []])
    lg = eng.step([(slots[0], [with_a[b_at]]), (slots[1], [without_a[b_at]])])
    close(lg[0], refs[0][b_at], dtype, ("old state, batched, with a",), tol=TIGHT)
    close(lg[1], refs[1][b_at], dtype, ("old state, batched, without a",), tol=TIGHT)


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
            lg = RP.forward(w, cfg, toks)[-1]
            slack = 1e-4 if dtype == torch.float32 else 0.05
            assert float(lg[tok]) >= float(lg.max()) - slack * float(lg.abs().max()), (len(toks), tok)
            toks.append(tok)


def test_command_line_and_trace_replay_take_the_design(models, tmp_path):
    """``python -m llogos_b200`` generates and benchmarks a Rukedra folder, and ``bin/trace_run`` replays steps on it (two
    requests started together, decoded together, the shorter one ending first), as they do for every model."""
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
        lg = RP.forward(w, cfg, toks)[-1]
        assert float(lg[tok]) >= float(lg.max()) - 1e-4 * float(lg.abs().max())
        toks.append(tok)
    p = subprocess.run(base + ["--bench", "--batch", "2", "--prompt-len", "20:40", "--context", "80", "--seed", "1"],
                       capture_output=True, text=True, env=env, cwd=root)
    assert p.returncode == 0 and "Decode step:" in p.stderr and "Prompt step:" in p.stderr, p.stderr
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
