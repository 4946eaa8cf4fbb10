"""The Rukedra decoder without a GPU: its configuration reader and spec, the plain implementation's mechanisms against
closed forms, and the engine's host logic (packing, cache, rings, recurrent state slots, a layer run twice with caches
of its own, expert layout) over the CPU stand-ins of the kernels against the plain implementation."""
import copy
import math

import pytest
import torch

import cpu_ops
import rukedra_models as RM
import rukedra_plain as RP


def test_reader_takes_every_size_from_the_file_and_names_the_key_of_an_error(llogos):
    raw = RM.CONFIGS["mixed"]
    cfg = llogos.config.registry.architecture_of(raw).read_config(raw)
    assert (cfg.vocab, cfg.width, cfg.norm_groups, cfg.norm_eps, cfg.logit_softcap, len(cfg.layers)) == (211, 72, 3, 1e-5, 9.0, 8)
    a, r, b = cfg.layers[0].mixer, cfg.layers[1].mixer, cfg.layers[2].mixer
    assert (a.heads, a.dim, a.rot_dim, a.vdim, a.kv_rank, a.q_rank, a.mask_size, a.out_gate) == (3, 16, 8, 20, 24, 12, 37, True)
    assert (a.rot.base, a.rot.scaling.factor, a.rot.scaling.original, a.rot.scaling.fast, a.rot.scaling.slow) == (5000.0, 4.0, 48.0, 8.0, 1.0)
    assert r.width == 40 and (b.heads, b.q_rank, b.mask_size, b.out_gate, b.scale) == (2, 0, 0, False, 0.21)
    m = cfg.layers[1].mlp
    assert (m.experts, m.top, m.ff, m.shared_ff, m.groups, m.keep_groups, m.scale) == (8, 3, 24, 16, 4, 2, 1.7)
    assert cfg.layers[2].mlp is None and cfg.layers[7].mlp.groups == 0 and cfg.layers[7].mlp.scale == 1.0
    assert [l.weights_of for l in cfg.layers] == [0, 1, 2, 0, 4, 5, 1, 7]
    assert llogos.config.registry.architecture_of(RM.CONFIGS["odd"]).read_config(RM.CONFIGS["odd"]).logit_softcap == 0.0
    ConfigError = llogos.config.ConfigError
    for path, value, word in ((("layers", 0, "mixer", "q_rank"), None, "q_rank"), (("layers", 2, "mixer", "rot_dim"), 7, "rot_dim"),
                              (("layers", 1, "mlp", "router", "top"), 5, "top"), (("layers", 0, "type"), "conv", "type"),
                              (("norm", "groups"), 5, "groups"), (("layers", 4, "mlp", "kind"), "sparse", "kind"),
                              (("layers", 3, "weights_of"), 1, "weights_of"), (("layers", 0, "mixer", "rot", "dims"), 6, "rot.dims"),
                              (("layers", 1, "mlp", "router", "groups", "count"), 3, "groups.count"),
                              (("layers", 1, "mixer", "width"), 0, "width"), (("logit_softcap",), -1.0, "logit_softcap")):
        bad = copy.deepcopy(raw)
        node = bad
        for k in path[:-1]:
            node = node[k]
        node[path[-1]] = value
        with pytest.raises(ConfigError, match=word):
            llogos.config.registry.architecture_of(bad).read_config(bad)


def test_spec_names_parts_tensors_and_cache_units(llogos):
    cfg = RM.CONFIGS["mixed"]
    model = llogos.weights.build_model(cfg, dtype=torch.float32, device="cpu", ops=cpu_ops)
    decls = model.tensor_decls()
    assert set(decls) == set(RM.random_weights(cfg, 0))
    assert decls["l0.mix.uq"].shape == (3 * 24, 12) and decls["l0.mix.g"].shape == (60, 72) and decls["l1.mlp.shared.sg"].shape == (1, 72)
    assert decls["l2.mix.q"].shape == (2 * 40, 72) and decls["l4.mix.z.b"].shape == (56,) and "l2.norm2" not in decls
    base = llogos.parts.base
    needs = model.cache_needs()
    assert [e.layer for e in model.spec.schedule] == [0, 1, 2, 0, 3, 4, 1, 5] and len(needs) == 8
    assert needs[0] == base.KvNeed(1, 24 + 8, 37, values_in_keys=True) == needs[3]
    assert needs[2] == base.KvNeed(1, 16 + 16, 0, values_in_keys=True)
    assert needs[1] == base.StateNeed((40,), torch.float32) == needs[6] and needs[4] == base.StateNeed((56,), torch.float32)
    assert [type(b).__name__ for b in model.blocks] == ["SandwichBlock"] * 6
    assert model.spec.head.params["softcap"] == 9.0 and len(model.spec.encodings) == 4


def test_plain_mechanisms_against_closed_forms():
    # the grouped norm: every group has unit mean square before the weight; one group is the ordinary norm
    x = torch.tensor([[3.0, 4.0, 0.0, 0.0, 1.0, 1.0, 1.0, 1.0]])
    y = RP.group_rms_norm(x, torch.ones(8), 0.0, 2)
    assert torch.allclose(y, torch.tensor([[1.2, 1.6, 0.0, 0.0, 1.0, 1.0, 1.0, 1.0]], dtype=torch.float64))
    assert torch.allclose(RP.group_rms_norm(x, torch.ones(8), 0.0, 1), RP.rms_norm(x, torch.ones(8), 0.0))
    assert torch.allclose(RP.group_rms_norm(x, 2 * torch.ones(8), 0.0, 4)[0, :2], torch.tensor([1.2, 1.6], dtype=torch.float64) * 2 * 2.5 / math.sqrt(12.5))
    # rotation of neighbours: position 0 changes nothing without scaling; lengths are kept; element 0 pairs with element 1
    rot = {"base": 100.0, "dims": 8}
    v = torch.arange(8.0).view(1, 1, 8) + 1
    assert torch.allclose(RP.rotate_pairs(v, torch.tensor([0]), rot), v.double())
    r = RP.rotate_pairs(v, torch.tensor([3]), rot)
    assert abs(float(r.norm() - v.double().norm())) < 1e-9
    f1 = 100.0 ** (-2 / 8)
    assert abs(float(r[0, 0, 0]) - (1 * math.cos(3) - 2 * math.sin(3))) < 1e-12
    assert abs(float(r[0, 0, 3]) - (4 * math.cos(3 * f1) + 3 * math.sin(3 * f1))) < 1e-12
    # stretched frequencies: fast pairs keep theirs, slow ones are divided by the factor, and the amplitude grows
    f, amp = RP.stretched_frequencies(32, 10000.0, {"factor": 4.0, "original": 256, "fast": 32.0, "slow": 1.0})
    plain_f, one = RP.stretched_frequencies(32, 10000.0, None)
    assert one == 1.0 and abs(amp - (0.1 * math.log(4.0) + 1.0)) < 1e-15
    assert float(f[0]) == float(plain_f[0]) and abs(float(f[-1]) - float(plain_f[-1]) / 4) < 1e-18
    lo, hi = math.floor(32 * math.log(256 / (2 * math.pi * 32)) / (2 * math.log(1e4))), math.ceil(32 * math.log(256 / (2 * math.pi)) / (2 * math.log(1e4)))
    mid = (lo + hi) // 2
    ramp = (mid - lo) / (hi - lo)
    assert 0 <= lo < mid < hi and abs(float(f[mid]) - float(plain_f[mid]) * (ramp / 4 + 1 - ramp)) < 1e-15
    # the window: a query sees itself and size - 1 keys before it
    wdw = RP.window_mask(7, 3)
    assert wdw[5].tolist() == [False, False, False, True, True, True, False] and wdw[1].tolist()[:3] == [True, True, False]
    assert RP.window_mask(4, None)[3].all()
    # the recurrence: a constant gate z and candidate c give S_t = c (1 - (1 - z)^t); the candidate's two branches meet at 1/2
    assert RP.mingru_candidate(torch.tensor([0.0, 2.0, -1e9, -0.0])).tolist() == [0.5, 2.5, 0.0, 0.5]
    d = 3
    w = {"m.z": torch.zeros(2, d), "m.z.b": torch.tensor([0.0, math.log(3.0)]), "m.x": torch.zeros(2, d), "m.x.b": torch.tensor([1.5, -50.0]),
         "m.g": torch.zeros(2, d), "m.o": torch.eye(2)}
    w["m.g"][:, 0] = 1.0
    h = torch.zeros(5, d)
    h[:, 0] = 2.0
    out = RP.mingru(h, w, "m.")
    silu2 = 2.0 / (1 + math.exp(-2.0))
    assert torch.allclose(out[:, 0], torch.tensor([2.0 * (1 - 0.5 ** t) * silu2 for t in range(1, 6)], dtype=torch.float64))
    assert float(out[:, 1].abs().max()) < 1e-20
    # routing: groups are judged by their two largest scores; the weights are the chosen scores over their sum, scaled
    logits = torch.tensor([[2.0, -9.0, -9.0, 1.0, 1.0, 1.0, 0.5, 3.0, -9.0]])       # groups of 3: sums of two largest
    w = {"r.router": torch.eye(9)}
    h = logits.clone()
    sg = torch.sigmoid(logits[0].double())
    idx, wt, margin = RP.route(h, w, "r.", {"experts": 9, "top": 2, "scale": 2.5, "groups": {"count": 3, "keep": 1}})
    assert idx.tolist() == [[7, 6]]           # group 2 (0.5, 3) beats group 1 (1, 1, 1) and group 0 (2 alone)
    assert torch.allclose(wt[0], 2.5 * torch.stack([sg[7], sg[6]]) / (sg[7] + sg[6]))
    assert abs(float(margin) - float(sg[6] + sg[7] - 2 * sg[3])) < 1e-12
    idx, _, _ = RP.route(h, w, "r.", {"experts": 9, "top": 3, "groups": {"count": 3, "keep": 2}})
    assert 7 in idx.tolist()[0] and set(idx.tolist()[0]) - {7} < {3, 4, 5}          # groups 2 and 1 stay
    idx, wt, _ = RP.route(h, w, "r.", {"experts": 9, "top": 2})
    assert idx.tolist() == [[7, 0]] and abs(float(wt.sum()) - 1.0) < 1e-12
    # the cap
    assert torch.allclose(RP.soft_cap(torch.tensor([0.0, 1e9, -3.0]).double(), 5.0), torch.tensor([0.0, 5.0, -5.0 * math.tanh(0.6)], dtype=torch.float64))
    assert RP.soft_cap(torch.tensor([7.0]), None).tolist() == [7.0]


@pytest.fixture(scope="module")
def small(llogos, tmp_path_factory):
    out = {}
    for i, name in enumerate(("mixed", "odd")):
        d = str(tmp_path_factory.mktemp("rukedra_" + name))
        w = RM.write_model(llogos, d, RM.CONFIGS[name], seed=31 + i)
        out[name] = (d, RM.CONFIGS[name], {k: v.float() for k, v in w.items()})
    return out


@pytest.mark.parametrize("name", ["mixed", "odd"])
def test_engine_host_logic_agrees_with_plain(llogos, small, name):
    d, cfg, w = small[name]
    model = llogos.weights.load_model(d, dtype=torch.float32, device="cpu", ops=cpu_ops)
    eng = llogos.engine.Engine(model, max_tokens=64 * 12, use_graphs=False)
    g = torch.Generator().manual_seed(0)
    seqs = [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in (1, 20, 75)]
    refs = [RP.forward(w, cfg, s) for s in seqs]
    tol = 2e-4
    for rnd in range(2):                                   # the second round uses slots, pages and state rows again
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
    # a prompt in portions of 2, 5 and the rest: the recurrent state and the windows carry over
    slot = eng.open()
    s, r = seqs[2], refs[2]
    got = [eng.step([(slot, s[a:b])], [list(range(b - a))]).clone() for a, b in ((0, 2), (2, 7), (7, len(s)))]
    assert float((torch.cat(got).double() - r).abs().max()) < tol
    eng.close(slot)


def test_cost_model_counts_a_layer_run_twice_and_the_chosen_experts(llogos):
    import importlib
    measure = importlib.import_module("daisi-llogos_b200.measure")
    cfg = RM.CONFIGS["mixed"]
    model = llogos.weights.build_model(cfg, dtype=torch.bfloat16, device="cpu", ops=cpu_ops)
    costs = measure.model_costs(model)
    d = cfg["width"]
    stored = active = 0
    for lay in cfg["layers"]:
        m = lay["mixer"]
        if lay["type"] == "mingru":
            n = 4 * d * m["width"]
        else:
            qw = m["heads"] * (m["dim"] + m["rot_dim"])
            n = (m["q_rank"] * (d + qw) + d * m["heads"] * m["vdim"]) if "q_rank" in m else d * qw
            n += d * (m["kv_rank"] + m["rot_dim"]) + m["kv_rank"] * m["heads"] * (m["dim"] + m["vdim"]) + d * m["heads"] * m["vdim"]
        n += d * d                                             # the gate on the mixer's output
        stored, active = stored + n, active + n
        ml = lay["mlp"]
        if not ml:
            continue
        stored, active = stored + d * d, active + d * d
        if ml["kind"] == "dense":
            stored, active = stored + 3 * d * ml["ff"], active + 3 * d * ml["ff"]
        else:
            e_n, top, ff, sh = ml["router"]["experts"], ml["router"]["top"], ml["expert"]["ff"], (ml.get("shared") or {}).get("ff", 0)
            gate_row = d if sh else 0
            stored += e_n * d + e_n * 3 * d * ff + 3 * d * sh + gate_row
            active += e_n * d + top * 3 * d * ff + 3 * d * sh
    assert costs.matrix_params == stored and abs(costs.active_params - active) <= 4 * d
    assert costs.kv_units[0] == ((24 + 8) * 2, 37) and len(costs.kv_units) == 5
