"""The Piratar decoder without a GPU: its configuration reader and spec, the plain implementation's mechanisms against
closed forms, and the engine's host logic (packing, cache units that keep several things, state slots used again, the
token before a step) over the CPU stand-ins of the kernels against the plain implementation."""
import copy
import math

import pytest
import torch

import cpu_ops
import piratar_models as PM
import piratar_plain as PP


def test_reader_takes_every_size_from_the_file_and_names_the_key_of_an_error(llogos):
    raw = PM.CONFIGS["mixed"]
    cfg = llogos.config.registry.architecture_of(raw).read_config(raw)
    assert (cfg.vocab, cfg.width, cfg.norm_eps, cfg.embed_scale, cfg.side_dim, len(cfg.layers)) == (173, 80, 1e-5, 4.0, 6, 5)
    assert (cfg.pair.buckets, cfg.pair.mul_prev, cfg.pair.mul_cur) == (97, 7, 13)
    r, p = cfg.layers[0].mixer, cfg.layers[1].mixer
    assert (r.width, r.blocks, r.conv) == (48, 3, 3)
    assert (p.left.heads, p.left.kv_heads, p.left.dim, p.left.vdim, p.left.conv, p.left.scale) == (4, 2, 16, 24, 4, 0.3)
    assert (p.left.rot.dims, p.left.rot.base, p.right.rot.base) == (8, 500.0, 100.0)
    assert (p.right.heads, p.right.dim, p.right.vdim, p.right.decay) == (3, 8, 12, (0.9, 0.97, 0.995))
    m = cfg.layers[1].mlp
    assert (m.experts, m.top, m.ff, m.shared_ff, m.scale) == (6, 2, 24, 16, 1.3)
    assert cfg.layers[2].mlp is None and cfg.layers[3].mlp.scale == 1.0 and cfg.layers[3].mlp.shared_ff == 0
    assert cfg.layers[4].mixer.left.rot is None and cfg.layers[0].mlp.ff == 56
    odd = llogos.config.registry.architecture_of(PM.CONFIGS["odd"]).read_config(PM.CONFIGS["odd"])
    assert odd.pair is None and odd.side_dim == 0 and odd.layers[1].mixer.left.conv == 0 and odd.layers[0].mixer.conv == 1
    ConfigError = llogos.config.ConfigError
    for path, value, word in ((("layers", 0, "mixer", "blocks"), 5, "blocks"), (("layers", 1, "mixer", "left", "kv_heads"), 3, "kv_heads"),
                              (("layers", 1, "mlp", "router", "top"), 7, "top"), (("layers", 0, "type"), "conv", "type"),
                              (("layers", 1, "mixer", "right", "decay"), [0.9, 0.8], "decay"), (("layers", 3, "mlp", "kind"), "sparse", "kind"),
                              (("layers", 1, "mixer", "left", "rot", "dims"), 7, "rot.dims"), (("layers", 1, "mixer", "right"), None, "right"),
                              (("embedding", "bigram", "buckets"), 0, "buckets"), (("token_side", "dim"), -1, "dim"),
                              (("layers", 0, "mixer", "width"), 0, "width"), (("norm", "eps"), 0.0, "eps")):
        bad = copy.deepcopy(raw)
        node = bad
        for k in path[:-1]:
            node = node[k]
        node[path[-1]] = value
        with pytest.raises(ConfigError, match=word):
            llogos.config.registry.architecture_of(bad).read_config(bad)


def test_spec_names_parts_tensors_and_cache_units(llogos):
    cfg = PM.CONFIGS["mixed"]
    model = llogos.weights.build_model(cfg, dtype=torch.float32, device="cpu", ops=cpu_ops)
    decls = model.tensor_decls()
    assert set(decls) == set(PM.random_weights(cfg, 0))
    assert decls["bigram"].shape == (98, 80) and decls["side.embed"].shape == (173, 30) and decls["l1.mlp.shared.sg"].shape == (1, 80)
    assert decls["l1.mix.left.g"].shape == (96, 80) and decls["l1.mix.left.k.conv"].shape == (32, 4) and "l2.norm2" not in decls
    assert decls["l0.mix.ra"].shape == (3, 16, 16) and decls["l3.mix.conv"].shape == (64, 2) and decls["l4.mix.right.o"].shape == (80, 8)
    base = llogos.parts.base
    needs = model.cache_needs()
    assert needs["embedding"] == base.StateNeed((1,), torch.int32) and len(needs) == 6
    assert dict(needs[0].needs) == {"state": base.StateNeed((48,), torch.float32), "conv": base.StateNeed((2, 48), torch.float32)}
    sides = dict(needs[1].needs)
    assert dict(sides["left"].needs) == {"kv": base.KvNeed(2, 16, 0, 24), "conv": base.StateNeed((3, 64 + 32 + 48), torch.float32)}
    assert sides["right"] == base.StateNeed((3, 8, 12), torch.float32)
    assert [type(b).__name__ for b in model.blocks] == ["TwoNormParallelBlock"] * 5 and len(model.spec.encodings) == 4
    odd = llogos.weights.build_model(PM.CONFIGS["odd"], dtype=torch.float32, device="cpu", ops=cpu_ops)
    assert "embedding" not in odd.cache_needs() and "side" not in odd.blocks[0].parts
    assert odd.cache_needs()[0] == base.StateNeed((30,), torch.float32)            # one tap: no inputs to keep
    assert dict(odd.cache_needs()[1].needs)["left"] == base.KvNeed(1, 10, 0, 6)    # no convolution: keys and values alone


def test_plain_mechanisms_against_closed_forms():
    # convolution: taps (1, 2, 3) on the sequence 1, 10, 100 with zeros before it
    u = torch.tensor([[1.0], [10.0], [100.0]])
    assert PP.causal_conv(u, torch.tensor([[1.0, 2.0, 3.0]])).flatten().tolist() == [3.0, 32.0, 321.0]
    # rotation by halves: a quarter turn of the pair (element 0, element 2) at position 1 with base 1 leaves the rest
    x = torch.tensor([[[1.0, 5.0, 0.0, 7.0, 9.0]]])
    y = PP.rotate_halves(x, torch.tensor([math.pi / 2], dtype=torch.float64), {"base": 1.0, "dims": 4})
    assert torch.allclose(y, torch.tensor([[[0.0, -7.0, 1.0, 5.0, 9.0]]], dtype=torch.float64), atol=1e-12)
    # retention with one head of one element, q = k = h, v = (h, 0), decay 1/2
    w = {"q": torch.tensor([[1.0]]), "k": torch.tensor([[1.0]]), "v": torch.tensor([[1.0], [0.0]]), "g": torch.full((2, 1), 50.0),
         "o": torch.eye(2)}
    h = torch.tensor([[1.0], [2.0], [4.0]])
    out = PP.retention(h, w, "", {"heads": 1, "dim": 1, "vdim": 2, "decay": [0.5]}, 1e-12)
    # o_t = (sum_j 2^-(t-j) h_j^2) h_t in column 0, 0 in column 1; unit rms over the two columns makes it sqrt(2); silu(50 h) = 50 h
    assert torch.allclose(out[:, 0], math.sqrt(2.0) * 50.0 * h[:, 0].double(), rtol=1e-9) and float(out[:, 1].abs().max()) == 0.0
    # router: weights are the chosen softmax scores over their sum, times the scale
    wr = {"router": torch.eye(3)}
    idx, wt, margin = PP.route(torch.tensor([[0.0, 2.0, 1.0]]), wr, "", {"experts": 3, "top": 2, "scale": 3.0})
    e = torch.exp(torch.tensor([2.0, 1.0], dtype=torch.float64))
    assert idx.tolist() == [[1, 2]] and torch.allclose(wt[0], 3.0 * e / e.sum()) and float(margin) > 0
    # the pair table's row
    cfg = {"embedding": {"scale": 2.0, "bigram": {"buckets": 5, "mul_prev": 3, "mul_cur": 4}}}
    we = {"embed": torch.arange(7.0)[:, None], "bigram": 100.0 * torch.arange(6.0)[:, None]}
    assert PP.embed(we, cfg, [6, 1, 2]).flatten().tolist() == [12.0 + 500.0, 2.0 + 100.0 * ((18 + 4) % 5), 4.0 + 100.0 * ((3 + 8) % 5)]
    # rglru with r -> 0 (a = 1) keeps the state; with a large rate it forgets: S_t -> i u
    wg = {"y": torch.zeros(1, 1), "y.b": torch.tensor([3.0]), "x": torch.ones(1, 1), "x.b": torch.zeros(1), "conv": torch.ones(1, 1),
          "conv.b": torch.zeros(1), "ra": torch.zeros(1, 1, 1), "ra.b": torch.tensor([[0.0]]), "ri": torch.zeros(1, 1, 1),
          "ri.b": torch.tensor([[100.0]]), "lam": torch.tensor([30.0]), "o": torch.ones(1, 1)}
    st = []
    PP.rglru(torch.tensor([[1.0], [2.0]]), wg, "", {"width": 1, "blocks": 1}, states_out=st)
    assert torch.allclose(st[0].flatten(), torch.tensor([1.0, 2.0], dtype=torch.float64))


@pytest.mark.parametrize("name", list(PM.CONFIGS))
def test_engine_host_logic_on_stand_ins(llogos, tmp_path, name):
    """Whole prompts, portions down to two tokens, a token decoded alone, unequal batches and slots used again give the
    plain model's logits when the kernels are the CPU stand-ins: packing, cache units, state rows and the token before a
    step are the engine's."""
    cfg = PM.CONFIGS[name]
    w = PM.write_model(llogos, str(tmp_path), cfg, seed=5)
    wf = {k: v.float() for k, v in w.items()}
    model = llogos.weights.load_model(str(tmp_path), dtype=torch.float32, device="cpu", ops=cpu_ops)
    eng = llogos.engine.Engine(model, max_tokens=64 * 12, n_slots=3, use_graphs=False)
    g = torch.Generator().manual_seed(3)
    seqs = [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in (1, 37, 70, 9)]
    refs = [PP.forward(wf, cfg, s) for s in seqs]

    def close(got, ref, what):
        err = float((got.double() - ref).abs().max() / ref.abs().max())
        assert err < 2e-4, (name, what, err)

    for rounds in range(2):                      # the second round finds slots, pages and state rows used before
        slot = eng.open()
        close(eng.step([(slot, seqs[2])], [list(range(70))]), refs[2], "whole")
        eng.close(slot)
        slot = eng.open()
        at, got = 0, []
        for s in (2, 2, 3, 1, 1, 29, 2, 30):
            got.append(eng.step([(slot, seqs[2][at:at + s])], [list(range(s))]).clone())
            at += s
        close(torch.cat(got), refs[2], "portions")
        eng.close(slot)
        slots = [eng.open() for _ in range(3)]
        order = [1, 0, 3] if rounds else [3, 1, 0]
        cut = {i: max(1, len(seqs[i]) - 5) for i in order}
        lg = eng.step([(slots[j], seqs[i][:cut[i]]) for j, i in enumerate(order)])
        for j, i in enumerate(order):
            close(lg[j], refs[i][cut[i] - 1], ("batched prompt", i))
        live = [(j, i) for j, i in enumerate(order) if cut[i] < len(seqs[i])]
        while live:
            lg = eng.step([(slots[j], [seqs[i][cut[i]]]) for j, i in live])
            for r, (j, i) in enumerate(live):
                close(lg[r], refs[i][cut[i]], ("batched decode", i, cut[i]))
                cut[i] += 1
            live = [(j, i) for j, i in live if cut[i] < len(seqs[i])]
        for s in slots:
            eng.close(s)
        eng.cache.audit()
    assert eng.cache.slots.free_count == eng.cache.slots.n_slots


def test_fixed_size_state_refuses_a_rollback(llogos, tmp_path):
    cfg = PM.CONFIGS["odd"]
    PM.write_model(llogos, str(tmp_path), cfg, seed=1)
    model = llogos.weights.load_model(str(tmp_path), dtype=torch.float32, device="cpu", ops=cpu_ops)
    eng = llogos.engine.Engine(model, max_tokens=128, n_slots=2, use_graphs=False)
    slot = eng.open()
    eng.step([(slot, [1, 2, 3])])
    with pytest.raises(llogos.engine.StepError, match="rolled back"):
        eng.truncate(slot, 1)
