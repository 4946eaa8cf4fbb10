"""Small Rukedra configurations with random weights for the tests: written as a model folder (config.json and
model.safetensors under the design's tensor names) so that the library loads them as it loads any checkpoint."""
import json
import math
import os

import torch


def rotation(dims, base=10000.0, scaling=None):
    r = {"base": base, "dims": dims}
    if scaling:
        factor, original, fast, slow = scaling
        r["scaling"] = {"factor": factor, "original": original, "fast": fast, "slow": slow}
    return r


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, window, base=10000.0, scaling=None, scale=None):
    """The windowed mixer: queries through a bottleneck of ``q_rank``, an output gate."""
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
         "mask": {"size": window}, "rot": rotation(rot_dim, base, scaling),
         "scale": float(scale if scale is not None else 1.0 / math.sqrt(dim + rot_dim))}
    return {"type": "latent_attention", "mixer": m}


def latent2(heads, dim, rot_dim, vdim, kv_rank, base=10000.0, scaling=None, scale=None):
    """The causal mixer: queries by one matrix, no gate."""
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
         "rot": rotation(rot_dim, base, scaling), "scale": float(scale if scale is not None else 1.0 / math.sqrt(dim + rot_dim))}
    return {"type": "latent_attention_2", "mixer": m}


def mingru(width):
    return {"type": "mingru", "mixer": {"width": width}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, shared, groups=None, scale=None):
    router = {"experts": experts, "top": top}
    if groups:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    if scale is not None:
        router["scale"] = scale
    m = {"kind": "moe", "router": router, "expert": {"ff": ff}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def layer(mixer, mlp):
    return dict(mixer, mlp=mlp)


def again(layers, j):
    """A layer that runs with layer j's tensors."""
    return dict(layers[j], weights_of=j)


def config(layers, *, vocab, width, groups, eps=1e-5, cap=None):
    c = {"architecture": "Rukedra", "vocab": vocab, "width": width, "norm": {"eps": eps, "groups": groups}, "layers": layers}
    if cap is not None:
        c["logit_softcap"] = cap
    return c


def _mixed():
    ls = [
        layer(latent(3, 16, 8, 20, 24, 12, 37, base=5000.0, scaling=(4.0, 48, 8.0, 1.0)), dense(40)),
        layer(mingru(40), moe(8, 3, 24, 16, groups=(4, 2), scale=1.7)),
        layer(latent2(2, 24, 16, 8, 16, base=300.0, scaling=(2.0, 64, 16.0, 2.0), scale=0.21), None),
    ]
    ls.append(again(ls, 0))
    ls.append(layer(mingru(56), dense(24)))
    ls.append(layer(latent2(5, 8, 4, 12, 20), moe(6, 2, 16, 0, groups=(3, 3))))
    ls.append(again(ls, 1))
    ls.append(layer(latent(2, 12, 6, 28, 10, 30, 70, base=800.0), moe(5, 1, 32, 24)))
    return config(ls, vocab=211, width=72, groups=3, cap=9.0)


def _tensor():
    # keys of 64 elements (the tensor-core attention kernels in bfloat16), widths whose products run on the tensor cores
    ls = [
        layer(latent(4, 32, 16, 32, 48, 64, 70, scaling=(8.0, 32, 4.0, 1.0)), moe(8, 2, 64, 96, groups=(2, 1), scale=2.0)),
        layer(mingru(192), dense(160)),
        layer(latent2(4, 64, 32, 64, 96, base=50000.0), moe(4, 2, 128, 0)),
        layer(mingru(128), None),
    ]
    ls.append(again(ls, 0))
    return config(ls, vocab=300, width=128, groups=4, eps=1e-6, cap=30.0)


def _odd():
    # sizes that fit no vector access and no tensor-core tile; one group (the ordinary RMS norm); a window of one
    # position; every expert chosen; one group of experts; one head; no cap on the logits
    ls = [
        layer(mingru(30), moe(3, 3, 10, 6, groups=(1, 1))),
        layer(latent(1, 10, 2, 6, 9, 7, 1), dense(14)),
        layer(latent2(5, 12, 4, 20, 20), moe(6, 4, 6, 10, groups=(3, 2), scale=0.5)),
        layer(latent(3, 6, 10, 10, 14, 5, 200, scaling=(3.0, 16, 2.0, 0.5)), None),
        layer(mingru(100), None),
    ]
    return config(ls, vocab=97, width=100, groups=1)


# Every size differs between the configurations and from one layer to the next; none is a size of a published model.
CONFIGS = {"mixed": _mixed(), "tensor": _tensor(), "odd": _odd()}

RESERVED = 8      # see random_weights(steady_routing=True)


def random_weights(cfg, seed, *, steady_routing=False):
    """bfloat16-valued tensors by the design's names.  Spreads are chosen so that activations stay of order one.

    ``steady_routing``: which experts a token gets hangs (nearly) on the token alone and never on a close call, for
    comparisons in bfloat16 where the router's input is rounded.  The last ``RESERVED`` elements of the width hold a code
    of the token that no sublayer changes (the norms that follow the sublayers have weight zero there), and the routers
    read those elements only."""
    g = torch.Generator().manual_seed(seed)

    def normal(shape, std, mean=0.0):
        return (mean + std * torch.randn(shape, generator=g)).to(torch.bfloat16)

    d = cfg["width"]
    w = {"embed": normal((cfg["vocab"], d), 1.0), "final.norm": normal((d,), 0.1, 1.0), "head": normal((cfg["vocab"], d), 2.0 * d ** -0.5)}
    if steady_routing:
        code = 1.0 + torch.rand((cfg["vocab"], RESERVED), generator=g)
        sign = torch.where(torch.rand((cfg["vocab"], RESERVED), generator=g) < 0.5, -1.0, 1.0)
        w["embed"][:, -RESERVED:] = (code * sign).to(torch.bfloat16)
    for i, lay in enumerate(cfg["layers"]):
        if "weights_of" in lay:
            continue
        m, p = lay["mixer"], f"l{i}."
        for n in ("norm1", "norm2", "norm1b", "norm2b") if lay.get("mlp") else ("norm1", "norm1b"):
            w[p + n] = normal((d,), 0.1, 1.0 if n[-1] != "b" else 0.6)
            if steady_routing:
                w[p + n][-RESERVED:] = 0.0 if n[-1] == "b" else 1.0
        for n in ("rg1", "rg2") if lay.get("mlp") else ("rg1",):
            w[p + n] = normal((d, d), 1.5 * d ** -0.5)
            w[p + n + ".b"] = normal((d,), 0.5, 0.5)
        if lay["type"] == "mingru":
            r = m["width"]
            w[p + "mix.z"], w[p + "mix.z.b"] = normal((r, d), 1.5 * d ** -0.5), normal((r,), 0.7, -0.5)
            w[p + "mix.x"], w[p + "mix.x.b"] = normal((r, d), 1.5 * d ** -0.5), normal((r,), 0.5)
            w[p + "mix.g"] = normal((r, d), 1.5 * d ** -0.5)
            w[p + "mix.o"] = normal((d, r), r ** -0.5)
        else:
            r, qw = m["kv_rank"], m["heads"] * (m["dim"] + m["rot_dim"])
            if "q_rank" in m:
                w[p + "mix.dq"] = normal((m["q_rank"], d), 1.5 * d ** -0.5)
                w[p + "mix.dq.norm"] = normal((m["q_rank"],), 0.2, 1.3)
                w[p + "mix.uq"] = normal((qw, m["q_rank"]), 1.5 * m["q_rank"] ** -0.5)
                w[p + "mix.g"] = normal((m["heads"] * m["vdim"], d), 1.5 * d ** -0.5)
            else:
                w[p + "mix.q"] = normal((qw, d), 1.5 * d ** -0.5)
            w[p + "mix.dkv"] = normal((r + m["rot_dim"], d), 1.5 * d ** -0.5)
            w[p + "mix.dkv.norm"] = normal((r,), 0.2, 1.2)
            w[p + "mix.uk"] = normal((m["heads"] * m["dim"], r), 1.5 * r ** -0.5)
            w[p + "mix.uv"] = normal((m["heads"] * m["vdim"], r), r ** -0.5)
            w[p + "mix.o"] = normal((d, m["heads"] * m["vdim"]), (m["heads"] * m["vdim"]) ** -0.5)
        ml = lay.get("mlp")
        if not ml:
            continue
        if ml["kind"] == "dense":
            ff = ml["ff"]
            w[p + "mlp.gate"], w[p + "mlp.up"] = normal((ff, d), 1.5 * d ** -0.5), normal((ff, d), 1.5 * d ** -0.5)
            w[p + "mlp.down"] = normal((d, ff), ff ** -0.5)
            continue
        e_n, ff = ml["router"]["experts"], ml["expert"]["ff"]
        if steady_routing:
            router = torch.zeros((e_n, d))
            router[:, -RESERVED:] = 0.6 * torch.randn((e_n, RESERVED), generator=g)
            w[p + "mlp.router"] = router.to(torch.bfloat16)
        else:
            w[p + "mlp.router"] = normal((e_n, d), 1.5 * d ** -0.5)
        for e in range(e_n):
            w[p + f"mlp.e{e}.gate"] = normal((ff, d), 1.5 * d ** -0.5)
            w[p + f"mlp.e{e}.up"] = normal((ff, d), 1.5 * d ** -0.5)
            w[p + f"mlp.e{e}.down"] = normal((d, ff), ff ** -0.5)
        if ml.get("shared"):
            sf = ml["shared"]["ff"]
            w[p + "mlp.shared.gate"] = normal((sf, d), d ** -0.5)
            w[p + "mlp.shared.up"] = normal((sf, d), d ** -0.5)
            w[p + "mlp.shared.down"] = normal((d, sf), sf ** -0.5)
            w[p + "mlp.shared.sg"] = normal((1, d), 2.0 * d ** -0.5)
    return w


def write_model(llogos, folder, cfg, seed, weights=None, **kw):
    os.makedirs(folder, exist_ok=True)
    w = weights if weights is not None else random_weights(cfg, seed, **kw)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    llogos.weights.write_safetensors(os.path.join(folder, "model.safetensors"), w, {"format": "pt"})
    return w
