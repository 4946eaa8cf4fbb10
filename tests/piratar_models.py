"""Small Piratar configurations with random weights for the tests: written as a model folder (config.json and
model.safetensors under the design's tensor names) so that the library loads them as it loads any checkpoint."""
import json
import os

import torch


def rotation(dims, base=10000.0):
    return {"base": base, "dims": dims}


def left(heads, kv_heads, dim, vdim, conv, rot_dims, base=10000.0, scale=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": float(scale if scale is not None else dim ** -0.5)}
    if conv:
        m["conv"] = conv
    if rot_dims:
        m["rot"] = rotation(rot_dims, base)
    return m


def right(heads, dim, vdim, decay, rot_dims, base=10000.0):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}
    if rot_dims:
        m["rot"] = rotation(rot_dims, base)
    return m


def parallel(le, ri):
    return {"type": "parallel", "mixer": {"left": le, "right": ri}}


def rglru(width, blocks, conv):
    return {"type": "rglru", "mixer": {"width": width, "blocks": blocks, "conv": conv}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, shared, scale=None):
    router = {"experts": experts, "top": top}
    if scale is not None:
        router["scale"] = scale
    m = {"kind": "moe", "router": router, "expert": {"ff": ff}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def layer(mixer, mlp):
    return dict(mixer, mlp=mlp)


def config(layers, *, vocab, width, eps=1e-5, scale=1.0, bigram=None, side=0):
    c = {"architecture": "Piratar", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers,
         "embedding": {"scale": scale}}
    if bigram:
        c["embedding"]["bigram"] = {"buckets": bigram[0], "mul_prev": bigram[1], "mul_cur": bigram[2]}
    if side:
        c["token_side"] = {"dim": side}
    return c


def _mixed():
    ls = [
        layer(rglru(48, 3, 3), dense(56)),
        layer(parallel(left(4, 2, 16, 24, 4, 8, base=500.0, scale=0.3), right(3, 8, 12, (0.9, 0.97, 0.995), 8, base=100.0)),
              moe(6, 2, 24, 16, scale=1.3)),
        layer(parallel(left(2, 2, 32, 32, 2, 32), right(2, 16, 16, (1.0, 0.75), 4)), None),
        layer(rglru(64, 1, 2), moe(5, 1, 32, 0)),
        layer(parallel(left(6, 3, 8, 40, 5, 0), right(1, 24, 8, (0.99,), 0)), dense(24)),
    ]
    return config(ls, vocab=173, width=80, scale=4.0, bigram=(97, 7, 13), side=6)


def _tensor():
    # heads of 64 elements with values of the same size (the tensor-core attention kernels in bfloat16), widths whose
    # products run on the tensor cores, gate blocks of 64 channels
    ls = [
        layer(parallel(left(4, 1, 64, 64, 4, 64, base=50000.0), right(2, 32, 64, (0.98, 0.999), 32)), moe(8, 2, 64, 96, scale=2.0)),
        layer(rglru(256, 4, 4), dense(160)),
        layer(parallel(left(2, 2, 128, 128, 3, 64), right(4, 64, 32, (0.9, 0.95, 0.99, 0.999), 16)), moe(4, 2, 128, 0)),
        layer(rglru(128, 2, 2), None),
    ]
    return config(ls, vocab=300, width=128, eps=1e-6, scale=11.0, bigram=(509, 3, 5), side=16)


def _odd():
    # sizes that fit no vector access and no tensor-core tile; no pair table, no per-token input; a left side without a
    # convolution and without rotation; every expert chosen; one head; one tap
    ls = [
        layer(rglru(30, 5, 1), moe(3, 3, 10, 6)),
        layer(parallel(left(3, 1, 10, 6, 0, 0), right(1, 10, 14, (0.5,), 0)), dense(14)),
        layer(parallel(left(1, 1, 12, 20, 7, 6), right(5, 6, 6, (0.9, 0.9, 1.0, 0.2, 0.999), 6, base=30.0)), moe(6, 4, 6, 10, scale=0.5)),
        layer(rglru(100, 4, 6), None),
    ]
    return config(ls, vocab=97, width=100)


# Every size differs between the configurations and from one layer to the next; none is a size of a published model.
CONFIGS = {"mixed": _mixed(), "tensor": _tensor(), "odd": _odd()}

RESERVED = 8      # see random_weights(steady_routing=True)


def random_weights(cfg, seed, *, steady_routing=False):
    """bfloat16-valued tensors by the design's names.  Spreads are chosen so that activations stay of order one.

    ``steady_routing``: which experts a token gets hangs (nearly) on the token alone and never on a close call, for
    comparisons in bfloat16 where the router's input is rounded.  The last ``RESERVED`` elements of the width hold a code
    of the token that no sublayer changes (whatever enters the residual has weight zero there), and the routers read
    those elements only."""
    g = torch.Generator().manual_seed(seed)

    def normal(shape, std, mean=0.0):
        return (mean + std * torch.randn(shape, generator=g)).to(torch.bfloat16)

    d, v = cfg["width"], cfg["vocab"]
    n_layers = len(cfg["layers"])
    w = {"embed": normal((v, d), 1.0), "embed.norm": normal((d,), 0.1), "final.norm": normal((d,), 0.1),
         "head": normal((v, d), 2.0 * d ** -0.5)}
    bg = cfg["embedding"].get("bigram")
    if bg:
        w["bigram"] = normal((bg["buckets"] + 1, d), 2.0)
    side = (cfg.get("token_side") or {}).get("dim", 0)
    if side:
        w["side.embed"] = normal((v, side * n_layers), 1.0)
    if steady_routing:
        code = 1.0 + torch.rand((v, RESERVED), generator=g)
        sign = torch.where(torch.rand((v, RESERVED), generator=g) < 0.5, -1.0, 1.0)
        w["embed"][:, -RESERVED:] = (code * sign * 4.0 / cfg["embedding"]["scale"]).to(torch.bfloat16)
        w["embed.norm"][-RESERVED:] = 0.0
        if bg:
            w["bigram"][:, -RESERVED:] = 0.0

    def into_residual(t):
        """A matrix [width, .] or vector [width] whose product enters the residual: nothing of it reaches the code."""
        if steady_routing:
            t[-RESERVED:] = 0.0
        return t

    for i, lay in enumerate(cfg["layers"]):
        m, p = lay["mixer"], f"l{i}."
        for n in ("norm1", "norm2") if lay.get("mlp") else ("norm1",):
            w[p + n] = normal((d,), 0.1)
        if lay["type"] == "rglru":
            r, b, k = m["width"], m["blocks"], m.get("conv") or 1
            bw = r // b
            w[p + "mix.y"], w[p + "mix.y.b"] = normal((r, d), 1.5 * d ** -0.5), normal((r,), 0.3)
            w[p + "mix.x"], w[p + "mix.x.b"] = normal((r, d), 1.5 * d ** -0.5), normal((r,), 0.3)
            w[p + "mix.conv"], w[p + "mix.conv.b"] = normal((r, k), 0.6), normal((r,), 0.2)
            w[p + "mix.ra"], w[p + "mix.ra.b"] = normal((b, bw, bw), bw ** -0.5), normal((b, bw), 0.5)
            w[p + "mix.ri"], w[p + "mix.ri.b"] = normal((b, bw, bw), bw ** -0.5), normal((b, bw), 0.5, 0.5)
            w[p + "mix.lam"] = normal((r,), 1.0, -2.5)
            w[p + "mix.o"] = into_residual(normal((d, r), 2.0 * r ** -0.5))
        else:
            le, ri = m["left"], m["right"]
            q, kv, vv = le["heads"] * le["dim"], le["kv_heads"] * le["dim"], le["kv_heads"] * le["vdim"]
            ov = le["heads"] * le["vdim"]
            w[p + "mix.left.q"], w[p + "mix.left.k"] = normal((q, d), 1.5 * d ** -0.5), normal((kv, d), 1.5 * d ** -0.5)
            w[p + "mix.left.v"], w[p + "mix.left.g"] = normal((vv, d), d ** -0.5), normal((ov, d), 1.5 * d ** -0.5)
            w[p + "mix.left.o"] = normal((d, ov), ov ** -0.5)
            if le.get("conv"):
                for n, c in (("q", q), ("k", kv), ("v", vv)):
                    w[p + f"mix.left.{n}.conv"] = normal((c, le["conv"]), 0.6)
            rq, rv = ri["heads"] * ri["dim"], ri["heads"] * ri["vdim"]
            w[p + "mix.right.q"], w[p + "mix.right.k"] = normal((rq, d), 1.5 * d ** -0.5), normal((rq, d), 1.5 * d ** -0.5)
            w[p + "mix.right.v"], w[p + "mix.right.g"] = normal((rv, d), d ** -0.5), normal((rv, d), 1.5 * d ** -0.5)
            w[p + "mix.right.o"] = normal((d, rv), rv ** -0.5)
            w[p + "mix.left.out"] = into_residual(normal((d,), 0.1, 0.8))
            w[p + "mix.right.out"] = into_residual(normal((d,), 0.1, 0.6))
        if side:
            w[p + "side.gate"], w[p + "side.proj"] = normal((side, d), d ** -0.5), normal((d, side), side ** -0.5)
            w[p + "side.norm"] = into_residual(normal((d,), 0.1, 0.5))
        ml = lay.get("mlp")
        if not ml:
            continue
        if ml["kind"] == "dense":
            ff = ml["ff"]
            w[p + "mlp.gate"], w[p + "mlp.up"] = normal((ff, d), 1.5 * d ** -0.5), normal((ff, d), 1.5 * d ** -0.5)
            w[p + "mlp.down"] = into_residual(normal((d, ff), ff ** -0.5))
            continue
        e_n, ff = ml["router"]["experts"], ml["expert"]["ff"]
        if steady_routing:
            router = torch.zeros((e_n, d))
            router[:, -RESERVED:] = 1.5 * torch.randn((e_n, RESERVED), generator=g)
            w[p + "mlp.router"] = router.to(torch.bfloat16)
            w[p + "norm2"][-RESERVED:] = 0.0
        else:
            w[p + "mlp.router"] = normal((e_n, d), 1.5 * d ** -0.5)
        for e in range(e_n):
            w[p + f"mlp.e{e}.gate"] = normal((ff, d), 1.5 * d ** -0.5)
            w[p + f"mlp.e{e}.up"] = normal((ff, d), 1.5 * d ** -0.5)
            w[p + f"mlp.e{e}.down"] = into_residual(normal((d, ff), ff ** -0.5))
        if ml.get("shared"):
            sf = ml["shared"]["ff"]
            w[p + "mlp.shared.gate"] = normal((sf, d), d ** -0.5)
            w[p + "mlp.shared.up"] = normal((sf, d), d ** -0.5)
            w[p + "mlp.shared.down"] = into_residual(normal((d, sf), sf ** -0.5))
            w[p + "mlp.shared.sg"] = normal((1, d), 2.0 * d ** -0.5)
    return w


def write_model(llogos, folder, cfg, seed, weights=None, **kw):
    os.makedirs(folder, exist_ok=True)
    w = weights if weights is not None else random_weights(cfg, seed, **kw)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    llogos.weights.write_safetensors(os.path.join(folder, "model.safetensors"), w, {"format": "pt"})
    return w
