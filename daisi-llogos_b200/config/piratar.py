"""Typed configuration of the Piratar decoder and its model builder.

Piratar's config.json is nested and names its architecture under ``architecture``:

    {"architecture": "Piratar", "vocab": V, "width": D, "norm": {"eps": e},
     "embedding": {"scale": s, "bigram": {"buckets": B, "mul_prev": a, "mul_cur": b} | null},
     "token_side": {"dim": d} | null,
     "layers": [{"type": "parallel",
                 "mixer": {"left": {"heads": H, "kv_heads": G, "dim": dq, "vdim": dv, "scale": c, "conv": K,
                                    "rot": {"base": b, "dims": R}},
                           "right": {"heads": H', "dim": dq', "vdim": dv', "decay": [...], "rot": {...}}},
                 "mlp": {"kind": "dense", "ff": F} |
                        {"kind": "moe", "router": {"experts": E, "top": k, "scale": r}, "expert": {"ff": F},
                         "shared": {"ff": Fs} | null} | null},
                {"type": "rglru", "mixer": {"width": W, "blocks": n, "conv": K}, "mlp": ...}, ...]}

Every layer names its own sizes and its kind of mixer, so the order of kinds and all sizes may differ from layer to
layer.  What the design fixes and no file says stands below as constants: a layer is ``x' = x + mixer(N1 x) + ff(N2 x)``
with two norms of the same x (parts/block.py: ``two_norm_parallel``), followed by the token's own input
(parts/embedding.py: ``token_side_input``); the model's norms store their weights as differences from one (``1 + w``); "parallel" is
softmax attention with short convolutions behind its projections and a sigmoid gate on its heads (parts/attention.py)
beside retention (parts/recurrent.py), each RMS-normed with a weight and the two averaged (``side_by_side``); "rglru" is the
recurrent block around a real-gated linear recurrent unit (parts/recurrent.py); the mixture's router takes a softmax
over all experts and divides the chosen scores by their sum (parts/moe.py); the embedding adds a row chosen by a hash
of the token and the one before it (parts/embedding.py: ``pair_hash_embedding``).  Tensor names: ``embed``, ``bigram``,
``embed.norm``, ``side.embed``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.left.{q,k,v,g,o}``, ``l<i>.mix.left.{q,k,v}.conv``,
``l<i>.mix.right.{q,k,v,g,o}``, ``l<i>.mix.{left,right}.out``, ``l<i>.mix.{y,x,conv,ra,ri}`` (+ ``.b``), ``l<i>.mix.{lam,o}``,
``l<i>.mlp.{gate,up,down}``, ``l<i>.mlp.router``, ``l<i>.mlp.e<j>.{gate,up,down}``, ``l<i>.mlp.shared.{gate,up,down,sg}``,
``l<i>.side.{gate,proj,norm}``, ``final.norm``, ``head``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple, Union

from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .dense import ConfigError, _need
from .fipavik import Rotation, _float, _rotation
from .karitar import _obj, _positive

NAME = "Piratar"

# what the design fixes
NORM_WEIGHT_OFFSET = 1.0            # the model's norms multiply by 1 + weight
MIXER_AVERAGE = 0.5                 # the two sides of a "parallel" mixer enter as half their sum
RGLRU_DECAY_SCALE = 8.0             # log a = -8 r softplus(lam)
ROUTER_SCORE = "softmax_all"        # scores are a softmax over all experts
ROUTER_SUM_EPS = 1e-20              # added to the chosen scores' sum
DENSE_ACTIVATION = "silu"
SIDE_ACTIVATION = "gelu_tanh"


@dataclass(frozen=True)
class PairHash:
    buckets: int
    mul_prev: int
    mul_cur: int


@dataclass(frozen=True)
class ConvAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    conv: int             # taps; 0: no convolution
    rot: Optional[Rotation]


@dataclass(frozen=True)
class RetentionSide:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]
    rot: Optional[Rotation]


@dataclass(frozen=True)
class SideBySideMixer:
    left: ConvAttention
    right: RetentionSide


@dataclass(frozen=True)
class RgLruMixer:
    width: int
    blocks: int
    conv: int


@dataclass(frozen=True)
class DenseMlp:
    ff: int


@dataclass(frozen=True)
class MoeMlp:
    experts: int
    top: int
    scale: float
    ff: int
    shared_ff: int        # 0: no shared expert


@dataclass(frozen=True)
class PiratarLayer:
    type: str             # "parallel" | "rglru"
    mixer: Union[SideBySideMixer, RgLruMixer]
    mlp: Union[None, DenseMlp, MoeMlp]


@dataclass(frozen=True)
class PiratarConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    embed_scale: float
    pair: Optional[PairHash]
    side_dim: int         # 0: no per-token input
    layers: Tuple[PiratarLayer, ...]

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "PiratarConfig":
        vocab = _positive(d, "vocab")
        width = _positive(d, "width")
        eps = _need(_obj(d, "norm"), "eps", float)
        if eps <= 0:
            raise ConfigError(f"config.json: norm.eps must be positive, got {eps}")
        em = d.get("embedding") or {}
        if not isinstance(em, Mapping):
            raise ConfigError("config.json: embedding must be an object")
        scale = _need(em, "scale", float, default=1.0, required=False)
        pair = None
        if em.get("bigram") is not None:
            bg = _obj(em, "bigram")
            buckets = _positive(bg, "buckets", "embedding.bigram.")
            # only a multiplier's remainder matters; taking it here keeps the products small and not negative
            pair = PairHash(buckets, _int(bg, "mul_prev", "embedding.bigram.", negative=True) % buckets,
                            _int(bg, "mul_cur", "embedding.bigram.", negative=True) % buckets)
        side_dim = 0
        if d.get("token_side") is not None:
            side_dim = _positive(_obj(d, "token_side"), "dim", "token_side.")
        raw_layers = d.get("layers")
        if not isinstance(raw_layers, (list, tuple)) or not raw_layers:
            raise ConfigError("config.json: missing key 'layers' (a non-empty list of layers)")
        layers = tuple(_layer(i, raw) for i, raw in enumerate(raw_layers))
        return cls(architecture=str(d.get("architecture", NAME)), vocab=vocab, width=width, norm_eps=eps,
                   embed_scale=scale, pair=pair, side_dim=side_dim, layers=layers)


def _int(d: Mapping[str, Any], key: str, where: str, negative: bool = False) -> int:
    try:
        v = _need(d, key, int)
    except ConfigError as e:
        raise ConfigError(str(e).replace(f"'{key}'", f"'{where}{key}'")) from None
    if v < 0 and not negative:
        raise ConfigError(f"config.json: key '{where}{key}' must not be negative, got {v}")
    return v


def _taps(m: Mapping[str, Any], where: str) -> int:
    if m.get("conv") is None:
        return 0
    return _int(m, "conv", where)


def _layer(i: int, raw: Any) -> PiratarLayer:
    where = f"layers[{i}]."
    if not isinstance(raw, Mapping):
        raise ConfigError(f"config.json: layers[{i}] must be an object")
    kind = raw.get("type")
    if kind not in ("parallel", "rglru"):
        raise ConfigError(f"config.json: {where}type = {kind!r} is not supported (known: 'parallel', 'rglru')")
    if not isinstance(raw.get("mixer"), Mapping):
        raise ConfigError(f"config.json: {where}mixer must be an object")
    m, mw = raw["mixer"], where + "mixer."
    if kind == "rglru":
        width, blocks = _positive(m, "width", mw), _positive(m, "blocks", mw)
        if width % blocks:
            raise ConfigError(f"config.json: {mw}width {width} is not a multiple of {mw}blocks {blocks}")
        mixer = RgLruMixer(width, blocks, max(1, _taps(m, mw)))
    else:
        for side in ("left", "right"):
            if not isinstance(m.get(side), Mapping):
                raise ConfigError(f"config.json: {mw}{side} must be an object")
        le, lw = m["left"], mw + "left."
        heads, kv_heads = _positive(le, "heads", lw), _positive(le, "kv_heads", lw)
        if heads % kv_heads:
            raise ConfigError(f"config.json: {lw}heads {heads} is not a multiple of {lw}kv_heads {kv_heads}")
        dim = _positive(le, "dim", lw)
        scale = _float(le, "scale", lw)
        if not scale > 0:
            raise ConfigError(f"config.json: {lw}scale must be positive, got {scale}")
        left = ConvAttention(heads, kv_heads, dim, _positive(le, "vdim", lw), scale, _taps(le, lw), _rotation(le, lw, dim, "dim"))
        ri, rw = m["right"], mw + "right."
        r_heads, r_dim = _positive(ri, "heads", rw), _positive(ri, "dim", rw)
        decay = ri.get("decay")
        if not isinstance(decay, (list, tuple)) or len(decay) != r_heads or \
                not all(isinstance(x, (int, float)) and not isinstance(x, bool) and 0 <= x <= 1 for x in decay):
            raise ConfigError(f"config.json: {rw}decay must list one number in [0, 1] per head ({r_heads})")
        right = RetentionSide(r_heads, r_dim, _positive(ri, "vdim", rw), tuple(float(x) for x in decay),
                              _rotation(ri, rw, r_dim, "dim"))
        mixer = SideBySideMixer(left, right)
    mlp = None
    if raw.get("mlp") is not None:
        ml, lw = raw["mlp"], where + "mlp."
        if not isinstance(ml, Mapping):
            raise ConfigError(f"config.json: {where}mlp must be an object or null")
        if ml.get("kind") == "dense":
            mlp = DenseMlp(_positive(ml, "ff", lw))
        elif ml.get("kind") == "moe":
            router = _obj(ml, "router")
            experts, top = _positive(router, "experts", lw + "router."), _positive(router, "top", lw + "router.")
            if top > experts:
                raise ConfigError(f"config.json: {lw}router.top {top} exceeds {lw}router.experts {experts}")
            r_scale = _need(router, "scale", float, default=1.0, required=False)
            ff = _positive(_obj(ml, "expert"), "ff", lw + "expert.")
            shared = 0
            if ml.get("shared") is not None:
                shared = _positive(_obj(ml, "shared"), "ff", lw + "shared.")
            mlp = MoeMlp(experts, top, r_scale, ff, shared)
        else:
            raise ConfigError(f"config.json: {lw}kind = {ml.get('kind')!r} is not supported (known: 'dense', 'moe')")
    return PiratarLayer(kind, mixer, mlp)


def _encoding(encodings: Dict[str, PartSpec], rot: Optional[Rotation]) -> Optional[str]:
    """The name of the rotary tables for ``rot`` (mixers with the same base and size share them)."""
    if rot is None:
        return None
    name = f"rot{rot.dims}@{rot.base!r}"
    if name not in encodings:
        encodings[name] = PartSpec("rotary", {"head_dim": rot.dims, "rotary_dim": rot.dims, "theta": rot.base,
                                              "scaling": None, "pairing": "half"})
    return name


_GATED = {"gate_proj.weight": "gate", "up_proj.weight": "up", "down_proj.weight": "down"}


def piratar_spec(cfg: PiratarConfig) -> ModelSpec:
    """Parts and run order of a Piratar model (see the module's text for what the design fixes)."""
    norm = {"size": cfg.width, "eps": cfg.norm_eps, "weight_offset": NORM_WEIGHT_OFFSET}
    encodings: Dict[str, PartSpec] = {}
    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = layer.mixer
        if layer.type == "rglru":
            mixer = PartSpec("rglru", {
                "hidden_size": cfg.width, "state_size": m.width, "blocks": m.blocks, "conv_taps": m.conv,
                "decay_scale": RGLRU_DECAY_SCALE,
                "tensor_names": {"y_proj.weight": "y", "y_proj.bias": "y.b", "x_proj.weight": "x", "x_proj.bias": "x.b",
                                 "conv.weight": "conv", "conv.bias": "conv.b", "a_gate.weight": "ra", "a_gate.bias": "ra.b",
                                 "i_gate.weight": "ri", "i_gate.bias": "ri.b", "lam": "lam", "o_proj.weight": "o"},
            }, p + "mix.")
        else:
            le, ri = m.left, m.right
            left = {"kind": "attention", "params": {
                "hidden_size": cfg.width, "num_heads": le.heads, "num_kv_heads": le.kv_heads, "head_dim": le.dim,
                "value_dim": le.vdim, "qkv_bias": False, "qk_norm": False, "window": 0, "softmax_scale": le.scale,
                "conv_taps": le.conv, "out_gate": True, "position": _encoding(encodings, le.rot),
                "tensor_names": {"q_proj.weight": "q", "k_proj.weight": "k", "v_proj.weight": "v", "o_proj.weight": "o",
                                 "g_proj.weight": "g", "q_proj.conv": "q.conv", "k_proj.conv": "k.conv",
                                 "v_proj.conv": "v.conv"}}}
            right = {"kind": "retention", "params": {
                "hidden_size": cfg.width, "num_heads": ri.heads, "head_dim": ri.dim, "value_dim": ri.vdim,
                "decay": list(ri.decay), "norm_eps": cfg.norm_eps, "position": _encoding(encodings, ri.rot),
                "tensor_names": {"q_proj.weight": "q", "k_proj.weight": "k", "v_proj.weight": "v", "g_proj.weight": "g",
                                 "o_proj.weight": "o"}}}
            mixer = PartSpec("side_by_side", {"hidden_size": cfg.width, "eps": cfg.norm_eps, "scale": MIXER_AVERAGE,
                                              "left": left, "right": right}, p + "mix.")
        parts = {"norm1": PartSpec("rmsnorm", dict(norm, tensor_names={"weight": "norm1"}), p), "mixer": mixer}
        ml = layer.mlp
        if ml is not None:
            parts["norm2"] = PartSpec("rmsnorm", dict(norm, out_name="norm.out2", tensor_names={"weight": "norm2"}), p)
            if isinstance(ml, DenseMlp):
                parts["ffn"] = PartSpec("swiglu", {"hidden_size": cfg.width, "intermediate_size": ml.ff,
                                                   "activation": DENSE_ACTIVATION, "tensor_names": dict(_GATED)}, p + "mlp.")
            else:
                parts["ffn"] = PartSpec("moe", {
                    "hidden_size": cfg.width, "num_experts": ml.experts, "top": ml.top, "expert_size": ml.ff,
                    "shared_size": ml.shared_ff, "router_bias": False, "score": ROUTER_SCORE,
                    "weight_scale": ml.scale, "weight_sum_eps": ROUTER_SUM_EPS, "shared_gate": bool(ml.shared_ff),
                    "shared_prefix": "shared.", "shared_names": dict(_GATED),
                    "tensor_names": {"router.weight": "router", "shared_gate.weight": "shared.sg",
                                     "experts.*.gate_proj.weight": "e*.gate", "experts.*.up_proj.weight": "e*.up",
                                     "experts.*.down_proj.weight": "e*.down"},
                }, p + "mlp.")
        if cfg.side_dim:
            parts["side"] = PartSpec("token_side_input", {
                "hidden_size": cfg.width, "dim": cfg.side_dim, "offset": i * cfg.side_dim, "eps": cfg.norm_eps,
                "activation": SIDE_ACTIVATION, "tied_to": "side.embed",
                "tensor_names": {"gate.weight": "gate", "proj.weight": "proj", "norm.weight": "norm"}}, p + "side.")
        layers.append(LayerSpec("two_norm_parallel", parts))
    embed_names = {"weight": "embed", "pair.weight": "bigram", "norm.weight": "embed.norm", "side.weight": "side.embed"}
    spec = ModelSpec(
        hidden_size=cfg.width,
        vocab_size=cfg.vocab,
        max_positions=None,                       # the rotation has no limit of its own: the cache's size is the limit
        embedding=PartSpec("pair_hash_embedding", {
            "vocab_size": cfg.vocab, "hidden_size": cfg.width, "scale": cfg.embed_scale,
            "pair": None if cfg.pair is None else {"buckets": cfg.pair.buckets, "mul_prev": cfg.pair.mul_prev,
                                                   "mul_cur": cfg.pair.mul_cur},
            "norm_eps": cfg.norm_eps, "norm_offset": NORM_WEIGHT_OFFSET,
            "side_width": cfg.side_dim * len(cfg.layers), "tensor_names": embed_names}, ""),
        encodings=encodings,
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in range(len(layers))),
        final_norm=PartSpec("rmsnorm", dict(norm, tensor_names={"weight": "final.norm"}), ""),
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "tied_to": None,
                                      "tensor_names": {"weight": "head"}}, ""),
    )
    spec.validate()
    return spec
