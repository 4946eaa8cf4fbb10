"""Typed configuration of the Rukedra decoder and its model builder.

Rukedra's config.json is nested and names its architecture under ``architecture``:

    {"architecture": "Rukedra", "vocab": V, "width": D, "norm": {"eps": e, "groups": G}, "logit_softcap": c,
     "layers": [{"type": "latent_attention",
                 "mixer": {"heads": H, "dim": dq, "rot_dim": dr, "vdim": dv, "kv_rank": L, "q_rank": Lq, "scale": s,
                           "mask": {"size": W}, "rot": {"base": b, "dims": dr, "scaling": {"factor": f, "original": n,
                                                                                           "fast": a, "slow": z}}},
                 "mlp": {"kind": "dense", "ff": F} | {"kind": "moe", "router": {"experts": E, "top": K, "scale": r,
                         "groups": {"count": C, "keep": M}}, "expert": {"ff": F}, "shared": {"ff": Fs}} | null},
                {"type": "latent_attention_2", "mixer": {... no q_rank, no mask ...}, "mlp": ...},
                {"type": "mingru", "mixer": {"width": R}, "mlp": ...},
                {"type": ..., "mixer": ..., "mlp": ..., "weights_of": j}, ...]}

Every layer names its own kind of mixer and its own sizes.  A layer with ``weights_of: j`` has no tensors: it runs with
layer j's (mixer, feed-forward, norms and gates) and keeps a cache or state of its own; in the run order it is a second
entry of layer j.  What the design fixes and no file says stands below as constants: every sublayer sits between two
grouped RMS norms and its output passes an element-wise sigmoid gate computed from the sublayer's input
(parts/sandwich.py); "latent_attention" sends its queries through a normed bottleneck, looks at a sliding window and
gates its concatenated heads; "latent_attention_2" projects its queries directly and sees every earlier key; both rotate
neighbouring pairs with stretched frequencies (parts/position.py: ``yarn``) and use an ordinary softmax
(parts/latent_attention.py); "mingru" is a gated recurrence with a fixed-size float32 state (parts/recurrent.py); the
dense feed-forward is gated with the tanh form of gelu, the mixture's experts with silu, its router scores are sigmoids
chosen within the best groups and normalised (parts/moe.py); the logits pass a tanh cap.  Tensor names: ``embed``,
``l<i>.norm{1,2}``, ``l<i>.norm{1,2}b``, ``l<i>.rg{1,2}`` (+ ``.b``), ``l<i>.mix.{dq,uq,q,dkv,uk,uv,g,o}``,
``l<i>.mix.{dq,dkv}.norm``, ``l<i>.mix.{z,x}`` (+ ``.b``), ``l<i>.mlp.{gate,up,down}``, ``l<i>.mlp.router``,
``l<i>.mlp.e<j>.{gate,up,down}``, ``l<i>.mlp.shared.{gate,up,down,sg}``, ``final.norm``, ``head``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple, Union

from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .dense import ConfigError, _need
from .fipavik import _float, _mask_size
from .karitar import _obj, _positive

NAME = "Rukedra"

# what the design fixes
DENSE_ACTIVATION = "gelu_tanh"      # the dense feed-forward's gate
EXPERT_ACTIVATION = "silu"          # the experts' gate
ROUTER_SCORE = "sigmoid"            # router scores; the chosen ones are divided by their sum
ROUTER_SUM_EPS = 1e-20              # added to that sum
GROUP_SCORE_TOP = 2                 # a group of experts is judged by the sum of this many of its largest scores
ROTATION_PAIRING = "adjacent"       # element 2i turns with element 2i + 1
YARN_AMPLITUDE_SLOPE = 0.1          # cos and sin are multiplied by slope * ln(factor) + 1
MIXER_KINDS = ("latent_attention", "latent_attention_2", "mingru")


@dataclass(frozen=True)
class RotationScaling:
    factor: float
    original: float
    fast: float
    slow: float


@dataclass(frozen=True)
class Rotation:
    base: float
    dims: int
    scaling: Optional[RotationScaling]


@dataclass(frozen=True)
class RukedraLatentAttention:
    heads: int
    dim: int              # unrotated elements of a query / key head
    rot_dim: int          # rotated elements
    vdim: int
    kv_rank: int
    q_rank: int           # 0: queries by one matrix
    scale: float
    mask_size: int        # 0: every earlier key
    rot: Optional[Rotation]
    out_gate: bool


@dataclass(frozen=True)
class RukedraMinGru:
    width: int


@dataclass(frozen=True)
class RukedraDense:
    ff: int


@dataclass(frozen=True)
class RukedraMoe:
    experts: int
    top: int
    ff: int
    shared_ff: int        # 0: no shared expert
    groups: int           # 0: every expert is eligible
    keep_groups: int
    scale: float


@dataclass(frozen=True)
class RukedraLayer:
    type: str
    mixer: Union[RukedraLatentAttention, RukedraMinGru]
    mlp: Union[None, RukedraDense, RukedraMoe]
    weights_of: int       # the layer whose tensors this one runs with (its own index where it has its own)


@dataclass(frozen=True)
class RukedraConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    norm_groups: int
    logit_softcap: float  # 0: none
    layers: Tuple[RukedraLayer, ...]

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "RukedraConfig":
        vocab = _positive(d, "vocab")
        width = _positive(d, "width")
        norm = _obj(d, "norm")
        eps = _need(norm, "eps", float)
        if eps <= 0:
            raise ConfigError(f"config.json: norm.eps must be positive, got {eps}")
        groups = 1 if norm.get("groups") is None else _positive(norm, "groups", "norm.")
        if width % groups:
            raise ConfigError(f"config.json: width {width} is not a multiple of norm.groups {groups}")
        cap = 0.0
        if d.get("logit_softcap") is not None:
            cap = _need(d, "logit_softcap", float)
            if not cap > 0:
                raise ConfigError(f"config.json: logit_softcap must be positive, got {cap}")
        raw_layers = d.get("layers")
        if not isinstance(raw_layers, (list, tuple)) or not raw_layers:
            raise ConfigError("config.json: missing key 'layers' (a non-empty list of layers)")
        layers = [_layer(i, raw, len(raw_layers)) for i, raw in enumerate(raw_layers)]
        for i, layer in enumerate(layers):
            j = layer.weights_of
            if j != i:
                if layers[j].weights_of != j:
                    raise ConfigError(f"config.json: layers[{i}].weights_of = {j} names a layer that has no tensors of its own")
                same = (layers[j].type, layers[j].mixer, layers[j].mlp) == (layer.type, layer.mixer, layer.mlp)
                if not same:
                    raise ConfigError(f"config.json: layers[{i}] runs with the tensors of layers[{j}] (weights_of), so its "
                                      f"type, mixer and mlp must equal that layer's")
        return cls(architecture=str(d.get("architecture", NAME)), vocab=vocab, width=width, norm_eps=eps,
                   norm_groups=groups, logit_softcap=cap, layers=tuple(layers))


def _rotation(m: Mapping[str, Any], where: str, rot_dim: int) -> Optional[Rotation]:
    rot = m.get("rot")
    if rot is None:
        return None
    if not isinstance(rot, Mapping):
        raise ConfigError(f"config.json: {where}rot must be an object or null")
    base = _float(rot, "base", where + "rot.")
    dims = _positive(rot, "dims", where + "rot.")
    if not base > 1:
        raise ConfigError(f"config.json: {where}rot.base must be above 1, got {base}")
    if dims % 2 or dims != rot_dim:
        raise ConfigError(f"config.json: {where}rot.dims {dims} must be even and equal rot_dim {rot_dim}")
    scaling = None
    if rot.get("scaling") is not None:
        s, sw = rot["scaling"], where + "rot.scaling."
        if not isinstance(s, Mapping):
            raise ConfigError(f"config.json: {where}rot.scaling must be an object or null")
        scaling = RotationScaling(_float(s, "factor", sw), _float(s, "original", sw), _float(s, "fast", sw), _float(s, "slow", sw))
        for key, v in (("factor", scaling.factor), ("original", scaling.original), ("fast", scaling.fast), ("slow", scaling.slow)):
            if not v > 0:
                raise ConfigError(f"config.json: {sw}{key} must be positive, got {v}")
    return Rotation(base, dims, scaling)


def _mlp(ml: Any, where: str):
    if ml is None:
        return None
    lw = where + "mlp."
    if not isinstance(ml, Mapping):
        raise ConfigError(f"config.json: {where}mlp must be an object or null")
    kind = ml.get("kind")
    if kind == "dense":
        return RukedraDense(_positive(ml, "ff", lw))
    if kind != "moe":
        raise ConfigError(f"config.json: {lw}kind = {kind!r} is not supported (known: 'dense', 'moe')")
    router = _obj(ml, "router")
    rw = lw + "router."
    experts, top = _positive(router, "experts", rw), _positive(router, "top", rw)
    groups = keep = 0
    if router.get("groups") is not None:
        g = router["groups"]
        if not isinstance(g, Mapping):
            raise ConfigError(f"config.json: {rw}groups must be an object or null")
        groups, keep = _positive(g, "count", rw + "groups."), _positive(g, "keep", rw + "groups.")
        if experts % groups:
            raise ConfigError(f"config.json: {rw}experts {experts} is not a multiple of {rw}groups.count {groups}")
        if keep > groups:
            raise ConfigError(f"config.json: {rw}groups.keep {keep} exceeds {rw}groups.count {groups}")
    eligible = experts if not groups else keep * (experts // groups)
    if top > eligible:
        raise ConfigError(f"config.json: {rw}top {top} exceeds the {eligible} experts a token can choose from")
    scale = 1.0 if router.get("scale") is None else _float(router, "scale", rw)
    ff = _positive(_obj(ml, "expert"), "ff", lw + "expert.")
    shared = 0
    if ml.get("shared") is not None:
        shared = _positive(_obj(ml, "shared"), "ff", lw + "shared.")
    return RukedraMoe(experts, top, ff, shared, groups, keep, scale)


def _layer(i: int, raw: Any, n_layers: int) -> RukedraLayer:
    where = f"layers[{i}]."
    if not isinstance(raw, Mapping):
        raise ConfigError(f"config.json: layers[{i}] must be an object")
    kind = raw.get("type")
    if kind not in MIXER_KINDS:
        known = ", ".join(repr(k) for k in MIXER_KINDS)
        raise ConfigError(f"config.json: {where}type = {kind!r} is not supported (known: {known})")
    if not isinstance(raw.get("mixer"), Mapping):
        raise ConfigError(f"config.json: {where}mixer must be an object")
    m, mw = raw["mixer"], where + "mixer."
    if kind == "mingru":
        mixer = RukedraMinGru(_positive(m, "width", mw))
    else:
        heads = _positive(m, "heads", mw)
        dim, vdim = _positive(m, "dim", mw), _positive(m, "vdim", mw)
        scale = _float(m, "scale", mw)
        if not scale > 0:
            raise ConfigError(f"config.json: {mw}scale must be positive, got {scale}")
        rot_dim = _need(m, "rot_dim", int, default=0, required=False)
        if rot_dim < 0 or rot_dim % 2:
            raise ConfigError(f"config.json: {mw}rot_dim must be even and not negative, got {rot_dim}")
        rot = _rotation(m, mw, rot_dim) if rot_dim else None
        if rot_dim and rot is None:
            raise ConfigError(f"config.json: {mw}rot is missing although rot_dim is {rot_dim}")
        first = kind == "latent_attention"
        q_rank = _positive(m, "q_rank", mw) if first else 0
        mixer = RukedraLatentAttention(heads, dim, rot_dim, vdim, _positive(m, "kv_rank", mw), q_rank, scale,
                                       _mask_size(m, mw) if first else 0, rot, out_gate=first)
    j = i
    if raw.get("weights_of") is not None:
        j = _need(raw, "weights_of", int)
        if not 0 <= j < n_layers or j == i:
            raise ConfigError(f"config.json: {where}weights_of = {j} must name another of the {n_layers} layers")
    return RukedraLayer(kind, mixer, _mlp(raw.get("mlp"), where), j)


def _encoding(encodings: Dict[str, PartSpec], rot: Optional[Rotation]) -> Optional[str]:
    """The name of the rotary tables for ``rot`` (layers with the same constants share them)."""
    if rot is None:
        return None
    s = rot.scaling
    name = f"rot{rot.dims}@{rot.base!r}" + (f"*{s.factor!r}/{s.original!r}/{s.fast!r}/{s.slow!r}" if s else "")
    if name not in encodings:
        scaling = None
        if s is not None:
            scaling = {"rope_type": "yarn", "factor": s.factor, "original_max_position_embeddings": s.original,
                       "beta_fast": s.fast, "beta_slow": s.slow, "amplitude_slope": YARN_AMPLITUDE_SLOPE}
        encodings[name] = PartSpec("rotary", {"head_dim": rot.dims, "rotary_dim": rot.dims, "theta": rot.base,
                                              "scaling": scaling, "pairing": ROTATION_PAIRING})
    return name


def rukedra_spec(cfg: RukedraConfig) -> ModelSpec:
    """Parts and run order of a Rukedra model (see the module's text for what the design fixes)."""
    norm = {"size": cfg.width, "eps": cfg.norm_eps, "groups": cfg.norm_groups}
    encodings: Dict[str, PartSpec] = {}
    layers, index_of = [], {}
    for i, layer in enumerate(cfg.layers):
        if layer.weights_of != i:
            continue
        index_of[i] = len(layers)
        p = f"l{i}."
        m = layer.mixer
        if layer.type == "mingru":
            mixer = PartSpec("mingru", {
                "hidden_size": cfg.width, "state_size": m.width,
                "tensor_names": {"z_proj.weight": "z", "z_proj.bias": "z.b", "x_proj.weight": "x", "x_proj.bias": "x.b",
                                 "gate_proj.weight": "g", "o_proj.weight": "o"},
            }, p + "mix.")
        else:
            names = {"kv_down_proj.weight": "dkv", "kv_norm.weight": "dkv.norm", "k_up_proj.weight": "uk",
                     "v_up_proj.weight": "uv", "o_proj.weight": "o", "gate_proj.weight": "g"}
            if m.q_rank:
                names.update({"q_down_proj.weight": "dq", "q_norm.weight": "dq.norm", "q_up_proj.weight": "uq"})
            else:
                names["q_proj.weight"] = "q"
            mixer = PartSpec("latent_attention", {
                "hidden_size": cfg.width, "num_heads": m.heads, "head_dim": m.dim, "rot_dim": m.rot_dim,
                "value_dim": m.vdim, "kv_rank": m.kv_rank, "q_rank": m.q_rank, "norm_eps": cfg.norm_eps,
                "window": m.mask_size, "mask": "window", "softmax_scale": m.scale, "sink": None,
                "out_gate": m.out_gate, "position": _encoding(encodings, m.rot), "tensor_names": names,
            }, p + "mix.")

        def between(name, gate):
            return PartSpec("gated_postnorm", dict(norm, tensor_names={"weight": name, "gate.weight": gate,
                                                                      "gate.bias": gate + ".b"}), p)

        parts = {"norm1": PartSpec("group_rmsnorm", dict(norm, tensor_names={"weight": "norm1"}), p),
                 "mixer": mixer, "post1": between("norm1b", "rg1")}
        ml = layer.mlp
        if ml is not None:
            parts["norm2"] = PartSpec("group_rmsnorm", dict(norm, tensor_names={"weight": "norm2"}), p)
            parts["post2"] = between("norm2b", "rg2")
            if isinstance(ml, RukedraDense):
                parts["ffn"] = PartSpec("swiglu", {
                    "hidden_size": cfg.width, "intermediate_size": ml.ff, "activation": DENSE_ACTIVATION,
                    "tensor_names": {"gate_proj.weight": "gate", "up_proj.weight": "up", "down_proj.weight": "down"},
                }, p + "mlp.")
            else:
                parts["ffn"] = PartSpec("moe", {
                    "hidden_size": cfg.width, "num_experts": ml.experts, "top": ml.top, "expert_size": ml.ff,
                    "shared_size": ml.shared_ff, "router_bias": False, "score": ROUTER_SCORE,
                    "groups": ml.groups, "keep_groups": ml.keep_groups, "group_score_top": GROUP_SCORE_TOP,
                    "weight_scale": ml.scale, "weight_sum_eps": ROUTER_SUM_EPS, "shared_gate": bool(ml.shared_ff),
                    "shared_prefix": "shared.",
                    "shared_names": {"gate_proj.weight": "gate", "up_proj.weight": "up", "down_proj.weight": "down"},
                    "tensor_names": {"router.weight": "router", "shared_gate.weight": "shared.sg",
                                     "experts.*.gate_proj.weight": "e*.gate", "experts.*.up_proj.weight": "e*.up",
                                     "experts.*.down_proj.weight": "e*.down"},
                }, p + "mlp.")
        layers.append(LayerSpec("sandwich", parts))
    spec = ModelSpec(
        hidden_size=cfg.width,
        vocab_size=cfg.vocab,
        max_positions=None,                       # the rotation has no limit of its own: the cache's size is the limit
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.width,
                                               "tensor_names": {"weight": "embed"}}, ""),
        encodings=encodings,
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(index_of[layer.weights_of]) for layer in cfg.layers),
        final_norm=PartSpec("group_rmsnorm", dict(norm, tensor_names={"weight": "final.norm"}), ""),
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "tied_to": None,
                                      "softcap": cfg.logit_softcap, "tensor_names": {"weight": "head"}}, ""),
    )
    spec.validate()
    return spec
