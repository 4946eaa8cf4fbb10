"""A plain, slow implementation of the Rukedra decoder, for tests only: whole sequences, no cache, float64,
one function per mechanism, and no code shared with the library under test (it reads config.json's keys and
looks tensors up by name on its own).

The design in this file's notation (T tokens, width D):

* a layer has four norms around two sublayers: ``x' = x + N1b(g1 * mixer(h))`` with ``h = N1(x)`` and
  ``g1 = sigmoid(R1 h + b1)`` (one gate value per element of the width), then the same with the feed-forward, ``N2``,
  ``N2b`` and ``R2``; a layer may have no feed-forward.  A layer that says ``weights_of: j`` runs with layer j's tensors.
* every norm is an RMS norm in ``norm.groups`` equal consecutive groups: each group is divided by its own root mean
  square, then the whole row is multiplied by one weight vector.
* mixer "latent_attention": queries through a low-rank bottleneck with an RMS norm (``dq``, ``dq.norm``, ``uq``); keys and
  values of all heads from one RMS-normed latent ``c`` per token (``uk``, ``uv``) and one rotated key part shared by all
  heads; sliding window; ordinary softmax; the concatenated heads are multiplied by ``sigmoid(G h)`` before ``o``.
* mixer "latent_attention_2": the same keys and values, queries by one matrix, every earlier key visible, no gate.
* both rotate pairs of neighbouring elements ``(2i, 2i+1)``, with frequencies stretched for long contexts: low
  frequencies are divided by ``factor``, high ones kept, a linear ramp between, and cos and sin scaled by
  ``0.1 ln(factor) + 1``.
* mixer "mingru": ``S_t = (1 - z_t) S_{t-1} + z_t c_t`` element by element with ``z = sigmoid(Z h + bz)``,
  ``u = X h + bx``, ``c = u + 1/2`` where ``u >= 0`` and ``sigmoid(u)`` where ``u < 0``; output ``O (S_t * silu(G h))``.
* feed-forward "dense": ``down(gelu_tanh(gate h) * up h)``.  "moe": scores ``s = sigmoid(router h)``; the experts form
  equal groups of neighbours, a group's score is the sum of its two largest ``s``, only the ``keep`` best groups stay
  eligible; the ``top`` eligible experts of largest ``s`` are weighted by ``s / (sum + 1e-20) * scale``; experts are
  ``down(silu(gate h) * up h)``; a shared expert of the same form is added times ``sigmoid(sg . h)``.
* output: the grouped norm with ``final.norm``, ``head``, then ``cap * tanh(logits / cap)``.
"""
from __future__ import annotations

import math
from typing import Dict, Optional, Sequence

import torch

F64 = torch.float64


# ---- mechanisms ---------------------------------------------------------------------------------

def linear(x, w, b=None):
    y = x.to(F64) @ w.to(F64).t()
    return y if b is None else y + b.to(F64)


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    x = x.to(F64)
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * weight.to(F64)


def group_rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, groups: int) -> torch.Tensor:
    """Each of ``groups`` equal consecutive parts of a row is divided by its own root mean square; one weight vector."""
    x = x.to(F64)
    t, d = x.shape
    parts = x.view(t, groups, d // groups)
    parts = parts / torch.sqrt((parts * parts).mean(-1, keepdim=True) + eps)
    return parts.reshape(t, d) * weight.to(F64)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def stretched_frequencies(dims: int, base: float, scaling: Optional[dict]):
    """(frequencies [dims / 2], amplitude): pair i turns by ``position * f_i``; cos and sin are scaled by the amplitude."""
    i = torch.arange(dims // 2, dtype=F64)
    f = float(base) ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, orig = float(scaling["factor"]), float(scaling["original"])

    def turn_dim(turns):           # the pair index whose wavelength makes `turns` turns over the original context
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(float(base)))

    lo = max(math.floor(turn_dim(float(scaling["fast"]))), 0)
    hi = min(math.ceil(turn_dim(float(scaling["slow"]))), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_pairs(x: torch.Tensor, positions: torch.Tensor, rot: dict) -> torch.Tensor:
    """x: [T, heads, d]; the first ``rot.dims`` elements of every head are rotated, element 2i with element 2i + 1."""
    dims = int(rot["dims"])
    f, amp = stretched_frequencies(dims, float(rot["base"]), rot.get("scaling"))
    ang = positions.to(F64)[:, None] * f[None, :]
    c, s = (amp * torch.cos(ang))[:, None, :], (amp * torch.sin(ang))[:, None, :]
    x = x.to(F64).clone()
    u, v = x[..., 0:dims:2].clone(), x[..., 1:dims:2].clone()
    x[..., 0:dims:2] = u * c - v * s
    x[..., 1:dims:2] = v * c + u * s
    return x


def window_mask(t: int, size: Optional[int]) -> torch.Tensor:
    """[t, t] bool: query i sees key j when 0 <= i - j < size (no size: every j <= i)."""
    i = torch.arange(t)[:, None]
    j = torch.arange(t)[None, :]
    vis = j <= i
    return vis if not size else vis & (i - j < size)


def latent_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, mx: dict, eps: float) -> torch.Tensor:
    """Both latent mixers: with ``q_rank`` the queries go through a normed bottleneck; with ``mask`` a window; with a
    tensor ``g`` an output gate."""
    t = h.shape[0]
    heads, dim, rdim, vdim, rank = int(mx["heads"]), int(mx["dim"]), int(mx["rot_dim"]), int(mx["vdim"]), int(mx["kv_rank"])
    pos = torch.arange(t)
    if p + "dq" in w:
        q = linear(rms_norm(linear(h, w[p + "dq"]), w[p + "dq.norm"], eps), w[p + "uq"])
    else:
        q = linear(h, w[p + "q"])
    q = q.view(t, heads, dim + rdim)
    q_plain, q_rot = q[..., :dim], rotate_pairs(q[..., dim:], pos, mx["rot"])
    down = linear(h, w[p + "dkv"])
    c = rms_norm(down[:, :rank], w[p + "dkv.norm"], eps)                     # [T, rank]
    k_rot = rotate_pairs(down[:, None, rank:], pos, mx["rot"])[:, 0]         # [T, rdim], one for all heads
    k_plain = linear(c, w[p + "uk"]).view(t, heads, dim)
    v = linear(c, w[p + "uv"]).view(t, heads, vdim)
    size = (mx.get("mask") or {}).get("size")
    vis = window_mask(t, size)
    out = torch.zeros(t, heads, vdim, dtype=F64)
    for hh in range(heads):
        s = (q_plain[:, hh] @ k_plain[:, hh].t() + q_rot[:, hh] @ k_rot.t()) * float(mx["scale"])
        out[:, hh] = torch.softmax(s.masked_fill(~vis, -math.inf), dim=-1) @ v[:, hh]
    out = out.reshape(t, heads * vdim)
    if p + "g" in w:
        out = out * torch.sigmoid(linear(h, w[p + "g"]))
    return linear(out, w[p + "o"])


def mingru_candidate(u):
    return torch.where(u >= 0, u + 0.5, torch.sigmoid(u))


def mingru(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, state: Optional[torch.Tensor] = None) -> torch.Tensor:
    z = torch.sigmoid(linear(h, w[p + "z"], w[p + "z.b"]))
    c = mingru_candidate(linear(h, w[p + "x"], w[p + "x.b"]))
    s = torch.zeros(z.shape[1], dtype=F64) if state is None else state.to(F64)
    states = []
    for t in range(h.shape[0]):
        s = (1.0 - z[t]) * s + z[t] * c[t]
        states.append(s)
    return linear(torch.stack(states) * silu(linear(h, w[p + "g"])), w[p + "o"])


def dense_mlp(h, w, p):
    return linear(gelu_tanh(linear(h, w[p + "gate"])) * linear(h, w[p + "up"]), w[p + "down"])


def expert(h, w, p):
    return linear(silu(linear(h, w[p + "gate"])) * linear(h, w[p + "up"]), w[p + "down"])


def route(h, w, p, router: dict):
    """(chosen experts [T, top], their weights [T, top], margin [T]): the margin is by how much the last chosen score
    beats the best eligible one left out, or, if less, by how much the last kept group's score beats the best group
    left out; infinite where nothing is left out."""
    n_exp, top = int(router["experts"]), int(router["top"])
    s = torch.sigmoid(linear(h, w[p + "router"]))
    eligible = torch.ones_like(s, dtype=torch.bool)
    margin = torch.full((s.shape[0],), math.inf, dtype=F64)
    groups = router.get("groups")
    if groups:
        count, keep = int(groups["count"]), int(groups["keep"])
        per = n_exp // count
        by_group = s.view(-1, count, per)
        group_score = torch.topk(by_group, min(2, per), dim=-1).values.sum(-1)          # [T, count]
        best = torch.topk(group_score, keep, dim=-1).indices
        ok = torch.zeros_like(group_score, dtype=torch.bool).scatter_(1, best, True)
        eligible = ok[:, :, None].expand(-1, -1, per).reshape(-1, n_exp)
        if keep < count:
            ordered = torch.sort(group_score, dim=-1, descending=True).values
            margin = ordered[:, keep - 1] - ordered[:, keep]
    masked = s.masked_fill(~eligible, -1.0)
    val, idx = torch.topk(masked, top, dim=-1)
    if top < int(eligible.sum(-1).min()):
        margin = torch.minimum(margin, val[:, -1] - torch.topk(masked, top + 1, dim=-1).values[:, -1])
    weights = val / (val.sum(-1, keepdim=True) + 1e-20) * float(router.get("scale", 1.0))
    return idx, weights, margin


def moe(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, ml: dict, margins: Optional[list] = None) -> torch.Tensor:
    n_exp = int(ml["router"]["experts"])
    idx, wt, margin = route(h, w, p, ml["router"])
    if margins is not None:
        margins.append(margin)
    out = torch.zeros(h.shape[0], w[p + "e0.down"].shape[0], dtype=F64)
    for e in range(n_exp):
        hit = idx == e                                      # [T, top]
        rows = hit.any(-1)
        if rows.any():
            out[rows] += (wt * hit).sum(-1)[rows, None] * expert(h[rows], w, f"{p}e{e}.")
    if ml.get("shared"):
        out = out + torch.sigmoid(linear(h, w[p + "shared.sg"])) * expert(h, w, p + "shared.")
    return out


def soft_cap(logits, cap: Optional[float]):
    return logits if not cap else float(cap) * torch.tanh(logits / float(cap))


# ---- the model ------------------------------------------------------------------------------------

def forward(weights: Dict[str, torch.Tensor], cfg: dict, tokens: Sequence[int], trace: Optional[list] = None,
            margins: Optional[list] = None) -> torch.Tensor:
    """float64 logits [T, vocab] of one whole sequence.  ``trace`` (a list) receives the residual after every layer,
    ``margins`` every router's margins (see ``route``)."""
    w = weights
    eps, groups = float(cfg["norm"]["eps"]), int(cfg["norm"].get("groups", 1))
    x = w["embed"].to(F64)[torch.as_tensor(list(tokens), dtype=torch.long)]

    def norm(v, name):
        return group_rms_norm(v, w[name], eps, groups)

    for li, layer in enumerate(cfg["layers"]):
        p = f"l{layer.get('weights_of', li)}."
        kind = layer["type"]
        h = norm(x, p + "norm1")
        if kind in ("latent_attention", "latent_attention_2"):
            y = latent_attention(h, w, p + "mix.", layer["mixer"], eps)
        elif kind == "mingru":
            y = mingru(h, w, p + "mix.")
        else:
            raise ValueError(f"layer type {kind!r}")
        x = x + norm(y * torch.sigmoid(linear(h, w[p + "rg1"], w[p + "rg1.b"])), p + "norm1b")
        ml = layer.get("mlp")
        if ml:
            h = norm(x, p + "norm2")
            y = dense_mlp(h, w, p + "mlp.") if ml["kind"] == "dense" else moe(h, w, p + "mlp.", ml, margins)
            x = x + norm(y * torch.sigmoid(linear(h, w[p + "rg2"], w[p + "rg2.b"])), p + "norm2b")
        if trace is not None:
            trace.append(x.clone())
    return soft_cap(linear(norm(x, "final.norm"), w["head"]), cfg.get("logit_softcap"))
