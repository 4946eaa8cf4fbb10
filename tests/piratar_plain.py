"""A plain, slow implementation of the Piratar decoder, for tests only: whole sequences, no cache, float64,
one function per mechanism, and no code shared with the library under test (it reads config.json's keys and
looks tensors up by name on its own).

The design in this file's notation (T tokens, width D, token ids ``tok``):

* embedding: ``x_t = scale * embed[tok_t] + bigram[r_t]`` with ``r_t = (mul_prev tok_{t-1} + mul_cur tok_t) mod buckets``
  and, for a sequence's first token, the table's last row; then ``N(x, embed.norm)``.
* ``N(x, w) = x / sqrt(mean(x^2) + eps) * (1 + w)``: the model's norm stores its weight as the difference from one.  ``P(x, w)`` is the
  same with a plain weight, ``U(x)`` the same with no weight.
* a layer: ``x' = x + mixer(N(x, norm1)) + ff(N(x, norm2))`` (both read the old x; a layer may lack the feed-forward),
  then the token's own input ``x'' = x' + P(proj(gelu(gate x') * e_t), side.norm)`` with ``e_t`` layer i's slice of
  ``side.embed[tok_t]``.
* mixer "rglru": ``y = gelu(Y h + b_y)``, ``u = conv(X h + b_x)`` (causal, per channel, with a bias); per block of
  channels ``r = sigmoid(A_b u_b + a_b)``, ``i = sigmoid(I_b u_b + i_b)``; ``a = exp(-8 r softplus(lam))``,
  ``S_t = a S_{t-1} + sqrt(1 - a^2) i u`` from ``S = 0``; output ``O (S * y)``.
* mixer "parallel": ``(P(left(h), left.out) + P(right(h), right.out)) / 2``.  Left: grouped-query softmax attention whose
  q, k, v pass a short causal convolution per channel before the rotation, with the concatenated heads multiplied by
  ``sigmoid(G h)``.  Right: retention, ``S_t = d_h S_{t-1} + k_t v_t^T``, ``o_t = S_t^T q_t`` per head with rotated q and k,
  k times ``dim^-1/2``; ``U(o)`` per head, times ``silu(G h)``, then ``O``.
* rotation by halves: element i of the first ``dims`` pairs with element ``i + dims / 2``; angle ``pos * base^(-2i/dims)``.
* feed-forward "dense": ``down(silu(gate h) * up h)``.  "moe": ``s = softmax(router h)`` over all experts, the ``top``
  largest, weights ``s / (sum of the chosen + 1e-20) * scale``; a shared expert times ``sigmoid(sg . h)``.
* output: ``head N(x, final.norm)``.
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


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    x = x.to(F64)
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_one_plus(x, weight, eps):
    return unit_rms(x, eps) * (1.0 + weight.to(F64))


def norm_plain(x, weight, eps):
    return unit_rms(x, eps) * weight.to(F64)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def embed(w: Dict[str, torch.Tensor], cfg: dict, tokens: Sequence[int]) -> torch.Tensor:
    tok = torch.as_tensor(list(tokens), dtype=torch.long)
    em = cfg["embedding"]
    x = w["embed"].to(F64)[tok] * float(em.get("scale", 1.0))
    bg = em.get("bigram")
    if bg:
        buckets = int(bg["buckets"])
        rows = torch.full_like(tok, buckets)
        rows[1:] = (tok[:-1] * int(bg["mul_prev"]) + tok[1:] * int(bg["mul_cur"])) % buckets
        x = x + w["bigram"].to(F64)[rows]
    return x


def causal_conv(u: torch.Tensor, taps: torch.Tensor, bias=None) -> torch.Tensor:
    """u: [T, C]; taps: [C, K], the last column weighs the current token; zeros before the start."""
    t, c = u.shape
    k = taps.shape[1]
    taps = taps.to(F64)
    padded = torch.cat([torch.zeros(k - 1, c, dtype=F64), u.to(F64)])
    out = torch.zeros(t, c, dtype=F64)
    for j in range(k):
        out += padded[j:j + t] * taps[:, j]
    return out if bias is None else out + bias.to(F64)


def rotate_halves(x: torch.Tensor, positions: torch.Tensor, rot: Optional[dict]) -> torch.Tensor:
    """x: [T, heads, d]; the first ``rot.dims`` elements of every head are rotated, element i with i + dims / 2."""
    if not rot:
        return x.to(F64)
    dims = int(rot["dims"])
    half = dims // 2
    f = float(rot["base"]) ** (-2.0 * torch.arange(half, dtype=F64) / dims)
    ang = positions.to(F64)[:, None] * f[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    x = x.to(F64).clone()
    a, b = x[..., :half].clone(), x[..., half:dims].clone()
    x[..., :half] = a * c - b * s
    x[..., half:dims] = b * c + a * s
    return x


def conv_attention(h, w, p, mx, pos=None, scores_out: Optional[list] = None) -> torch.Tensor:
    """The left mixer: projections, convolutions, rotation, causal softmax attention, sigmoid gate, output."""
    t = h.shape[0]
    heads, kvh, dim, vdim = int(mx["heads"]), int(mx["kv_heads"]), int(mx["dim"]), int(mx["vdim"])
    pos = torch.arange(t) if pos is None else pos
    q, k, v = linear(h, w[p + "q"]), linear(h, w[p + "k"]), linear(h, w[p + "v"])
    if mx.get("conv"):
        q, k, v = causal_conv(q, w[p + "q.conv"]), causal_conv(k, w[p + "k.conv"]), causal_conv(v, w[p + "v.conv"])
    q = rotate_halves(q.view(t, heads, dim), pos, mx.get("rot"))
    k = rotate_halves(k.view(t, kvh, dim), pos, mx.get("rot"))
    v = v.view(t, kvh, vdim)
    i = torch.arange(t)
    hidden = i[None, :] > i[:, None]
    out = torch.zeros(t, heads, vdim, dtype=F64)
    for hh in range(heads):
        g = hh // (heads // kvh)
        s = (q[:, hh] @ k[:, g].t()) * float(mx["scale"])
        pr = torch.softmax(s.masked_fill(hidden, -math.inf), dim=-1)
        if scores_out is not None:
            scores_out.append(pr)
        out[:, hh] = pr @ v[:, g]
    out = out.reshape(t, heads * vdim) * torch.sigmoid(linear(h, w[p + "g"]))
    return linear(out, w[p + "o"])


def retention(h, w, p, mx, eps, pos=None) -> torch.Tensor:
    """The right mixer, token by token: ``S <- d S + k v^T``, ``o = S^T q``."""
    t = h.shape[0]
    heads, dim, vdim = int(mx["heads"]), int(mx["dim"]), int(mx["vdim"])
    pos = torch.arange(t) if pos is None else pos
    q = rotate_halves(linear(h, w[p + "q"]).view(t, heads, dim), pos, mx.get("rot"))
    k = rotate_halves(linear(h, w[p + "k"]).view(t, heads, dim), pos, mx.get("rot")) * dim ** -0.5
    v = linear(h, w[p + "v"]).view(t, heads, vdim)
    decay = torch.as_tensor([float(d) for d in mx["decay"]], dtype=F64)
    state = torch.zeros(heads, dim, vdim, dtype=F64)
    out = torch.zeros(t, heads, vdim, dtype=F64)
    for n in range(t):
        state = decay[:, None, None] * state + k[n][:, :, None] * v[n][:, None, :]
        out[n] = torch.einsum("hdv,hd->hv", state, q[n])
    out = unit_rms(out, eps).reshape(t, heads * vdim) * silu(linear(h, w[p + "g"]))
    return linear(out, w[p + "o"])


def side_by_side(h, w, p, mx, eps) -> torch.Tensor:
    left = norm_plain(conv_attention(h, w, p + "left.", mx["left"]), w[p + "left.out"], eps)
    right = norm_plain(retention(h, w, p + "right.", mx["right"], eps), w[p + "right.out"], eps)
    return 0.5 * (left + right)


def rglru(h, w, p, mx, states_out: Optional[list] = None) -> torch.Tensor:
    t = h.shape[0]
    width, blocks = int(mx["width"]), int(mx["blocks"])
    y = gelu_tanh(linear(h, w[p + "y"], w[p + "y.b"]))
    u = causal_conv(linear(h, w[p + "x"], w[p + "x.b"]), w[p + "conv"], w[p + "conv.b"])
    ub = u.view(t, blocks, width // blocks)
    r = torch.sigmoid(torch.einsum("boi,tbi->tbo", w[p + "ra"].to(F64), ub) + w[p + "ra.b"].to(F64)).reshape(t, width)
    i = torch.sigmoid(torch.einsum("boi,tbi->tbo", w[p + "ri"].to(F64), ub) + w[p + "ri.b"].to(F64)).reshape(t, width)
    log_a = -8.0 * r * torch.nn.functional.softplus(w[p + "lam"].to(F64))
    a = torch.exp(log_a)
    drive = torch.sqrt(1.0 - a * a) * i * u
    s = torch.zeros(width, dtype=F64)
    states = []
    for n in range(t):
        s = a[n] * s + drive[n]
        states.append(s)
    states = torch.stack(states)
    if states_out is not None:
        states_out.append(states)
    return linear(states * y, w[p + "o"])


def expert(h, w, p):
    return linear(silu(linear(h, w[p + "gate"])) * linear(h, w[p + "up"]), w[p + "down"])


def route(h, w, p, router: dict):
    """(chosen experts [T, top], weights [T, top], margin [T]): the margin is by how much the last chosen score beats the
    next, as a share of the chosen scores' sum; infinite where nothing is left out, or where the last chosen expert's
    share of the sum is below 1/100 (then it hardly matters which of the two is taken)."""
    top = int(router["top"])
    s = torch.softmax(linear(h, w[p + "router"]), dim=-1)
    val, idx = torch.topk(s, top, dim=-1)
    margin = torch.full((s.shape[0],), math.inf, dtype=F64)
    if top < s.shape[1]:
        total = val.sum(-1)
        margin = (val[:, -1] - torch.topk(s, top + 1, dim=-1).values[:, -1]) / total
        margin = torch.where(val[:, -1] / total < 0.01, torch.full_like(margin, math.inf), margin)
    weights = val / (val.sum(-1, keepdim=True) + 1e-20) * float(router.get("scale", 1.0))
    return idx, weights, margin


def moe(h, w, p, ml, margins: Optional[list] = None) -> torch.Tensor:
    n_exp = int(ml["router"]["experts"])
    idx, wt, margin = route(h, w, p, ml["router"])
    if margins is not None:
        margins.append(margin)
    out = torch.zeros(h.shape[0], w[p + "e0.down"].shape[0], dtype=F64)
    for e in range(n_exp):
        hit = idx == e
        rows = hit.any(-1)
        if rows.any():
            out[rows] += (wt * hit).sum(-1)[rows, None] * expert(h[rows], w, f"{p}e{e}.")
    if ml.get("shared"):
        out = out + torch.sigmoid(linear(h, w[p + "shared.sg"])) * expert(h, w, p + "shared.")
    return out


def token_side(x, w, p, cfg, li: int, tokens, eps) -> torch.Tensor:
    dim = int(cfg["token_side"]["dim"])
    tok = torch.as_tensor(list(tokens), dtype=torch.long)
    e = w["side.embed"].to(F64)[tok][:, li * dim:(li + 1) * dim]
    y = linear(gelu_tanh(linear(x, w[p + "side.gate"])) * e, w[p + "side.proj"])
    return x + norm_plain(y, w[p + "side.norm"], eps)


# ---- the model ------------------------------------------------------------------------------------

def forward(weights: Dict[str, torch.Tensor], cfg: dict, tokens: Sequence[int], trace: Optional[list] = None,
            margins: Optional[list] = None) -> torch.Tensor:
    """float64 logits [T, vocab] of one whole sequence.  ``trace`` (a list) receives the residual after every layer,
    ``margins`` every router's margins (see ``route``)."""
    w = weights
    eps = float(cfg["norm"]["eps"])
    x = norm_one_plus(embed(w, cfg, tokens), w["embed.norm"], eps)
    for li, layer in enumerate(cfg["layers"]):
        p = f"l{li}."
        h = norm_one_plus(x, w[p + "norm1"], eps)
        if layer["type"] == "rglru":
            y = rglru(h, w, p + "mix.", layer["mixer"])
        elif layer["type"] == "parallel":
            y = side_by_side(h, w, p + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(f"layer type {layer['type']!r}")
        ml = layer.get("mlp")
        if ml:
            h2 = norm_one_plus(x, w[p + "norm2"], eps)
            y = y + (expert(h2, w, p + "mlp.") if ml["kind"] == "dense" else moe(h2, w, p + "mlp.", ml, margins))
        x = x + y
        if cfg.get("token_side"):
            x = token_side(x, w, p, cfg, li, tokens, eps)
        if trace is not None:
            trace.append(x.clone())
    return linear(norm_one_plus(x, w["final.norm"], eps), w["head"])
