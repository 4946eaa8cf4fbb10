"""Recurrent mixers: a fixed-size state per sequence instead of keys and values.

``MinGru``: a gated recurrence whose gates read the current token only,

    z_t = sigmoid(W_z h_t + b_z),   u_t = W_x h_t + b_x,   c_t = u_t + 1/2 (u_t >= 0) | sigmoid(u_t) (u_t < 0)
    S_t = (1 - z_t) S_{t-1} + z_t c_t        (element by element, S before a sequence's first token = 0)
    y_t = W_o (S_t * silu(W_g h_t))

The three input projections are one product; ``ops.mingru_scan`` adds its float32 partial sums, runs the recurrence
along every sequence of the step from the state the cache holds (float32 ``[slots, state_size]``, zeroed when a
sequence starts), leaves the last state there and writes ``S_t * silu(g_t)`` in the compute type for the output
product.  Because the recurrence is linear in S, a step's tokens are scanned in pieces that are joined afterwards, so a
prompt does not run token by token; gates, candidates and the state are float32 whatever the compute type.

``RgLru`` (a block around a real-gated linear recurrent unit, with a short convolution ahead of it), ``Retention`` (a
matrix-valued state per head under a fixed decay, read out by the query) and ``SideBySide`` (two mixers over the same
input, each normed and the two weighed) follow the same pattern: one input product, float32 kernels for what enters the
recurrence, a state per sequence in the cache (several things per sequence are a ``MultiNeed``), pieces for long prompts.
"""
from __future__ import annotations

import torch

from ..kernels.linear import linear
from .base import Branch, Mixer, MultiNeed, StateNeed, TensorDecl, Term, as_f32, part_class, register_part


class MinGru(Mixer):
    """params: hidden_size, state_size.  Tensors: ``z_proj``, ``x_proj`` (weight [state, hidden] and bias [state]),
    ``gate_proj.weight`` [state, hidden], ``o_proj.weight`` [hidden, state]."""

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        self.hidden = int(params["hidden_size"])
        self.size = int(params["state_size"])
        if self.size <= 0:
            raise ValueError(f"mingru: state_size must be positive, got {self.size}")
        self.w_in = self.bias = self.w_o = None

    def tensors(self):
        return {"z_proj.weight": TensorDecl((self.size, self.hidden)), "z_proj.bias": TensorDecl((self.size,), "bias"),
                "x_proj.weight": TensorDecl((self.size, self.hidden)), "x_proj.bias": TensorDecl((self.size,), "bias"),
                "gate_proj.weight": TensorDecl((self.size, self.hidden)),
                "o_proj.weight": TensorDecl((self.hidden, self.size))}

    def bind(self, tensors):
        ws = [tensors["z_proj.weight"], tensors["x_proj.weight"], tensors["gate_proj.weight"]]
        if len({w.dtype for w in ws}) != 1:
            raise ValueError(f"{self.prefix}: the input projections are stored with different types")
        self.w_in = torch.cat(ws, dim=0).contiguous()                       # rows: z | x | g
        self.bias = torch.cat([as_f32(tensors["z_proj.bias"], self.env), as_f32(tensors["x_proj.bias"], self.env)]).contiguous()
        self.w_o = tensors["o_proj.weight"]

    def cache_need(self):
        return StateNeed((self.size,), torch.float32)

    def forward(self, x, ctx, cache) -> Branch:
        n = x.shape[0]
        rows = linear(ctx, x, self.w_in, "mingru.in", torch.float32)        # [P, N, 3 size]
        out = ctx.buffer("mingru.out", (n, self.size))
        carry = None
        pieces = ctx.ops.mingru_pieces(ctx.max_count)
        if pieces > 1:
            carry = ctx.buffer("mingru.carry", (ctx.n_seqs, pieces, 2, self.size), torch.float32)
        ctx.ops.mingru_scan(rows, self.bias, cache.state, ctx.slots, ctx.cu_tokens, out, carry)
        return Branch(linear(ctx, out, self.w_o, "mingru.proj", torch.float32))


class RgLru(Mixer):
    """A recurrent block around a real-gated linear recurrent unit.  Two branches of ``state_size`` channels from one input
    product: ``y = gelu_tanh(W_y h + b_y)`` and ``u = conv(W_x h + b_x)``, a short causal convolution per channel with a bias.
    The channels form ``blocks`` equal blocks; in block b ``r = sigmoid(A_b u_b + a_b)``, ``i = sigmoid(I_b u_b + i_b)`` with
    square matrices per block; ``a = exp(-decay_scale r softplus(lam))``, ``S_t = a S_{t-1} + sqrt(1 - a^2) i u`` element by
    element from ``S = 0``; output ``W_o (S_t * y_t)``.  Per sequence the cache keeps S (float32) and the convolution's
    last ``taps - 1`` inputs.  The gates' products take ``u`` in the compute type and leave float32 sums
    (``ops.head_linear`` with the block as the head); sigmoids, decay, state and the drive are float32.

    params: hidden_size, state_size, blocks, conv_taps, decay_scale (default 8).  Tensors: ``y_proj``, ``x_proj`` (weight
    [state, hidden], bias [state]), ``conv.weight`` [state, taps], ``conv.bias`` [state], ``a_gate``, ``i_gate`` (weight
    [blocks, state / blocks, state / blocks], bias [blocks, state / blocks]), ``lam`` [state], ``o_proj.weight`` [hidden, state]."""

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        self.hidden = int(params["hidden_size"])
        self.size = int(params["state_size"])
        self.blocks = int(params["blocks"])
        self.taps = int(params.get("conv_taps", 1) or 1)
        self.decay_scale = float(params.get("decay_scale", 8.0))
        if self.size <= 0 or self.blocks <= 0 or self.size % self.blocks:
            raise ValueError(f"rglru: {self.size} channels do not split into {self.blocks} equal blocks")
        limit = getattr(env.ops, "CONV_MAX_TAPS", None)
        if self.taps < 1 or (limit is not None and self.taps > limit):
            raise ValueError(f"rglru: {self.taps} convolution taps (1 to {limit})")
        self.bw = self.size // self.blocks
        self.w_in = self.b_y = self.b_x = self.w_conv = self.b_conv = self.w_gates = self.b_gates = self.lam = self.w_o = None

    def tensors(self):
        s, h, b, bw = self.size, self.hidden, self.blocks, self.bw
        return {"y_proj.weight": TensorDecl((s, h)), "y_proj.bias": TensorDecl((s,), "bias"),
                "x_proj.weight": TensorDecl((s, h)), "x_proj.bias": TensorDecl((s,), "bias"),
                "conv.weight": TensorDecl((s, self.taps), "conv"), "conv.bias": TensorDecl((s,), "bias"),
                "a_gate.weight": TensorDecl((b, bw, bw)), "a_gate.bias": TensorDecl((b, bw), "bias"),
                "i_gate.weight": TensorDecl((b, bw, bw)), "i_gate.bias": TensorDecl((b, bw), "bias"),
                "lam": TensorDecl((s,), "rate"), "o_proj.weight": TensorDecl((h, s))}

    def bind(self, tensors):
        ws = [tensors["y_proj.weight"], tensors["x_proj.weight"]]
        gs = [tensors["a_gate.weight"], tensors["i_gate.weight"]]
        if len({w.dtype for w in ws + gs}) != 1:
            raise ValueError(f"{self.prefix}: the projections and gate matrices are stored with different types")
        self.w_in = torch.cat(ws, dim=0).contiguous()                               # rows: y | x
        self.b_y, self.b_x = as_f32(tensors["y_proj.bias"], self.env), as_f32(tensors["x_proj.bias"], self.env)
        self.w_conv, self.b_conv = as_f32(tensors["conv.weight"], self.env), as_f32(tensors["conv.bias"], self.env)
        self.w_gates = torch.cat(gs, dim=1).contiguous()                            # [blocks, 2 bw, bw]: r's rows, then i's
        self.b_gates = torch.cat([as_f32(tensors["a_gate.bias"], self.env), as_f32(tensors["i_gate.bias"], self.env)],
                                 dim=1).contiguous()
        self.lam = as_f32(tensors["lam"], self.env)
        self.w_o = tensors["o_proj.weight"]

    def cache_need(self):
        state = StateNeed((self.size,), torch.float32)
        if self.taps > 1:
            return MultiNeed.of(state=state, conv=StateNeed((self.taps - 1, self.size), torch.float32))
        return state

    def forward(self, x, ctx, cache) -> Branch:
        ops = ctx.ops
        n = x.shape[0]
        conv_state = None
        if self.taps > 1:
            cache, conv_state = cache["state"], cache["conv"].state
        rows = linear(ctx, x, self.w_in, "rglru.in", torch.float32)                 # [P, N, 2 size]: y | x
        u = ctx.buffer("rglru.u", (n, self.size), torch.float32)
        u_c = u if x.dtype == torch.float32 else ctx.buffer("rglru.u_c", (n, self.size))
        ops.causal_conv(rows, self.size, self.w_conv, conv_state, ctx.slots, ctx.cu_tokens, ctx.seq_of_token,
                        ctx.len_before, u, in_bias=self.b_x, bias=self.b_conv, out2=None if u_c is u else u_c)
        gates = ctx.buffer("rglru.gates", (n, self.blocks, 2 * self.bw), torch.float32)
        ops.head_linear(u_c.view(n, self.blocks, self.bw), self.w_gates, gates)
        out = ctx.buffer("rglru.out", (n, self.size))
        carry = None
        pieces = ops.mingru_pieces(ctx.max_count)
        if pieces > 1:
            carry = ctx.buffer("rglru.carry", (ctx.n_seqs, pieces, 2, self.size), torch.float32)
        ops.rglru_scan(rows, 0, self.b_y, u, gates, self.b_gates, self.lam, self.decay_scale, cache.state, ctx.slots,
                       ctx.cu_tokens, out, carry)
        return Branch(linear(ctx, out, self.w_o, "rglru.proj", torch.float32))


class Retention(Mixer):
    """Linear attention with a fixed decay per head and neither softmax nor denominator:

        S_t = decay_h S_{t-1} + k_t v_t^T,    o_t = S_t^T q_t        (per head; S is [dim, vdim], zero before a sequence)

    with q and k rotated by position (k then times ``dim^-1/2``), every head's ``o`` divided by its root mean square (no
    weight), the concatenated heads multiplied by ``silu(W_g h)`` and projected by ``W_o``.  q, k, v and the gate's arguments
    come from one product; the rotation, the state and everything that enters it are float32 (``ops.retention``); the
    cache keeps S per sequence.

    params: hidden_size, num_heads, head_dim, value_dim, decay (a list, one per head), norm_eps, position (name of a
    rotary encoding or None).  Tensors: ``q_proj``, ``k_proj``, ``v_proj``, ``g_proj``, ``o_proj`` (weights)."""

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        p = params
        self.hidden = int(p["hidden_size"])
        self.nh = int(p["num_heads"])
        self.hd = int(p["head_dim"])
        self.vd = int(p.get("value_dim") or self.hd)
        self.decay = [float(d) for d in p["decay"]]
        if len(self.decay) != self.nh:
            raise ValueError(f"retention: {len(self.decay)} decays for {self.nh} heads")
        self.eps = float(p["norm_eps"])
        fits = getattr(env.ops, "retention_supported", None)
        if fits is not None and not fits(self.hd, self.vd):
            raise ValueError(f"retention: a head's state of {self.hd} x {self.vd} elements fits neither the registers nor "
                             f"the shared memory of one block")
        self.k_scale = float(self.hd) ** -0.5
        enc = p.get("position")
        self.encoding = env.encodings[enc] if enc is not None else None
        self.w_in = self.w_o = self.decay_t = None

    def tensors(self):
        qk, v = self.nh * self.hd, self.nh * self.vd
        return {"q_proj.weight": TensorDecl((qk, self.hidden)), "k_proj.weight": TensorDecl((qk, self.hidden)),
                "v_proj.weight": TensorDecl((v, self.hidden)), "g_proj.weight": TensorDecl((v, self.hidden)),
                "o_proj.weight": TensorDecl((self.hidden, v))}

    def bind(self, tensors):
        ws = [tensors[n + "_proj.weight"] for n in ("q", "k", "v", "g")]
        if len({w.dtype for w in ws}) != 1:
            raise ValueError(f"{self.prefix}: the input projections are stored with different types")
        self.w_in = torch.cat(ws, dim=0).contiguous()                               # rows: q | k | v | g
        self.w_o = tensors["o_proj.weight"]
        self.decay_t = torch.tensor(self.decay, dtype=torch.float32).to(self.w_o.device)

    def cache_need(self):
        return StateNeed((self.nh, self.hd, self.vd), torch.float32)

    def forward(self, x, ctx, cache) -> Branch:
        ops = ctx.ops
        n = x.shape[0]
        qk, v = self.nh * self.hd, self.nh * self.vd
        rot = self.encoding.rotation() if self.encoding is not None else None
        if rot is not None and rot.pairing != 0:
            raise ValueError("retention: the rotation pairs halves")
        rows = linear(ctx, x, self.w_in, "retention.in", torch.float32)
        out = ctx.buffer("retention.out", (n, v))
        carry = None
        pieces = ops.retention_pieces(ctx.max_count)
        if pieces > 1:
            carry = ctx.buffer("retention.carry", (ctx.n_seqs, pieces, self.nh, self.hd, self.vd), torch.float32)
        ops.retention(rows, q_col=0, k_col=qk, v_col=2 * qk, g_col=2 * qk + v, n_heads=self.nh, dim=self.hd, vdim=self.vd,
                      cos=rot.cos if rot else None, sin=rot.sin if rot else None, rotary_dim=rot.rotary_dim if rot else 0,
                      positions=ctx.positions, decay=self.decay_t, k_scale=self.k_scale, eps=self.eps, state=cache.state,
                      slots=ctx.slots, cu_tokens=ctx.cu_tokens, out=out, carry=carry)
        return Branch(linear(ctx, out, self.w_o, "retention.proj", torch.float32))


class SideBySide(Mixer):
    """Two mixers that read the same input; each one's output is RMS-normed over the model width with a weight of its
    own, and ``scale`` times each enters the residual: ``scale * (N(left(h), w_l) + N(right(h), w_r))``.  The norms are not
    computed here: the branch names them (``Branch.terms``) and the norm that adds the branch applies them in its launch.

    params: hidden_size, eps, scale (default 1/2), left and right (each {"kind": a registered mixer, "params": {...}};
    their tensors lie under ``left.`` and ``right.``).  Tensors of its own: ``left.out``, ``right.out`` [hidden]."""

    SIDES = ("left", "right")

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        self.hidden = int(params["hidden_size"])
        self.eps = float(params["eps"])
        self.scale = float(params.get("scale", 0.5))
        self.sides = {}
        for side in self.SIDES:
            sub = params[side]
            self.sides[side] = part_class("mixer", sub["kind"])(sub["params"], prefix + side + ".", env)
        self.out_w = {}

    def tensor_name(self, rel: str) -> str:
        side, _, rest = rel.partition(":")
        if rest and side in self.sides:
            return self.sides[side].tensor_name(rest)
        return super().tensor_name(rel)

    def tensors(self):
        t = {side + ".out": TensorDecl((self.hidden,), "norm") for side in self.SIDES}
        for side, part in self.sides.items():
            for rel, d in part.tensors().items():
                t[side + ":" + rel] = d
        return t

    def bind(self, tensors):
        for side, part in self.sides.items():
            self.out_w[side] = as_f32(tensors[side + ".out"], self.env)
            part.bind({rel[len(side) + 1:]: t for rel, t in tensors.items() if rel.startswith(side + ":")})

    def cache_need(self):
        return MultiNeed.of(**{side: part.cache_need() for side, part in self.sides.items()})

    def forward(self, x, ctx, cache) -> Branch:
        terms = []
        for side, part in self.sides.items():
            view = cache[side] if part.cache_need() is not None else None
            b = part.forward(x, ctx, view)
            if b.more or b.terms or b.scale != 1.0 or b.write is not None:
                raise ValueError("side by side: a side's branch must be plain partials")
            terms.append(Term(b.data, self.out_w[side], self.eps, self.scale))
        return Branch.of_terms(terms)


register_part("mixer", "mingru", MinGru)
register_part("mixer", "rglru", RgLru)
register_part("mixer", "retention", Retention)
register_part("mixer", "side_by_side", SideBySide)
