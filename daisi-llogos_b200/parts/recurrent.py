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
"""
from __future__ import annotations

import torch

from ..kernels.linear import linear
from .base import Branch, Mixer, StateNeed, TensorDecl, as_f32, register_part


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


register_part("mixer", "mingru", MinGru)
