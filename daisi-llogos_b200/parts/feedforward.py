"""Feed-forward parts: the gated ``SwiGLU`` and the ungated ``DenseMLP`` (up, activation, down).

``SwiGLU``: ``down( silu(gate(x)) * up(x) )`` without biases
(Inference/ForwardPass.cs:242-246; silu(g) = g / (1 + exp(-g)), Daisi.Llogos.Cpu/Silu.cs:9-16).
The gate and up matrices are stored as one matrix (gate rows, then up rows, each part filled up to a
multiple of 128 rows), so that the gating is the epilogue of one product.
"""
from __future__ import annotations

import torch

from ..kernels.linear import activated_linear, gated_layout, gated_linear, linear
from .base import Branch, FeedForward, TensorDecl, register_part


class SwiGLU(FeedForward):
    """``down(act(gate(x)) * up(x))``.  params: hidden_size, intermediate_size, activation (of the gate: one of
    ``ops.GATE_ACTIVATIONS``, "silu" by default, or "gelu_tanh")."""

    TAKES_ROW_SCALE = True

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        self.hidden = int(params["hidden_size"])
        self.inter = int(params["intermediate_size"])
        self.activation = str(params.get("activation", "silu"))
        known = getattr(env.ops, "GATE_ACTIVATIONS", ("silu",))
        if self.activation not in known:
            raise ValueError(f"swiglu: gate activation '{self.activation}' is not known ({', '.join(known)})")
        self.w_gate_up = None
        self.w_down = None

    def tensors(self):
        return {
            "gate_proj.weight": TensorDecl((self.inter, self.hidden)),
            "up_proj.weight": TensorDecl((self.inter, self.hidden)),
            "down_proj.weight": TensorDecl((self.hidden, self.inter)),
        }

    def bind(self, tensors):
        g, u = tensors["gate_proj.weight"], tensors["up_proj.weight"]
        if g.dtype != u.dtype:
            raise ValueError(f"{self.prefix}: gate_proj and up_proj are stored with different types")
        self.w_gate_up = gated_layout(g, u)
        self.w_down = tensors["down_proj.weight"]

    def forward(self, x, ctx, row_scale=None) -> Branch:
        act = ctx.buffer("ffn.act", (x.shape[0], self.inter))
        gated_linear(ctx, x, self.w_gate_up, act, row_scale, self.activation)
        return Branch(linear(ctx, act, self.w_down, "ffn.out", torch.float32))


class DenseMLP(FeedForward):
    """``down(act(up(x)))`` without a gate and without biases.  params: hidden_size, intermediate_size, activation
    (one of ``ops.ACTIVATIONS``: "relu2" = the square of relu, "gelu_tanh", "silu", "relu").  The activation sees the
    up product's float32 sums and its result is rounded to the compute type once (``kernels.linear.activated_linear``)."""

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        self.hidden = int(params["hidden_size"])
        self.inter = int(params["intermediate_size"])
        self.activation = str(params["activation"])
        known = getattr(env.ops, "ACTIVATIONS", None)
        if known is not None and self.activation not in known:
            raise ValueError(f"dense_mlp: activation '{self.activation}' is not known ({', '.join(known)})")
        self.w_up = self.w_down = None

    def tensors(self):
        return {"up_proj.weight": TensorDecl((self.inter, self.hidden)),
                "down_proj.weight": TensorDecl((self.hidden, self.inter))}

    def bind(self, tensors):
        self.w_up, self.w_down = tensors["up_proj.weight"], tensors["down_proj.weight"]

    def forward(self, x, ctx) -> Branch:
        act = ctx.buffer("ffn.act", (x.shape[0], self.inter))
        activated_linear(ctx, x, self.w_up, act, self.activation)
        return Branch(linear(ctx, act, self.w_down, "ffn.out", torch.float32))


register_part("ffn", "swiglu", SwiGLU)
register_part("ffn", "dense_mlp", DenseMLP)
