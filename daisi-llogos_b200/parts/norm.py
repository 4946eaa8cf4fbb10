"""RMSNorm fused with the residual add.

``out = v / sqrt(mean(v^2) + eps) * weight`` with ``v = residual + branch``; eps is added to
the mean inside the root and the weight multiplies after normalisation
(Daisi.Llogos.Cpu/RmsNorm.cs:14-65; fused forms IComputeBackend.cs:417-438).  The residual
stream and the statistics are float32.

For a consumer that takes a row scale, bfloat16 models write ``v * weight`` and hand the division on as the
row's sum of squares (whole, or in parts that add up to it): a product is linear in its rows, so the consumer's
first product scales its result instead.  Nothing then has to see a whole row, and the few rows of a decode
step are spread over many blocks, each adding up the partial sums of its own columns.
"""
from __future__ import annotations

from typing import Optional

import torch

from .base import Branch, Norm, TensorDecl, as_f32, register_part


class RmsNorm(Norm):
    """params: size, eps, weight_offset (default 0; 1 for a weight that holds its difference from one: the row is multiplied by
    ``1 + weight``), out_name (the workspace buffer of the output, default "norm.out": two norms whose outputs are alive
    together name two).

    With ``weight_offset`` the norm runs on ``ops.multi_add_rmsnorm``, which also takes a pending branch of several
    terms, each with a norm and a factor of its own (``Branch.terms``), and can norm the same row for a second norm in
    the same launch (``forward_many``).  Without it everything is as before."""

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        if self.eps <= 0:
            raise ValueError("RMSNorm eps must be positive")
        self.weight_offset = float(params.get("weight_offset", 0.0) or 0.0)
        self.out_name = str(params.get("out_name", "norm.out"))
        self.weight: Optional[torch.Tensor] = None

    def tensors(self):
        # such a weight is drawn near zero
        return {"weight": TensorDecl((self.size,), "bias" if self.weight_offset else "norm")}

    def bind(self, tensors):
        self.weight = as_f32(tensors["weight"], self.env) if self.weight_offset else tensors["weight"]

    def forward_many(self, residual, branch: Optional[Branch], ctx, others=(), rows=None):
        """Adds the pending branch and norms the sum for this norm and for ``others`` (norms of the same size and eps
        with weights of their own) in one launch; returns the outputs in that order."""
        norms = (self,) + tuple(others)
        for o in norms:
            if not isinstance(o, RmsNorm) or o.size != self.size or o.eps != self.eps:
                raise ValueError("rmsnorm: norms that share a launch share their size and eps")
        m = residual.shape[0] if rows is None else rows.numel()
        names = [o.out_name for o in norms]
        if len(set(names)) != len(names):
            raise ValueError(f"rmsnorm: norms that share a launch write to buffers of their own (out_name), got {names}")
        outs = [ctx.buffer(o.out_name, (m, self.size)) for o in norms]
        terms = () if branch is None else branch.as_terms()
        ws = [o.weight if o.weight.dtype == torch.float32 else as_f32(o.weight, self.env) for o in norms]
        ctx.ops.multi_add_rmsnorm(residual, [(t.data, t.weight, t.eps, t.scale) for t in terms],
                                  [(out, w, o.weight_offset) for out, w, o in zip(outs, ws, norms)], self.eps, rows)
        return outs

    def forward(self, residual, branch: Optional[Branch], ctx, rows=None):
        if self.weight_offset or (branch is not None and branch.terms):
            return self.forward_many(residual, branch, ctx, (), rows)[0]
        self.check_plain(branch, "rmsnorm")
        m = residual.shape[0] if rows is None else rows.numel()
        out = ctx.buffer("norm.out", (m, self.size))
        ctx.ops.add_rmsnorm(residual, branch.data if branch is not None else None, self.weight, self.eps, out, rows)
        return out

    def forward_unscaled(self, residual, branch: Optional[Branch], ctx, rows=None):
        ops = ctx.ops
        make_scale = getattr(ops, "RowScale", None)
        if make_scale is None or ctx.dtype != torch.bfloat16 or self.weight_offset or (branch is not None and branch.terms):
            return self.forward(residual, branch, ctx, rows), None
        self.check_plain(branch, "rmsnorm")
        m = residual.shape[0] if rows is None else rows.numel()
        out = ctx.buffer("norm.out", (m, self.size))
        ss = ctx.buffer("norm.ss", (m, ops.norm_ss_parts(m, self.size)), torch.float32)
        ops.add_rmsnorm(residual, branch.data if branch is not None else None, self.weight, self.eps, out, rows, ss_out=ss)
        return out, make_scale(ss, self.size, self.eps)


class LayerNorm(Norm):
    """Layer norm fused with the residual add: ``v = residual + scale * (sum of the pending branch's partials)``,
    ``out = (v - mean(v)) / sqrt(var(v) + eps) * weight + bias`` with the variance as the mean of the squared
    deviations.  Takes a branch of several sublayers' outputs and a scale on their sum (``Branch.more``,
    ``Branch.scale``).  Statistics, the residual and its sum are float32.  params: size, eps."""

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        if self.eps <= 0:
            raise ValueError("layer norm eps must be positive")
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None

    def tensors(self):
        return {"weight": TensorDecl((self.size,), "norm"), "bias": TensorDecl((self.size,), "bias")}

    def bind(self, tensors):
        self.weight, self.bias = tensors["weight"], tensors["bias"]
        if self.weight.dtype != self.bias.dtype:
            raise ValueError(f"{self.prefix}: a layer norm's weight and bias are stored with different types")

    def forward(self, residual, branch: Optional[Branch], ctx, rows=None):
        if residual.dim() != 2:
            raise ValueError("layernorm: the residual must be one stream [tokens, hidden]")
        m = residual.shape[0] if rows is None else rows.numel()
        out = ctx.buffer("norm.out", (m, self.size))
        parts = () if branch is None else (branch.data,) + tuple(branch.more)
        ctx.ops.add_layernorm(residual, parts, branch.scale if branch is not None else 1.0, self.weight, self.bias,
                              self.eps, out, rows)
        return out


register_part("norm", "rmsnorm", RmsNorm)
register_part("norm", "layernorm", LayerNorm)
