"""Sublayers between two norms, with a gate on what they add to the residual.

    h = N(x);   y = f(h);   x <- x + N'(sigmoid(R h + b) * y)

``N`` and ``N'`` are RMS norms in groups: a row is cut into ``groups`` equal consecutive parts, every part is divided by
its own root mean square (eps inside the root), and the whole row is multiplied by one weight vector; with one group
this is the ordinary RMS norm.  The gate has one value per element of the row and is computed from the sublayer's input.

Three parts.  ``GroupRmsNorm`` is the norm ``N`` fused with the residual add, as ``RmsNorm`` is: it adds the pending
branch and norms the sum in ONE kernel (``ops.gated_add_group_rmsnorm``).  ``GatedPostNorm`` holds what stands between a
sublayer's output and the residual (``R``, ``b`` and the weight of ``N'``; the gate and the norm can each be left out);
the block attaches it to the sublayer's ``Branch`` with the gate's arguments, and the next norm, whichever block it is in,
applies gate, ``N'`` and the add before its own norm.  ``SandwichBlock`` arranges norm1, mixer, post1 and, where the
layer has a feed-forward, norm2, ffn, post2.  The residual, the gate, both norms' statistics and every sum are float32.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels.linear import linear
from .base import Block, Branch, Norm, Part, TensorDecl, as_f32, register_part


class GatedPostNorm(Part):
    """What a sublayer's output passes on its way into the residual.  params: size, eps, groups, gate (default True:
    tensors ``gate.weight`` [size, size] and ``gate.bias`` [size]), norm (default True: tensor ``weight`` [size])."""

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.groups = int(params.get("groups", 1))
        self.gated = bool(params.get("gate", True))
        self.normed = bool(params.get("norm", True))
        if self.groups < 1 or self.size % self.groups:
            raise ValueError(f"gated_postnorm: {self.size} elements do not split into {self.groups} equal groups")
        self.weight = self.w_gate = self.b_gate = None

    def tensors(self):
        t = {}
        if self.normed:
            t["weight"] = TensorDecl((self.size,), "norm")
        if self.gated:
            t["gate.weight"] = TensorDecl((self.size, self.size))
            t["gate.bias"] = TensorDecl((self.size,), "bias")
        return t

    def bind(self, tensors):
        self.weight = tensors.get("weight")
        if self.gated:
            self.w_gate, self.b_gate = tensors["gate.weight"], as_f32(tensors["gate.bias"], self.env)

    def gate_arguments(self, h, ctx) -> Optional[torch.Tensor]:
        """float32 partial sums ``[S, N, size]`` of ``R h`` (the bias joins them in the norm's kernel)."""
        if not self.gated:
            return None
        return linear(ctx, h, self.w_gate, "post.gate", torch.float32)


class GroupRmsNorm(Norm):
    """RMS norm in groups fused with the residual add.  params: size, eps, groups (default 1).  A pending branch is
    added as it is, or, where the block attached a ``GatedPostNorm`` (``Branch.write``) and the gate's arguments
    (``Branch.more[0]``), gated and normed first."""

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.groups = int(params.get("groups", 1))
        if self.eps <= 0:
            raise ValueError("RMSNorm eps must be positive")
        if self.groups < 1 or self.size % self.groups:
            raise ValueError(f"group_rmsnorm: {self.size} elements do not split into {self.groups} equal groups")
        limit = getattr(env.ops, "NORM_MAX_GROUPS", None)
        if limit is not None and self.groups > limit:
            raise ValueError(f"group_rmsnorm: {self.groups} groups; the kernel takes up to {limit}")
        self.weight: Optional[torch.Tensor] = None

    def tensors(self):
        return {"weight": TensorDecl((self.size,), "norm")}

    def bind(self, tensors):
        self.weight = tensors["weight"]

    def forward(self, residual, branch: Optional[Branch], ctx, rows=None):
        if residual.dim() != 2:
            raise ValueError("group_rmsnorm: the residual must be one stream [tokens, hidden]")
        m = residual.shape[0] if rows is None else rows.numel()
        out = ctx.buffer("norm.out", (m, self.size))
        data = gate = gate_bias = post_w = None
        post_groups, post_eps = 1, self.eps
        if branch is not None:
            if branch.scale != 1.0:
                raise ValueError("group_rmsnorm: the pending branch carries a scale; this norm adds outputs as they are")
            data, post = branch.data, branch.write
            if post is None:
                if branch.more:
                    raise ValueError("group_rmsnorm: the pending branch carries several sublayers' outputs")
            elif not isinstance(post, GatedPostNorm) or post.size != self.size:
                raise ValueError("group_rmsnorm: the pending branch's write is no gated_postnorm part of this width")
            else:
                if len(branch.more) != (1 if post.gated else 0):
                    raise ValueError("group_rmsnorm: a gated branch carries its gate's arguments and nothing else")
                if post.gated:
                    gate, gate_bias = branch.more[0], post.b_gate
                post_w, post_groups, post_eps = post.weight, post.groups, post.eps
        ctx.ops.gated_add_group_rmsnorm(residual, data, gate, gate_bias, post_w, post_groups, post_eps,
                                        self.weight, self.groups, self.eps, out, rows)
        return out


class SandwichBlock(Block):
    """roles: norm1, mixer, post1 and, where the layer has a feed-forward, norm2, ffn, post2 (the posts are
    ``gated_postnorm`` parts, the norms whatever norm takes their branches: ``group_rmsnorm``).  The block hands its last
    sublayer's branch on with the post attached; the next block's first norm (or the model's final norm) applies it."""

    ROLES = {"norm1": "norm", "mixer": "mixer", "post1": "connection",
             "norm2": "norm", "ffn": "ffn", "post2": "connection"}

    def __init__(self, params, prefix, env, parts):
        super().__init__(params, prefix, env, parts)
        for role in ("norm1", "mixer", "post1"):
            if role not in parts:
                raise ValueError(f"sandwich: no part for the role '{role}'")
        if ("ffn" in parts) != ("norm2" in parts) or ("ffn" in parts) != ("post2" in parts):
            raise ValueError("sandwich: norm2, ffn and post2 come together or not at all")

    @staticmethod
    def _through(post: GatedPostNorm, branch: Branch, h, ctx) -> Branch:
        if branch.more or branch.scale != 1.0 or branch.write is not None:
            raise ValueError("sandwich: a sublayer's branch must be plain partials")
        gate = post.gate_arguments(h, ctx)
        return Branch(branch.data, write=post, more=() if gate is None else (gate,))

    def forward(self, residual, pending: Optional[Branch], ctx, cache) -> Optional[Branch]:
        p = self.parts
        h = p["norm1"].forward(residual, pending, ctx)
        a = self._through(p["post1"], p["mixer"].forward(h, ctx, cache), h, ctx)
        if "ffn" not in p:
            return a
        h = p["norm2"].forward(residual, a, ctx)
        return self._through(p["post2"], p["ffn"].forward(h, ctx), h, ctx)


register_part("connection", "gated_postnorm", GatedPostNorm)
register_part("norm", "group_rmsnorm", GroupRmsNorm)
register_part("block", "sandwich", SandwichBlock)
