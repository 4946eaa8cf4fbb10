"""A feed-forward of many small experts of which every token uses a few, beside an optional shared expert.

Router: ``z = W_r h + b`` with float32 sums; the ``top`` experts of largest ``z`` are chosen per token and weighted by a
softmax over the chosen logits alone.  Or (``score = "softmax_all"``) the scores are the softmax over ALL experts' logits,
the ``top`` largest are chosen and weighted by ``s / (sum of the chosen s + weight_sum_eps) * weight_scale``.  Or, by parameter (``score = "sigmoid"``): every expert's score is ``s = sigmoid(z)``; the
experts form ``groups`` equal groups of neighbours, a group is judged by the sum of its ``group_score_top`` largest scores,
and only the experts of the ``keep_groups`` best groups can be chosen; the ``top`` eligible experts of largest score are
weighted by ``s / (sum of the chosen s + weight_sum_eps) * weight_scale``.  Every expert is the gated form ``W_down (silu(W_gate h) * W_up h)`` without
biases; the token's output is the weighted sum of its experts' outputs, plus the shared expert's (which every token
runs) where the layer has one; with ``shared_gate`` the shared expert's output is multiplied by ``sigmoid(w_sg . h)``, one
number per token, whose row ``w_sg`` rides in the router's product.

On the device the step's (token, choice) pairs are put in the order of their experts, every expert's run of rows
filled up to a whole tile (``ops.moe_plan``), so that two grouped products (gate/up with the gating as its epilogue,
then down) work tile by tile, each tile with one expert's matrices (a prompt step in bfloat16: tiles of 128 rows on the
grouped tcgen05 product of csrc/gemm_tc.cu; otherwise tiles of 32 rows on the kernels of csrc/moe.cu); ``ops.moe_combine`` adds a token's rows with their
weights, and the shared expert's partial sums, into one float32 set of partials.  Nothing comes back to the host: the
same launches serve any routing, so a decode step can be recorded once and replayed.
"""
from __future__ import annotations

import torch

from ..kernels.linear import gated_layout, linear
from .base import Branch, FeedForward, TensorDecl, as_f32, part_class, register_part


class MoeFeedForward(FeedForward):
    """params: hidden_size, num_experts, top, expert_size (an expert's inner size), shared_size (0 or None: no shared
    expert), router_bias (bool), shared_prefix (where the shared expert's tensors lie under this part's prefix,
    default "shared."), shared_names (its ``tensor_names``), score ("softmax", the default, "softmax_all" or "sigmoid"), groups and
    keep_groups (0: every expert is eligible), group_score_top (default 2), weight_scale (default 1), weight_sum_eps
    (default 0), shared_gate (bool: a tensor ``shared_gate.weight`` [1, hidden]).  Tensors: ``router.weight`` [experts, hidden],
    ``router.bias`` [experts], and per expert i ``experts.<i>.{gate_proj,up_proj,down_proj}.weight``."""

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        p = params
        self.hidden = int(p["hidden_size"])
        self.n_exp = int(p["num_experts"])
        self.top = int(p["top"])
        self.inter = int(p["expert_size"])
        if not 0 < self.top <= self.n_exp:
            raise ValueError(f"moe: top {self.top} of {self.n_exp} experts")
        limit = getattr(env.ops, "MOE_MAX_EXPERTS", None)
        if limit is not None and self.n_exp > limit:
            raise ValueError(f"moe: {self.n_exp} experts; the routing kernels take up to {limit}")
        top_limit = getattr(env.ops, "MOE_MAX_TOP", None)
        if top_limit is not None and self.top > top_limit:
            raise ValueError(f"moe: top {self.top}; the routing kernels take up to {top_limit}")
        self.router_bias = bool(p.get("router_bias", False))
        self.score = str(p.get("score", "softmax"))
        if self.score not in ("softmax", "sigmoid", "softmax_all"):
            raise ValueError(f"moe: score '{self.score}' is not known (softmax, sigmoid, softmax_all)")
        self.groups, self.keep_groups = int(p.get("groups") or 0), int(p.get("keep_groups") or 0)
        if self.groups:
            if self.score != "sigmoid":
                raise ValueError("moe: groups of experts go with sigmoid scores")
            if self.n_exp % self.groups or not 0 < self.keep_groups <= self.groups:
                raise ValueError(f"moe: {self.n_exp} experts in {self.groups} groups of which {self.keep_groups} are kept")
            if self.top > self.keep_groups * (self.n_exp // self.groups):
                raise ValueError(f"moe: top {self.top} exceeds the experts of {self.keep_groups} groups")
        self.group_score_top = int(p.get("group_score_top", 2))
        self.weight_scale = float(p.get("weight_scale", 1.0))
        self.weight_sum_eps = float(p.get("weight_sum_eps", 0.0))
        self.shared_gate = bool(p.get("shared_gate", False))
        if self.shared_gate and not int(p.get("shared_size") or 0):
            raise ValueError("moe: a shared gate needs a shared expert")
        self.shared = None
        shared = int(p.get("shared_size") or 0)
        if shared:
            sp = {"hidden_size": self.hidden, "intermediate_size": shared}
            if p.get("shared_names"):
                sp["tensor_names"] = dict(p["shared_names"])
            self.shared_rel = str(p.get("shared_prefix", "shared."))
            self.shared = part_class("ffn", "swiglu")(sp, prefix + self.shared_rel, env)
        self.w_router = self.b_router = self.w_gate_up = self.w_down = None

    def _expert(self, i: int, what: str) -> str:
        return f"experts.{i}.{what}_proj.weight"

    def tensor_name(self, rel: str) -> str:
        names = self.params.get("tensor_names", {})
        if rel in names:
            return self.prefix + names[rel]
        if rel.startswith("experts."):                       # "experts.<i>.gate_proj.weight" by the pattern's name
            _, i, what = rel.split(".", 2)
            pattern = names.get("experts.*." + what)
            if pattern is not None:
                return self.prefix + pattern.replace("*", i)
        if self.shared is not None and rel.startswith("shared:"):
            return self.shared.tensor_name(rel[len("shared:"):])
        return self.prefix + rel

    def tensors(self):
        t = {"router.weight": TensorDecl((self.n_exp, self.hidden))}
        if self.router_bias:
            t["router.bias"] = TensorDecl((self.n_exp,), "bias")
        if self.shared_gate:
            t["shared_gate.weight"] = TensorDecl((1, self.hidden))
        for i in range(self.n_exp):
            t[self._expert(i, "gate")] = TensorDecl((self.inter, self.hidden))
            t[self._expert(i, "up")] = TensorDecl((self.inter, self.hidden))
            t[self._expert(i, "down")] = TensorDecl((self.hidden, self.inter))
        if self.shared is not None:
            for rel, d in self.shared.tensors().items():
                t["shared:" + rel] = d
        return t

    def bind(self, tensors):
        # A router stored in the compute type goes through the matrix product every other projection takes (the products
        # of bfloat16 values are exact in float32 and are added in float32); one stored wider keeps its own kernel.
        w_r = tensors["router.weight"]
        if self.shared_gate:
            # the shared expert's gate is one more row of the router's product
            if tensors["shared_gate.weight"].dtype != w_r.dtype:
                raise ValueError(f"{self.prefix}: the router and the shared expert's gate are stored with different types")
            w_r = torch.cat([w_r, tensors["shared_gate.weight"].view(1, self.hidden)], dim=0).contiguous()
        self.w_router_same = w_r if w_r.dtype == self.env.dtype else None
        self.w_router = as_f32(w_r, self.env) if self.w_router_same is None else None
        self.b_router = as_f32(tensors["router.bias"], self.env) if self.router_bias else None
        per = {what: [tensors[self._expert(i, what)] for i in range(self.n_exp)] for what in ("gate", "up", "down")}
        if len({w.dtype for ws in per.values() for w in ws}) != 1:
            raise ValueError(f"{self.prefix}: the experts' matrices are stored with different types")
        # every expert's gate and up matrices as one matrix in the gated layout (gate rows, filled up to a multiple of
        # 128, then the up rows): what the gating epilogue of the tensor-core product reads, and the other kernels too
        self.w_gate_up = torch.stack([gated_layout(g, u) for g, u in zip(per["gate"], per["up"])]).contiguous()
        self.w_down = torch.stack(per["down"]).contiguous()          # [E, hidden, inner]
        if self.shared is not None:
            self.shared.bind({rel[len("shared:"):]: t for rel, t in tensors.items() if rel.startswith("shared:")})

    def active_matrix_params(self) -> int:
        """Elements of the matrices one token passes through: the router, ``top`` experts, the shared expert."""
        shared = 3 * self.hidden * self.shared.inter if self.shared is not None else 0
        return self.n_exp * self.hidden + self.top * 3 * self.hidden * self.inter + shared

    def forward(self, x, ctx) -> Branch:
        ops = ctx.ops
        n = x.shape[0]
        pairs = n * self.top
        choice = ctx.buffer("moe.choice", (n, self.top), torch.int32)
        weight = ctx.buffer("moe.weight", (n, self.top), torch.float32)
        plain = self.score == "softmax" and not self.shared_gate
        shared_scale = ctx.buffer("moe.shared_scale", (n,), torch.float32) if self.shared_gate else None
        rule = {} if plain else dict(rule=ops.RouterRule(self.score, self.groups, self.keep_groups, self.group_score_top,
                                                        self.weight_scale, self.weight_sum_eps), extra_out=shared_scale)
        if self.w_router_same is not None and x.dtype == self.w_router_same.dtype and hasattr(ops, "moe_topk"):
            ops.moe_topk(linear(ctx, x, self.w_router_same, "moe.logits", torch.float32), self.b_router, choice, weight, **rule)
        else:
            if self.w_router is None:
                self.w_router = as_f32(self.w_router_same, self.env)
            ops.moe_route(x, self.w_router, self.b_router, choice, weight, **rule)
        tile = ops.moe_tile_rows(x.dtype, pairs, self.n_exp, self.hidden, self.inter)
        cap = ops.moe_row_capacity(pairs, self.n_exp, tile)
        row_of_pair = ctx.buffer("moe.row_of_pair", (pairs,), torch.int32)
        token_of_row = ctx.buffer("moe.token_of_row", (cap,), torch.int32)
        tile_expert = ctx.buffer("moe.tile_expert", (cap // tile,), torch.int32)
        ops.moe_plan(choice, self.n_exp, row_of_pair, token_of_row, tile_expert)
        act = ctx.buffer("moe.act", (cap, self.inter))
        if tile == ops.MOE_TILE_ROWS:
            ops.moe_gated(x, token_of_row, tile_expert, self.w_gate_up, act)
        else:
            # a prompt step on the tensor cores: the layout's rows as a matrix of their own, then the grouped tcgen05 product
            rows = ctx.buffer("moe.rows", (cap, self.hidden))
            ops.moe_gather_rows(x, token_of_row, rows)
            ops.moe_gated(rows, None, tile_expert, self.w_gate_up, act)
        y = ctx.buffer("moe.y", (cap, self.hidden), torch.float32)
        ops.moe_down(act, tile_expert, self.w_down, y)
        shared = self.shared.forward(x, ctx).data if self.shared is not None else None
        out = ctx.buffer("moe.out", (1, n, self.hidden), torch.float32)
        if shared_scale is not None:
            ops.moe_combine(y, row_of_pair, weight, shared, out[0], shared_scale=shared_scale)
        else:
            ops.moe_combine(y, row_of_pair, weight, shared, out[0])
        return Branch(out)


register_part("ffn", "moe", MoeFeedForward)
