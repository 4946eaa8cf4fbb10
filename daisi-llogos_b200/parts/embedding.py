"""Token embedding and output head.

The embedding copies one table row per token, unscaled, into the float32 residual stream
(Inference/ForwardPass.cs:205).  The head is a matrix product of the final norm's output with
the vocabulary matrix, which is the embedding table itself when the model ties them
(Model/ModelWeights.cs:29); logits are float32.
"""
from __future__ import annotations

import torch

from ..kernels.linear import linear
from .base import Branch, Part, StateNeed, TensorDecl, Term, as_f32, register_part


class TokenEmbedding(Part):
    """params: vocab_size, hidden_size, streams (0: the residual is one ``[N, hidden]`` array; S >= 1: it is S
    streams ``[S, N, hidden]`` that all start as the embedding)."""

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        self.vocab = int(params["vocab_size"])
        self.hidden = int(params["hidden_size"])
        self.streams = int(params.get("streams", 0) or 0)
        self.weight = None

    def tensors(self):
        return {"weight": TensorDecl((self.vocab, self.hidden), "table")}

    def bind(self, tensors):
        self.weight = tensors["weight"]

    def forward(self, ctx) -> torch.Tensor:
        if self.streams:
            residual = ctx.buffer("residual", (self.streams, ctx.n_tokens, self.hidden), torch.float32)
            ctx.ops.embed_rows(self.weight, ctx.token_ids, residual)       # every stream starts as the embedding
            return residual
        residual = ctx.buffer("residual", (ctx.n_tokens, self.hidden), torch.float32)
        ctx.ops.embed_rows(self.weight, ctx.token_ids, residual)
        return residual


class PairHashEmbedding(Part):
    """``x = scale * table[token] + pair_table[(previous token * mul_prev + token * mul_cur) mod buckets]``, then an RMS norm
    of the sum into the residual; a sequence's first token takes the pair table's last row (row ``buckets``).  The token
    before a step's first one is part of the sequence's state (one int32 per slot), so a prompt cut into steps and a token
    decoded alone see the same pair as the whole prompt does.

    params: vocab_size, hidden_size, scale (default 1), pair (None, or {"buckets", "mul_prev", "mul_cur"}: a tensor
    ``pair.weight`` [buckets + 1, hidden]), norm_eps (None: no norm; else a tensor ``norm.weight`` [hidden]),
    norm_offset (added to the norm's weight, default 0), side_width (0, or the width of a second table
    ``side.weight`` [vocab, side_width] that other parts read by the token's id: they name it with ``tied_to``)."""

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        self.vocab = int(params["vocab_size"])
        self.hidden = int(params["hidden_size"])
        self.scale = float(params.get("scale", 1.0))
        pair = params.get("pair")
        self.pair = None
        if pair:
            self.pair = (int(pair["buckets"]), int(pair["mul_prev"]), int(pair["mul_cur"]))
            if self.pair[0] <= 0:
                raise ValueError(f"pair embedding: {self.pair[0]} buckets")
        eps = params.get("norm_eps")
        self.norm_eps = None if eps is None else float(eps)
        self.norm_offset = float(params.get("norm_offset", 0.0) or 0.0)
        self.side_width = int(params.get("side_width", 0) or 0)
        self.weight = self.pair_table = self.norm_w = self.side_table = None

    def tensors(self):
        t = {"weight": TensorDecl((self.vocab, self.hidden), "table")}
        if self.pair:
            t["pair.weight"] = TensorDecl((self.pair[0] + 1, self.hidden), "table")
        if self.norm_eps is not None:
            t["norm.weight"] = TensorDecl((self.hidden,), "bias" if self.norm_offset else "norm")
        if self.side_width:
            t["side.weight"] = TensorDecl((self.vocab, self.side_width), "table")
        return t

    def bind(self, tensors):
        self.weight = tensors["weight"]
        self.pair_table = tensors.get("pair.weight")
        self.side_table = tensors.get("side.weight")
        if self.norm_eps is not None:
            self.norm_w = as_f32(tensors["norm.weight"], self.env)

    def cache_need(self):
        return StateNeed((1,), torch.int32) if self.pair else None

    def forward(self, ctx, cache=None) -> torch.Tensor:
        residual = ctx.buffer("residual", (ctx.n_tokens, self.hidden), torch.float32)
        buckets, mul_prev, mul_cur = self.pair or (0, 0, 0)
        if self.pair and cache is None:
            raise ValueError("pair embedding: the step brought no state for the sequences' last tokens")
        ctx.ops.hash_embed(self.weight, self.scale, self.pair_table, buckets, mul_prev, mul_cur, ctx.token_ids,
                           ctx.positions, ctx.seq_of_token, ctx.cu_tokens, ctx.slots,
                           cache.state if self.pair else None, self.norm_w, self.norm_offset,
                           self.norm_eps if self.norm_eps is not None else 1.0, residual)
        return residual


class TokenSideInput(Part):
    """A sublayer that reads the residual AFTER the pending branch has been added and adds a small per-token input:

        e = table[token][offset : offset + dim];   y = W_proj (act(W_gate x) * e);   x <- x + y / rms(y) * weight

    ``forward(residual, pending, ctx)`` adds the pending branch (one launch, which also leaves the sum in the compute
    type for the gate's product), runs the two small products and returns ``y`` as a branch whose term carries the norm.
    params: hidden_size, dim, offset, eps, activation (default "gelu_tanh"), tied_to (full name of the table's tensor,
    declared by the embedding).  Tensors: ``gate.weight`` [dim, hidden], ``proj.weight`` [hidden, dim], ``norm.weight``
    [hidden]."""

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        self.hidden = int(params["hidden_size"])
        self.dim = int(params["dim"])
        self.offset = int(params.get("offset", 0))
        self.eps = float(params["eps"])
        self.activation = str(params.get("activation", "gelu_tanh"))
        known = getattr(env.ops, "ACTIVATIONS", None)
        if known is not None and self.activation not in known:
            raise ValueError(f"token side input: activation '{self.activation}' is not known ({', '.join(known)})")
        self.tied_to = params.get("tied_to")
        if not self.tied_to:
            raise ValueError("token side input: 'tied_to' must name the table's tensor")
        self.table = self.w_gate = self.w_proj = self.norm_w = None

    def tensors(self):
        return {"gate.weight": TensorDecl((self.dim, self.hidden)), "proj.weight": TensorDecl((self.hidden, self.dim)),
                "norm.weight": TensorDecl((self.hidden,), "norm")}

    def bind(self, tensors):
        self.table = tensors["weight"]                       # the tensor ``tied_to`` names
        if self.table.dim() != 2 or self.table.shape[1] < self.offset + self.dim:
            raise ValueError(f"token side input: the table {tuple(self.table.shape)} has no columns "
                             f"[{self.offset}, {self.offset + self.dim})")
        self.w_gate, self.w_proj = tensors["gate.weight"], tensors["proj.weight"]
        self.norm_w = as_f32(tensors["norm.weight"], self.env)

    def forward(self, residual, pending, ctx) -> Branch:
        n = residual.shape[0]
        x = ctx.buffer("side.x", (n, self.hidden))
        terms = () if pending is None else pending.as_terms()
        ctx.ops.multi_add_rmsnorm(residual, [(t.data, t.weight, t.eps, t.scale) for t in terms], [(x, None, 0.0)], self.eps)
        gate = linear(ctx, x, self.w_gate, "side.gate", torch.float32)
        g = ctx.buffer("side.g", (n, self.dim))
        ctx.ops.table_gate(gate, self.table, self.offset, ctx.token_ids, g, self.activation)
        y = linear(ctx, g, self.w_proj, "side.proj", torch.float32)
        return Branch.of_terms([Term(y, self.norm_w, self.eps, 1.0)])


class LinearHead(Part):
    """params: vocab_size, hidden_size, tied_to (full name of the tensor to share, or None), softcap (0 or None: none;
    c: the logits become ``c tanh(logits / c)``)."""

    TAKES_ROW_SCALE = True

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        self.vocab = int(params["vocab_size"])
        self.hidden = int(params["hidden_size"])
        self.tied_to = params.get("tied_to")
        self.softcap = float(params.get("softcap") or 0.0)
        if self.softcap < 0:
            raise ValueError(f"output head: softcap must not be negative, got {self.softcap}")
        self.weight = None

    def tensors(self):
        if self.tied_to:
            return {}
        return {"weight": TensorDecl((self.vocab, self.hidden))}

    def bind(self, tensors):
        self.weight = tensors["weight"]
        if tuple(self.weight.shape) != (self.vocab, self.hidden):
            raise ValueError(f"output head: shared tensor has shape {tuple(self.weight.shape)}, "
                             f"expected {(self.vocab, self.hidden)}")

    def forward(self, x, ctx, row_scale=None) -> torch.Tensor:
        # the logits go to samplers and callers as they are: one product, no partial sums to add up
        logits = linear(ctx, x, self.weight, "head.logits", torch.float32, split_k=False, row_scale=row_scale)[0]
        if self.softcap:
            ctx.ops.tanh_cap(logits, self.softcap)
        return logits


register_part("embedding", "token_embedding", TokenEmbedding)
register_part("embedding", "pair_hash_embedding", PairHashEmbedding)
register_part("connection", "token_side_input", TokenSideInput)
register_part("head", "linear_head", LinearHead)
