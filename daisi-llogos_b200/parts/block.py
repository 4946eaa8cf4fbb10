"""Arrangements of norms, a mixer and a feed-forward around the residual stream.

``PreNormBlock`` is the reference's order (Inference/ForwardPass.cs:215-250): the output of the
previous feed-forward is added to the residual inside this block's first norm; the attention
output is added inside the second norm; the block returns its feed-forward output still to
be added (by the next block's first norm, or by the model's final norm).
"""
from __future__ import annotations

from typing import Optional

from .base import Block, Branch, register_part


class PreNormBlock(Block):
    """roles: norm1, mixer, norm2, ffn (a layer without a feed-forward leaves norm2 and ffn out)."""

    ROLES = {"norm1": "norm", "mixer": "mixer", "norm2": "norm", "ffn": "ffn"}

    def forward(self, residual, pending: Optional[Branch], ctx, cache) -> Optional[Branch]:
        p = self.parts
        h, kw = normed_for(p["norm1"], p["mixer"], residual, pending, ctx)
        a = p["mixer"].forward(h, ctx, cache, **kw)
        if "ffn" not in p:
            return a
        h, kw = normed_for(p["norm2"], p["ffn"], residual, a, ctx)
        return p["ffn"].forward(h, ctx, **kw)


class ParallelBlock(Block):
    """One norm whose output feeds the mixer and the feed-forward side by side; both outputs enter the residual
    together, times ``residual_scale``: ``x' = x + s (mixer(h) + ffn(h))`` with ``h = norm1(x)``.  roles: norm1, mixer,
    ffn (a layer may have no feed-forward).  The norm that adds the block's pending branch must take several sets
    of partials and a scale (``layernorm`` does).  params: residual_scale (default 1)."""

    ROLES = {"norm1": "norm", "mixer": "mixer", "ffn": "ffn"}

    def __init__(self, params, prefix, env, parts):
        super().__init__(params, prefix, env, parts)
        for role in ("norm1", "mixer"):
            if role not in parts:
                raise ValueError(f"parallel block: no part for the role '{role}'")
        self.scale = float(self.params.get("residual_scale", 1.0))

    def forward(self, residual, pending: Optional[Branch], ctx, cache) -> Optional[Branch]:
        p = self.parts
        # neither consumer gets a row scale: both read the same finished rows
        h = p["norm1"].forward(residual, pending, ctx)
        a = p["mixer"].forward(h, ctx, cache)
        if a.more or a.scale != 1.0 or a.write is not None:
            raise ValueError("parallel block: the mixer's branch must be plain partials")
        if "ffn" not in p:
            return Branch(a.data, scale=self.scale)
        f = p["ffn"].forward(h, ctx)
        return Branch(a.data, more=(f.data,) + tuple(f.more), scale=self.scale)


class TwoNormParallelBlock(Block):
    """Mixer and feed-forward side by side, each behind a norm of its own over the SAME residual, and an optional last
    sublayer that reads the residual once both have been added:

        x' = x + mixer(norm1(x)) + ffn(norm2(x));     x'' = x' + side(x')

    roles: norm1, mixer, and optionally norm2 + ffn and side (family "connection": a part with
    ``forward(residual, pending, ctx) -> Branch`` that adds the pending branch itself, because it reads the sum).  Both
    norms run in one launch (``norm1.forward_many``), which also adds the branch the block before left pending.  The
    sublayers' branches may be several terms with norms and factors of their own; they are handed on as one branch of
    terms, so the norm that adds them must take terms."""

    ROLES = {"norm1": "norm", "mixer": "mixer", "norm2": "norm", "ffn": "ffn", "side": "connection"}

    def __init__(self, params, prefix, env, parts):
        super().__init__(params, prefix, env, parts)
        for role in ("norm1", "mixer"):
            if role not in parts:
                raise ValueError(f"two-norm parallel block: no part for the role '{role}'")
        if ("ffn" in parts) != ("norm2" in parts):
            raise ValueError("two-norm parallel block: norm2 and ffn come together or not at all")
        if not hasattr(parts["norm1"], "forward_many"):
            raise ValueError("two-norm parallel block: norm1 must be a norm that can share its launch (rmsnorm)")

    def forward(self, residual, pending: Optional[Branch], ctx, cache) -> Optional[Branch]:
        p = self.parts
        if "ffn" in p:
            h1, h2 = p["norm1"].forward_many(residual, pending, ctx, (p["norm2"],))
        else:
            (h1,) = p["norm1"].forward_many(residual, pending, ctx, ())
        terms = p["mixer"].forward(h1, ctx, cache).as_terms()
        if "ffn" in p:
            terms = terms + p["ffn"].forward(h2, ctx).as_terms()
        out = Branch.of_terms(terms)
        if "side" in p:
            out = p["side"].forward(residual, out, ctx)
        return out


def normed_for(norm, consumer, residual, pending, ctx, rows=None):
    """``(x, keyword arguments)`` for ``consumer.forward``: a consumer that takes a row scale lets the norm leave
    its division to the consumer's first product."""
    if getattr(consumer, "TAKES_ROW_SCALE", False):
        x, scale = norm.forward_unscaled(residual, pending, ctx, rows)
        return x, {"row_scale": scale}
    return norm.forward(residual, pending, ctx, rows), {}


register_part("block", "prenorm", PreNormBlock)
register_part("block", "parallel", ParallelBlock)
register_part("block", "two_norm_parallel", TwoNormParallelBlock)
