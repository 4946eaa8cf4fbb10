"""Attention whose keys and values of all heads come from one small latent vector per token.

Per token the mixer's input ``h`` gives

* queries ``q = W_q h``, head by head ``[dim unrotated | rot_dim rotated]``;
* ``W_dkv h`` = ``[kv_rank | rot_dim]``: the first part, RMS-normed with a weight, is the latent ``c``; the second,
  rotated by the token's position, is one key part that every head shares;
* per head ``k_h = [W_uk,h c | shared rotated part]`` and ``v_h = W_uv,h c``.

Only ``c`` and the rotated key part are kept per position.  The products with ``W_uk`` and ``W_uv`` are moved to the
query's side (they are linear): ``q_h . W_uk,h c = (W_uk,h^T q_h) . c`` and ``sum_j p_j W_uv,h c_j = W_uv,h sum_j p_j c_j``.
So attention runs over ONE key/value head whose keys are ``[c | rotated part]`` (``kv_rank + rot_dim`` elements) and
whose values are ``c``, with queries ``[W_uk,h^T q_h,unrotated | q_h,rotated]``, in the same kernels, cache pages and
rings as every other attention; the score's scale, the mask (sliding window or chunks) and a learned sink per head are
parameters.  The cache holds one row per position: the key's pages are read as the values too (a value head as long as a
key head, so that the tensor-core kernels take it), and the per-head product with ``W_uv`` reads the first ``kv_rank``
elements of what attention returns; the rest (the weighted rotated parts) is never looked at.  One kernel (``ops.latent_prep``) adds the input product's partial sums, norms
the latent, rotates and writes queries, keys and values; ``ops.head_linear`` is the per-head product on either side.
Norm statistics, angles, scores and softmax weights are float32 whatever the compute type.

Two further forms, by parameter.  ``q_rank``: the queries pass a bottleneck of their own, ``q = W_uq RMSnorm(W_dq h)``
(the norm with a weight of ``q_rank`` elements); the input product then yields the queries' latent, which the same
kernel norms, and a second product makes the queries.  ``out_gate``: the concatenated heads are multiplied element by
element by ``sigmoid(W_g h)`` before the output product; ``W_g`` rides in the input product and ``ops.sigmoid_gate``
applies it to the per-head products' result.  Which elements a rotation pairs (halves, or neighbours) is the position
encoding's.
"""
from __future__ import annotations

import torch

from ..kernels.linear import linear
from .base import Branch, KvNeed, Mixer, TensorDecl, as_f32, register_part

_Q, _DKV, _UK, _UV, _O = "q_proj.weight", "kv_down_proj.weight", "k_up_proj.weight", "v_up_proj.weight", "o_proj.weight"


class LatentAttention(Mixer):
    """params: hidden_size, num_heads, head_dim (unrotated elements of a query/key head), rot_dim (rotated elements),
    value_dim, kv_rank, norm_eps (of the latent's norm), window (0 = all keys), mask ("window" or "chunk"),
    softmax_scale, sink (None or "learned": a tensor ``sink`` [num_heads]), position (name of a rotary encoding over
    ``rot_dim`` elements), q_rank (0: queries by one matrix ``q_proj``; else ``q_down_proj`` [q_rank, hidden],
    ``q_norm.weight`` [q_rank], ``q_up_proj``), out_gate (bool: a tensor ``gate_proj.weight`` [num_heads value_dim, hidden])."""

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        p = params
        self.hidden = int(p["hidden_size"])
        self.nh = int(p["num_heads"])
        self.dim = int(p["head_dim"])
        self.rdim = int(p["rot_dim"])
        self.vdim = int(p["value_dim"])
        self.rank = int(p["kv_rank"])
        for what, v in (("num_heads", self.nh), ("head_dim", self.dim), ("value_dim", self.vdim), ("kv_rank", self.rank)):
            if v <= 0:
                raise ValueError(f"latent_attention: {what} must be positive, got {v}")
        if self.rdim < 0 or self.rdim % 2:
            raise ValueError(f"latent_attention: rot_dim {self.rdim} must be even and not negative")
        self.kd = self.rank + self.rdim                      # elements of a cached key
        limit = getattr(env.ops, "ATTN_MAX_HEAD_DIM", None)
        if limit is not None and self.kd > limit:
            raise ValueError(f"latent_attention: kv_rank + rot_dim = {self.kd}; the attention kernels take keys of up to {limit}")
        self.eps = float(p["norm_eps"])
        self.window = int(p.get("window", 0) or 0)
        self.mask = p.get("mask", "window")
        if self.mask not in ("window", "chunk"):
            raise ValueError(f"latent_attention: mask '{self.mask}' is not known (window, chunk)")
        self.scale = float(p["softmax_scale"])
        if not self.scale > 0:
            raise ValueError("latent_attention: the score scale must be positive")
        self.sink_kind = p.get("sink")
        if self.sink_kind not in (None, "learned"):
            raise ValueError(f"latent_attention: sink '{self.sink_kind}' is not known (None, 'learned')")
        enc = p.get("position")
        self.encoding = env.encodings[enc] if enc is not None else None
        if (self.encoding is None) != (self.rdim == 0):
            raise ValueError("latent_attention: rotated elements and a position encoding come together")
        self.q_rank = int(p.get("q_rank") or 0)
        self.out_gate = bool(p.get("out_gate", False))
        self.w_in = self.w_o = self.w_absorb = self.w_uv = self.c_norm_w = self.sinks = self.form = None
        self.w_uq = self.q_norm_w = None

    def tensors(self):
        qw = self.nh * (self.dim + self.rdim)
        if self.q_rank:
            t = {"q_down_proj.weight": TensorDecl((self.q_rank, self.hidden)),
                 "q_norm.weight": TensorDecl((self.q_rank,), "norm"),
                 "q_up_proj.weight": TensorDecl((qw, self.q_rank))}
        else:
            t = {_Q: TensorDecl((qw, self.hidden))}
        if self.out_gate:
            t["gate_proj.weight"] = TensorDecl((self.nh * self.vdim, self.hidden))
        t.update({
             _DKV: TensorDecl((self.rank + self.rdim, self.hidden)),
             "kv_norm.weight": TensorDecl((self.rank,), "norm"),
             _UK: TensorDecl((self.nh * self.dim, self.rank)),
             _UV: TensorDecl((self.nh * self.vdim, self.rank)),
             _O: TensorDecl((self.hidden, self.nh * self.vdim))})
        if self.sink_kind == "learned":
            t["sink"] = TensorDecl((self.nh,), "bias")
        return t

    def bind(self, tensors):
        # rows of the input product: [queries, or their latent | latent and rotated key part | gate arguments]
        ws = [tensors["q_down_proj.weight"] if self.q_rank else tensors[_Q], tensors[_DKV]]
        if self.out_gate:
            ws.append(tensors["gate_proj.weight"])
        if len({w.dtype for w in ws}) != 1:
            raise ValueError(f"{self.prefix}: the input projections are stored with different types")
        self.w_in = torch.cat(ws, dim=0).contiguous()
        if self.q_rank:
            self.w_uq, self.q_norm_w = tensors["q_up_proj.weight"], tensors["q_norm.weight"]
        # [head][rank][dim]: the key up-projection as it meets the query
        self.w_absorb = tensors[_UK].view(self.nh, self.dim, self.rank).transpose(1, 2).contiguous()
        self.w_uv = tensors[_UV].view(self.nh, self.vdim, self.rank).contiguous()
        self.w_o = tensors[_O]
        self.c_norm_w = tensors["kv_norm.weight"]
        if self.sink_kind == "learned":
            self.sinks = as_f32(tensors["sink"], self.env)
        self.form = self.env.ops.AttentionForm(sinks=self.sinks, chunked=self.mask == "chunk")

    def cache_need(self):
        return KvNeed(1, self.kd, self.window, values_in_keys=True)

    def forward(self, x, ctx, cache) -> Branch:
        ops = ctx.ops
        n = x.shape[0]
        rot = self.encoding.rotation() if self.encoding is not None else None
        rows = linear(ctx, x, self.w_in, "lattn.in", torch.float32)
        q_plain = ctx.buffer("lattn.q_plain", (n, self.nh, self.dim))
        q = ctx.buffer("lattn.q", (n, self.nh, self.kd))
        q_cols = self.q_rank or self.nh * (self.dim + self.rdim)             # the first columns of ``rows``
        common = dict(n_heads=self.nh, head_dim=self.dim, rot_dim=self.rdim, kv_rank=self.rank, c_norm_w=self.c_norm_w,
                      norm_eps=self.eps, cos=rot.cos if rot else None, sin=rot.sin if rot else None,
                      pairing=rot.pairing if rot else 0, positions=ctx.positions, kv_col=q_cols)
        queries = dict(q_plain_out=q_plain, q_out=q)
        pages = dict(k_pages=cache.k_pages, page_table=cache.page_table,
                     ring_pages=cache.ring_pages, seq_of_token=ctx.seq_of_token, slots=ctx.slots)
        write_now = ctx.decode or self.window == 0       # a ring's pages may hold keys that this step's queries still need
        k_new = None if ctx.decode else ctx.buffer("lattn.k_new", (n, 1, self.kd))
        kv = dict(k_new=k_new, **(pages if write_now else {}))
        if self.q_rank:
            # keys and the queries' normed latent first, then the queries from their own product
            cq = ctx.buffer("lattn.cq", (n, self.q_rank))
            ops.latent_prep(rows, **common, **kv, q_col=-1, cq_col=0, cq_norm_w=self.q_norm_w, cq_out=cq)
            q_rows = linear(ctx, cq, self.w_uq, "lattn.q_rows", torch.float32)
            ops.latent_prep(q_rows, **dict(common, kv_col=-1), **queries, q_col=0)
        else:
            ops.latent_prep(rows, **common, **kv, **queries, q_col=0)
        ops.head_linear(q_plain, self.w_absorb, q[:, :, :self.rank])
        mixed = ctx.buffer("lattn.mixed", (n, self.nh, self.kd))            # per head sum_j p_j [c_j | rotated part]
        if ctx.decode:
            plan = ops.attn_decode_plan(q.dtype, ctx.n_seqs, self.nh, 1, self.kd, ctx.max_len_after, self.form)
            scratch = ctx.buffer("attn.scratch", (max(1, plan.scratch_floats),), torch.float32)
            counters = None
            if plan.n_counters:
                counters = ctx.buffer("attn.counters", (plan.n_counters,), torch.int32, zero=True)
            ops.attn_decode(q, cache.k_pages, cache.v_pages, cache.page_table, cache.ring_pages, ctx.slots,
                            ctx.len_before, mixed.view(n, self.nh * self.kd), scratch, scale=self.scale,
                            window=self.window, plan=plan, counters=counters, form=self.form)
        else:
            tq = ops.prefill_tile_queries(q.dtype, self.kd, self.form)
            ops.attn_prefill(q, k_new, k_new, cache.k_pages, cache.v_pages, cache.page_table, cache.ring_pages,
                             ctx.query_tiles(tq), ctx.cu_tokens, ctx.len_before, ctx.slots,
                             mixed.view(n, self.nh * self.kd), scale=self.scale, window=self.window,
                             tile_queries=tq, form=self.form)
            if not write_now:
                ops.kv_write(k_new, k_new, cache.k_pages, cache.v_pages, cache.page_table, cache.ring_pages,
                             ctx.positions, ctx.seq_of_token, ctx.slots, ctx.cu_tokens, ctx.len_before)
        out = ctx.buffer("lattn.out", (n, self.nh, self.vdim))
        ops.head_linear(mixed[:, :, :self.rank], self.w_uv, out)
        if self.out_gate:
            ops.sigmoid_gate(out.view(n, self.nh * self.vdim), rows, q_cols + self.kd)
        return Branch(linear(ctx, out.view(n, self.nh * self.vdim), self.w_o, "lattn.proj", torch.float32))


register_part("mixer", "latent_attention", LatentAttention)
