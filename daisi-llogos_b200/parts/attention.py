"""Grouped-query attention with rotary positions over the paged cache.

Order of operations as in the reference (Inference/ForwardPass.cs:329-405): q, k, v
projections; optional per-head RMSNorm of q and k (:372-376); optional biases (:380-382);
rotation of q and k (:385); keys and values into the cache (:388); causal softmax attention
with ``scale = 1/sqrt(head_dim)`` applied to the dot product (:336, :399-400); output
projection (:404).  A window of W makes a query see only the last W keys, its own included
(Inference/AttentionStrategy.cs:64-71).  The reference leaves the biases out of its batched
prompt path (:783-794); here every path applies them.

Beyond the reference, all by parameter: value heads of another size than the key heads; a mask by chunks (a query sees
the keys of its own chunk of ``window`` positions, chunks counted from position 0) instead of the sliding window; a
learned sink per query head in the softmax's denominator (``p_j = e^{s_j} / (e^{sink_h} + sum e^{s_j})``, no key, no
value, not scaled); and values blended across layers: the first layer of a group keeps its own values and lends them
(float32, per step) to the others, which cache ``(1 - lam) v + lam v_first`` with a learned number ``lam`` each.
"""
from __future__ import annotations

import math

import torch

from ..kernels.linear import linear
from .base import Branch, KvNeed, Mixer, MultiNeed, StateNeed, TensorDecl, as_f32, register_part


class Attention(Mixer):
    """params: hidden_size, num_heads, num_kv_heads, head_dim, qkv_bias, qk_norm, qk_norm_eps,
    window (0 = all keys), position (name of a position encoding or None), softmax_scale
    (None = 1/sqrt(head_dim)), own_kv (False: no k/v projections, reads another entry's cache), value_dim (None =
    head_dim), mask ("window": the last ``window`` keys; "chunk": the keys of the query's own chunk of ``window``
    positions), sink (None or "learned": a tensor ``sink`` [num_heads]), value_blend (None, or the name of a group of
    layers that blend their values with the group's first layer's; every member has a tensor ``vmix`` [], which the
    first does not use), conv_taps (0, or the taps of a short causal convolution over time on every channel of q, k and v,
    directly behind the projections: tensors ``q_proj.conv``, ``k_proj.conv``, ``v_proj.conv`` [channels, taps], the last
    column the current token's; the last ``taps - 1`` projected rows of a sequence are kept as float32 state beside the
    keys and values), out_gate (False, or True: the concatenated heads are multiplied by ``sigmoid(g_proj x)`` before
    the output projection; a tensor ``g_proj.weight`` [num_heads * value_dim, hidden])."""

    TAKES_ROW_SCALE = True

    def __init__(self, params, prefix, env):
        super().__init__(params, prefix, env)
        p = params
        self.hidden = int(p["hidden_size"])
        self.nh = int(p["num_heads"])
        self.nkv = int(p["num_kv_heads"])
        self.hd = int(p["head_dim"])
        if self.nh % self.nkv:
            raise ValueError(f"{self.nh} heads are not a multiple of {self.nkv} key/value heads")
        # said when the model is built, not at its first step
        limit = getattr(env.ops, "ATTN_MAX_HEAD_DIM", None)
        if limit is not None and not 0 < self.hd <= limit:
            raise ValueError(f"head_dim {self.hd}: the attention kernels take head sizes from 1 to {limit}")
        self.qkv_bias = bool(p.get("qkv_bias", False))
        self.qk_norm = bool(p.get("qk_norm", False))
        self.qk_norm_eps = float(p.get("qk_norm_eps", 1e-6))
        self.window = int(p.get("window", 0) or 0)
        self.own_kv = bool(p.get("own_kv", True))
        self.vd = int(p.get("value_dim") or self.hd)
        if limit is not None and not 0 < self.vd <= limit:
            raise ValueError(f"value_dim {self.vd}: the attention kernels take head sizes from 1 to {limit}")
        self.mask = p.get("mask", "window")
        if self.mask not in ("window", "chunk"):
            raise ValueError(f"attention: mask '{self.mask}' is not known (window, chunk)")
        if self.mask == "chunk" and self.window <= 0:
            raise ValueError("attention: a mask by chunks needs the chunk's size as 'window'")
        self.sink_kind = p.get("sink")
        if self.sink_kind not in (None, "learned"):
            raise ValueError(f"attention: sink '{self.sink_kind}' is not known (None, 'learned')")
        self.blend_group = p.get("value_blend")
        if self.blend_group is not None and not self.own_kv:
            raise ValueError("attention: values are blended by the layer that projects them (own_kv)")
        self.conv_taps = int(p.get("conv_taps", 0) or 0)
        taps_limit = getattr(env.ops, "CONV_MAX_TAPS", None)
        if self.conv_taps < 0 or (taps_limit is not None and self.conv_taps > taps_limit):
            raise ValueError(f"attention: {self.conv_taps} convolution taps (0 to {taps_limit})")
        if self.conv_taps and not self.own_kv:
            raise ValueError("attention: the convolution goes with the layer that projects its keys and values (own_kv)")
        self.out_gate = bool(p.get("out_gate", False))
        self.special = (self.vd != self.hd or self.mask != "window" or self.sink_kind is not None or bool(self.conv_taps)
                        or self.out_gate)
        self.w_gate = self.w_conv = None
        if self.conv_taps:
            self.TAKES_ROW_SCALE = False      # the convolution mixes rows: every row arrives finished
        self.form = None
        self.sinks = self.v_lambda = None
        scale = p.get("softmax_scale")
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.hd)
        enc = p.get("position")
        self.encoding = env.encodings[enc] if enc is not None else None
        self.w_qkv = self.w_o = self.b_qkv = self.q_norm_w = self.k_norm_w = None

    # ---- tensors -------------------------------------------------------------------------
    def tensors(self):
        q, kv = self.nh * self.hd, self.nkv * self.hd
        t = {"q_proj.weight": TensorDecl((q, self.hidden)), "o_proj.weight": TensorDecl((self.hidden, self.nh * self.vd))}
        if self.own_kv:
            t["k_proj.weight"] = TensorDecl((kv, self.hidden))
            t["v_proj.weight"] = TensorDecl((self.nkv * self.vd, self.hidden))
        if self.qkv_bias:
            t["q_proj.bias"] = TensorDecl((q,), "bias")
            if self.own_kv:
                t["k_proj.bias"] = TensorDecl((kv,), "bias")
                t["v_proj.bias"] = TensorDecl((self.nkv * self.vd,), "bias")
        if self.qk_norm:
            t["q_norm.weight"] = TensorDecl((self.hd,), "norm")
            if self.own_kv:
                t["k_norm.weight"] = TensorDecl((self.hd,), "norm")
        if self.sink_kind == "learned":
            t["sink"] = TensorDecl((self.nh,), "bias")
        if self.blend_group is not None:
            t["vmix"] = TensorDecl((), "bias")
        if self.conv_taps:
            t["q_proj.conv"] = TensorDecl((q, self.conv_taps), "conv")
            t["k_proj.conv"] = TensorDecl((kv, self.conv_taps), "conv")
            t["v_proj.conv"] = TensorDecl((self.nkv * self.vd, self.conv_taps), "conv")
        if self.out_gate:
            t["g_proj.weight"] = TensorDecl((self.nh * self.vd, self.hidden))
        return t

    def bind(self, tensors):
        names = ["q_proj", "k_proj", "v_proj"] if self.own_kv else ["q_proj"]
        ws = [tensors[n + ".weight"] for n in names]
        if len({w.dtype for w in ws}) != 1:
            raise ValueError(f"{self.prefix}: q/k/v projections are stored with different types")
        self.w_qkv = torch.cat(ws, dim=0).contiguous() if len(ws) > 1 else ws[0]
        self.w_o = tensors["o_proj.weight"]
        if self.qkv_bias:
            bs = [tensors[n + ".bias"] for n in names]
            self.b_qkv = torch.cat(bs, dim=0).contiguous() if len(bs) > 1 else bs[0]
        if self.qk_norm:
            self.q_norm_w = tensors["q_norm.weight"]
            self.k_norm_w = tensors["k_norm.weight"] if self.own_kv else None
            if self.b_qkv is not None and self.b_qkv.dtype != self.q_norm_w.dtype:
                self.b_qkv = self.b_qkv.to(self.q_norm_w.dtype)
        if self.sink_kind == "learned":
            self.sinks = as_f32(tensors["sink"], self.env)
        if self.blend_group is not None:
            self.v_lambda = as_f32(tensors["vmix"], self.env).reshape(1)
        self.qkv_width = self.qkv_width_of() if self.own_kv else self.w_qkv.shape[0]
        if self.conv_taps:
            self.w_conv = torch.cat([as_f32(tensors[n + ".conv"], self.env) for n in names], dim=0).contiguous()
        if self.out_gate:
            self.w_gate = tensors["g_proj.weight"]
            if self.conv_taps and self.w_gate.dtype == self.w_qkv.dtype:
                # behind a convolution the preparation reads a buffer of its own, so the gate's rows can ride in the
                # projections' product
                self.w_qkv = torch.cat([self.w_qkv, self.w_gate], dim=0).contiguous()
                self.w_gate = None
        if self.vd != self.hd or self.mask != "window" or self.sink_kind is not None:
            self.form = self.env.ops.AttentionForm(value_dim=self.vd, sinks=self.sinks, chunked=self.mask == "chunk")

    def cache_need(self):
        if not self.own_kv:
            return None
        kv = KvNeed(self.nkv, self.hd, self.window, 0 if self.vd == self.hd else self.vd)
        if self.conv_taps > 1:
            return MultiNeed.of(kv=kv, conv=StateNeed((self.conv_taps - 1, self.qkv_width_of()), torch.float32))
        return kv

    def qkv_width_of(self) -> int:
        """Columns of the q | k | v rows of a layer that projects its own keys and values."""
        return (self.nh + self.nkv) * self.hd + self.nkv * self.vd

    def check_borrowed(self, need) -> None:
        if self.own_kv:
            raise ValueError("an attention part that reads another entry's cache must have own_kv = False")
        if not isinstance(need, KvNeed):
            raise ValueError("attention can only read a cache of keys and values")
        mine = (self.nkv, self.hd, self.window, self.vd)
        theirs = (need.num_kv_heads, need.head_dim, need.window, need.value_dim or need.head_dim)
        if theirs != mine:
            raise ValueError(f"the owner keeps (key/value heads, head size, window, value head size) = "
                             f"{theirs}, this reader expects {mine}")

    # ---- one step ------------------------------------------------------------------------
    def forward(self, x, ctx, cache, row_scale=None) -> Branch:
        ops = ctx.ops
        n = x.shape[0]
        nkv_in = self.nkv if self.own_kv else 0
        conv_state = None
        if self.conv_taps > 1:
            cache, conv_state = cache["kv"], cache["conv"].state
        rot = self.encoding.rotation() if self.encoding is not None else None
        # A large prompt step on the tensor cores prepares q and k in the projection's own epilogue.  Otherwise the
        # projection writes float32 (partials when the product splits K) and a second kernel prepares them; either
        # way the row scale, bias, norm and rotation see the unrounded sums, so q and k are rounded once.
        fused_qkv = getattr(ops, "gemm_tc_qkv_supported", None)
        scale_kw = {"row_scale": row_scale} if row_scale is not None else {}
        form_kw = {"form": self.form} if self.form is not None else {}
        extra = {}                    # what only the general preparation kernel does
        if self.vd != self.hd:
            extra["value_dim"] = self.vd
        if self.blend_group is not None:
            # the group's first layer of this step lends its values; the others blend theirs with them
            key = ("value_blend", self.blend_group)
            lent = ctx.extras.get(key)
            if lent is None:
                lent = ctx.extras[key] = ctx.buffer(f"attn.v_first.{self.blend_group}", (n, self.nkv, self.vd), torch.float32)
                extra["v_first_out"] = lent
            else:
                if tuple(lent.shape) != (n, self.nkv, self.vd):
                    raise ValueError(f"attention: layers of the value group '{self.blend_group}' differ in their values' shape")
                extra["v_first_in"], extra["v_mix"] = lent, self.v_lambda
        if (not ctx.decode and fused_qkv is not None and not extra and not self.conv_taps and not self.out_gate
                and fused_qkv(x, self.w_qkv, self.hd, rot.rotary_dim if rot else 0, rot.pairing if rot else 0)):
            def prep(qkv_, **kw):
                ops.gemm_tc_qkv(x, self.w_qkv, **kw, **scale_kw)
            qkv = None
        else:
            def prep(qkv_, **kw):
                ops.qk_prep(qkv_, **kw, **scale_kw, **extra)
            qkv = linear(ctx, x, self.w_qkv, "attn.qkv", torch.float32)
        gate, gate_col = None, 0
        if self.out_gate:
            if self.w_gate is None:
                gate, gate_col = qkv, self.qkv_width                 # the gate's arguments lie behind q, k, v in the same rows
            else:
                gate = linear(ctx, x, self.w_gate, "attn.gate", torch.float32)
        if self.conv_taps:
            # the convolution sees the projections' float32 sums and leaves one set of float32 rows of q | k | v for the
            # preparation
            if row_scale is not None:
                raise ValueError("attention: a convolution behind the projections takes finished rows (no row scale)")
            mixed = ctx.buffer("attn.conv", (1, n, self.qkv_width), torch.float32)
            ops.causal_conv(qkv, 0, self.w_conv, conv_state, ctx.slots, ctx.cu_tokens, ctx.seq_of_token, ctx.len_before,
                            mixed[0])
            qkv = mixed
        q = ctx.buffer("attn.q", (n, self.nh, self.hd))
        out = ctx.buffer("attn.out", (n, self.nh * self.vd))
        common = dict(n_heads=self.nh, n_kv_heads=nkv_in, head_dim=self.hd,
                      q_norm_w=self.q_norm_w, k_norm_w=self.k_norm_w, norm_eps=self.qk_norm_eps,
                      bias=self.b_qkv, cos=rot.cos if rot else None, sin=rot.sin if rot else None,
                      rotary_dim=rot.rotary_dim if rot else 0, pairing=rot.pairing if rot else 0,
                      positions=ctx.positions, q_out=q)
        if ctx.decode:
            if self.own_kv:
                prep(qkv, **common, k_pages=cache.k_pages, v_pages=cache.v_pages,
                     page_table=cache.page_table, ring_pages=cache.ring_pages,
                     seq_of_token=ctx.seq_of_token, slots=ctx.slots)
            else:
                prep(qkv, **common)
            # which kernel runs and how it splits the keys is the kernels' business: the plan says what scratch it wants
            plan = ops.attn_decode_plan(q.dtype, ctx.n_seqs, self.nh, self.nkv, self.hd, ctx.max_len_after, **form_kw)
            scratch = ctx.buffer("attn.scratch", (max(1, plan.scratch_floats),), torch.float32)
            counters = None
            if plan.n_counters:
                counters = ctx.buffer("attn.counters", (plan.n_counters,), torch.int32, zero=True)
            ops.attn_decode(q, cache.k_pages, cache.v_pages, cache.page_table, cache.ring_pages, ctx.slots,
                            ctx.len_before, out, scratch, scale=self.scale, window=self.window, plan=plan,
                            counters=counters, **form_kw)
        else:
            # A group that keeps every key can take the step's keys and values into its pages right away
            # (the step reads them from the packed buffer, never from the pages).  A ring must wait until
            # the attention has read the old keys that the new ones overwrite.
            write_now = self.own_kv and self.window == 0
            if self.own_kv:
                suffix = f".{cache.unit}" if cache.keep_step_kv else ""
                k_new = ctx.buffer("attn.k_new" + suffix, (n, self.nkv, self.hd))
                v_new = ctx.buffer("attn.v_new" + suffix, (n, self.nkv, self.vd))
                if write_now:
                    prep(qkv, **common, k_new=k_new, v_new=v_new, k_pages=cache.k_pages, v_pages=cache.v_pages,
                         page_table=cache.page_table, ring_pages=cache.ring_pages,
                         seq_of_token=ctx.seq_of_token, slots=ctx.slots)
                else:
                    prep(qkv, **common, k_new=k_new, v_new=v_new)
                cache.shared["k_new"], cache.shared["v_new"] = k_new, v_new
            else:
                prep(qkv, **common)
                k_new, v_new = cache.shared["k_new"], cache.shared["v_new"]
            tq = ops.prefill_tile_queries(q.dtype, self.hd, **form_kw)
            ops.attn_prefill(q, k_new, v_new, cache.k_pages, cache.v_pages, cache.page_table, cache.ring_pages,
                             ctx.query_tiles(tq), ctx.cu_tokens, ctx.len_before, ctx.slots, out,
                             scale=self.scale, window=self.window, tile_queries=tq, **form_kw)
            if self.own_kv and not write_now:
                def write_ring():
                    ops.kv_write(k_new, v_new, cache.k_pages, cache.v_pages, cache.page_table, cache.ring_pages,
                                 ctx.positions, ctx.seq_of_token, ctx.slots, ctx.cu_tokens, ctx.len_before)
                if cache.keep_step_kv:
                    # later entries of the run order read this ring in the same step: the new keys must not
                    # replace old ones before the last of them has run
                    cache.shared.setdefault("after_last_reader", []).append(write_ring)
                else:
                    write_ring()
        if gate is not None:
            ops.sigmoid_gate(out, gate, gate_col)
        return Branch(linear(ctx, out, self.w_o, "attn.proj", torch.float32))


register_part("mixer", "attention", Attention)
