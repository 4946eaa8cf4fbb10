"""Stand-ins for the CUDA kernels, for tests of the host logic where there is no GPU.

Each function has the signature and the contract of its namesake in the library's
``kernels.ops`` and is written with plain torch operations on CPU tensors.  Only tests pass
this module to the engine (as ``ops=``); the library itself never falls back to it.
"""
from __future__ import annotations

import torch

PAGE = 64


def sm_count():
    return 4


def require_gpu():
    pass


def embed_rows(table, token_ids, out_residual):
    rows = table[token_ids.long()].float()
    out_residual.copy_(rows if out_residual.dim() == 2 else rows.expand_as(out_residual))


def add_rmsnorm(residual, branch, weight, eps, out, rows=None):
    if branch is not None:
        if rows is None:
            residual += branch.sum(0)
        else:
            residual[rows.long()] += branch.sum(0)[rows.long()]
    x = residual if rows is None else residual[rows.long()]
    y = x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * weight.float()
    out.copy_(y.to(out.dtype))


def gemm_simt(x, w, out):
    out.copy_((x.float() @ w.float().t()).to(out.dtype))


def _rows_of(page_table, ring_pages, slot, pos, kvh, nkv):
    page = int(page_table[slot, (pos // PAGE) % ring_pages])
    return page, kvh, pos % PAGE


def qk_prep(qkv, *, n_heads, n_kv_heads, head_dim, q_norm_w, k_norm_w, norm_eps, bias, cos, sin, rotary_dim,
            pairing, positions, q_out, k_new=None, v_new=None, k_pages=None, v_pages=None, page_table=None,
            ring_pages=0, seq_of_token=None, slots=None, value_dim=0, v_mix=None, v_first_in=None, v_first_out=None):
    x = qkv.float().sum(0)
    n = x.shape[0]
    nh, nkv, hd = n_heads, n_kv_heads, head_dim
    vd = value_dim or hd
    v_part = x[:, (nh + nkv) * hd:].reshape(n, nkv, vd).clone() if nkv else None
    if bias is not None and nkv:
        v_part = v_part + bias.float()[(nh + nkv) * hd:].view(1, nkv, vd)
    if v_first_out is not None:
        v_first_out.copy_(v_part)
    if v_first_in is not None:
        lam = v_mix.float().reshape(())
        v_part = (1.0 - lam) * v_part + lam * v_first_in
    if bias is not None:
        bias = torch.cat([bias.float()[:(nh + nkv) * hd], torch.zeros(nkv * hd)])
    x = torch.cat([x[:, :(nh + nkv) * hd], torch.zeros(n, nkv * hd)], dim=1).view(n, nh + 2 * nkv, hd).clone()

    def norm(t, w):
        return t * torch.rsqrt((t * t).mean(-1, keepdim=True) + norm_eps) * w.float()

    if q_norm_w is not None:
        x[:, :nh] = norm(x[:, :nh], q_norm_w)
    if k_norm_w is not None and nkv:
        x[:, nh:nh + nkv] = norm(x[:, nh:nh + nkv], k_norm_w)
    if bias is not None:
        x = x + bias.float().view(1, nh + 2 * nkv, hd)
    if cos is not None:
        half = rotary_dim // 2
        c = cos[positions.long()][:, None, :]
        s = sin[positions.long()][:, None, :]
        r = x[:, :nh + nkv]
        if pairing == 0:
            a, b = r[..., :half].clone(), r[..., half:2 * half].clone()
            r[..., :half] = a * c - b * s
            r[..., half:2 * half] = a * s + b * c
        else:
            a, b = r[..., 0:2 * half:2].clone(), r[..., 1:2 * half:2].clone()
            r[..., 0:2 * half:2] = a * c - b * s
            r[..., 1:2 * half:2] = a * s + b * c
    q_out.copy_(x[:, :nh].to(q_out.dtype))
    if nkv == 0:
        return
    k = x[:, nh:nh + nkv].to(q_out.dtype)
    v = v_part.to(q_out.dtype)
    _store_kv(k, v, positions, k_new, v_new, k_pages, v_pages, page_table, ring_pages, seq_of_token, slots)


def _store_kv(k, v, positions, k_new, v_new, k_pages, v_pages, page_table, ring_pages, seq_of_token, slots):
    n, nkv = k.shape[0], k.shape[1]
    if k_new is not None:
        k_new.copy_(k)
        v_new.copy_(v)
    if k_pages is not None:
        for t in range(n):
            slot = int(slots[int(seq_of_token[t])])
            pos = int(positions[t])
            for h in range(nkv):
                pg, hh, off = _rows_of(page_table, ring_pages, slot, pos, h, nkv)
                k_pages[pg, hh, off] = k[t, h]
                v_pages[pg, hh, off] = v[t, h]


def add_layernorm(residual, parts, scale, weight, bias, eps, out, rows=None):
    idx = slice(None) if rows is None else rows.long()
    if parts:
        total = sum(p.sum(0) for p in parts)
        residual[idx] += float(scale) * total[idx]
    x = residual[idx]
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    out.copy_(((x - mu) * torch.rsqrt(var + eps) * weight.float() + bias.float()).to(out.dtype))


def latent_prep(rows, *, n_heads, head_dim, rot_dim, kv_rank, c_norm_w, norm_eps, cos, sin, positions, q_plain_out=None,
                q_out=None, k_new=None, v_new=None, k_pages=None, v_pages=None, page_table=None, ring_pages=0, seq_of_token=None,
                slots=None, pairing=0, q_col=0, kv_col=None, cq_col=-1, cq_norm_w=None, cq_out=None):
    x = rows.float().sum(0)
    n = x.shape[0]
    qw = n_heads * (head_dim + rot_dim)
    if kv_col is None:
        kv_col = qw

    def rotate(t):                      # [..., rot_dim] with a leading token axis
        half = rot_dim // 2
        cs, sn = cos[positions.long()], sin[positions.long()]
        while cs.dim() < t.dim():
            cs, sn = cs.unsqueeze(1), sn.unsqueeze(1)
        if pairing == 0:
            a, b = t[..., :half], t[..., half:]
            return torch.cat([a * cs - b * sn, b * cs + a * sn], dim=-1)
        a, b = t[..., 0::2], t[..., 1::2]
        return torch.stack([a * cs - b * sn, b * cs + a * sn], dim=-1).flatten(-2)

    if cq_col >= 0:
        cq = x[:, cq_col:cq_col + cq_out.shape[1]]
        cq_out.copy_((cq * torch.rsqrt((cq * cq).mean(-1, keepdim=True) + norm_eps) * cq_norm_w.float()).to(cq_out.dtype))
    if q_col >= 0:
        q = x[:, q_col:q_col + qw].view(n, n_heads, head_dim + rot_dim)
        q_plain_out.copy_(q[..., :head_dim].to(q_plain_out.dtype))
        if rot_dim:
            q_out[..., kv_rank:] = rotate(q[..., head_dim:]).to(q_out.dtype)
    if kv_col < 0:
        return
    c = x[:, kv_col:kv_col + kv_rank]
    kr = x[:, kv_col + kv_rank:kv_col + kv_rank + rot_dim]
    c = c * torch.rsqrt((c * c).mean(-1, keepdim=True) + norm_eps) * c_norm_w.float()
    if rot_dim:
        kr = rotate(kr)
    dtype = (k_new if k_new is not None else k_pages).dtype
    k = torch.cat([c, kr], dim=-1).view(n, 1, kv_rank + rot_dim).to(dtype)
    v = c.view(n, 1, kv_rank).to(dtype)
    if v_new is None and v_pages is None:          # the caller reads its values out of the keys
        v, v_new, v_pages = k, k_new, k_pages
    _store_kv(k, v, positions, k_new, v_new, k_pages, v_pages, page_table, ring_pages, seq_of_token, slots)


def sigmoid_gate(x, gate, col0, bias=None):
    z = gate.float().sum(0)[:, col0:col0 + x.shape[1]]
    if bias is not None:
        z = z + bias.float()
    x.copy_((x.float() * torch.sigmoid(z)).to(x.dtype))


NORM_MAX_GROUPS = 65536


def gated_add_group_rmsnorm(residual, branch, gate, gate_bias, post_w, post_groups, post_eps, weight, groups, eps, out,
                            rows=None):
    def grouped(v, g, e):
        p = v.view(v.shape[0], g, -1)
        return (p * torch.rsqrt((p * p).mean(-1, keepdim=True) + e)).reshape(v.shape)

    idx = slice(None) if rows is None else rows.long()
    if branch is not None:
        y = branch.sum(0)[idx]
        if gate is not None:
            z = gate.sum(0)[idx]
            if gate_bias is not None:
                z = z + gate_bias.float()
            y = y * torch.sigmoid(z)
        if post_w is not None:
            y = grouped(y, post_groups, post_eps) * post_w.float()
        residual[idx] += y
    out.copy_((grouped(residual[idx], groups, eps) * weight.float()).to(out.dtype))


MINGRU_PIECE = 4


def mingru_pieces(max_count):
    return -(-max_count // MINGRU_PIECE)


def mingru_scan(rows, bias, state, slots, cu_tokens, out, carry=None):
    x = rows.float().sum(0)
    size = out.shape[1]
    z = torch.sigmoid(x[:, :size] + bias[:size].float())
    u = x[:, size:2 * size] + bias[size:].float()
    cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    g = x[:, 2 * size:]
    for b in range(slots.numel()):
        s = state[int(slots[b])].clone()
        for t in range(int(cu_tokens[b]), int(cu_tokens[b + 1])):
            s = (1 - z[t]) * s + z[t] * cand[t]
            out[t] = (s * g[t] * torch.sigmoid(g[t])).to(out.dtype)
        state[int(slots[b])] = s


def multi_add_rmsnorm(residual, terms, outs, eps, rows=None):
    idx = slice(None) if rows is None else rows.long()
    for data, w, w_eps, scale in terms:
        y = data.float().sum(0)[idx]
        if w is not None:
            y = y * torch.rsqrt((y * y).mean(-1, keepdim=True) + w_eps) * w.float()
        residual[idx] += scale * y
    x = residual[idx]
    inv = torch.rsqrt((x * x).mean(-1, keepdim=True) + eps)
    for out, w, offset in outs:
        out.copy_((x if w is None else x * inv * (offset + w.float())).to(out.dtype))


def hash_embed(table, scale, pair_table, buckets, mul_prev, mul_cur, token_ids, positions, seq_of_token, cu_tokens, slots,
               last_token, norm_w, norm_offset, eps, out_residual):
    tok = token_ids.long()
    x = table[tok].float() * scale
    if pair_table is not None:
        rows = torch.empty_like(tok)
        for n in range(tok.numel()):
            b = int(seq_of_token[n])
            if int(positions[n]) == 0:
                rows[n] = buckets
                continue
            prev = int(tok[n - 1]) if n > int(cu_tokens[b]) else int(last_token[int(slots[b]), 0])
            rows[n] = (prev * mul_prev + int(tok[n]) * mul_cur) % buckets
        for b in range(slots.numel()):
            last_token[int(slots[b]), 0] = int(tok[int(cu_tokens[b + 1]) - 1])
        x = x + pair_table[rows].float()
    if norm_w is not None:
        x = x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * (norm_offset + norm_w.float())
    out_residual.copy_(x)


def table_gate(rows, table, col0, token_ids, out, kind):
    z = rows.float().sum(0)
    e = table[token_ids.long()][:, col0:col0 + z.shape[1]].float()
    out.copy_((_act(z, kind) * e).to(out.dtype))


def _act(z, kind):
    if kind == "relu2":
        return torch.relu(z) ** 2
    if kind == "gelu_tanh":
        return 0.5 * z * (1 + torch.tanh(0.7978845608028654 * (z + 0.044715 * z ** 3)))
    if kind == "silu":
        return z * torch.sigmoid(z)
    return torch.relu(z)


CONV_MAX_TAPS = 16
RETENTION_PIECE = 4


def causal_conv(rows, col0, weight, state, slots, cu_tokens, seq_of_token, len_before, out, in_bias=None, bias=None, out2=None):
    c, k = weight.shape
    x = rows.float().sum(0)[:, col0:col0 + c]
    if in_bias is not None:
        x = x + in_bias.float()
    for b in range(slots.numel()):
        t0, t1 = int(cu_tokens[b]), int(cu_tokens[b + 1])
        past = state[int(slots[b])].float() if k > 1 else x.new_zeros((0, c))
        seq = torch.cat([past, x[t0:t1]])               # the state holds zeros where the sequence had not begun
        for t in range(t1 - t0):
            y = (seq[t:t + k] * weight.float().t()).sum(0)
            out[t0 + t] = y if bias is None else y + bias.float()
        if k > 1:
            state[int(slots[b])] = seq[seq.shape[0] - (k - 1):]
    if out2 is not None:
        out2.copy_(out.to(out2.dtype))


def rglru_scan(rows, y_col, y_bias, u, gates, gate_bias, lam, decay_scale, state, slots, cu_tokens, out, carry=None):
    n, size = out.shape
    bw = gates.shape[2] // 2
    y = rows.float().sum(0)[:, y_col:y_col + size]
    if y_bias is not None:
        y = y + y_bias.float()
    g = gates.float() + gate_bias.float()
    r = torch.sigmoid(g[:, :, :bw]).reshape(n, size)
    i = torch.sigmoid(g[:, :, bw:]).reshape(n, size)
    a = torch.exp(-decay_scale * r * torch.nn.functional.softplus(lam.float()))
    drive = torch.sqrt(1 - a * a) * i * u.float()
    for b in range(slots.numel()):
        s = state[int(slots[b])].clone()
        for t in range(int(cu_tokens[b]), int(cu_tokens[b + 1])):
            s = a[t] * s + drive[t]
            out[t] = (s * _act(y[t], "gelu_tanh")).to(out.dtype)
        state[int(slots[b])] = s


def retention_pieces(max_count):
    return -(-max_count // RETENTION_PIECE)


def retention(rows, *, q_col, k_col, v_col, g_col, n_heads, dim, vdim, cos, sin, rotary_dim, positions, decay, k_scale, eps,
              state, slots, cu_tokens, out, carry=None):
    x = rows.float().sum(0)
    n = x.shape[0]
    q = x[:, q_col:q_col + n_heads * dim].reshape(n, n_heads, dim).clone()
    k = x[:, k_col:k_col + n_heads * dim].reshape(n, n_heads, dim).clone()
    v = x[:, v_col:v_col + n_heads * vdim].reshape(n, n_heads, vdim)
    g = x[:, g_col:g_col + n_heads * vdim].reshape(n, n_heads, vdim)
    if cos is not None and rotary_dim:
        half = rotary_dim // 2
        c, s = cos[positions.long()][:, None, :], sin[positions.long()][:, None, :]
        for t in (q, k):
            a, b2 = t[..., :half].clone(), t[..., half:rotary_dim].clone()
            t[..., :half] = a * c - b2 * s
            t[..., half:rotary_dim] = b2 * c + a * s
    k = k * k_scale
    for b in range(slots.numel()):
        st = state[int(slots[b])].clone()
        for t in range(int(cu_tokens[b]), int(cu_tokens[b + 1])):
            st = decay.float()[:, None, None] * st + k[t][:, :, None] * v[t][:, None, :]
            o = torch.einsum("hdv,hd->hv", st, q[t])
            o = o * torch.rsqrt((o * o).mean(-1, keepdim=True) + eps) * (g[t] * torch.sigmoid(g[t]))
            out[t] = o.reshape(-1).to(out.dtype)
        state[int(slots[b])] = st


def tanh_cap(x, cap):
    x.copy_(cap * torch.tanh(x / cap))


def head_linear(x, w, y):
    y.copy_(torch.einsum("nha,hba->nhb", x.float(), w.float()).to(y.dtype))


MOE_TILE_ROWS = 8
MOE_MAX_EXPERTS = 1024
MOE_MAX_TOP = 32


def moe_tile_rows(dtype, pairs, n_experts, hidden, inner):
    return MOE_TILE_ROWS


def moe_row_capacity(pairs, n_experts, tile=MOE_TILE_ROWS):
    cap = pairs + n_experts * (tile - 1)
    return -(-cap // tile) * tile


class RouterRule:
    def __init__(self, score="softmax", groups=0, keep_groups=0, group_score_top=2, weight_scale=1.0, weight_sum_eps=0.0):
        self.score, self.groups, self.keep_groups, self.group_score_top = score, groups, keep_groups, group_score_top
        self.weight_scale, self.weight_sum_eps = weight_scale, weight_sum_eps


def moe_route(x, w_router, b_router, choice, weight, rule=None, extra_out=None):
    z = x.float() @ w_router.float().t()
    if extra_out is not None:
        extra_out.copy_(torch.sigmoid(z[:, -1]))
        z = z[:, :-1]
    if b_router is not None:
        z = z + b_router.float()
    top = choice.shape[1]
    if rule is None or rule.score == "softmax":
        val, idx = torch.topk(z, top, dim=-1)
        choice.copy_(idx.to(torch.int32))
        weight.copy_(torch.softmax(val, dim=-1))
        return
    s = torch.softmax(z, dim=-1) if rule.score == "softmax_all" else torch.sigmoid(z)
    n, n_exp = s.shape
    masked = s
    if rule.groups:
        per = n_exp // rule.groups
        gs = torch.topk(s.view(n, rule.groups, per), min(rule.group_score_top, per), dim=-1).values.sum(-1)
        best = torch.topk(gs, rule.keep_groups, dim=-1).indices
        ok = torch.zeros_like(gs, dtype=torch.bool).scatter_(1, best, True)
        masked = s.masked_fill(~ok[:, :, None].expand(-1, -1, per).reshape(n, n_exp), -1.0)
    val, idx = torch.topk(masked, top, dim=-1)
    choice.copy_(idx.to(torch.int32))
    weight.copy_(val / (val.sum(-1, keepdim=True) + rule.weight_sum_eps) * rule.weight_scale)


def moe_plan(choice, n_experts, row_of_pair, token_of_row, tile_expert):
    top = choice.shape[1]
    flat = choice.reshape(-1).tolist()
    token_of_row.fill_(-1)
    tile_expert.fill_(-1)
    row = 0
    for e in range(n_experts):
        mine = [p for p, c in enumerate(flat) if c == e]
        for p in reversed(mine):                 # any order inside an expert's run is allowed
            row_of_pair[p] = row
            token_of_row[row] = p // top
            row += 1
        while row % MOE_TILE_ROWS:
            row += 1
        for t in range((row - 1) // MOE_TILE_ROWS, -1, -1):
            if tile_expert[t] != -1:
                break
            if mine:
                tile_expert[t] = e
        # tiles of an expert without rows stay -1 (it has none)


def moe_gated(x, token_of_row, tile_expert, w_gate_up, act):
    act.zero_()
    inner, pad = act.shape[1], w_gate_up.shape[1] // 2
    for r in range(token_of_row.numel()):
        t = int(token_of_row[r])
        if t < 0:
            continue
        e = int(tile_expert[r // MOE_TILE_ROWS])
        g = w_gate_up[e, :inner].float() @ x[t].float()
        u = w_gate_up[e, pad:pad + inner].float() @ x[t].float()
        act[r] = (g / (1 + torch.exp(-g)) * u).to(act.dtype)


def moe_down(act, tile_expert, w_down, y):
    y.zero_()
    for r in range(act.shape[0]):
        e = int(tile_expert[r // MOE_TILE_ROWS])
        if e >= 0:
            y[r] = w_down[e].float() @ act[r].float()


def moe_combine(y, row_of_pair, weight, shared, out, shared_scale=None):
    n, top = weight.shape
    rows = row_of_pair.view(n, top).long()
    out.copy_((weight[:, :, None] * y[rows]).sum(1))
    if shared is not None:
        out += shared.sum(0) if shared_scale is None else shared.sum(0) * shared_scale[:, None]


def kv_write(k_new, v_new, k_pages, v_pages, page_table, ring_pages, positions, seq_of_token, slots,
             cu_tokens, len_before):
    n, nkv, hd = k_new.shape
    for t in range(n):
        b = int(seq_of_token[t])
        pos = int(positions[t])
        len_after = int(len_before[b]) + int(cu_tokens[b + 1] - cu_tokens[b])
        if pos < len_after - ring_pages * PAGE:
            continue
        slot = int(slots[b])
        for h in range(nkv):
            pg, hh, off = _rows_of(page_table, ring_pages, slot, pos, h, nkv)
            k_pages[pg, hh, off] = k_new[t, h]
            v_pages[pg, hh, off] = v_new[t, h]


GATE_ACTIVATIONS = ("silu", "gelu_tanh")


def silu_mul(gate_up, out, activation="silu"):
    x = gate_up.float().sum(0)
    inter = out.shape[1]
    half = x.shape[1] // 2
    g, u = x[:, :inter], x[:, half:half + inter]
    if activation == "gelu_tanh":
        a = 0.5 * g * (1 + torch.tanh(0.7978845608028654 * (g + 0.044715 * g ** 3)))
    else:
        a = g / (1 + torch.exp(-g))
    out.copy_((a * u).to(out.dtype))


def hc_max_streams():
    return 16


def hc_add_rmsnorm(streams, branch, mix, write, read, weight, eps, out, rows=None):
    idx = slice(None) if rows is None else rows.long()
    x = streams[:, idx]
    if branch is not None:
        y = branch.sum(0)[idx]
        x = torch.einsum("st,snd->tnd", mix, x) + write[:, None, None] * y[None]
        streams[:, idx] = x
    u = x.sum(0) if read is None else torch.einsum("s,snd->nd", read, x)
    out.copy_((u * torch.rsqrt((u * u).mean(-1, keepdim=True) + eps) * weight.float()).to(out.dtype))


def qkv_row_prep(qkvg, *, n_heads, n_kv_heads, head_dim, value_dim, bias, q_norm_w, k_norm_w, norm_eps, positions,
                 q_out, gate_out=None, k_new=None, v_new=None, k_pages=None, v_pages=None, page_table=None,
                 ring_pages=0, seq_of_token=None, slots=None):
    x = qkvg.float().sum(0)
    n = x.shape[0]
    qw, kw, vw = n_heads * head_dim, n_kv_heads * head_dim, n_kv_heads * value_dim
    if bias is not None:
        x[:, :qw + kw + vw] += bias.float()
    q, k, v = x[:, :qw], x[:, qw:qw + kw], x[:, qw + kw:qw + kw + vw]

    def norm(t, w):
        return t * torch.rsqrt((t * t).mean(-1, keepdim=True) + norm_eps) * w.float()

    if q_norm_w is not None:
        q = norm(q, q_norm_w)
    if k_norm_w is not None:
        k = norm(k, k_norm_w)
    q_out.copy_(q.view(n, n_heads, head_dim).to(q_out.dtype))
    if gate_out is not None:
        gate_out.copy_(torch.sigmoid(x[:, qw + kw + vw:]))
    k = k.reshape(n, n_kv_heads, head_dim).to(q_out.dtype)
    v = v.reshape(n, n_kv_heads, value_dim).to(q_out.dtype)
    if k_new is not None:
        k_new.copy_(k)
        v_new.copy_(v)
    if k_pages is not None:
        for t in range(n):
            slot = int(slots[int(seq_of_token[t])])
            pos = int(positions[t])
            for h in range(n_kv_heads):
                pg, hh, off = _rows_of(page_table, ring_pages, slot, pos, h, n_kv_heads)
                k_pages[pg, hh, off] = k[t, h]
                v_pages[pg, hh, off] = v[t, h]


ACTIVATIONS = {"relu2": 0, "gelu_tanh": 1, "silu": 2, "relu": 3}


def act_rows(x, out, kind):
    z = x.float().sum(0)
    if kind == "relu2":
        y = torch.relu(z) ** 2
    elif kind == "gelu_tanh":
        y = torch.nn.functional.gelu(z, approximate="tanh")
    elif kind == "silu":
        y = z / (1 + torch.exp(-z))
    else:
        y = torch.relu(z)
    out.copy_(y.to(out.dtype))


def scatter_i32(dst, idx, val):
    dst.view(-1)[idx.long()] = val


def gather_i32(dst, src, idx):
    dst.copy_(src.view(-1)[idx.long()])


def zero_rows(base, rows):
    base[rows.long()] = 0


class AttentionForm:
    def __init__(self, value_dim=0, sink=None, gated=False, sinks=None, chunked=False):
        self.value_dim, self.sink, self.gated = int(value_dim), sink, bool(gated)
        self.sinks, self.chunked = sinks, bool(chunked)

    def plain(self, head_dim):
        return self.value_dim in (0, head_dim) and self.sink is None and not self.gated

    def vd(self, head_dim):
        return self.value_dim or head_dim


PLAIN_ATTENTION = AttentionForm()


def _lowest(form, window, pos):
    """The first position a query at ``pos`` sees."""
    if window <= 0:
        return 0
    return (pos // window) * window if form.chunked else max(0, pos - window + 1)


def _attend(q, keys, vals, scale, form=PLAIN_ATTENTION, gate=None, head=0):
    s = (keys.float() @ q.float()) * scale
    sink = form.sink if form.sinks is None else float(form.sinks[head])
    if sink is not None:
        s = torch.cat([s, torch.tensor([float(sink)])])
        p = torch.softmax(s, 0)[:-1]
    else:
        p = torch.softmax(s, 0)
    o = p @ vals.float()
    return o if gate is None else o * gate


def _gather(k_pages, v_pages, page_table, ring_pages, slot, positions, kvh):
    ks, vs = [], []
    for pos in positions:
        pg, hh, off = _rows_of(page_table, ring_pages, slot, pos, kvh, k_pages.shape[1])
        ks.append(k_pages[pg, hh, off])
        vs.append(v_pages[pg, hh, off])
    return ks, vs


def prefill_tile_queries(dtype, head_dim, form=PLAIN_ATTENTION):
    return 16


def attn_prefill(q, k_new, v_new, k_pages, v_pages, page_table, ring_pages, tiles, cu_tokens, len_before,
                 slots, out, *, scale, window, tile_queries=16, form=PLAIN_ATTENTION, gate=None):
    n, nh, hd = q.shape
    nkv = k_new.shape[1]
    g = nh // nkv
    o = out.view(n, nh, form.vd(hd))
    for b in range(slots.numel()):
        t0, t1 = int(cu_tokens[b]), int(cu_tokens[b + 1])
        lb = int(len_before[b])
        slot = int(slots[b])
        for t in range(t0, t1):
            pos = lb + (t - t0)
            lo = _lowest(form, window, pos)
            for h in range(nh):
                kvh = h // g
                old = [p for p in range(lo, pos + 1) if p < lb]
                ks, vs = _gather(k_pages, v_pages, page_table, ring_pages, slot, old, kvh)
                for p in range(max(lo, lb), pos + 1):
                    ks.append(k_new[t0 + p - lb, kvh])
                    vs.append(v_new[t0 + p - lb, kvh])
                o[t, h] = _attend(q[t, h], torch.stack(ks), torch.stack(vs), scale, form,
                                  None if gate is None else gate[t, h], h).to(out.dtype)


class _Plan:
    scratch_floats, n_counters = 1, 0


def attn_decode_plan(dtype, n_seqs, n_heads, n_kv_heads, head_dim, max_len, form=PLAIN_ATTENTION):
    return _Plan()


def attn_decode(q, k_pages, v_pages, page_table, ring_pages, slots, len_before, out, scratch, *,
                scale, window, plan=None, n_splits=0, counters=None, balance=False, form=PLAIN_ATTENTION, gate=None):
    b_n, nh, hd = q.shape
    nkv = k_pages.shape[1]
    g = nh // nkv
    o = out.view(b_n, nh, form.vd(hd))
    for b in range(b_n):
        length = int(len_before[b]) + 1
        lo = _lowest(form, window, length - 1)
        slot = int(slots[b])
        for h in range(nh):
            ks, vs = _gather(k_pages, v_pages, page_table, ring_pages, slot, range(lo, length), h // g)
            o[b, h] = _attend(q[b, h], torch.stack(ks), torch.stack(vs), scale, form,
                              None if gate is None else gate[b, h], h).to(out.dtype)


def argmax(logits, out):
    out.copy_(torch.argmax(logits, dim=-1).to(torch.int32))
