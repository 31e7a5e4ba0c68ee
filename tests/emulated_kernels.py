"""Stand-ins for the CUDA kernels, written with torch on the CPU, for tests only.

The engine has no CPU path. To check the host side of the engine on a machine without
a GPU (batch building, block tables, page reuse, the scheduler's loop), the `-m "not gpu"`
tests swap the functions of `tgo_b200.kernels.ops` for these through `install(monkeypatch)`.
They mirror the kernels' contracts (in-place writes, strided views, the cache layout
[page, kv_head, offset, head_dim]) and nothing of this file is importable from the
package itself.
"""
from __future__ import annotations

import math

import torch


def embed(table, ids, out, scale=1.0):
    out.copy_(table[ids.long()].float() * float(torch.tensor(scale, dtype=torch.float32)))


def add_rmsnorm(h, delta, gain, eps, out, rows=None):
    if rows is None:
        if delta is not None:
            h += delta.float()
        x = h
    else:
        x = h[rows.long()]
        if delta is not None:
            x = x + delta[rows.long()].float()
    scale = torch.rsqrt((x * x).mean(-1, keepdim=True) + eps)
    out.copy_(((x * scale) * gain).to(out.dtype))


def residual_add(h, delta):
    h += delta.float()


def _gate(gate_up, f, interleaved):
    if interleaved:
        v = gate_up.reshape(gate_up.shape[0], f // 8, 2, 8)
        return v[:, :, 0].reshape(-1, f).float(), v[:, :, 1].reshape(-1, f).float()
    return gate_up[:, :f].float(), gate_up[:, f:].float()


def swiglu(gate_up, out, interleaved=False):
    g, u = _gate(gate_up, out.shape[1], interleaved)
    out.copy_((g / (1 + torch.exp(-g)) * u).to(out.dtype))


def rope_table(positions, inv_freq, mag=1.0):
    ang = positions.double()[:, None] * inv_freq[None, :]
    return (torch.cat([ang.cos(), ang.sin()], dim=1) * mag).float()


def qk_norm_rope_cache(q, k, v, num_heads, num_kv_heads, head_dim, q_gain, k_gain, eps, rope,
                       rotary_dim, slots, k_cache, v_cache, page_size):
    T = q.shape[0]

    def treat(x, heads, gain):
        y = x.reshape(T, heads, head_dim).float()
        if gain is not None:
            y = (y * torch.rsqrt((y * y).mean(-1, keepdim=True) + eps)) * gain
        if rope is not None:
            half = rotary_dim // 2
            cos, sin = rope[:, None, :half], rope[:, None, half:]
            lo, hi = y[..., :half].clone(), y[..., half:rotary_dim].clone()
            y[..., :half] = lo * cos - hi * sin
            y[..., half:rotary_dim] = lo * sin + hi * cos
        return y

    q.copy_(treat(q, num_heads, q_gain).reshape(T, -1).to(q.dtype))
    if k is not None:
        kk = treat(k, num_kv_heads, k_gain)
        if k_cache is None:
            k.copy_(kk.reshape(T, -1).to(k.dtype))
    if k_cache is not None:
        vv = v.reshape(T, num_kv_heads, head_dim) if v is not None else None
        for t in range(T):
            s = int(slots[t])
            if s < 0:
                continue
            page, off = s // page_size, s % page_size
            k_cache[page, :, off, :] = kk[t].to(k_cache.dtype)
            if vv is not None:
                v_cache[page, :, off, :] = vv[t]


def attention_generic(q, out, num_heads, num_kv_heads, head_dim, k_cache, v_cache, page_size,
                      block_tables, seq_ids, positions, scale, window, value_dim=None, sinks=None,
                      softcap=0.0, value_row=0, keep_first=0, dist_bias=None):
    T = q.shape[0]
    group = num_heads // num_kv_heads
    dv = value_dim or head_dim
    scale = float(torch.tensor(scale, dtype=torch.float32))
    for t in range(T):
        p, b = int(positions[t]), int(seq_ids[t])
        if p < 0:
            out[t] = 0
            continue
        lo = max(0, p - window + 1) if window > 0 else 0
        idx = torch.arange(lo, p + 1)
        if window > 0 and keep_first:
            idx = torch.cat([torch.arange(0, min(keep_first, lo)), idx])
        pages = block_tables[b].long()[idx // page_size]
        offs = idx % page_size
        for h in range(num_heads):
            g = h // group
            K = k_cache[pages, g, offs, :].float()
            V = v_cache[pages, g, offs, :dv].float()
            qv = q[t, h * head_dim:(h + 1) * head_dim].float()
            s = (K @ qv) * scale
            if softcap:
                s = softcap * torch.tanh(s / softcap)
            if dist_bias is not None:
                s = s + dist_bias[torch.clamp(p - idx, max=dist_bias.shape[0] - 1), h]
            if sinks is not None:
                w = torch.softmax(torch.cat([s, sinks[h:h + 1].float()]), dim=0)[:-1]
            else:
                w = torch.softmax(s, dim=0)
            out[t, h * dv:(h + 1) * dv] = (w @ V).to(out.dtype)


def paged_attention(q, out, num_heads, num_kv_heads, head_dim, cache, ctx, scale, window):
    attention_generic(q, out, num_heads, num_kv_heads, head_dim, cache.k, cache.v,
                      cache.page_size, cache.block_tables, ctx.seq_ids, ctx.positions, scale,
                      window)


def linear(x, w, out_dtype=None, residual=None):
    y = x.float() @ w.float().t()
    if residual is not None:
        residual += y
        return None
    return y.to(out_dtype or x.dtype)


def gated_linear(x, w_gate_up, interleaved, activation="silu", bias=None):
    gu = (x.float() @ w_gate_up.float().t()).to(x.dtype)
    out = torch.empty((x.shape[0], w_gate_up.shape[0] // 2), dtype=x.dtype)
    if activation == "silu" and bias is None:
        swiglu(gu, out, interleaved)
    else:
        gated_act(gu, out, interleaved, activation, bias)
    return out


def gated_act(gate_up, out, interleaved, activation, bias=None):
    if bias is not None:
        gate_up = gate_up.float() + bias
    g, u = _gate(gate_up, out.shape[1], interleaved)
    if activation == "relu":
        a = torch.relu(g)
    elif activation == "gelu_tanh":
        a = 0.5 * g * (1 + torch.tanh(math.sqrt(2 / math.pi) * (g + 0.044715 * g ** 3)))
    else:
        a = g / (1 + torch.exp(-g))
    out.copy_((a * u).to(out.dtype))


def cast_rows(h, out):
    out.copy_(h.to(out.dtype))


def _group_norm(x, eps, groups):
    n, d = x.shape
    g = x.reshape(n, groups, d // groups)
    return (g * torch.rsqrt((g * g).mean(-1, keepdim=True) + eps)).reshape(n, d)


def group_norm_scale_add(h, y, gain, scale, eps, groups, act=None):
    v = _group_norm(y.float(), eps, groups) * gain
    if scale is not None:
        v = v * scale
    h += v
    if act is not None:
        act.copy_(h.to(act.dtype))


def group_norm_rows(h, rows, gain, eps, groups, out):
    x = h if rows is None else h[rows.long()]
    out.copy_((_group_norm(x, eps, groups) * gain).to(out.dtype))


def softcap(x, cap):
    x.copy_(cap * torch.tanh(x / cap))


def value_norm_share_cache(v, num_kv_heads, value_dim, norm, eps, blend, shared, mode, slots,
                           v_cache, page_size):
    T = v.shape[0]
    x = v.reshape(T, num_kv_heads, value_dim).float()
    if norm:
        x = x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps)
    if mode == 1:
        shared.copy_(x.reshape(T, -1))
    elif mode == 2:
        lam = float(blend[0])
        x = (1 - lam) * x + lam * shared.reshape(T, num_kv_heads, value_dim)
    for t in range(T):
        s = int(slots[t])
        if s >= 0:
            v_cache[s // page_size, :, s % page_size, :] = x[t].to(v_cache.dtype)


def head_norm_gate(o, gate, out, heads, value_dim, eps):
    T = o.shape[0]
    x = o.reshape(T, heads, value_dim)
    x = (x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps)).reshape(T, -1)
    if gate is not None:
        g = gate.float()
        x = x * (g / (1 + torch.exp(-g)))
    out.copy_(x.to(out.dtype))


def attention_mixed(q, out, num_heads, num_kv_heads, key_dim, value_dim, k_cache, v_cache,
                    page_size, block_tables, seq_ids, positions, mix, scale, window):
    T = q.shape[0]
    group = num_heads // num_kv_heads
    scale = float(torch.tensor(scale, dtype=torch.float32))
    for t in range(T):
        p, b = int(positions[t]), int(seq_ids[t])
        if p < 0:
            out[t] = 0
            continue
        lo = max(0, p - window + 1) if window > 0 else 0
        idx = torch.arange(lo, p + 1)
        if window > 0 and keep_first:
            idx = torch.cat([torch.arange(0, min(keep_first, lo)), idx])
        pages = block_tables[b].long()[idx // page_size]
        offs = idx % page_size
        w = []
        for h in range(num_heads):
            K = k_cache[pages, h // group, offs, :].float()
            w.append(torch.softmax((K @ q[t, h * key_dim:(h + 1) * key_dim].float()) * scale, 0))
        w = torch.stack(w)
        if mix is not None:
            w = mix @ w
        for h in range(num_heads):
            V = v_cache[pages, h // group, offs, :].float()
            out[t, h * value_dim:(h + 1) * value_dim] = (w[h] @ V).to(out.dtype)


def retention(q, k, v, out, num_seqs, num_heads, key_dim, value_dim, decay, k_scale, rope,
              rotary_dim, q_start, state_slots, state, act=0):
    T = q.shape[0]
    taken = (lambda x: x.float() * torch.sigmoid(x.float())) if act == 1 else (lambda x: x.float())

    def turn(x):
        y = taken(x.reshape(T, num_heads, key_dim)).clone()
        if rope is not None:
            half = rotary_dim // 2
            cos, sin = rope[:, None, :half], rope[:, None, half:]
            lo, hi = y[..., :half].clone(), y[..., half:rotary_dim].clone()
            y[..., :half] = lo * cos - hi * sin
            y[..., half:rotary_dim] = lo * sin + hi * cos
        return y
    qq, kk = turn(q), turn(k) * k_scale
    vv = taken(v.reshape(T, num_heads, value_dim))
    for b in range(num_seqs):
        S = state[int(state_slots[b])]
        for t in range(int(q_start[b]), int(q_start[b + 1])):
            S.mul_(decay[:, None, None]).add_(kk[t][:, :, None] * vv[t][:, None, :])
            out[t] = torch.einsum("hdv,hd->hv", S, qq[t]).reshape(-1)


def sgemm_tn(x, w, out):
    out.copy_(x @ w.t())


def argmax(logits, out):
    import plain_qwen3 as plain
    for r in range(logits.shape[0]):
        out[r] = plain.argmax_lowest(logits[r].numpy())


def sample(logits, temperature, top_k, top_p, draws, out, report=None, logprob=None,
           top_ids=None, top_logprobs=None):
    import plain_qwen3 as plain
    for r in range(logits.shape[0]):
        ids, w, total = plain.policy_distribution(
            logits[r].numpy(), temperature=float(temperature[r]), top_k=int(top_k[r]),
            top_p=float(top_p[r]))
        out[r] = plain.walk(ids, w, total, float(draws[r]))
        if report is not None and int(report[r]) >= 0:
            lp, top = plain.token_logprobs(ids, w, total, int(out[r]), int(report[r]),
                                           logits.shape[1])
            logprob[r] = lp
            for j, (i, v) in enumerate(top):
                top_ids[r, j] = i
                top_logprobs[r, j] = v


def logits_adjust(row, bias_ids, bias, ids, counts, repetition, presence, frequency):
    if bias_ids is not None:
        for i, b in zip(bias_ids.tolist(), bias.tolist()):
            row[i] += b
    if ids is not None:
        for i, c in zip(ids.tolist(), counts.tolist()):
            x = float(row[i])
            if repetition not in (0.0, 1.0):
                x = x / repetition if x > 0 else x * repetition
            x -= presence + frequency * c
            row[i] = x


def retention_chunked(q, k, v, out, num_seqs, num_heads, key_dim, value_dim, decay, k_scale, rope,
                      rotary_dim, q_start, state_slots, state, chunk_tok0=None, chunk_ntok=None,
                      chunk_first=None, act=0):
    if chunk_tok0 is not None:          # the lists the host made must describe the step
        T, at = q.shape[0], 0
        starts = [int(x) for x in q_start]
        for b in range(num_seqs):
            assert int(chunk_first[b]) == at
            o = starts[b]
            while o < starts[b + 1]:
                assert int(chunk_tok0[at]) == o and 0 < int(chunk_ntok[at]) <= retention_chunk_tokens()
                o += int(chunk_ntok[at])
                at += 1
            assert o == starts[b + 1]
        assert at == chunk_tok0.numel() and starts[-1] == T
    retention(q, k, v, out, num_seqs, num_heads, key_dim, value_dim, decay, k_scale, rope,
              rotary_dim, q_start, state_slots, state, act=act)


def retention_chunk_tokens():
    return 64


def retention_chunked_supports(num_heads, key_dim, value_dim):
    return True


def _gate_value(z, act):
    z = z.float()
    return z * torch.sigmoid(z) if act == "silu" else torch.sigmoid(z) if act == "sigmoid" else z


def gated_group_norm(o, gate, gain, out, groups, eps, gate_activation, gate_first):
    T, W = o.shape
    x = o.float()
    if gate is not None and gate_first:
        x = x * _gate_value(gate, gate_activation)
    x = x.reshape(T, groups, W // groups)
    x = (x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps)).reshape(T, W)
    if gain is not None:
        x = x * gain
    if gate is not None and not gate_first:
        x = x * _gate_value(gate, gate_activation)
    out.copy_(x.to(out.dtype))


def qkv_bias_rope_cache(q, k, v, num_heads, num_kv_heads, key_dim, value_dim, q_bias, k_bias,
                        v_bias, rope, rotary_dim, interleaved, slots, k_cache, v_cache, page_size):
    T = q.shape[0]

    def treat(x, heads, bias):
        y = x.float() + (bias if bias is not None else 0.0)
        y = y.reshape(T, heads, key_dim).clone()
        if rope is not None:
            half = rotary_dim // 2
            cos, sin = rope[:, None, :half], rope[:, None, half:]
            if interleaved:
                a, b = y[..., 0:rotary_dim:2].clone(), y[..., 1:rotary_dim:2].clone()
                y[..., 0:rotary_dim:2] = a * cos - b * sin
                y[..., 1:rotary_dim:2] = b * cos + a * sin
            else:
                a, b = y[..., :half].clone(), y[..., half:rotary_dim].clone()
                y[..., :half] = a * cos - b * sin
                y[..., half:rotary_dim] = a * sin + b * cos
        return y
    q.copy_(treat(q, num_heads, q_bias).reshape(T, -1).to(q.dtype))
    if k is not None:
        kk = treat(k, num_kv_heads, k_bias)
        vv = None
        if v is not None:
            vv = (v.float() + (v_bias if v_bias is not None else 0.0)).reshape(T, num_kv_heads, value_dim)
        for t in range(T):
            s = int(slots[t])
            if s >= 0:
                k_cache[s // page_size, :, s % page_size, :] = kk[t].to(k_cache.dtype)
                if vv is not None:
                    v_cache[s // page_size, :, s % page_size, :] = vv[t].to(v_cache.dtype)


def causal_conv_act(x, w, bias, y, num_seqs, seq_ids, q_start, state_slots, state, conv_offset):
    C, taps = w.shape
    keep = taps - 1
    for b in range(num_seqs):
        t0, t1 = int(q_start[b]), int(q_start[b + 1])
        row = state[int(state_slots[b])]
        kept = row[conv_offset:conv_offset + keep * C].reshape(keep, C)
        full = torch.cat([kept, x[t0:t1].float()], dim=0)
        for t in range(t1 - t0):
            a = (full[t:t + taps] * w.t()).sum(0) + (bias if bias is not None else 0.0)
            y[t0 + t] = a * torch.sigmoid(a)
        if keep:
            kept.copy_(full[full.shape[0] - keep:])


def selective_scan(xbc, dt_raw, dt_bias, a_log, d_skip, y, num_seqs, heads, groups, state_dim,
                   value_dim, q_start, state_slots, state, ssm_offset):
    H, G, N, P = heads, groups, state_dim, value_dim
    inner = H * P
    A = torch.exp(a_log.float())
    for b in range(num_seqs):
        S = state[int(state_slots[b])][ssm_offset:ssm_offset + H * N * P].reshape(H, N, P)
        for t in range(int(q_start[b]), int(q_start[b + 1])):
            x = xbc[t, :inner].reshape(H, P)
            Bm = xbc[t, inner:inner + G * N].reshape(G, N).repeat_interleave(H // G, dim=0)
            Cm = xbc[t, inner + G * N:].reshape(G, N).repeat_interleave(H // G, dim=0)
            dt = torch.nn.functional.softplus(dt_raw[t].float() + (dt_bias if dt_bias is not None else 0.0),
                                              threshold=1e9)
            S.mul_(torch.exp(-A * dt)[:, None, None]).add_((dt[:, None] * Bm)[:, :, None] * x[:, None, :])
            out = torch.einsum("hnp,hn->hp", S, Cm)
            if d_skip is not None:
                out = out + d_skip[:, None] * x
            y[t] = out.reshape(-1)


def _plain_act(z, activation):
    if activation == "relu_squared":
        return torch.relu(z) ** 2
    if activation == "relu":
        return torch.relu(z)
    if activation == "gelu_tanh":
        return torch.nn.functional.gelu(z, approximate="tanh")
    return torch.nn.functional.silu(z)


def moe_feed_forward(x, w_router, b_router, w_gate, w_up, w_down, top, activation, extra=None,
                     scores="chosen", correction=None, identity=0, extra_gated=False):
    T, d = x.shape
    E = w_up.shape[0]
    outputs = E + identity
    z = x.float() @ w_router.float().t()
    gate = torch.sigmoid(z[:, outputs]) if extra_gated else None
    z = z[:, :outputs] + (b_router if b_router is not None else 0.0)
    out = torch.zeros((T, d), dtype=torch.float32)
    for t in range(T):
        if scores == "all":
            sc = torch.softmax(z[t], dim=0)
            choice = sc + (correction if correction is not None else 0.0)
            order = sorted(range(outputs), key=lambda e: (-float(choice[e]), e))[:top]
            w = sc[order] / (sc[order].sum() + 1e-20)
        else:
            order = sorted(range(outputs), key=lambda e: (-float(z[t, e]), e))[:top]
            w = torch.softmax(z[t, order], dim=0)
        for e, we in zip(order, w):
            if e >= E:
                out[t] += we * x[t].float()
                continue
            u = x[t].float() @ w_up[e].float().t()
            if w_gate is not None:
                hid = _plain_act(x[t].float() @ w_gate[e].float().t(), activation) * u
            else:
                hid = _plain_act(u, activation)
            out[t] += we * (hid.to(x.dtype).float() @ w_down[e].float().t())
    if extra is not None:
        out += extra * gate[:, None] if gate is not None else extra
    return out


def act_rows(x, activation):
    x.copy_(_plain_act(x.float(), activation).to(x.dtype))


def stream_spread(h, x):
    x.copy_(h.unsqueeze(0).expand_as(x))


def _normed(u, gain, eps):
    return u * torch.rsqrt((u * u).mean(-1, keepdim=True) + eps) * gain


def stream_read_norm(x, cin, gain, eps, out):
    out.copy_(_normed(torch.tensordot(cin, x, 1), gain, eps).to(out.dtype))


def stream_write(x, y, mix, cout, eps=0.0, next_in=None, next_gain=None, next_out=None, sum_out=None):
    S = x.shape[0]
    new = torch.einsum("st,snd->tnd", mix.reshape(S, S), x) + cout[:, None, None] * y.float()[None]
    x.copy_(new)
    if next_out is not None:
        next_out.copy_(_normed(torch.tensordot(next_in, x, 1), next_gain, eps).to(next_out.dtype))
    if sum_out is not None:
        sum_out.copy_(x.sum(0))


def qkv_conv_rope_norm_cache(qkv, q_out, num_heads, num_kv_heads, key_dim, value_dim, conv_w, num_seqs,
                             seq_ids, q_start, state_slots, state, conv_offset, rope, rotary_dim,
                             interleaved, unit_norm, eps, slots, k_cache, v_cache, page_size):
    T, C = qkv.shape
    u = qkv.float()
    y = u.clone()
    taps = conv_w.shape[1] if conv_w is not None else 0
    if taps:
        keep = taps - 1
        for b in range(num_seqs):
            s, e = int(q_start[b]), int(q_start[b + 1])
            kept = state[int(state_slots[b])][conv_offset:conv_offset + keep * C].view(keep, C) if keep \
                else torch.zeros((0, C))
            rows = torch.cat([kept.clone(), u[s:e]])
            for t in range(s, e):
                y[t] = (rows[t - s:t - s + taps] * conv_w.t()).sum(0)
            if keep:
                kept.copy_(rows[rows.shape[0] - keep:])
    qw, kw = num_heads * key_dim, num_kv_heads * key_dim

    def treat(z, heads):
        z = _turn(z.reshape(T, heads, key_dim).clone(), rope, rotary_dim, interleaved)
        if unit_norm:
            z = z * torch.rsqrt((z * z).mean(-1, keepdim=True) + eps)
        return z

    q_out.copy_(treat(y[:, :qw], num_heads).reshape(T, -1).to(q_out.dtype))
    kk = treat(y[:, qw:qw + kw], num_kv_heads)
    vv = y[:, qw + kw:].reshape(T, num_kv_heads, value_dim)
    for t in range(T):
        s = int(slots[t])
        if s < 0:
            continue
        page, off = s // page_size, s % page_size
        k_cache[page, :, off, :] = kk[t].to(k_cache.dtype)
        v_cache[page, :, off, :] = vv[t].to(v_cache.dtype)


def weighted_sum(parts, scales, out):
    out.zero_()
    for p, s in zip(parts, scales):
        out.add_(p.float() * float(torch.tensor(s, dtype=torch.float32)))


def scaled_add_norm(h, y, bias, alpha, gain, eps, act=None):
    s = float(torch.tensor(alpha, dtype=torch.float32)) * h + y.float()
    if bias is not None:
        s = s + bias
    h.copy_(s * torch.rsqrt((s * s).mean(-1, keepdim=True) + eps) * gain)
    if act is not None:
        act.copy_(h.to(act.dtype))


def add_bias(y, bias):
    y.copy_((y.float() + bias).to(y.dtype))


def _turn(y, rope, rot, interleaved):
    """y [T, heads, width] float32: the first `rot` channels rotated by rope [T, rot]."""
    if rope is None or rot == 0:
        return y
    half = rot // 2
    cos, sin = rope[:, None, :half], rope[:, None, half:]
    if interleaved:
        a, b = y[..., 0:rot:2].clone(), y[..., 1:rot:2].clone()
        y[..., 0:rot:2] = a * cos - b * sin
        y[..., 1:rot:2] = b * cos + a * sin
    else:
        a, b = y[..., :half].clone(), y[..., half:rot].clone()
        y[..., :half] = a * cos - b * sin
        y[..., half:rot] = b * cos + a * sin
    return y


def qk_rownorm_rope_cache(q, k, v, num_heads, num_kv_heads, key_dim, value_dim, q_gain, k_gain, eps,
                          rope, rotary_dim, interleaved, slots, k_cache, v_cache, page_size,
                          positions=None, temp_coef=0.0, temp_every=0):
    T = q.shape[0]

    def treat(x, heads, gain):
        y = x.float()
        if gain is not None:
            y = y * torch.rsqrt((y * y).mean(-1, keepdim=True) + eps) * gain
        return _turn(y.reshape(T, heads, key_dim).clone(), rope, rotary_dim, interleaved)

    qq = treat(q, num_heads, q_gain).reshape(T, -1)
    if positions is not None and temp_every > 0:
        steps = torch.div(positions.clamp(min=-1) + 1, temp_every, rounding_mode="floor") + 1
        qq = qq * (1.0 + float(torch.tensor(temp_coef, dtype=torch.float32)) *
                   torch.log(steps.float()))[:, None]
    q.copy_(qq.to(q.dtype))
    if k is None:
        return
    kk = treat(k, num_kv_heads, k_gain)
    vv = v.reshape(T, num_kv_heads, value_dim) if v is not None else None
    for t in range(T):
        s = int(slots[t])
        if s < 0:
            continue
        page, off = s // page_size, s % page_size
        k_cache[page, :, off, :] = kk[t].to(k_cache.dtype)
        if vv is not None:
            v_cache[page, :, off, :] = vv[t]


def latent_row_cache(kv, rank, width, gain, eps, rope, rotary_dim, interleaved, slots, cache,
                     page_size):
    T = kv.shape[0]
    c = kv[:, :rank].float()
    c = c * torch.rsqrt((c * c).mean(-1, keepdim=True) + eps) * gain
    r = _turn(kv[:, rank:].float().reshape(T, 1, width).clone(), rope, rotary_dim, interleaved)
    row = torch.cat([c, r.reshape(T, width)], dim=1).to(cache.dtype)
    flat = cache.reshape(-1, rank + width)
    for t in range(T):
        s = int(slots[t])
        if s >= 0:
            flat[s] = row[t]


def rope_slice(src, src_head, src_off, dst, dst_head, dst_off, num_heads, width, rope, rotary_dim,
               interleaved):
    T = src.shape[0]
    y = torch.stack([src[:, h * src_head + src_off:h * src_head + src_off + width]
                     for h in range(num_heads)], dim=1).float()
    y = _turn(y.clone(), rope, rotary_dim, interleaved)
    for h in range(num_heads):
        dst[:, h * dst_head + dst_off:h * dst_head + dst_off + width] = y[:, h].to(dst.dtype)


def head_linear(x, x_head, w, y, y_head):
    H, N, K = w.shape
    for h in range(H):
        y[:, h * y_head:h * y_head + N] = \
            (x[:, h * x_head:h * x_head + K].float() @ w[h].float().t()).to(y.dtype)


def mlstm(q, k, v, gate_i, gate_f, bias_i, bias_f, cap, q_scale, out, num_seqs, num_heads, key_dim,
          value_dim, q_start, state_slots, state):
    H, dk, dv = num_heads, key_dim, value_dim
    cap = float(torch.tensor(cap, dtype=torch.float32))
    q_scale = float(torch.tensor(q_scale, dtype=torch.float32))
    for b in range(num_seqs):
        row = state[int(state_slots[b])]
        S = row[:H * dk * dv].view(H, dk, dv)
        n = row[H * dk * dv:H * dk * dv + H * dk].view(H, dk)
        m = row[H * dk * dv + H * dk:H * dk * dv + H * dk + H]
        for t in range(int(q_start[b]), int(q_start[b + 1])):
            qt = q[t].float().reshape(H, dk) * q_scale
            kt = k[t].float().reshape(H, dk)
            vt = v[t].float().reshape(H, dv)
            li = cap * torch.tanh((gate_i[t] + bias_i) / cap)
            lf = torch.nn.functional.logsigmoid(cap * torch.tanh((gate_f[t] + bias_f) / cap))
            m_new = torch.maximum(lf + m, li)
            keep, take = torch.exp(lf + m - m_new), torch.exp(li - m_new)
            S.copy_(keep[:, None, None] * S + take[:, None, None] * kt[:, :, None] * vt[:, None, :])
            n.copy_(keep[:, None] * n + take[:, None] * kt)
            m.copy_(m_new)
            num = torch.einsum("hkv,hk->hv", S, qt)
            den = torch.maximum((n * qt).sum(-1).abs(), torch.exp(-m_new)) + 1e-6
            out[t] = (num / den[:, None]).reshape(-1)


def _chunk_lists_describe_step(q, num_seqs, q_start, chunk_tok0, chunk_ntok, chunk_first, most):
    T, at = q.shape[0], 0
    starts = [int(x) for x in q_start]
    for b in range(num_seqs):
        assert int(chunk_first[b]) == at
        o = starts[b]
        while o < starts[b + 1]:
            assert int(chunk_tok0[at]) == o and 0 < int(chunk_ntok[at]) <= most
            o += int(chunk_ntok[at])
            at += 1
        assert o == starts[b + 1]
    assert at == chunk_tok0.numel() and starts[-1] == T


def mlstm_chunked(q, k, v, gate_i, gate_f, bias_i, bias_f, cap, q_scale, out, num_seqs, num_heads,
                  key_dim, value_dim, q_start, state_slots, state, chunk_tok0=None, chunk_ntok=None,
                  chunk_first=None):
    if chunk_tok0 is not None:          # the lists the host made must describe the step
        _chunk_lists_describe_step(q, num_seqs, q_start, chunk_tok0, chunk_ntok, chunk_first,
                                   mlstm_chunk_tokens())
    else:
        assert q.shape[0] == num_seqs
    mlstm(q, k, v, gate_i, gate_f, bias_i, bias_f, cap, q_scale, out, num_seqs, num_heads, key_dim,
          value_dim, q_start, state_slots, state)


def mlstm_chunk_tokens():
    return 64


def mlstm_chunked_supports(num_heads, key_dim, value_dim):
    return True


def attention_sink_supports(num_heads, num_kv_heads, key_dim, value_dim):
    return False


def attention_sink_wide_supports(num_heads, num_kv_heads, key_dim, value_dim):
    return False


NAMES = ["act_rows", "stream_spread", "stream_read_norm", "stream_write", "qkv_conv_rope_norm_cache",
         "scaled_add_norm", "add_bias", "qk_rownorm_rope_cache", "latent_row_cache", "rope_slice",
         "head_linear", "mlstm", "mlstm_chunked", "mlstm_chunk_tokens", "mlstm_chunked_supports",
         "gated_group_norm", "qkv_bias_rope_cache", "causal_conv_act", "selective_scan",
         "moe_feed_forward", "weighted_sum", "attention_sink_supports", "attention_sink_wide_supports", "rope_table", "argmax", "sample", "logits_adjust", "embed", "add_rmsnorm", "residual_add", "swiglu", "qk_norm_rope_cache",
         "attention_generic", "linear", "gated_linear", "sgemm_tn", "gated_act", "cast_rows",
         "group_norm_scale_add", "group_norm_rows", "softcap", "value_norm_share_cache",
         "head_norm_gate", "attention_mixed", "retention", "retention_chunked",
         "retention_chunk_tokens", "retention_chunked_supports"]


def install(monkeypatch):
    from tgo_b200.kernels import ops
    from tgo_b200.parts import attention
    here = globals()
    for name in NAMES:
        monkeypatch.setattr(ops, name, here[name])
    monkeypatch.setattr(attention, "paged_attention", paged_attention)
