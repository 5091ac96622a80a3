"""Plain PyTorch statements of what each CUDA launcher computes, with the launchers' signatures.

Used two ways: the GPU tests compare every kernel with its function here, and the CPU tests
install these functions in place of the launchers (``install(monkeypatch)``) so that the host
side of the engine (batch packing, cache, scheduling) can be exercised where there is no GPU.
They are test code only: the product has no CPU path.
Math is float64 inside; outputs are rounded once to the output tensor's dtype.
"""
from __future__ import annotations

import math

import torch

D = torch.float64


def embed(table, tokens, out, status, accumulate=False, scale=1.0):
    tok = tokens.long()
    bad = (tok < 0) | (tok >= table.shape[0])
    if bad.any():
        status |= 4 if accumulate else 1
    rows = (table[tok.clamp(0, table.shape[0] - 1)].to(torch.float32) * torch.tensor(scale, dtype=torch.float32)).to(torch.float32)
    rows[bad] = 0
    out.copy_(out + rows if accumulate else rows)


def gather_tokens(dst, src, idx):
    m = idx >= 0
    dst[m] = src[idx[m].long()]


def add_rmsnorm(h, delta, weight, out, eps, rows=None):
    idx = torch.arange(out.shape[0], device=h.device) if rows is None else rows.long()
    if delta is not None:
        if delta.dim() == 3:                                  # a stack of float32 partial sums
            delta = delta.to(D).sum(0)
        h[idx] = (h[idx].to(D) + delta[idx].to(D)).to(torch.float32)
    x = h[idx].to(D)
    y = x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * weight.to(D)
    out.copy_(y.to(out.dtype))


def residual_add(h, delta):
    if delta.dim() == 3:
        delta = delta.to(D).sum(0)
    h.copy_((h.to(D) + delta.to(D)).to(torch.float32))


def swiglu(gate_up, out, activation="silu"):
    I = out.shape[1]
    g, u = gate_up[:, :I].to(D), gate_up[:, I:].to(D)
    if activation == "gelu_tanh":
        a = 0.5 * g * (1 + torch.tanh(math.sqrt(2 / math.pi) * (g + 0.044715 * g ** 3)))
    else:
        a = g / (1 + torch.exp(-g))
    out.copy_((a * u).to(out.dtype))


def add_layernorm(h, delta, weight, out, eps, rows=None, post=None):
    idx = torch.arange(out.shape[0], device=h.device) if rows is None else rows.long()
    if delta is not None:
        if delta.dim() == 3:
            delta = delta.to(D).sum(0)
        h[idx] = (h[idx].to(D) + delta[idx].to(D)).to(torch.float32)
    x = h[idx].to(D)
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    out.copy_(((x - mu) * torch.rsqrt(var + eps) * weight.to(D)).to(out.dtype))
    if post is not None:
        h[idx] = (h[idx].to(D) + post.to(D)).to(torch.float32)


def qkv_prep(qkv, q_out, q_weight, k_weight, inv_freq, k_pages, v_pages, table, positions, row_entry, n_q, n_k, n_v,
             dim, vdim, eps, status, *, whole=False, q_temp_coef=0.0, q_temp_every=1, half_pairing=False, unit_norm=False):
    n = qkv.shape[0]
    x = qkv.to(D)
    q = x[:, : n_q * dim].reshape(n, n_q, dim)
    k = x[:, n_q * dim:(n_q + n_k) * dim].reshape(n, n_k, dim)
    v = x[:, (n_q + n_k) * dim:(n_q + n_k) * dim + n_v * vdim].reshape(n, n_v, vdim)      # columns behind v are the caller's

    def norm(t, w):
        if w is None and unit_norm:
            return t * torch.rsqrt((t * t).mean(-1, keepdim=True) + eps)
        if w is None:
            return t
        if whole:                                                 # one norm over all heads of the row
            flat = t.reshape(n, -1)
            return (flat * torch.rsqrt((flat * flat).mean(-1, keepdim=True) + eps) * w.to(D)).reshape(t.shape)
        return t * torch.rsqrt((t * t).mean(-1, keepdim=True) + eps) * w.to(D)

    def rot(t):
        if inv_freq is None or inv_freq.numel() == 0:
            return t
        r = 2 * inv_freq.numel()
        ang = (positions.to(torch.float32)[:, None] * inv_freq[None, :]).to(D)          # float32 angle
        c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
        o = t.clone()
        if half_pairing:
            a, b = t[..., :r // 2], t[..., r // 2:r]
            o[..., :r // 2], o[..., r // 2:r] = a * c - b * s, b * c + a * s
            return o
        a, b = t[..., 0:r:2], t[..., 1:r:2]
        o[..., 0:r:2], o[..., 1:r:2] = a * c - b * s, b * c + a * s
        return o

    q, k = norm(q, q_weight), norm(k, k_weight)
    if q_temp_coef:
        steps = torch.div(positions.long() + 1, int(q_temp_every), rounding_mode="floor") + 1
        q = q * (1.0 + q_temp_coef * torch.log(steps.to(D)))[:, None, None]
    q, k = rot(q), rot(k)
    valid = row_entry >= 0
    qo = q.reshape(n, -1).to(q_out.dtype)
    qo[~valid] = 0
    q_out.copy_(qo)
    if n_k or n_v:
        ps = k_pages.shape[2]
        for r in range(n):
            if not bool(valid[r]):
                continue
            pos = int(positions[r])
            page = int(table[int(row_entry[r]), pos // ps])
            if page < 0 or page >= k_pages.shape[0]:
                status |= 2
                continue
            k_pages[page, :, pos % ps] = k[r].to(k_pages.dtype)
            v_pages[page, :, pos % ps] = v[r].to(v_pages.dtype)


def mapped_attention(q, k_pages, v_pages, table, positions, row_entry, out, n_heads, n_maps, window, keep_first, scale,
                     softcap, lam, head_norm, post_scale, eps, n_splits=1, partial=None, slopes=None, sinks=None, chunk=0):
    n = q.shape[0]
    P, n_k, ps, dim = k_pages.shape
    n_g, vdim = v_pages.shape[1], v_pages.shape[3]
    group = n_heads // n_g
    for r in range(n):
        e = int(row_entry[r])
        if e < 0:
            out[r] = 0
            continue
        pos = int(positions[r])
        lo = max(0, pos - window + 1) if window else 0
        if chunk:
            lo = max(lo, (pos // chunk) * chunk)
        kp = torch.tensor([j for j in range(pos + 1) if j >= lo or j < keep_first], device=q.device)
        pages = table[e, kp // ps].long()
        K = k_pages[pages, :, kp % ps].to(D)             # [keys, n_g * n_maps, dim]
        Vv = v_pages[pages, :, kp % ps].to(D)            # [keys, n_g, vdim]
        qr = q[r].to(D).reshape(n_heads, n_maps, dim)
        o = torch.empty(n_heads, vdim, dtype=D, device=q.device)
        for h in range(n_heads):
            g = h // group
            a = []
            for m in range(n_maps):
                s = (K[:, g * n_maps + m] @ qr[h, m]) * scale
                if softcap:
                    s = softcap * torch.tanh(s / softcap)
                if slopes is not None:
                    s = s - slopes[h].to(D) * (pos - kp).to(D)
                if sinks is not None:                              # one more term of the denominator, without a value
                    w = torch.softmax(torch.cat([s, sinks[h].to(D).reshape(1)]), 0)[:-1]
                else:
                    w = torch.softmax(s, 0)
                a.append(w @ Vv[:, g])
            y = a[0] if n_maps == 1 else a[0] - lam * a[1]
            if head_norm:
                y = y * torch.rsqrt((y * y).mean() + eps) * post_scale
            o[h] = y
        out[r] = o.reshape(-1).to(out.dtype)


def gated_delta(p, conv_weight, a_log, dt_bias, norm_weight, conv_state, state, conv_out, o_raw, out, cu_q, ctx_before, slots,
                row_entry, n_entries, max_q, n_heads, n_qk_heads, key_dim, value_dim, eps, chunk_scratch=None):
    nH, nG, dk, dv = n_heads, n_qk_heads, key_dim, value_dim
    C = 2 * nG * dk + nH * dv
    L = conv_weight.shape[1]
    cu = cu_q.tolist()
    out[row_entry < 0] = 0
    for e in range(n_entries):
        q0, q1 = cu[e], cu[e + 1]
        if q1 == q0:
            continue
        T = q1 - q0
        ctx, slot = int(ctx_before[e]), int(slots[e])
        rows = p[q0:q1].to(D)
        old = conv_state[slot].to(D).clone()
        for j in range(L - 1):
            if ctx - (L - 1) + j < 0:
                old[j] = 0
        u = torch.cat([old, rows[:, :C]])
        c = torch.zeros(T, C, dtype=D, device=p.device)
        for k in range(L):
            c += conv_weight[:, k].to(D) * u[k:k + T]
        conv_state[slot] = u[-(L - 1):].to(torch.float32)
        c = c * torch.sigmoid(c)
        unit = lambda t: t / torch.sqrt((t * t).sum(-1, keepdim=True) + 1e-6)
        qh = unit(c[:, :nG * dk].reshape(T, nG, dk)) * dk ** -0.5
        kh = unit(c[:, nG * dk:2 * nG * dk].reshape(T, nG, dk))
        vh = c[:, 2 * nG * dk:].reshape(T, nH, dv)
        gate = rows[:, C:C + nH * dv].reshape(T, nH, dv)
        a, b = rows[:, C + nH * dv:C + nH * dv + nH], rows[:, C + nH * dv + nH:]
        beta = torch.sigmoid(b)
        g = torch.exp(-torch.exp(a_log.to(D)) * torch.nn.functional.softplus(a + dt_bias.to(D)))
        S = state[slot].to(D).clone() if ctx > 0 else torch.zeros(nH, dk, dv, dtype=D, device=p.device)
        o = torch.zeros(T, nH, dv, dtype=D, device=p.device)
        rep = nH // nG
        for t in range(T):
            kt, qt = kh[t].repeat_interleave(rep, 0), qh[t].repeat_interleave(rep, 0)
            S = S * g[t][:, None, None]
            uu = beta[t][:, None] * (vh[t] - torch.einsum("hkv,hk->hv", S, kt))
            S = S + kt[:, :, None] * uu[:, None, :]
            o[t] = torch.einsum("hkv,hk->hv", S, qt)
        state[slot] = S.to(torch.float32)
        y = o * torch.rsqrt((o * o).mean(-1, keepdim=True) + eps) * norm_weight.to(D) * (gate * torch.sigmoid(gate))
        out[q0:q1] = y.reshape(T, nH * dv).to(out.dtype)


def pair_embed(table, tokens, state, cu_q, ctx_before, slots, row_entry, h, n_entries, vocab, buckets, mul_prev, mul_cur, status):
    cu = cu_q.tolist()
    for e in range(n_entries):
        q0, q1 = cu[e], cu[e + 1]
        for r in range(q0, q1):
            if r > q0:
                prev = int(tokens[r - 1])
            else:
                prev = int(state[int(slots[e])]) if int(ctx_before[e]) > 0 else -1
            idx = buckets if prev < 0 else (prev * mul_prev + int(tokens[r]) * mul_cur) % buckets
            h[r] += table[idx].to(h.dtype)
        if q1 > q0:
            state[int(slots[e])] = tokens[q1 - 1]


def pair_norm_mean(a, b, wa, wb, out, eps, act_dtype, accumulate=False):
    def whole(t):
        return t.to(D).sum(0).to(act_dtype).to(D) if t.dim() == 3 and t.shape[0] > 1 else t.reshape(out.shape).to(D)
    x, y = whole(a), whole(b)
    over = lambda t: t * torch.rsqrt((t * t).mean(-1, keepdim=True) + eps)
    v = 0.5 * (over(x) * wa.to(D) + over(y) * wb.to(D))
    out.copy_(((out.to(D) + v) if accumulate else v).to(out.dtype))


def relu_squared_(x):
    x.copy_((torch.relu(x.to(D)) ** 2).to(x.dtype))


def softcap_(x, cap):
    x.copy_((cap * torch.tanh(x.to(D) / cap)).to(x.dtype))


def moe_router_sigmoid(x, w_router, correction, w_shared_gate, weights, top_k, n_groups=1, keep_groups=1, *,
                       softmax_scores=False, group_max=False, route_scale=1.0):
    n, E = x.shape[0], w_router.shape[0]
    logits = x.to(D) @ w_router.to(D).T
    s = torch.softmax(logits, -1) if softmax_scores else torch.sigmoid(logits)
    choice = s + (correction.to(D) if correction is not None else 0.0)
    per = E // n_groups
    weights.zero_()
    for r in range(n):
        c = choice[r].clone()
        if keep_groups < n_groups:
            gs = []
            for g in range(n_groups):
                top2 = sorted(c[g * per:(g + 1) * per].tolist(), reverse=True)[:1 if group_max else 2]
                gs.append(sum(top2))
            order = sorted(range(n_groups), key=lambda g: (-gs[g], g))
            for g in order[keep_groups:]:
                c[g * per:(g + 1) * per] = -math.inf
        chosen = sorted(range(E), key=lambda e: (-float(c[e]), e))[:top_k]
        total = sum(float(s[r, e]) for e in chosen) + 1e-20
        for e in chosen:
            weights[r, e] = float(s[r, e]) / total * route_scale
    if w_shared_gate is not None:
        weights[:, E] = torch.sigmoid(x.to(D) @ w_shared_gate.to(D)).to(weights.dtype)


def moe_clamped_glu_scaled(gate_up, weights, out, n_experts, expert_ff, limit, shared_limit, alpha, shared_gated):
    n, I = out.shape
    g, u = gate_up[:, :I].to(D), gate_up[:, I:].to(D)
    routed = n_experts * expert_ff
    lim = torch.cat([torch.full((routed,), float(limit), dtype=D), torch.full((I - routed,), float(shared_limit), dtype=D)]).to(g.device)
    g = torch.minimum(g, lim)
    u = torch.maximum(torch.minimum(u, lim), -lim)
    w = weights[:, :n_experts].to(D).repeat_interleave(expert_ff, dim=1)
    tail = weights[:, n_experts:n_experts + 1].to(D) if shared_gated else torch.ones(n, 1, dtype=D, device=g.device)
    w = torch.cat([w, tail.expand(n, I - routed)], dim=1)
    out.copy_((g * torch.sigmoid(alpha * g) * (u + 1.0) * w).to(out.dtype))


def gemm_f32(a, w, bias, out):
    r = a.to(D) @ w.to(D).T
    if bias is not None:
        r = r + bias.to(D)
    out.copy_(r.to(out.dtype))


def linear(x, weight, bias, out):
    gemm_f32(x, weight, bias, out)


def shortconv(p, weight, bias, state, out, cu_q, ctx_before, slots, n_entries, max_q):
    H = out.shape[1]
    L = weight.shape[1]
    if p.dim() == 3:                                          # float32 partial sums, rounded where the product would be
        p = p.to(D).sum(0).to(out.dtype)
    cu = cu_q.tolist()
    for e in range(n_entries):
        q0, q1 = cu[e], cu[e + 1]
        if q1 == q0:
            continue
        ctx, slot = int(ctx_before[e]), int(slots[e])
        rows = p[q0:q1].to(D)
        Bg, Cg, x = rows[:, :H], rows[:, H:2 * H], rows[:, 2 * H:]
        u_new = Bg * x
        old = state[slot].to(D).clone()                       # [L-1, H], positions ctx-(L-1)..ctx-1
        for j in range(L - 1):
            if ctx - (L - 1) + j < 0:
                old[j] = 0
        u = torch.cat([old, u_new])                           # index i <-> chunk index i-(L-1)
        c = torch.zeros(q1 - q0, H, dtype=D, device=p.device)
        for k in range(L):
            c += weight[:, k].to(D) * u[k:k + (q1 - q0)]
        if bias is not None:
            c = c + bias.to(D)
        out[q0:q1] = (Cg * c).to(out.dtype)
        state[slot] = u[-(L - 1):].to(torch.float32)


def rope_cache(qkv, q_out, q_weight, k_weight, inv_freq, half_pairing, pos_scale, k_pages, v_pages, table,
               positions, row_entry, n_heads, n_kv_heads, head_dim, eps, status):
    if qkv.dim() == 3:
        qkv = qkv.to(D).sum(0).to(q_out.dtype)
    n = qkv.shape[0]
    hd = head_dim
    x = qkv.to(D)
    q = x[:, : n_heads * hd].reshape(n, n_heads, hd)
    k = x[:, n_heads * hd:(n_heads + n_kv_heads) * hd].reshape(n, n_kv_heads, hd)
    v = x[:, (n_heads + n_kv_heads) * hd:].reshape(n, n_kv_heads, hd)

    def norm(t, w):
        return t * torch.rsqrt((t * t).mean(-1, keepdim=True) + eps) * w.to(D)

    def rot(t):
        if inv_freq is None:
            return t
        ang = ((positions.to(torch.float32) / pos_scale)[:, None] * inv_freq[None, :]).to(D)   # float32 angle
        c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
        o = torch.empty_like(t)
        if half_pairing:
            a, b = t[..., : hd // 2], t[..., hd // 2:]
            o[..., : hd // 2], o[..., hd // 2:] = a * c - b * s, a * s + b * c
        else:
            a, b = t[..., 0::2], t[..., 1::2]
            o[..., 0::2], o[..., 1::2] = a * c - b * s, a * s + b * c
        return o

    if q_weight is not None:
        q = norm(q, q_weight)
        if n_kv_heads:
            k = norm(k, k_weight)
    q, k = rot(q), (rot(k) if n_kv_heads else k)
    valid = row_entry >= 0
    qo = q.reshape(n, -1).to(q_out.dtype)
    qo[~valid] = 0
    q_out.copy_(qo)
    if n_kv_heads:
        ps = k_pages.shape[2]
        for r in range(n):
            if not bool(valid[r]):
                continue
            pos = int(positions[r])
            page = int(table[int(row_entry[r]), pos // ps])
            if page < 0 or page >= k_pages.shape[0]:
                status |= 2
                continue
            k_pages[page, :, pos % ps] = k[r].to(k_pages.dtype)
            v_pages[page, :, pos % ps] = v[r].to(v_pages.dtype)


def attention_generic(q, k_pages, v_pages, table, positions, row_entry, out, n_heads, window, scale, slopes=None):
    n = q.shape[0]
    P, n_kv, ps, hd = k_pages.shape
    group = n_heads // n_kv
    for r in range(n):
        e = int(row_entry[r])
        if e < 0:
            out[r] = 0
            continue
        pos = int(positions[r])
        lo = max(0, pos - window + 1) if window else 0
        kp = torch.arange(lo, pos + 1, device=q.device)
        pages = table[e, kp // ps].long()
        K = k_pages[pages, :, kp % ps].to(D)             # [keys, n_kv, hd]
        Vv = v_pages[pages, :, kp % ps].to(D)
        qr = q[r].to(D).reshape(n_heads, hd)
        o = torch.empty(n_heads, hd, dtype=D, device=q.device)
        for h in range(n_heads):
            s = (K[:, h // group] @ qr[h]) * scale
            if slopes is not None:
                s = s - float(slopes[h]) * (pos - kp).to(D)
            o[h] = torch.softmax(s, 0) @ Vv[:, h // group]
        out[r] = o.reshape(-1).to(out.dtype)


def sample(logits, temperature, top_p, uniform, out, scratch):
    W, V = logits.shape
    for r in range(W):
        lg = logits[r].to(D)
        t = float(temperature[r]) if temperature is not None else 0.0
        if not t > 0:
            out[r] = int(torch.argmax(lg))
            continue
        e = torch.exp((lg - lg.max()) / t)
        p = float(top_p[r]) if top_p is not None else 1.0
        if 0 < p < 1:
            vals = torch.sort(e, descending=True).values
            cs = torch.cumsum(vals, 0)
            cut = int(torch.nonzero(cs >= p * e.sum())[0]) if (cs >= p * e.sum()).any() else V - 1
            e = torch.where(e >= vals[cut], e, torch.zeros_like(e))
        c = torch.cumsum(e, 0)
        target = float(uniform[r]) * float(c[-1])
        hit = torch.nonzero(target < c)
        out[r] = int(hit[0]) if len(hit) else int(torch.argmax(lg))


# ------------------------------------------------------------------------------------------------ Dodilix's launchers
def scale_(x, factor):
    x.mul_(factor)


def gate_mul(y, gate, activation="sigmoid", scale=1.0):
    f = torch.full_like(y, scale, dtype=D)
    if gate is not None:
        g = gate.to(D)
        f = f * (torch.sigmoid(g) if activation == "sigmoid" else g * torch.sigmoid(g))
    y.copy_((y.to(D) * f).to(y.dtype))


def hc_step(streams, n_streams, *, x0=None, delta=None, mix=None, out_w=None, in_w=None, norm_w=None, out=None, sum_out=None,
            eps=0.0, act_dtype=None):
    n, S = streams.shape[0], n_streams
    H = streams.shape[1] // S
    X = x0.to(D)[:, None, :].expand(n, S, H).clone() if x0 is not None else streams.to(D).reshape(n, S, H)
    if delta is not None:
        y = (delta.sum(0) if delta.dim() == 3 else delta).to(D)
        X = torch.einsum("st,nsh->nth", mix.to(D).reshape(S, S), X) + out_w.to(D)[None, :, None] * y[:, None, :]
    if x0 is not None or delta is not None:
        streams.copy_(X.reshape(n, S * H).to(streams.dtype))
    if in_w is not None:
        u = torch.einsum("s,nsh->nh", in_w.to(D), X)
        out.copy_((u * torch.rsqrt((u * u).mean(-1, keepdim=True) + eps) * norm_w.to(D)).to(out.dtype))
    if sum_out is not None:
        sum_out.copy_(X.sum(1).to(sum_out.dtype))


def moe_swiglu_scaled(gate_up, weights, out, expert_ff, shared_gated=False):
    n, I = out.shape
    E = weights.shape[1] - int(bool(shared_gated))
    g, u = gate_up[:, :I].to(D), gate_up[:, I:].to(D)
    w = weights[:, :E].to(D).repeat_interleave(expert_ff, dim=1)
    tail = weights[:, E:E + 1].to(D) if shared_gated else torch.ones(n, 1, dtype=D)
    w = torch.cat([w, tail.expand(n, I - E * expert_ff)], dim=1)
    out.copy_((g * torch.sigmoid(g) * u * w).to(out.dtype))


def gated_linear(x, z, norm_w, state, out, cu_q, ctx_before, slots, n_entries, n_heads, key_dim, value_dim, tau, eps,
                 out_scale=1.0, scratch=None, state_scratch=None, max_q=0):
    H, dk, dv = n_heads, key_dim, value_dim
    for e in range(n_entries):
        r0, r1 = int(cu_q[e]), int(cu_q[e + 1])
        slot = int(slots[e])
        S = state[slot].to(D).clone() if int(ctx_before[e]) > 0 else torch.zeros(H, dk, dv, dtype=D)
        for r in range(r0, r1):
            row = x[r].to(D)
            q = row[:H * dk].reshape(H, dk) * dk ** -0.5
            k = row[H * dk:2 * H * dk].reshape(H, dk)
            v = row[2 * H * dk:2 * H * dk + H * dv].reshape(H, dv)
            g = row[2 * H * dk + H * dv:].reshape(H, dv)
            alpha = torch.sigmoid(z[r].to(D)).pow(1.0 / tau).reshape(H, dk)
            S = alpha[:, :, None] * S + k[:, :, None] * v[:, None, :]
            o = torch.einsum("hkv,hk->hv", S, q)
            o = o * torch.rsqrt((o * o).mean(-1, keepdim=True) + eps) * norm_w.to(D) * (g * torch.sigmoid(g)) * out_scale
            out[r] = o.reshape(-1).to(out.dtype)
        if r1 > r0:
            state[slot] = S.to(state.dtype)


def latent_prep(x, wq, wkv, cq_out, pages, gate_out, table, positions, row_entry, n_heads, eps, status, *, rot=0,
                inv_freq=None, half_pairing=False):
    n, rq = cq_out.shape
    rkv = wkv.numel() if wkv is not None else 0
    xd = x.to(D)
    a = xd[:, :rq]
    cq_out.copy_((a * torch.rsqrt((a * a).mean(-1, keepdim=True) + eps) * wq.to(D)).to(cq_out.dtype))
    gate_out.copy_(torch.sigmoid(xd[:, rq + rkv + rot:]).to(gate_out.dtype))
    if not rkv:
        return
    c = xd[:, rq:rq + rkv]
    c = c * torch.rsqrt((c * c).mean(-1, keepdim=True) + eps) * wkv.to(D)
    kr = _rotate_tail(xd[:, rq + rkv:rq + rkv + rot], positions, inv_freq, half_pairing) if rot else xd[:, :0]
    ps, rp = pages.shape[2], pages.shape[3]
    for r in range(n):
        e = int(row_entry[r])
        if e < 0:
            continue
        pos = int(positions[r])
        page = int(table[e, pos // ps])
        rowv = torch.zeros(rp, dtype=D)
        rowv[:rkv], rowv[rkv:rkv + rot] = c[r], kr[r]
        pages[page, 0, pos % ps] = rowv.to(pages.dtype)


def _rotate_tail(t, positions, inv_freq, half_pairing):
    r = t.shape[-1]
    ang = (positions.to(torch.float32)[:, None] * inv_freq[None, :]).to(D)
    c, s = torch.cos(ang), torch.sin(ang)
    o = t.clone()
    if half_pairing:
        a, b = t[..., :r // 2], t[..., r // 2:]
        o[..., :r // 2], o[..., r // 2:] = a * c - b * s, b * c + a * s
    else:
        a, b = t[..., 0::2], t[..., 1::2]
        o[..., 0::2], o[..., 1::2] = a * c - b * s, b * c + a * s
    return o


def latent_rope_q(q, positions, row_entry, inv_freq, n_heads, offset, half_pairing=False):
    n = q.shape[0]
    rot = 2 * inv_freq.numel()
    qv = q.view(n, n_heads, -1)
    for h in range(n_heads):
        qv[:, h, offset:offset + rot] = _rotate_tail(qv[:, h, offset:offset + rot].to(D), positions, inv_freq,
                                                     half_pairing).to(q.dtype)


def latent_core(q, pages, table, positions, row_entry, gate, out, n_heads, window, scale, n_splits=1, partial=None):
    n = q.shape[0]
    ps, rp = pages.shape[2], pages.shape[3]
    for r in range(n):
        e = int(row_entry[r])
        if e < 0:
            out[r] = 0
            continue
        pos = int(positions[r])
        lo = max(0, pos - window + 1) if window else 0
        kp = torch.arange(lo, pos + 1)
        C = pages[table[e, kp // ps].long(), 0, kp % ps].to(D)                  # [keys, rp]
        qr = q[r].to(D).reshape(n_heads, rp)
        w = torch.softmax(qr @ C.T * scale, -1)
        o = w @ C
        if gate is not None:
            o = o * gate[r].to(D)[:, None]
        out[r] = o.reshape(-1).to(out.dtype)


def head_up_gate(o, w, gate, out):
    n = o.shape[0]
    H, dv, rank = w.shape
    y = torch.einsum("hvr,nhr->nhv", w.to(D), o.to(D).reshape(n, H, -1)[:, :, :rank]).reshape(n, H * dv)
    if gate is not None:
        y = y * gate.to(D)
    out.copy_(y.to(out.dtype))


_NAMES = ["scale_", "gate_mul", "hc_step", "moe_swiglu_scaled", "gated_linear", "latent_prep", "latent_rope_q", "latent_core",
          "head_up_gate", "gather_tokens", "embed", "add_rmsnorm", "residual_add", "swiglu", "gemm_f32", "linear", "shortconv", "rope_cache",
          "attention_generic", "sample", "add_layernorm", "qkv_prep", "mapped_attention", "gated_delta", "pair_embed",
          "pair_norm_mean", "relu_squared_", "softcap_", "moe_router_sigmoid", "moe_clamped_glu_scaled"]


def install(monkeypatch):
    """Replace the launchers of ``neurogrid_b200.csrc.ops`` with the functions above."""
    from neurogrid_b200.csrc import ops
    for n in _NAMES:
        monkeypatch.setattr(ops, n, globals()[n])


def _rows_of(cu_q, single: bool):
    cu = cu_q.tolist()
    rows, entries = [], []
    for e in range(len(cu) - 1):
        n = cu[e + 1] - cu[e]
        if (n == 1) == single and n > 0:
            rows += list(range(cu[e], cu[e + 1]))
            entries += [e] * n
    return rows, entries


def _attend_rows(q, k_pages, v_pages, table, cu_q, ctx_before, out, n_heads, window, scale, single, slopes=None):
    rows, entries = _rows_of(cu_q, single)
    cu = cu_q.tolist()
    n = q.shape[0]
    pos = torch.zeros(n, dtype=torch.int32, device=q.device)
    re = torch.full((n,), -1, dtype=torch.int32, device=q.device)
    for r, e in zip(rows, entries):
        pos[r] = int(ctx_before[e]) + (r - cu[e])
        re[r] = e
    tmp = out.clone()
    attention_generic(q, k_pages, v_pages, table, pos, re, tmp, n_heads, window, scale, slopes)
    for r in rows:
        out[r] = tmp[r]


def attn_prefill_bf16(q, k_pages, v_pages, table, cu_q, ctx_before, out, n_entries, max_q, n_heads, window, scale,
                      skip_single, slopes=None):
    _attend_rows(q, k_pages, v_pages, table, cu_q, ctx_before, out, n_heads, window, scale, False, slopes)
    if not skip_single:
        _attend_rows(q, k_pages, v_pages, table, cu_q, ctx_before, out, n_heads, window, scale, True, slopes)


def attn_decode_bf16(q, k_pages, v_pages, table, cu_q, ctx_before, out, scratch, n_entries, n_heads, window, scale,
                     n_splits, max_ctx, slopes=None):
    _attend_rows(q, k_pages, v_pages, table, cu_q, ctx_before, out, n_heads, window, scale, True, slopes)


def attn_prefill_sm100(q, k_pages, v_pages, table, cu_q, ctx_before, out, n_entries, max_q, n_heads, window, scale,
                       skip_single, slopes=None, scratch=None, n_splits=1):
    attn_prefill_bf16(q, k_pages, v_pages, table, cu_q, ctx_before, out, n_entries, max_q, n_heads, window, scale,
                      skip_single, slopes)


_NAMES += ["attn_prefill_bf16", "attn_decode_bf16", "attn_prefill_sm100"]
# ops.linear_to_residual is host logic over ops.linear: it is not replaced
