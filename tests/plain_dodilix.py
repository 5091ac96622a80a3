"""A plain, slow statement of the Dodilix decoder: float64, whole sequences, one function per mechanism.

Shares no code with the package.  ``cfg`` is the dictionary of config.json, ``w`` maps tensor names to float64
tensors; a sequence is a list of token ids, positions count from 0.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms_div(x, eps):
    """x over its root mean square along the last axis (eps inside the root)."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, weight, eps):
    return rms_div(x, eps) * weight


def silu(z):
    return z * torch.sigmoid(z)


def rotate(x, positions, dims, base, interleaved):
    """x [T, heads, d]: the first ``dims`` coordinates of every head are turned by the angle position * base^(-2i/dims);
    pair i is (i, i + dims/2), or (2i, 2i + 1) when ``interleaved``."""
    if not dims:
        return x
    half = dims // 2
    i = torch.arange(half, dtype=F64)
    ang = positions.to(F64)[:, None] * base ** (-2.0 * i / dims)[None, :]           # [T, half]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    out = x.clone()
    if interleaved:
        a, b = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = a * c - b * s
        out[..., 1:dims:2] = b * c + a * s
    else:
        a, b = x[..., :half], x[..., half:dims]
        out[..., :half] = a * c - b * s
        out[..., half:dims] = b * c + a * s
    return out


# ------------------------------------------------------------------------------------------------ mixers
def chunk_attention(h, w, pre, m, eps):
    """The left side of a parallel mixer: grouped-query attention inside chunks, with a sink and an output gate."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = (h @ w[pre + "q"].T).view(T, H, d)
    k = (h @ w[pre + "k"].T).view(T, G, d)
    v = (h @ w[pre + "v"].T).view(T, G, dv)
    rot = m.get("rot")
    if rot:
        q = rotate(q, pos, rot["dims"], rot["base"], False)
        k = rotate(k, pos, rot["dims"], rot["base"], False)
    q, k = rms_div(q, eps), rms_div(k, eps)
    size = m["mask"]["size"] if m.get("mask") else None
    out = torch.zeros(T, H, dv, dtype=F64)
    for hd in range(H):
        g = hd // (H // G)
        for t in range(T):
            lo = (t // size) * size if size else 0
            s = (k[lo:t + 1, g] @ q[t, hd]) * m["scale"]
            sink = w[pre + "sink"][hd]
            top = torch.maximum(s.max(), sink)
            e = torch.exp(s - top)
            out[t, hd] = (e[:, None] * v[lo:t + 1, g]).sum(0) / (e.sum() + torch.exp(sink - top))
    gate = torch.sigmoid(h @ w[pre + "g"].T)
    return (out.reshape(T, H * dv) * gate) @ w[pre + "o"].T


def gated_linear_attention(h, w, pre, m, eps, state=None):
    """The right side: per head S <- diag(alpha_t) S + k_t v_t^T, o_t = S^T q_t, with a decay per key channel."""
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ w[pre + "q"].T).view(T, H, d) * d ** -0.5
    k = (h @ w[pre + "k"].T).view(T, H, d)
    v = (h @ w[pre + "v"].T).view(T, H, dv)
    z = (h @ w[pre + "a1"].T) @ w[pre + "a2"].T + w[pre + "a2.b"]
    alpha = torch.sigmoid(z).pow(1.0 / m["tau"]).view(T, H, d)
    S = torch.zeros(H, d, dv, dtype=F64) if state is None else state.clone()
    o = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = rms_norm(o, w[pre + "norm"], eps).reshape(T, H * dv)
    return (o * silu(h @ w[pre + "g"].T)) @ w[pre + "o"].T, S


def parallel_mixer(h, w, pre, m, eps):
    left = chunk_attention(h, w, pre + "left.", m["left"], eps)
    right, _ = gated_linear_attention(h, w, pre + "right.", m["right"], eps)
    return m.get("left_scale", 1.0) * left + m.get("right_scale", 1.0) * right


def latent_kv(h, w, pre, m, eps):
    """What a latent layer keeps of every token: the normed latent and the rotated key part all heads share."""
    T = h.shape[0]
    r = m["kv_rank"]
    d = h @ w[pre + "dkv"].T
    c = rms_norm(d[:, :r], w[pre + "dkv.norm"], eps)
    rot = m.get("rot") or {}
    kr = rotate(d[:, None, r:], torch.arange(T), rot.get("dims", m.get("rot_dim", 0)) if rot else 0, rot.get("base", 1.0), True)[:, 0]
    return c, kr


def latent_attention(h, w, pre, m, eps, kv):
    """Causal softmax attention whose keys and values are expanded from ``kv`` = (latent, rotated key part)."""
    T = h.shape[0]
    H, d, dr, dv = m["heads"], m["dim"], m.get("rot_dim", 0), m["vdim"]
    c, kr = kv
    cq = rms_norm(h @ w[pre + "dq"].T, w[pre + "dq.norm"], eps)
    q = (cq @ w[pre + "uq"].T).view(T, H, d + dr)
    qn = q[..., :d]
    rot = m.get("rot") or {}
    qr = rotate(q[..., d:], torch.arange(T), rot.get("dims", dr) if rot else 0, rot.get("base", 1.0), True)
    kn = (c @ w[pre + "uk"].T).view(T, H, d)
    v = (c @ w[pre + "uv"].T).view(T, H, dv)
    out = torch.zeros(T, H, dv, dtype=F64)
    for hd in range(H):
        s = (qn[:, hd] @ kn[:, hd].T + qr[:, hd] @ kr.T) * m["scale"]
        s = s.masked_fill(torch.ones(T, T).triu(1).bool(), -math.inf)
        out[:, hd] = torch.softmax(s, -1) @ v[:, hd]
    gate = torch.sigmoid(h @ w[pre + "g"].T)
    return (out.reshape(T, H * dv) * gate) @ w[pre + "o"].T


# ------------------------------------------------------------------------------------------------ feed-forward
def gated_ff(h, w, pre):
    return (silu(h @ w[pre + "gate"].T) * (h @ w[pre + "up"].T)) @ w[pre + "down"].T


def route(h, w, pre, r):
    """[T, experts] routing weights: softmax scores, the best groups by their largest score, the largest scores among
    those groups' experts, the chosen scores over their sum, times the router's scale."""
    E, top = r["experts"], r["top"]
    s = torch.softmax(h @ w[pre + "router"].T, -1)
    allowed = torch.ones_like(s, dtype=torch.bool)
    groups = r.get("groups")
    if groups:
        n, keep = groups["count"], groups["keep"]
        best = s.view(-1, n, E // n).max(-1).values                       # [T, groups]
        kept = torch.zeros_like(best, dtype=torch.bool)
        kept.scatter_(1, best.topk(keep, dim=1).indices, True)
        allowed = kept[:, :, None].expand(-1, -1, E // n).reshape(-1, E)
    idx = s.masked_fill(~allowed, -1.0).topk(top, dim=1).indices
    chosen = torch.zeros_like(s).scatter(1, idx, s.gather(1, idx))
    return chosen / (chosen.sum(1, keepdim=True) + 1e-20) * r.get("scale", 1.0)


def moe_ff(h, w, pre, mlp):
    weights = route(h, w, pre, mlp["router"])
    y = torch.zeros_like(h)
    for e in range(mlp["router"]["experts"]):
        y = y + weights[:, e:e + 1] * gated_ff(h, w, f"{pre}e{e}.")
    if mlp.get("shared"):
        y = y + torch.sigmoid(h @ w[pre + "shared.sg"].T) * gated_ff(h, w, pre + "shared.")
    return y


def feed_forward(h, w, pre, mlp):
    return gated_ff(h, w, pre) if mlp.get("kind", "dense") == "dense" else moe_ff(h, w, pre, mlp)


# ------------------------------------------------------------------------------------------------ the model
def forward(cfg, w, tokens, *, return_layers=False):
    """Logits [T, vocab] of a whole sequence (and the stream, summed over its copies, after every layer)."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.as_tensor(tokens)] * cfg.get("embedding", {}).get("scale", 1.0)
    n_streams = cfg.get("streams")
    xs = [x.clone() for _ in range(n_streams)] if n_streams else None
    kept, after = {}, []
    for i, layer in enumerate(cfg["layers"]):
        pre, m = f"l{i}.", layer["mixer"]
        subs = [(1, "norm1")] + ([(2, "norm2")] if layer.get("mlp") is not None else [])
        for q, norm in subs:
            if xs is None:
                u = x
            else:
                a = w[f"{pre}hc{q}.in"]
                u = sum(a[s] * xs[s] for s in range(n_streams))
            hn = rms_norm(u, w[pre + norm], eps)
            if q == 2:
                y = feed_forward(hn, w, pre + "mlp.", layer["mlp"])
            elif layer["type"] == "parallel":
                y = parallel_mixer(hn, w, pre + "mix.", m, eps)
            else:
                src = m.get("kv_from")
                if src is None:
                    kept[i] = latent_kv(hn, w, pre + "mix.", m, eps)
                    src = i
                y = latent_attention(hn, w, pre + "mix.", m, eps, kept[src])
            if xs is None:
                x = x + y
            else:
                mix, b = w[f"{pre}hc{q}.mix"], w[f"{pre}hc{q}.out"]
                xs = [sum(mix[s, t] * xs[s] for s in range(n_streams)) + b[t] * y for t in range(n_streams)]
        after.append(sum(xs) if xs is not None else x)
    x = after[-1] if after else (sum(xs) if xs is not None else x)
    logits = rms_norm(x, w["final.norm"], eps) @ w["head"].T * cfg.get("logit_scale", 1.0)
    return (logits, after) if return_layers else logits
