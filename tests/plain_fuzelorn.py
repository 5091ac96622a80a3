"""A plain, slow statement of the Fuzelorn decoder in float64: one function per mechanism, whole sequences at
once, nothing shared with the package's parts or kernels.  ``cfg`` is the dictionary of a ``config.json``,
``w`` maps tensor names to tensors.

Notation: T tokens, D the model's width; positions count from 0.  Left mixer: H query heads, G key/value heads,
d the query/key size, dv the value size.  Right mixer: Hr value heads, Gr query/key heads, dr, dvr.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def over_rms(x, eps):
    """x over the root of (its mean square + eps), along the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


# ------------------------------------------------------------------------------------------ embedding
def bigram_rows(tokens, big):
    """Row of the bigram table for every token: (previous * mul_prev + token * mul_cur) mod buckets, and the row
    number ``buckets`` for a sequence's first token."""
    rows = []
    for t, tok in enumerate(tokens):
        if t == 0:
            rows.append(int(big["buckets"]))
        else:
            rows.append((int(tokens[t - 1]) * int(big["mul_prev"]) + int(tok) * int(big["mul_cur"])) % int(big["buckets"]))
    return torch.tensor(rows, dtype=torch.long)


def embed(cfg, w, tokens):
    emb = cfg.get("embedding") or {}
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)] * float(emb.get("scale", 1.0))
    if emb.get("bigram"):
        x = x + w["bigram"][bigram_rows(list(tokens), emb["bigram"])]
    return x


# ------------------------------------------------------------------------------------------ left: windowed attention with a sink
def query_temperature(positions, q_temp):
    """1 + coef * ln(floor((p + 1) / every) + 1) per position."""
    if not q_temp:
        return torch.ones(len(positions), dtype=F64)
    p = positions.to(torch.long)
    return 1.0 + float(q_temp["coef"]) * torch.log((torch.div(p + 1, int(q_temp["every"]), rounding_mode="floor") + 1).to(F64))


def distance_slopes(H):
    return torch.tensor([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)], dtype=F64)


def window_visible(T, mask):
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if mask:
        ok = ok & ((i - j) < int(mask["size"]))
    return ok


def softmax_with_sink(scores, ok, sink):
    """Rows of weights exp(s_j) / (exp(sink) + sum over the visible j' of exp(s_j')); the sink has no value."""
    s = scores.masked_fill(~ok, -math.inf)
    m = torch.maximum(s.max(-1, keepdim=True).values, torch.as_tensor(sink, dtype=F64))
    e = torch.exp(s - m)
    return e / (e.sum(-1, keepdim=True) + torch.exp(sink - m))


def left_mixer(h, w, pre, m, positions, eps):
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = over_rms(h @ w[pre + "q"].T, eps) * w[pre + "q.norm"]          # over the whole projection, before the heads
    k = over_rms(h @ w[pre + "k"].T, eps) * w[pre + "k.norm"]
    v = (h @ w[pre + "v"].T).view(T, G, dv)
    q = (q * query_temperature(positions, m.get("q_temp"))[:, None]).view(T, H, d)
    k = k.view(T, G, d)
    ok = window_visible(T, m.get("mask"))
    dist = (positions[:, None] - positions[None, :]).to(F64)
    slopes = distance_slopes(H)
    out = torch.zeros(T, H, dv, dtype=F64)
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * float(m["scale"]) - slopes[hd] * dist
        out[:, hd] = softmax_with_sink(s, ok, w[pre + "sink"][hd]) @ v[:, g]
    return out.reshape(T, H * dv) @ w[pre + "o"].T


# ------------------------------------------------------------------------------------------ right: gated delta rule
def causal_conv(x, taps):
    """x [T, C], taps [C, L] (last column on the current token), zeros before the start."""
    T, C = x.shape
    L = taps.shape[1]
    padded = torch.cat([torch.zeros(L - 1, C, dtype=x.dtype), x])
    y = torch.zeros_like(x)
    for j in range(L):
        y = y + padded[j:j + T] * taps[:, j]
    return y


def unit(x):
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + 1e-6)


def delta_rule(q, k, v, beta, g):
    """q, k [T, Hr, dr], v [T, Hr, dvr], beta, g [T, Hr] -> o [T, Hr, dvr].  Per head, token by token:
    S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q."""
    T, Hr, dr = q.shape
    dvr = v.shape[-1]
    S = torch.zeros(Hr, dr, dvr, dtype=F64)
    o = torch.zeros(T, Hr, dvr, dtype=F64)
    for t in range(T):
        S = S * g[t][:, None, None]
        u = beta[t][:, None] * (v[t] - torch.einsum("hkv,hk->hv", S, k[t]))
        S = S + torch.einsum("hk,hv->hkv", k[t], u)
        o[t] = torch.einsum("hkv,hk->hv", S, q[t])
    return o


def right_mixer(h, w, pre, m, eps):
    T = h.shape[0]
    Hr, Gr, dr, dvr = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(h @ w[pre + "q"].T, w[pre + "q.conv"])).view(T, Gr, dr)
    k = silu(causal_conv(h @ w[pre + "k"].T, w[pre + "k.conv"])).view(T, Gr, dr)
    v = silu(causal_conv(h @ w[pre + "v"].T, w[pre + "v.conv"])).view(T, Hr, dvr)
    q = unit(q) * dr ** -0.5
    k = unit(k)
    rep = Hr // Gr
    q, k = q.repeat_interleave(rep, dim=1), k.repeat_interleave(rep, dim=1)      # head h uses q/k head h // rep
    beta = torch.sigmoid(h @ w[pre + "b"].T)
    g = torch.exp(-torch.exp(w[pre + "A_log"]) * torch.nn.functional.softplus(h @ w[pre + "a"].T + w[pre + "dt_bias"]))
    o = delta_rule(q, k, v, beta, g)
    o = over_rms(o, eps) * w[pre + "norm"] * silu(h @ w[pre + "g"].T).view(T, Hr, dvr)
    return o.reshape(T, Hr * dvr) @ w[pre + "o"].T


def parallel_mixer(h, w, pre, m, positions, eps):
    """Half the sum of the two mixers' outputs, each over its root mean square across the width times its weight."""
    left = left_mixer(h, w, pre + "left.", m["left"], positions, eps)
    right = right_mixer(h, w, pre + "right.", m["right"], eps)
    return 0.5 * (over_rms(left, eps) * w[pre + "left.out"] + over_rms(right, eps) * w[pre + "right.out"])


# ------------------------------------------------------------------------------------------ feed-forward
def dense_ff(h, w, pre):
    z = torch.relu(h @ w[pre + "up"].T + w[pre + "up.b"])
    return (z * z) @ w[pre + "down"].T + w[pre + "down.b"]


def expert(h, w, pre, limit):
    g = torch.clamp(h @ w[pre + "gate"].T, max=limit)
    u = torch.clamp(h @ w[pre + "up"].T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[pre + "down"].T


def route(z, correction, router):
    """z [T, E] router logits -> weights [T, E], zero where an expert is not chosen."""
    T, E = z.shape
    top = int(router["top"])
    s = torch.sigmoid(z)
    choice = s + correction
    groups = router.get("groups")
    if groups:
        n, keep = int(groups["count"]), int(groups["keep"])
        per = E // n
        grouped = choice.view(T, n, per)
        score = grouped.topk(min(2, per), dim=-1).values.sum(-1)            # a group's two largest choice scores
        best = score.topk(keep, dim=-1).indices
        allowed = torch.zeros(T, n, dtype=torch.bool)
        allowed.scatter_(1, best, True)
        choice = choice.masked_fill(~allowed[:, :, None].expand(T, n, per).reshape(T, E), -math.inf)
    chosen = choice.topk(top, dim=-1).indices
    picked = torch.gather(s, 1, chosen)
    weights = torch.zeros(T, E, dtype=F64)
    weights.scatter_(1, chosen, picked / (picked.sum(-1, keepdim=True) + 1e-20))
    return weights


def moe_ff(h, w, pre, mlp):
    router = mlp["router"]
    E = int(router["experts"])
    weights = route(h @ w[pre + "router"].T, w[pre + "correction"], router)
    y = torch.zeros(h.shape[0], w[pre + "e0.down"].shape[0], dtype=F64)
    for e in range(E):
        y = y + weights[:, e:e + 1] * expert(h, w, f"{pre}e{e}.", float(mlp["expert"]["limit"]))
    shared = mlp.get("shared")
    if shared:
        y = y + torch.sigmoid(h @ w[pre + "shared.sg"].T) * expert(h, w, pre + "shared.", float(shared["limit"]))
    return y


def feed_forward(h, w, pre, mlp):
    return dense_ff(h, w, pre) if mlp.get("kind", "dense") == "dense" else moe_ff(h, w, pre, mlp)


# ------------------------------------------------------------------------------------------ the model
def layer_runs(cfg):
    """Indices of the layers in the order they run: layers start .. stop-1 ``times`` times in a row, then the rest."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def forward(cfg, w, tokens, return_stream=False):
    """Logits [T, vocab] of a whole sequence (and the residual stream after every layer run, [runs, T, D])."""
    w = {k: v.to(F64) for k, v in w.items() if v.dtype.is_floating_point}
    T = len(tokens)
    positions = torch.arange(T)
    eps = float(cfg["norm"]["eps"])
    x = embed(cfg, w, tokens)
    stream = []
    for i in layer_runs(cfg):
        layer, pre = cfg["layers"][i], f"l{i}."
        if layer["type"] != "parallel":
            raise ValueError(layer["type"])
        x = x + parallel_mixer(over_rms(x, eps) * w[pre + "norm1"], w, pre + "mix.", layer["mixer"], positions, eps)
        if layer.get("mlp") is not None:
            x = x + feed_forward(over_rms(x, eps) * w[pre + "norm2"], w, pre + "mlp.", layer["mlp"])
        stream.append(x)
    logits = (over_rms(x, eps) * w["final.norm"]) @ w["head"].T
    cap = cfg.get("logit_softcap")
    if cap:
        logits = float(cap) * torch.tanh(logits / float(cap))
    return (logits, torch.stack(stream)) if return_stream else logits
