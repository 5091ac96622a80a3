"""Fuzelorn on the GPU against the plain statement: each mechanism alone (with weights or inputs made so that a fault
shows), then whole models under every way of cutting the work, then generation through the engine's own entry point
and the replay program."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import fuzelorn_models as fm
import plain_fuzelorn as plain
import scenarios
from helpers import make_ctx, make_runner, rel_err
from neurogrid_b200.config import (DistanceBiasSpec, GatedDeltaSpec, MLPSpec, MappedAttentionSpec, MoESpec, SideBySideSpec)
from neurogrid_b200.engine import StepEntry
from neurogrid_b200.parts import PagedView, SlotView, build

pytestmark = pytest.mark.gpu
DEV = "cuda"
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TOL = {torch.float32: 1e-4, torch.bfloat16: 3e-2}
DTYPES = [torch.float32, torch.bfloat16]
F64 = torch.float64


def ops():
    from neurogrid_b200.csrc import ops as o
    return o


def _close(got, want, dtype):
    """float32: within the tolerance everywhere.  bfloat16: rows are judged one by one against the largest logit
    (peaked attention and the layers amplify one another's rounding): nine in ten within twice the tolerance of a
    single part and the median within it."""
    if dtype == torch.float32:
        return rel_err(got, want) < TOL[dtype]
    d = (got.double().cpu() - want.double().cpu()).abs().amax(-1) / want.double().cpu().abs().max()
    return float(torch.quantile(d, 0.9)) < 2 * TOL[dtype] and float(d.median()) < TOL[dtype]


def _x(shape, dtype, seed=1, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (scale * torch.randn(*shape, generator=g)).to(torch.bfloat16).to(dtype).to(DEV)


def _i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


def _pages(n_tokens, ps, n_k, dim, n_v, vdim, dtype, seed=0):
    """Pages in a scrambled order with stale content, and the block table of one request."""
    n_pages = -(-n_tokens // ps) + 3
    g = torch.Generator().manual_seed(seed)
    order = torch.randperm(n_pages, generator=g)[: -(-n_tokens // ps)]
    table = torch.full((1, n_pages), -1, dtype=torch.int32)
    table[0, : len(order)] = order.to(torch.int32)
    kp = (5 * torch.randn(n_pages, n_k, ps, dim, generator=g)).to(dtype).to(DEV)
    vp = (5 * torch.randn(n_pages, n_v, ps, vdim, generator=g)).to(dtype).to(DEV)
    return kp, vp, table.to(DEV)


# ------------------------------------------------------------------------------------------ embedding of token pairs
@pytest.mark.parametrize("dtype", DTYPES)
def test_token_pairs_across_steps_and_slots(dtype):
    """A request's first token takes the last row; the previous token crosses steps through the slot; a slot that
    another request used before starts afresh; products larger than 32 bits."""
    V, H, big = 50000, 40, {"buckets": 97, "mul_prev": 1000003, "mul_cur": 999983}
    table = _x((98, H), dtype, seed=3)
    seqs = {2: [7, 49999, 49998, 3, 3, 12], 0: [5, 5, 40000, 1]}
    state = _i32([11, 22, 33, 44])                            # stale: what other requests left
    fed = {2: 0, 0: 0}
    got = {2: [], 0: []}
    for lens in ([(2, 3), (0, 1)], [(0, 2)], [(2, 1), (0, 1)], [(2, 2)]):
        ctx = make_ctx([n for _, n in lens], [fed[s] for s, _ in lens], [s for s, _ in lens], dtype=dtype)
        toks = sum((seqs[s][fed[s]:fed[s] + n] for s, n in lens), [])
        h = torch.zeros(len(toks), H, device=DEV)
        ops().pair_embed(table, _i32(toks), state, ctx.cu_q, ctx.ctx_before, ctx.slots, ctx.row_entry, h, len(lens), V,
                         big["buckets"], big["mul_prev"], big["mul_cur"], ctx.status)
        at = 0
        for s, n in lens:
            got[s].append(h[at:at + n].clone())
            fed[s] += n
            at += n
        assert int(ctx.status.item()) == 0
    for s, toks in seqs.items():
        want = table.double().cpu()[plain.bigram_rows(toks, big)]
        assert rel_err(torch.cat(got[s]), want) < 1e-6
    assert state.tolist() == [1, 22, 12, 44]


# ------------------------------------------------------------------------------------------ left: preparation
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n_q,n_k,dim,vdim,every", [(4, 2, 16, 24, 5), (3, 1, 10, 6, 1), (2, 2, 64, 64, 64), (6, 3, 40, 8, 1000)])
def test_norm_over_the_whole_projection_and_query_temperature(dtype, n_q, n_k, dim, vdim, every):
    T, ps, before, coef = 45, 8, 60, 0.7
    qkv = _x((T, (n_q + n_k) * dim + n_k * vdim), dtype, scale=2.0)
    # heads of unequal size: a norm per head would give another result than one over the whole projection
    qkv[:, :dim] *= 4.0
    qkv[:, n_q * dim:n_q * dim + dim] *= 3.0
    qw = (1 + 0.3 * torch.randn(n_q * dim)).to(DEV)
    kw = (1 + 0.3 * torch.randn(n_k * dim)).to(DEV)
    kp, vp, table = _pages(before + T, ps, n_k, dim, n_k, vdim, dtype)
    ctx = make_ctx([T], [before], [0], dtype=dtype)
    q = torch.empty(T, n_q * dim, dtype=dtype, device=DEV)
    ops().qkv_prep(qkv, q, qw, kw, None, kp, vp, table, ctx.positions, ctx.row_entry, n_q, n_k, n_k, dim, vdim, 1e-5, ctx.status,
                   whole=True, q_temp_coef=coef, q_temp_every=every)
    x = qkv.double().cpu()
    pos = torch.arange(before, before + T)
    temp = plain.query_temperature(pos, {"coef": coef, "every": every})
    assert every > before + T or float(temp.max()) > float(temp.min())
    qd = plain.over_rms(x[:, : n_q * dim], 1e-5) * qw.double().cpu() * temp[:, None]
    kd = plain.over_rms(x[:, n_q * dim:(n_q + n_k) * dim], 1e-5) * kw.double().cpu()
    assert rel_err(q, qd) < TOL[dtype]
    per_head = plain.over_rms(x[:, : n_q * dim].view(T, n_q, dim), 1e-5).reshape(T, -1) * qw.double().cpu() * temp[:, None]
    assert rel_err(per_head, qd) > 0.1
    pg = table[0, (pos // ps).to(DEV)].long()
    assert rel_err(kp[pg, :, (pos % ps).to(DEV)].reshape(T, -1), kd) < TOL[dtype]
    assert torch.equal(vp[pg, :, (pos % ps).to(DEV)].reshape(T, -1), qkv[:, (n_q + n_k) * dim:])
    assert int(ctx.status.item()) == 0


# ------------------------------------------------------------------------------------------ left: the attention core
def _attention_case(dtype, T, H, G, dim, vdim, targets, seed=0):
    """q, k, v in which the keys at ``targets`` stand out for every query that sees them: all queries share a
    direction u and the target keys point along it, so one score towers over the rest where the mask lets it."""
    g = torch.Generator().manual_seed(seed)
    u = torch.randn(dim, generator=g)
    u = u / u.norm()
    q = 0.3 * torch.randn(T, H, dim, generator=g) + 3.0 * u
    k = 0.5 * torch.randn(T, G, dim, generator=g)
    v = torch.randn(T, G, vdim, generator=g)
    for j in targets:
        k[j] += 4.0 * u
        v[j] += 6.0
    r = lambda t: t.to(torch.bfloat16).to(dtype)
    return r(q), r(k), r(v)


def _plain_core(q, k, v, window, scale, sinks, slopes=True):
    T, H, _ = q.shape
    G = k.shape[1]
    ok = plain.window_visible(T, {"size": window} if window else None)
    dist = (torch.arange(T)[:, None] - torch.arange(T)[None, :]).to(F64)
    sl = plain.distance_slopes(H) if slopes else torch.zeros(H, dtype=F64)
    out = torch.zeros(T, H, v.shape[2], dtype=F64)
    for h in range(H):
        s = (q[:, h] @ k[:, h // (H // G)].T) * scale - sl[h] * dist
        out[:, h] = plain.softmax_with_sink(s, ok, sinks[h]) @ v[:, h // (H // G)]
    return out.reshape(T, -1)


def _run_core(dtype, q, k, v, window, ps, scale, sinks, cuts, kind="rows", n_splits=1):
    T, H, dim = q.shape
    G, vdim = v.shape[1], v.shape[2]
    o = ops()
    kp, vp, table = _pages(T, ps, G, dim, G, vdim, dtype, seed=3)
    slopes = build("position", DistanceBiasSpec(H), device=DEV).kernel_args().score_slopes
    sk = sinks.float().to(DEV)
    got = []
    for at, n in cuts:
        ctx = make_ctx([n], [at], [0], dtype=dtype)
        qkv = torch.cat([q[at:at + n].reshape(n, -1), k[at:at + n].reshape(n, -1), v[at:at + n].reshape(n, -1)], 1).contiguous().to(DEV)
        qo = torch.empty(n, H * dim, dtype=dtype, device=DEV)
        o.qkv_prep(qkv, qo, None, None, None, kp, vp, table, ctx.positions, ctx.row_entry, H, G, G, dim, vdim, 1e-5, ctx.status)
        out = torch.full((n, H * vdim + 16), 9.0, dtype=dtype, device=DEV)
        block = out[:, 8:8 + H * vdim]
        if kind == "mma" and n > 1:
            o.mapped_attention_mma(qo, kp, vp, table, ctx.cu_q, ctx.ctx_before, block, 1, n, H, 1, window, 0, scale, 0.0, 0.0,
                                   False, 1.0, 1e-5, slopes=slopes, sinks=sk)
        elif kind == "mma":
            partial = torch.full((H * n_splits * (vdim + 2),), float("nan"), device=DEV)
            o.mapped_attention_group(qo, kp, vp, table, ctx.cu_q, ctx.ctx_before, ctx.row_entry, block, partial, 1, H, 1, window,
                                     0, scale, 0.0, 0.0, False, 1.0, 1e-5, n_splits, slopes=slopes, sinks=sk)
        else:
            s = n_splits if n == 1 else 1
            partial = torch.empty(max(1, o.mapped_attention_partial_floats(n, H, 1, vdim, s)), device=DEV) if s > 1 else None
            o.mapped_attention(qo, kp, vp, table, ctx.positions, ctx.row_entry, block, H, 1, window, 0, scale, 0.0, 0.0, False,
                               1.0, 1e-5, s, partial, slopes=slopes, sinks=sk)
        assert bool((out[:, :8] == 9).all()) and bool((out[:, 8 + H * vdim:] == 9).all())
        got.append(block.float().clone())
    return torch.cat(got)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,dim,vdim,window", [
    (4, 2, 16, 24, 37), (3, 1, 24, 8, 20), (2, 2, 32, 80, 44), (2, 1, 10, 5, 9), (1, 1, 64, 64, None), (6, 3, 64, 32, 80),
    (8, 1, 48, 16, 64), (2, 1, 12, 200, 1)])
def test_windowed_attention_with_sink_and_distance_bias(dtype, H, G, dim, vdim, window):
    """Keys that stand out just inside and just outside the window, at page borders and far back; sinks that weigh as
    much as the keys; as a whole prompt, in portions cut across those edges, and token by token with the keys cut into
    runs; the row-by-row kernel and, where it takes the sizes, the tensor-core kernels."""
    T, ps, scale = 300, 8, 0.4
    w = window or T
    targets = sorted({0, 7, 8, 63, 64, 100, 100 + w - 1, 180, T - w, T - 2} & set(range(T)))
    q, k, v = _attention_case(dtype, T, H, G, dim, vdim, targets)
    sinks = torch.linspace(-1.0, 5.0, H, dtype=F64) if H > 1 else torch.tensor([4.0], dtype=F64)
    qd, kd, vd = q.double(), k.double(), v.double()
    want = _plain_core(qd, kd, vd, window, scale, sinks)
    # the standout keys make a window that is one token off a gross error; so is a sink left out or a bias of slope * j
    if window and window > 1:
        assert rel_err(_plain_core(qd, kd, vd, window + 1, scale, sinks), want) > 0.05
        assert rel_err(_plain_core(qd, kd, vd, window - 1, scale, sinks), want) > 0.05
    assert rel_err(_plain_core(qd, kd, vd, window, scale, sinks - 30.0), want) > 0.02
    if w > 4:
        assert rel_err(_plain_core(qd, kd, vd, window, scale, sinks, slopes=False), want) > 1e-3
    tol = TOL[dtype] if dtype == torch.float32 else 2e-2
    whole = _run_core(dtype, q, k, v, window, ps, scale, sinks, [(0, T)])
    assert rel_err(whole, want) < tol
    cuts, at = [], 0
    for n in [2, 5, 1, 56, 2, 40, 3, 33, 64, 2, 92]:
        cuts.append((at, min(n, T - at)))
        at += cuts[-1][1]
    assert at == T
    assert rel_err(_run_core(dtype, q, k, v, window, ps, scale, sinks, cuts), want) < tol
    single = [(0, T - 110)] + [(i, 1) for i in range(T - 110, T)]
    got = _run_core(dtype, q, k, v, window, ps, scale, sinks, single, n_splits=3)
    assert rel_err(got, want) < tol
    if dtype == torch.float32:                                # runs and cuts change the order of the sums only
        assert rel_err(got, whole) < 1e-5
    elif ops().mapped_attention_group_takes(dim, vdim, H, G, dtype):
        for c, s in (([(0, T)], 1), (cuts, 2), ([(0, T - 40)] + [(i, 1) for i in range(T - 40, T)], 3)):
            got = _run_core(dtype, q, k, v, window, ps, scale, sinks, c, kind="mma", n_splits=s)
            assert rel_err(got, want) < tol
            assert rel_err(got, whole) < 1.5e-2


def test_first_tokens_see_the_sink_only_beside_themselves():
    """The first tokens of a sequence, one by one and as a portion: with a large sink the output is nearly nothing,
    with a very negative one the token's own value."""
    dtype, H, G, dim, vdim = torch.float32, 2, 1, 8, 6
    q, k, v = _attention_case(dtype, 5, H, G, dim, vdim, [])
    for sink, cuts in ((20.0, [(0, 5)]), (20.0, [(i, 1) for i in range(5)]), (-40.0, [(0, 1), (1, 4)])):
        sinks = torch.tensor([sink, sink], dtype=F64)
        got = _run_core(dtype, q, k, v, 3, 8, 0.4, sinks, cuts)
        want = _plain_core(q.double(), k.double(), v.double(), 3, 0.4, sinks)
        assert (got.double().cpu() - want).abs().max() < 1e-5
        if sink > 0:
            assert got.abs().max() < 1e-3
        else:
            assert rel_err(got[0].view(H, vdim), v[0, 0].expand(H, vdim)) < 1e-5


# ------------------------------------------------------------------------------------------ right: the gated delta rule
def _draw(part, seed, gains=None):
    """bfloat16 weights for a part alone, and the same as float64 under the prefix "m."."""
    g = torch.Generator().manual_seed(seed)
    w = {}
    for name, d in part.tensors().items():
        leaf = name.split(".")[-1]
        if leaf in ("norm", "out"):
            t = 1 + 0.2 * torch.randn(d.shape, generator=g)
        elif leaf == "A_log":
            t = torch.linspace(-6.0, 0.5, d.shape[0])          # from nearly no decay to a forgetful head
        elif leaf == "conv":
            t = 0.6 * torch.randn(d.shape, generator=g)
        elif len(d.shape) == 1:
            t = 0.5 * torch.randn(d.shape, generator=g)
        else:
            t = (gains or {}).get(leaf, 1.5) * torch.randn(d.shape, generator=g) / d.shape[-1] ** 0.5
        w[name] = t.to(torch.bfloat16)
    part.bind(w)
    return {"m." + k: v.double() for k, v in w.items()}


def _gd_state(part, n_slots, seed=0):
    """Slots full of stale numbers: a request that starts must not read them."""
    g = torch.Generator().manual_seed(seed)
    return tuple(SlotView((7 * torch.randn(n_slots, *need.shape, generator=g)).to(DEV)) for need in part.cache_need())


def _run_gd(part, x, cuts, dtype, views, slot=0):
    got = []
    for at, n in cuts:
        ctx = make_ctx([n], [at], [slot], dtype=dtype)
        y = part.forward(x[at:at + n].contiguous(), ctx, views)
        got.append((y.sum(0) if y.dim() == 3 else y).float().clone())
    return torch.cat(got)


GD_SIZES = [(4, 2, 8, 12, 3), (2, 1, 24, 20, 4), (1, 1, 8, 8, 1), (2, 2, 5, 7, 2), (4, 1, 72, 36, 3), (2, 2, 128, 64, 4),
            (3, 3, 40, 130, 8), (2, 1, 200, 16, 2)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("Hr,Gr,dk,dv,taps", GD_SIZES)
def test_gated_delta_rule_whole_cut_and_token_by_token(dtype, Hr, Gr, dk, dv, taps):
    D, T = 48, 150
    part = build("mixer", GatedDeltaSpec(hidden=D, n_heads=Hr, n_qk_heads=Gr, key_dim=dk, value_dim=dv, taps=taps, eps=1e-5),
                 dtype=dtype, device=DEV)
    w = _draw(part, 3)
    x = _x((T, D), dtype)
    m = {"heads": Hr, "kv_heads": Gr, "dim": dk, "vdim": dv, "conv": taps}
    want = plain.right_mixer(x.double().cpu(), w, "m.", m, 1e-5)
    # the state carries the first token to the last one: a state lost at a cut shows
    x0 = x.double().cpu().clone()
    x0[0] = -x0[0]
    assert rel_err(plain.right_mixer(x0, w, "m.", m, 1e-5)[-1], want[-1]) > 1e-3
    tol = TOL[dtype]
    views = _gd_state(part, 3)
    whole = _run_gd(part, x, [(0, T)], dtype, views, slot=1)
    assert rel_err(whole, want) < tol
    cuts, at = [], 0
    for n in [2, 1, 3, 2, 17, 2, 5, 31, 2, 64, 21]:
        cuts.append((at, n))
        at += n
    assert at == T
    got = _run_gd(part, x, cuts, dtype, views, slot=1)          # the slot is used again: its state starts afresh
    assert rel_err(got, want) < tol
    single = [(0, T - 60)] + [(i, 1) for i in range(T - 60, T)]
    got1 = _run_gd(part, x, single, dtype, views, slot=2)
    assert rel_err(got1, want) < tol
    if dtype == torch.float32:
        assert rel_err(got, whole) < 1e-5 and rel_err(got1, whole) < 1e-5


@pytest.mark.parametrize("dtype", DTYPES)
def test_gated_delta_rule_batch_of_unequal_entries(dtype):
    """Portions and single tokens of four requests in one launch, each in a slot of its own, against each alone."""
    D, Hr, Gr, dk, dv, taps = 40, 4, 2, 24, 20, 4
    part = build("mixer", GatedDeltaSpec(hidden=D, n_heads=Hr, n_qk_heads=Gr, key_dim=dk, value_dim=dv, taps=taps, eps=1e-6),
                 dtype=dtype, device=DEV)
    w = _draw(part, 5)
    lens = [70, 3, 41, 19]
    xs = [_x((n, D), dtype, seed=10 + i) for i, n in enumerate(lens)]
    m = {"heads": Hr, "kv_heads": Gr, "dim": dk, "vdim": dv, "conv": taps}
    want = [plain.right_mixer(x.double().cpu(), w, "m.", m, 1e-6) for x in xs]
    views = _gd_state(part, 4)
    slots = [3, 0, 2, 1]
    fed = [0] * 4
    got = [[] for _ in lens]
    for step in ([40, 2, 1, 17], [1, 1, 38, 1], [29, 0, 2, 1]):
        live = [i for i, n in enumerate(step) if n]
        ctx = make_ctx([step[i] for i in live], [fed[i] for i in live], [slots[i] for i in live], dtype=dtype)
        x = torch.cat([xs[i][fed[i]:fed[i] + step[i]] for i in live]).contiguous()
        y = part.forward(x, ctx, views)
        y = (y.sum(0) if y.dim() == 3 else y).float()
        at = 0
        for i in live:
            got[i].append(y[at:at + step[i]].clone())
            at += step[i]
            fed[i] += step[i]
    assert fed == lens
    for i in range(4):
        assert rel_err(torch.cat(got[i]), want[i]) < TOL[dtype], i


def _gd_op(o, p, w, state, conv_state, lens, before, slots, nH, nG, dk, dv, chunked):
    """The launcher alone on float32 rows: outputs, with the states updated in place."""
    n, C = p.shape[0], 2 * nG * dk + nH * dv
    cu = [0]
    for q in lens:
        cu.append(cu[-1] + q)
    re = [e for e, q in enumerate(lens) for _ in range(q)]
    conv = torch.empty(n, C, device=DEV)
    raw = torch.empty(n, nH * dv, device=DEV)
    out = torch.empty(n, nH * dv, device=DEV)
    scratch = None
    if chunked:
        scratch = torch.full((o.gated_delta_chunked_scratch(n, len(lens), nH, dk, dv),), float("nan"), device=DEV)
    o.gated_delta(p, w["conv"], w["a_log"], w["dt_bias"], w["norm"], conv_state, state, conv, raw, out, _i32(cu), _i32(before),
                  _i32(slots), _i32(re), len(lens), max(lens), nH, nG, dk, dv, 1e-5, chunk_scratch=scratch)
    return out


@pytest.mark.parametrize("nH,nG,dk,dv,taps", [(4, 2, 64, 32, 3), (2, 1, 128, 128, 4), (2, 2, 256, 48, 2), (3, 1, 20, 16, 4),
                                              (8, 4, 128, 64, 4)])
def test_gated_delta_rule_chunk_by_chunk_equals_token_by_token(nH, nG, dk, dv, taps):
    """The regrouped recurrence against the token-by-token one, both float32, over entries whose lengths fall on, just
    under and just over a chunk's edge, beside single tokens; requests that go on start from states of size, not zero;
    a second step goes on from the states the first one left.  Heads from nearly no decay to forgetful ones."""
    o = ops()
    assert o.gated_delta_chunked_takes(dk, dv) and not o.gated_delta_chunked_takes(dk + 1, dv)
    g = torch.Generator().manual_seed(dk + dv)
    C = 2 * nG * dk + nH * dv
    w = {"conv": (0.6 * torch.randn(C, taps, generator=g)).to(DEV), "a_log": torch.linspace(-6.0, 0.5, nH).to(DEV),
         "dt_bias": (0.5 * torch.randn(nH, generator=g)).to(DEV), "norm": (1 + 0.2 * torch.randn(dv, generator=g)).to(DEV)}
    states = (0.3 * torch.randn(6, nH, dk, dv, generator=g)).to(DEV)
    convs = torch.randn(6, taps - 1, C, generator=g).to(DEV)
    steps = [([130, 1, 64, 33, 7, 95], [0, 12, 5, 0, 3, 40], [4, 1, 0, 5, 2, 3]), ([63, 32, 1, 65, 31, 2], [130, 13, 69, 33, 10, 135], [4, 1, 0, 5, 2, 3])]
    got = {}
    for chunked in (False, True):
        st, cs, outs = states.clone(), convs.clone(), []
        for i, (lens, before, slots) in enumerate(steps):
            gp = torch.Generator().manual_seed(100 + i)
            p = (1.5 * torch.randn(sum(lens), C + nH * dv + 2 * nH, generator=gp)).to(DEV)
            outs.append(_gd_op(o, p, w, st, cs, lens, before, slots, nH, nG, dk, dv, chunked))
        got[chunked] = (torch.cat(outs), st, cs)
    assert torch.isfinite(got[True][0]).all()
    assert rel_err(got[True][0], got[False][0]) < 2e-5
    assert rel_err(got[True][1], got[False][1]) < 2e-5
    assert torch.equal(got[True][2], got[False][2])


def test_gated_delta_rule_long_portions_in_chunks():
    """A bfloat16 part over portions long enough for the chunk-by-chunk kernels, short ones between them, against the
    plain statement: the state passes from one kind of kernel to the other at every cut."""
    D, T, Hr, Gr, dk, dv, taps = 48, 420, 4, 2, 64, 32, 4
    part = build("mixer", GatedDeltaSpec(hidden=D, n_heads=Hr, n_qk_heads=Gr, key_dim=dk, value_dim=dv, taps=taps, eps=1e-5),
                 dtype=torch.bfloat16, device=DEV)
    w = _draw(part, 9)
    x = _x((T, D), torch.bfloat16)
    m = {"heads": Hr, "kv_heads": Gr, "dim": dk, "vdim": dv, "conv": taps}
    want = plain.right_mixer(x.double().cpu(), w, "m.", m, 1e-5)
    views = _gd_state(part, 3)
    cuts, at = [], 0
    for n in [97, 2, 64, 33, 129, 1, 94]:
        cuts.append((at, n))
        at += n
    assert at == T
    assert rel_err(_run_gd(part, x, cuts, torch.bfloat16, views, slot=2), want) < TOL[torch.bfloat16]
    assert rel_err(_run_gd(part, x, [(0, T)], torch.bfloat16, views, slot=2), want) < TOL[torch.bfloat16]


# ------------------------------------------------------------------------------------------ the two mixers side by side
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("accumulate", [False, True])
@pytest.mark.parametrize("H", [300, 2048, 2500])
def test_mean_of_two_normed_inputs(dtype, accumulate, H):
    n = 9
    a, b = _x((n, H), dtype, seed=1, scale=5.0), torch.randn(3, n, H, device=DEV)           # b: a stack of partial sums
    wa, wb = (1 + 0.3 * torch.randn(H)).to(DEV), (1 + 0.3 * torch.randn(H)).to(DEV)
    out = torch.randn(n, H, device=DEV)
    before = out.double().cpu()
    ops().pair_norm_mean(a, b, wa, wb, out, 1e-5, dtype, accumulate=accumulate)
    want = 0.5 * (plain.over_rms(a.double().cpu(), 1e-5) * wa.double().cpu()
                  + plain.over_rms(b.double().cpu().sum(0), 1e-5) * wb.double().cpu())
    # a stack's sum is rounded to the activation type, as the unsplit product would have been stored
    assert rel_err(out, want + before if accumulate else want) < (1e-5 if dtype == torch.float32 else 5e-3)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("layer", [("S", 0), ("S", 1), ("S", 3), ("U", 0), ("U", 1), ("W", 0), ("W", 1)])
def test_side_by_side_mixer_alone(dtype, layer):
    from neurogrid_b200.config import config_from_dict
    name, i = layer
    cfg = fm.CONFIGS[name][0]
    eps = cfg["norm"]["eps"]
    spec = config_from_dict(cfg)._mixer_spec(cfg["layers"][i])
    assert isinstance(spec, SideBySideSpec) and isinstance(spec.left, MappedAttentionSpec)
    part = build("mixer", spec, dtype=dtype, device=DEV)
    w = _draw(part, 7, gains={"q": 2.5, "k": 2.5})
    D, T, ps = cfg["width"], 130, 8
    x = _x((T, D), dtype)
    mix = cfg["layers"][i]["mixer"]
    want = plain.parallel_mixer(x.double().cpu(), w, "m.", mix, torch.arange(T), eps)
    l = mix["left"]
    for cuts in ([(0, T)], [(0, 2), (2, 61), (63, 3), (66, 1), (67, 63)], [(0, 100)] + [(i, 1) for i in range(100, T)]):
        kp, vp, table = _pages(T, ps, l["kv_heads"], l["dim"], l["kv_heads"], l["vdim"], dtype, seed=len(cuts))
        views = (PagedView(kp, vp, table),) + _gd_state(part.right, 2)
        got = []
        for at, n in cuts:
            ctx = make_ctx([n], [at], [1], dtype=dtype)
            y = part.forward(x[at:at + n].contiguous(), ctx, views)
            got.append((y.sum(0) if y.dim() == 3 else y).float().clone())
            assert int(ctx.status.item()) == 0
        assert rel_err(torch.cat(got), want) < TOL[dtype]


# ------------------------------------------------------------------------------------------ feed-forwards
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n", [3, 70, 300])
def test_feed_forward_with_squared_relu_and_biases(dtype, n):
    H, I = 72, 88
    part = build("ffn", MLPSpec(H, I), dtype=dtype, device=DEV)
    g = torch.Generator().manual_seed(n)
    w = {k: ((1.5 * torch.randn(d.shape, generator=g) / d.shape[-1] ** 0.5) if len(d.shape) == 2
             else 0.8 * torch.randn(d.shape, generator=g)).to(torch.bfloat16) for k, d in part.tensors().items()}
    assert set(w) == {"up", "up.b", "down", "down.b"}
    part.bind(w)
    x = _x((n, H), dtype)
    ctx = make_ctx([n], [0], [0], dtype=dtype)
    y = part.forward(x, ctx)
    want = plain.dense_ff(x.double().cpu(), {"m." + k: v.double() for k, v in w.items()}, "m.")
    assert rel_err(y.sum(0) if y.dim() == 3 else y, want) < TOL[dtype]


@pytest.mark.parametrize("n,H,I", [(1, 64, 96), (8, 72, 200), (33, 128, 136), (64, 256, 320)])
def test_squared_relu_in_the_product_equals_a_pass_over_it(n, H, I):
    """Few rows: the tensor-core product squares what is positive of its rounded result in the epilogue; the same bits
    as the product followed by the elementwise kernel, with and without a bias, beside the plain statement."""
    o = ops()
    g = torch.Generator().manual_seed(n + I)
    x = torch.randn(n, H, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(I, H, generator=g) / H ** 0.5).to(torch.bfloat16).to(DEV)
    for bias in (None, (0.5 * torch.randn(I, generator=g)).to(torch.bfloat16).to(DEV)):
        assert o.gemm_sm100_ok(x, w)
        fused = torch.full((n, I), 7.0, dtype=torch.bfloat16, device=DEV)
        o.linear_relu_squared(x, w, bias, fused)
        apart = torch.empty_like(fused)
        o.linear(x, w, bias, apart)
        o.relu_squared_(apart)
        assert torch.equal(fused, apart)
        y = x.double() @ w.double().t() + (0 if bias is None else bias.double())
        assert rel_err(fused, torch.relu(y) ** 2) < TOL[torch.bfloat16]
        assert (fused >= 0).all() and (fused == 0).any() and (fused > 0).any()


def _route_on_gpu(z, corr, router):
    """The router kernel on logits given outright: the router's matrix is the identity."""
    E = z.shape[1]
    groups = router.get("groups") or {"count": 1, "keep": 1}
    weights = torch.full((z.shape[0], E), 7.0, device=DEV)
    ops().moe_router_sigmoid(z.float().to(DEV), torch.eye(E, device=DEV), corr.float().to(DEV), None, weights, router["top"],
                             groups["count"], groups["keep"])
    return weights.double().cpu()


def test_router_choice_by_corrected_scores_within_the_best_groups():
    z = torch.tensor([[2.0, 1.9, -9.0, -9.0, 0.1, 0.0]], dtype=F64)
    corr = torch.tensor([0.0, 0.0, -0.9, -0.9, 0.5, 0.6], dtype=F64)
    cases = [(z, corr, {"experts": 6, "top": 3, "groups": {"count": 3, "keep": 2}}, [0, 4, 5]),
             (z, corr, {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 1}}, [4, 5]),
             (z, corr, {"experts": 6, "top": 1, "groups": {"count": 6, "keep": 1}}, [5]),
             (z, corr, {"experts": 6, "top": 2}, [4, 5]),
             # every choice score of the best group is negative: an excluded expert's score counts as minus infinity, not 0
             (torch.tensor([[-3.0, -2.0, 5.0, 5.0]], dtype=F64), torch.tensor([0.0, 0.0, -2.0, -2.0], dtype=F64),
              {"experts": 4, "top": 2, "groups": {"count": 2, "keep": 1}}, [0, 1]),
             (torch.tensor([[-4.0, -5.0, -6.0, 3.0]], dtype=F64), torch.tensor([-2.0, -2.0, -2.0, -9.0], dtype=F64),
              {"experts": 4, "top": 2, "groups": {"count": 2, "keep": 1}}, [0, 1])]
    for zz, cc, router, chosen in cases:
        want = plain.route(zz, cc, router)
        assert (want[0] > 0).nonzero().flatten().tolist() == chosen
        got = _route_on_gpu(zz, cc, router)
        assert (got - want).abs().max() < 1e-6, (router, got, want)
    # many tokens, random logits and corrections, every grouping of 12 experts
    g = torch.Generator().manual_seed(4)
    zz, cc = 2.0 * torch.randn(500, 12, generator=g, dtype=F64).float().double(), torch.randn(12, generator=g, dtype=F64).float().double()
    for count, keep, top in [(1, 1, 12), (2, 1, 6), (3, 2, 5), (4, 2, 1), (6, 3, 4), (12, 5, 5), (12, 12, 3), (4, 4, 7)]:
        router = {"experts": 12, "top": top, "groups": {"count": count, "keep": keep}}
        assert (_route_on_gpu(zz, cc, router) - plain.route(zz, cc, router)).abs().max() < 1e-5, router


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("E,top,ff,limit,groups,shared", [
    (6, 2, 24, 1.5, (3, 2), (32, 0.8)), (2, 1, 12, 1.0, None, None), (3, 3, 8, 0.6, (3, 3), None), (8, 3, 16, 0.9, (2, 1), (16, 2.5)),
    (4, 2, 16, 1.2, (4, 3), (24, 1.0)), (16, 4, 40, 0.5, (4, 2), (8, 0.3))])
def test_routed_experts_with_clamped_activation_and_gated_shared_expert(dtype, E, top, ff, limit, groups, shared):
    H, n = 56, 90
    spec = MoESpec(hidden=H, n_experts=E, top_k=top, expert_ff=ff, shared_ff=shared[0] if shared else 0, scoring="sigmoid",
                   correction=True, n_groups=groups[0] if groups else 1, keep_groups=groups[1] if groups else 1,
                   activation="clamped_glu", limit=limit, shared_limit=shared[1] if shared else 0.0, glu_alpha=1.702,
                   shared_gate=bool(shared))
    part = build("ffn", spec, dtype=dtype, device=DEV)
    g = torch.Generator().manual_seed(E)
    calm = dtype == torch.bfloat16            # routers that hardly look at the token: no close call flips an expert
    w = {}
    for k, d in part.tensors().items():
        if k == "correction":
            t = torch.linspace(-0.5, 0.5, E)[torch.randperm(E, generator=g)]
        elif k == "router":
            t = (0.02 if calm else 3.0) * torch.randn(d.shape, generator=g) / H ** 0.5
        else:
            t = 3.0 * torch.randn(d.shape, generator=g) / d.shape[-1] ** 0.5          # gates and ups beyond the limits
        w[k] = t.to(torch.bfloat16)
    part.bind(w)
    x = _x((n, H), dtype)
    ctx = make_ctx([n], [0], [0], dtype=dtype)
    y = part.forward(x, ctx)
    mlp = {"router": {"experts": E, "top": top}, "expert": {"ff": ff, "limit": limit}}
    if groups:
        mlp["router"]["groups"] = {"count": groups[0], "keep": groups[1]}
    if shared:
        mlp["shared"] = {"ff": shared[0], "limit": shared[1]}
    wd = {"m." + k: v.double() for k, v in w.items()}
    xd = x.double().cpu()
    want = plain.moe_ff(xd, wd, "m.", mlp)
    assert rel_err(y.sum(0) if y.dim() == 3 else y, want) < TOL[dtype]
    other = dict(mlp, expert={"ff": ff, "limit": 10.0})
    assert rel_err(plain.moe_ff(xd, wd, "m.", other), want) > 0.05          # the limit bites with these weights


# ------------------------------------------------------------------------------------------ whole models
LENS = {"S": [1, 9, 40, 131, 64, 23, 77], "U": [3, 50, 97, 30, 64], "W": [2, 17, 150, 33], "V": [200, 2, 100, 70]}


def _dir(dirs, name, dtype):
    return dirs[name if dtype == torch.float32 else name + "_calm"]


def _replay(runner, steps):
    got = []
    for s in steps:
        lg = runner.step([StepEntry(e["id"], e["tokens"], e["want"]) for e in s["entries"]])
        got.append(lg.clone())
        for r in s["end"]:
            runner.finish(r)
    runner.check_status()
    runner.cache.check()
    return scenarios.collect(steps, lambda i: got[i])


@pytest.fixture(scope="module")
def plain_logits(fuzelorn_dirs):
    out = {}
    for name in LENS:
        for key in (name, name + "_calm"):
            cfg, w = fm.load_plain(fuzelorn_dirs[key])
            reqs = scenarios.make_requests(LENS[name], cfg["vocab"], seed=7)
            out[key] = (reqs, {r: plain.forward(cfg, w, t) for r, t in reqs.items()})
    return out


def test_residual_stream_after_every_layer_run(fuzelorn_dirs):
    """float32, layer by layer: the stream after every run of a layer (a looped layer counts each time)."""
    cfg, w = fm.load_plain(fuzelorn_dirs["S"])
    toks = scenarios.make_requests([37], cfg["vocab"], seed=1)["r0"]
    _, stream = plain.forward(cfg, w, toks, return_stream=True)
    runner = make_runner(fuzelorn_dirs["S"], dtype=torch.float32, device="cuda", page_size=8, num_pages=16)
    seen = []
    model = runner.model
    run_entries = model.run_entries

    def spy(ctx, caches, entries, h, pending):
        for e in entries:                                        # one run at a time; the sum not yet added is folded in for the record
            pending = run_entries(ctx, caches, [e], h, pending)
            add = 0 if pending is None else (pending.sum(0) if pending.dim() == 3 else pending).double()
            seen.append((h.double() + add)[: len(toks)].cpu())
        return pending

    model.run_entries = spy
    runner.step([StepEntry("x", toks, [len(toks) - 1])])
    assert len(seen) == stream.shape[0] == 6
    for i, s in enumerate(seen):
        assert rel_err(s, stream[i]) < 1e-4, i


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["S", "U", "W", "V"])
@pytest.mark.parametrize("cut", ["whole", "tail_decode", "portions", "mixed"])
def test_cuts_against_plain(fuzelorn_dirs, plain_logits, name, dtype, cut):
    key = name if dtype == torch.float32 else name + "_calm"
    reqs, want = plain_logits[key]
    ps = fm.PAGE_SIZE[name]
    cap = 256 if cut == "mixed" else 512                     # tokens; mixed: pages and slots are used again
    runner = make_runner(fuzelorn_dirs[key], dtype=dtype, device="cuda", page_size=ps, num_pages=cap // ps,
                         max_requests=4, max_seq_len=cap)
    steps = {"whole": scenarios.whole, "tail_decode": scenarios.tail_decode, "portions": scenarios.portions,
             "mixed": lambda r: scenarios.mixed(r, cap, round_to=ps)}[cut](reqs)
    got = _replay(runner, steps)
    allg, allw = torch.cat([got[r] for r in reqs]), torch.cat([want[r] for r in reqs])
    assert allg.shape == allw.shape
    assert _close(allg, allw, dtype), rel_err(allg, allw)
    if dtype == torch.float32:
        for r in reqs:
            assert rel_err(got[r], want[r]) < TOL[dtype], (r, rel_err(got[r], want[r]))
    assert all(f == cap // ps for f in runner.cache.pages_free()) and runner.cache.slots_free() == 4


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["S", "W"])
def test_first_tokens_and_long_decode(fuzelorn_dirs, name, dtype):
    """The first tokens one by one (windows that reach before the start, an empty state, the pair table's last row), then
    decoding far beyond every window and across many page edges, with graphs replayed and pages given back."""
    folder = _dir(fuzelorn_dirs, name, dtype)
    cfg, w = fm.load_plain(folder)
    toks = scenarios.make_requests([230], cfg["vocab"], seed=11)["r0"]
    want = plain.forward(cfg, w, toks)
    runner = make_runner(folder, dtype=dtype, device="cuda", page_size=8, num_pages=32, max_seq_len=256)
    got = torch.cat([runner.step([StepEntry("x", [t], [0])]).clone() for t in toks])
    runner.check_status()
    assert _close(got, want, dtype), rel_err(got, want)
    if dtype == torch.float32:
        assert rel_err(got[:14], want[:14]) < TOL[dtype]
    assert runner.graph_replays > 100
    assert max(runner.cache.pages_held("x")) <= (11 if name == "W" else 6)      # the pages behind the windows came back


@pytest.mark.parametrize("name", ["S", "W"])
def test_float32_cuts_agree_closely(fuzelorn_dirs, name):
    cfg, _ = fm.load_plain(fuzelorn_dirs[name])
    reqs = scenarios.make_requests([120], cfg["vocab"], seed=3)
    runner = make_runner(fuzelorn_dirs[name], dtype=torch.float32, device="cuda", num_pages=64, page_size=8)
    a = _replay(runner, scenarios.whole(reqs))["r0"]
    b = _replay(runner, scenarios.portions(reqs))["r0"]
    c = _replay(runner, scenarios.tail_decode(reqs))["r0"]
    assert rel_err(a, b) < 2e-5 and rel_err(a, c) < 2e-5


@pytest.mark.parametrize("dtype", DTYPES)
def test_batch_of_unequal_requests_equals_each_alone(fuzelorn_dirs, dtype):
    folder = _dir(fuzelorn_dirs, "S", dtype)
    cfg, _ = fm.load_plain(folder)
    reqs = scenarios.make_requests([5, 70, 2, 33], cfg["vocab"], seed=5)
    runner = make_runner(folder, dtype=dtype, device="cuda", num_pages=64, page_size=8)
    alone = _replay(runner, scenarios.whole(reqs))
    lg = runner.step([StepEntry(r, t, list(range(len(t)))) for r, t in reqs.items()])
    at = 0
    for r, t in reqs.items():
        if dtype == torch.float32:
            assert rel_err(lg[at:at + len(t)], alone[r]) < 2e-5
        else:
            assert _close(lg[at:at + len(t)], alone[r], dtype)
        at += len(t)


def test_greedy_generation_through_the_engine(fuzelorn_dirs):
    """Engine.generate (scheduler, portions, decode graphs, device sampler) against greedy decoding with the oracle."""
    from neurogrid_b200 import Engine
    cfg, w = fm.load_plain(fuzelorn_dirs["W"])
    prompts = list(scenarios.make_requests([12, 30, 5], cfg["vocab"], seed=9).values())
    eng = Engine(fuzelorn_dirs["W"], dtype="float32", max_seq_len=128, page_size=8, max_requests=2,
                 max_tokens_per_step=32, chunk_size=16)
    outs = eng.generate(prompts, max_new_tokens=24, ignore_eos=True)
    for p, o in zip(prompts, outs):
        seq = list(p)
        for tok in o:
            lg = plain.forward(cfg, w, seq)[-1]
            top2 = torch.topk(lg, 2).values
            assert tok == int(torch.argmax(lg)) or float(top2[0] - top2[1]) < 1e-4 * float(lg.abs().max())
            seq.append(tok)
        assert len(o) == 24
    assert eng.stats()["slots_free"] == 2


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_program(fuzelorn_dirs, tmp_path, dtype):
    folder = fuzelorn_dirs["S" if dtype == "float32" else "S_calm"]
    cfg, w = fm.load_plain(folder)
    V = cfg["vocab"]
    reqs = scenarios.make_requests([9, 70, 33, 120, 41], V, seed=5)
    cap = 256
    steps = scenarios.number(scenarios.portions(reqs) + scenarios.mixed(reqs, cap, round_to=64))
    out = tmp_path / "out"
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder,
                           "--dtype", dtype, "--out", str(out), "--max-tokens", str(cap)],
                          input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-3000:]
    got = scenarios.collect(steps, lambda i: torch.from_numpy(np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, V)))
    want = {r: plain.forward(cfg, w, t) for r, t in reqs.items()}
    assert _close(torch.cat([got[r] for r in reqs]), torch.cat([torch.cat([want[r], want[r]]) for r in reqs]),
                  torch.float32 if dtype == "float32" else torch.bfloat16)
