"""Dodilix on the GPU against the plain statement: each mechanism alone (with weights or inputs made so that a fault
shows), then whole models under every way of cutting the work, then generation through the engine's own entry point
and the replay program."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import dodilix_models as dm
import kernel_refs as refs
import plain_dodilix as plain
import scenarios
from helpers import make_ctx, make_runner, rel_err
from neurogrid_b200.engine import StepEntry

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
    """float32: within the tolerance everywhere.  bfloat16: rows are judged one by one against the largest logit: nine
    in ten within twice the tolerance of a single part and the median within it."""
    if dtype == torch.float32:
        return rel_err(got, want) < TOL[dtype]
    d = (got.double().cpu() - want.double().cpu()).abs().amax(-1) / want.double().cpu().abs().max()
    return float(torch.quantile(d, 0.9)) < 2 * TOL[dtype] and float(d.median()) < TOL[dtype]


def _x(shape, dtype, seed=1, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (scale * torch.randn(*shape, generator=g)).to(torch.bfloat16).to(dtype).to(DEV)


def _i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


def _cpu(*ts):
    return [t.detach().cpu().clone() if isinstance(t, torch.Tensor) else t for t in ts]


def _pages(n_tokens, ps, n_k, dim, n_v, vdim, dtype, seed=0):
    """Pages in a scrambled order with stale content, and the block table of one request."""
    n_pages = -(-n_tokens // ps) + 3
    g = torch.Generator().manual_seed(seed)
    order = torch.randperm(n_pages, generator=g)[: -(-n_tokens // ps)]
    table = torch.full((1, n_pages), -1, dtype=torch.int32)
    table[0, : len(order)] = order.to(torch.int32)
    kp = (5 * torch.randn(n_pages, n_k, ps, dim, generator=g)).to(dtype).to(DEV)
    vp = (5 * torch.randn(n_pages, n_v, ps, vdim, generator=g)).to(dtype).to(DEV) if n_v else None
    return kp, vp, table.to(DEV)


# ------------------------------------------------------------------------------------------ the copies of the stream
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("S,H,n", [(1, 40, 5), (3, 56, 9), (4, 2056, 3), (7, 192, 70), (16, 64, 2), (5, 50, 4), (9, 31, 3)])
def test_stream_copies_between_two_sublayers(dtype, S, H, n):
    g = torch.Generator().manual_seed(S)
    x0 = torch.randn(n, H, generator=g).to(DEV)
    mix = (0.5 * torch.eye(S) + 0.3 * torch.randn(S, S, generator=g)).to(DEV)
    ow, iw = torch.randn(S, generator=g).to(DEV), torch.randn(S, generator=g).to(DEV)
    nw = (1 + 0.2 * torch.randn(H, generator=g)).to(DEV)
    deltas = [_x((n, H), dtype, seed=3), torch.randn(3, n, H, generator=g).to(DEV), _x((n, H), dtype, seed=4)]
    X = torch.full((n, S * H), 7.0, device=DEV)                       # stale: what another step left
    Xr = X.cpu().clone()
    out, total = torch.empty(n, H, dtype=dtype, device=DEV), torch.empty(n, H, device=DEV)
    outr, totalr = out.cpu().clone(), total.cpu().clone()
    calls = [dict(x0=x0, in_w=iw, norm_w=nw, out=out, eps=1e-5)]
    calls += [dict(delta=d, mix=mix, out_w=ow, in_w=iw, norm_w=nw, out=out, eps=1e-5) for d in deltas[:2]]
    calls += [dict(delta=deltas[2], mix=mix, out_w=ow, sum_out=total, act_dtype=dtype)]
    for kw in calls:
        ops().hc_step(X, S, **kw)
        kr = {k: (outr if k == "out" else totalr if k == "sum_out" else _cpu(v)[0]) for k, v in kw.items()}
        refs.hc_step(Xr, S, **kr)
        assert rel_err(X, Xr) < 1e-5
        if "out" in kw:
            assert rel_err(out, outr) < TOL[dtype]
    assert rel_err(total, totalr) < 1e-5
    assert rel_err(total, Xr.view(n, S, H).sum(1)) < 1e-5


@pytest.mark.parametrize("dtype", DTYPES)
def test_output_gate_on_a_block_of_columns(dtype):
    n, I = 11, 70
    wide, logits = _x((n, 3 * I + 5), dtype, seed=2), _x((n, 2 * I), dtype, seed=5, scale=2.0)
    for act, scale, gate in (("sigmoid", 0.7, logits[:, I:]), ("silu", 1.2, logits[:, :I]), ("sigmoid", 1.3, None)):
        y = wide.clone()
        want = y.cpu().clone()
        ops().gate_mul(y[:, I:2 * I], gate, act, scale)
        refs.gate_mul(want[:, I:2 * I], gate.cpu() if gate is not None else None, act, scale)
        assert rel_err(y, want) < TOL[dtype] / 3
        assert torch.equal(y[:, :I], wide[:, :I]) and torch.equal(y[:, 2 * I:], wide[:, 2 * I:])


# ------------------------------------------------------------------------------------------ left: preparation
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n_q,n_k,dim,vdim,rot,extra", [(4, 2, 16, 12, 8, 48), (3, 1, 10, 6, 10, 0), (2, 2, 64, 64, 32, 128),
                                                       (6, 3, 40, 8, 0, 7), (8, 2, 128, 64, 32, 512)])
def test_rotation_in_halves_and_norm_without_weights(dtype, n_q, n_k, dim, vdim, rot, extra):
    """Pairs (i, i + rot/2) inside the rotated coordinates, the rest unchanged, each head over its root mean square; the
    columns behind v (the gate's logits) are left alone."""
    T, ps, before = 45, 8, 60
    qkv = _x((T, (n_q + n_k) * dim + n_k * vdim + extra), dtype, scale=2.0)
    inv = (1000.0 ** (-2.0 * torch.arange(rot // 2, dtype=F64) / max(rot, 1))).float().to(DEV) if rot else None
    kp, vp, table = _pages(before + T, ps, n_k, dim, n_k, vdim, dtype)
    ctx = make_ctx([T], [before], [0], dtype=dtype)
    q = torch.empty(T, n_q * dim, dtype=dtype, device=DEV)
    ops().qkv_prep(qkv, q, None, None, inv, kp, vp, table, ctx.positions, ctx.row_entry, n_q, n_k, n_k, dim, vdim, 1e-5,
                   ctx.status, half_pairing=True, unit_norm=True)
    x = qkv.double().cpu()
    pos = torch.arange(before, before + T)
    qd = plain.rms_div(plain.rotate(x[:, : n_q * dim].view(T, n_q, dim), pos, rot, 1000.0, False), 1e-5)
    kd = plain.rms_div(plain.rotate(x[:, n_q * dim:(n_q + n_k) * dim].view(T, n_k, dim), pos, rot, 1000.0, False), 1e-5)
    assert rel_err(q, qd.reshape(T, -1)) < TOL[dtype]
    if rot:                                                         # the other pairing gives something else
        assert rel_err(plain.rms_div(plain.rotate(x[:, : n_q * dim].view(T, n_q, dim), pos, rot, 1000.0, True), 1e-5), qd) > 0.1
    pg = table[0, (pos // ps).to(DEV)].long()
    assert rel_err(kp[pg, :, (pos % ps).to(DEV)].reshape(T, -1), kd.reshape(T, -1)) < TOL[dtype]
    assert torch.equal(vp[pg, :, (pos % ps).to(DEV)].reshape(T, -1), qkv[:, (n_q + n_k) * dim:(n_q + n_k) * dim + n_k * vdim])
    assert int(ctx.status.item()) == 0


# ------------------------------------------------------------------------------------------ left: the chunked mask
def _attention_case(dtype, T, H, G, dim, vdim, targets, seed=0):
    """q, k, v in which the keys at ``targets`` stand out for every query that sees them: all queries share a direction
    u and the target keys point along it, so one score towers over the rest where the mask lets it."""
    g = torch.Generator().manual_seed(seed)
    u = torch.randn(dim, generator=g)
    u = u / u.norm()
    q = 0.3 * torch.randn(T, H, dim, generator=g) + 3.0 * u
    k = 0.3 * torch.randn(T, G, dim, generator=g)
    for t in targets:
        if 0 <= t < T:
            k[t] += 4.0 * u
    v = torch.randn(T, G, vdim, generator=g)
    rnd = lambda t: t.to(torch.bfloat16).to(dtype)
    return rnd(q), rnd(k), rnd(v)


def _fill(kp, vp, table, k, v, ps):
    T = k.shape[0]
    pos = torch.arange(T)
    pg = table[0, (pos // ps).to(DEV)].long()
    kp[pg, :, (pos % ps).to(DEV)] = k.to(DEV)
    vp[pg, :, (pos % ps).to(DEV)] = v.to(DEV)


def _run_attention(kind, q, kp, vp, table, ctx, H, chunk, scale, sinks, n_splits=1):
    n, vdim = q.shape[0], vp.shape[3]
    out = torch.empty(n, H * vdim, dtype=q.dtype, device=DEV)
    if kind == "rows":
        partial = torch.empty(max(1, ops().mapped_attention_partial_floats(n, H, 1, vdim, n_splits)), device=DEV) if n_splits > 1 else None
        ops().mapped_attention(q, kp, vp, table, ctx.positions, ctx.row_entry, out, H, 1, None, 0, scale, 0.0, 0.0, False, 1.0,
                               1e-6, n_splits, partial, sinks=sinks, chunk=chunk)
    elif kind == "tiles":
        ops().mapped_attention_mma(q, kp, vp, table, ctx.cu_q, ctx.ctx_before, out, ctx.n_entries, ctx.max_q, H, 1, None, 0,
                                   scale, 0.0, 0.0, False, 1.0, 1e-6, sinks=sinks, chunk=chunk)
    else:
        partial = torch.empty(n * H * n_splits * (vdim + 2), device=DEV)
        ops().mapped_attention_group(q, kp, vp, table, ctx.cu_q, ctx.ctx_before, ctx.row_entry, out, partial, ctx.n_entries,
                                     H, 1, None, 0, scale, 0.0, 0.0, False, 1.0, 1e-6, n_splits, sinks=sinks, chunk=chunk)
    return out


@pytest.mark.parametrize("kind,dtype", [("rows", torch.float32), ("rows", torch.bfloat16), ("tiles", torch.bfloat16)])
@pytest.mark.parametrize("chunk,ps", [(88, 16), (13, 8), (64, 16), (1, 4), (100, 32), (300, 16)])
def test_chunked_mask_in_prompts(kind, dtype, chunk, ps):
    """Keys that stand out sit on both sides of every chunk's first position: a row must see the one inside its chunk
    and never the one just outside; portions are cut across the chunks' edges and across pages."""
    T, H, G, dim, vdim = 230, 4, 2, 32, 32
    targets = [c * chunk + d for c in range(T // chunk + 1) for d in (-1, 0)] if chunk > 1 else [50, 51]
    q, k, v = _attention_case(dtype, T, H, G, dim, vdim, targets)
    kp, vp, table = _pages(T, ps, G, dim, G, vdim, dtype)
    _fill(kp, vp, table, k, v, ps)
    sinks = torch.linspace(-1.0, 2.0, H).to(DEV)
    want = torch.empty(T, H * vdim, dtype=F64)
    ctx_all = make_ctx([T], [0], [0], dtype=dtype, device="cpu")
    refs.mapped_attention(q.reshape(T, -1), kp.cpu(), vp.cpu(), table.cpu(), ctx_all.positions, ctx_all.row_entry, want, H, 1,
                          None, 0, 0.7, 0.0, 0.0, False, 1.0, 1e-6, sinks=sinks.cpu(), chunk=chunk)
    for cuts in ([T], [chunk - 1 if chunk > 2 else 3, 2, 70, T]):
        at, got = 0, []
        for c in cuts:
            n = min(c, T - at)
            if n <= 0:
                break
            ctx = make_ctx([n], [at], [0], dtype=dtype)
            got.append(_run_attention(kind, q[at:at + n].reshape(n, -1).to(DEV), kp, vp, table, ctx, H, chunk, 0.7, sinks))
            at += n
        assert rel_err(torch.cat(got), want) < TOL[dtype], cuts
    if chunk >= T:
        return
    # the mask matters: with another chunk size the result is another
    other = torch.empty(T, H * vdim, dtype=F64)
    refs.mapped_attention(q.reshape(T, -1), kp.cpu(), vp.cpu(), table.cpu(), ctx_all.positions, ctx_all.row_entry, other, H, 1,
                          None, 0, 0.7, 0.0, 0.0, False, 1.0, 1e-6, sinks=sinks.cpu(), chunk=chunk + 1)
    assert rel_err(other, want) > 0.05


@pytest.mark.parametrize("kind,dtype", [("rows", torch.float32), ("rows", torch.bfloat16), ("group", torch.bfloat16)])
@pytest.mark.parametrize("chunk", [88, 40, 7])
def test_chunked_mask_token_by_token(kind, dtype, chunk):
    """Single tokens of several requests in one launch, at positions around their chunks' edges, keys cut into runs."""
    T, H, G, dim, vdim, ps = 400, 8, 2, 64, 64, 16
    targets = [c * chunk + d for c in range(T // chunk + 1) for d in (-1, 0)]
    q, k, v = _attention_case(dtype, T, H, G, dim, vdim, targets, seed=3)
    kp, vp, table = _pages(T, ps, G, dim, G, vdim, dtype, seed=2)
    _fill(kp, vp, table, k, v, ps)
    sinks = torch.linspace(-2.0, 1.0, H).to(DEV)
    spots = sorted({p for c in range(1, T // chunk) for p in (c * chunk - 1, c * chunk, c * chunk + 1)} | {0, 1, T - 1})[:24]
    tables = table.expand(len(spots), -1).contiguous()
    ctx = make_ctx([1] * len(spots), spots, list(range(len(spots))), dtype=dtype)
    qs = q[spots].reshape(len(spots), -1).to(DEV)
    want = torch.empty(len(spots), H * vdim, dtype=F64)
    refs.mapped_attention(qs.cpu(), kp.cpu(), vp.cpu(), tables.cpu(), ctx.positions.cpu(), ctx.row_entry.cpu(), want, H, 1,
                          None, 0, 0.5, 0.0, 0.0, False, 1.0, 1e-6, sinks=sinks.cpu(), chunk=chunk)
    for n_splits in (1, 3):
        got = _run_attention(kind, qs, kp, vp, tables, ctx, H, chunk, 0.5, sinks, n_splits)
        assert rel_err(got, want) < TOL[dtype], n_splits


# ------------------------------------------------------------------------------------------ right: the recurrence
def _gla_inputs(dtype, T, H, dk, dv, seed=0):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, 2 * H * (dk + dv), generator=g)
    z = 2.0 * torch.randn(T, H * dk, generator=g) + torch.linspace(-6.0, 9.0, H * dk)     # forgetful to nearly no decay
    z[:, 0] = -60.0                                                                        # a channel that forgets at once
    z[:, 1] = 60.0                                                                         # and one that never does
    rnd = lambda t: t.to(torch.bfloat16).to(dtype).to(DEV)
    return rnd(x), rnd(z), (1 + 0.2 * torch.randn(dv, generator=g)).to(DEV)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,dk,dv,tau", [(2, 32, 48, 12.0), (3, 8, 10, 7.0), (1, 128, 64, 1.0), (2, 24, 12, 3.0), (1, 5, 7, 2.0)])
def test_recurrence_whole_cut_and_token_by_token(dtype, H, dk, dv, tau):
    T = 150
    x, z, nw = _gla_inputs(dtype, T, H, dk, dv)
    want, st = torch.empty(T, H * dv, dtype=F64), torch.zeros(4, H, dk, dv, dtype=F64)
    c = make_ctx([T], [0], [2], dtype=dtype, device="cpu")
    refs.gated_linear(x.cpu(), z.cpu(), nw.cpu(), st, want, c.cu_q, c.ctx_before, c.slots, 1, H, dk, dv, tau, 1e-5, 0.9)
    for cuts in ([T], [1, 2, 60, 1, 1, 85], [1] * 40 + [110]):
        state = torch.full((4, H, dk, dv), 9.0, device=DEV)          # stale: the first step must not read it
        wide = torch.zeros(T, H * dv + 6, dtype=dtype, device=DEV)   # the output as a block of columns
        at = 0
        for n in cuts:
            ctx = make_ctx([n], [at], [2], dtype=dtype)
            ops().gated_linear(x[at:at + n], z[at:at + n], nw, state, wide[at:at + n, 3:3 + H * dv], ctx.cu_q, ctx.ctx_before,
                               ctx.slots, 1, H, dk, dv, tau, 1e-5, 0.9)
            at += n
        assert rel_err(wide[:, 3:3 + H * dv], want) < TOL[dtype], cuts
        assert rel_err(state[2], st[2]) < TOL[dtype] and float(wide[:, :3].abs().max()) == 0
        assert float((state[1] - 9.0).abs().max()) == 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_recurrence_batch_of_unequal_entries(dtype):
    H, dk, dv, tau = 2, 16, 24, 5.0
    lens, before, slots = [1, 37, 2, 90], [5, 0, 40, 12], [3, 0, 2, 1]
    N = sum(lens)
    x, z, nw = _gla_inputs(dtype, N, H, dk, dv, seed=4)
    state = _x((4, H, dk, dv), torch.float32, seed=8)
    st = state.double().cpu()
    ctx = make_ctx(lens, before, slots, dtype=dtype)
    out, want = torch.empty(N, H * dv, dtype=dtype, device=DEV), torch.empty(N, H * dv, dtype=F64)
    ops().gated_linear(x, z, nw, state, out, ctx.cu_q, ctx.ctx_before, ctx.slots, 4, H, dk, dv, tau, 1e-5)
    refs.gated_linear(x.cpu(), z.cpu(), nw.cpu(), st, want, ctx.cu_q.cpu(), ctx.ctx_before.cpu(), ctx.slots.cpu(), 4, H, dk, dv,
                      tau, 1e-5)
    assert rel_err(out, want) < TOL[dtype] and rel_err(state, st) < TOL[dtype]


@pytest.mark.parametrize("H,dk,dv,tau", [(2, 32, 16, 12.0), (3, 16, 48, 2.0), (1, 128, 128, 8.0), (2, 64, 16, 1.0)])
def test_recurrence_chunk_by_chunk_against_token_by_token(H, dk, dv, tau):
    """Lengths on, just under and just over a chunk's edge, from states that are not zero, channels that forget at once."""
    if not ops().gated_linear_chunked_takes(dk, dv):
        pytest.skip("the chunk-by-chunk kernels do not take these head sizes")
    dtype, C = torch.bfloat16, ops().GATED_LINEAR_CHUNK
    lens, before, slots = [2 * C, 3 * C - 1, C + 1, 64 + 5 * C, 1], [0, 7, 3, 100, 9], [0, 3, 1, 2, 3]
    lens, before, slots = lens[:4], before[:4], slots[:4]
    N = sum(lens)
    x, z, nw = _gla_inputs(dtype, N, H, dk, dv, seed=6)
    start = _x((4, H, dk, dv), torch.float32, seed=8)
    ctx = make_ctx(lens, before, slots, dtype=dtype)
    a, b = torch.empty(N, H * dv, dtype=dtype, device=DEV), torch.empty(N, H * dv, dtype=dtype, device=DEV)
    sa, sb = start.clone(), start.clone()
    ops().gated_linear(x, z, nw, sa, a, ctx.cu_q, ctx.ctx_before, ctx.slots, 4, H, dk, dv, tau, 1e-5, 1.1)
    scratch = torch.empty(N, H * dv, device=DEV)
    states = torch.empty(ops().gated_linear_chunked_scratch(N, 4, H, dk, dv), device=DEV)
    ops().gated_linear(x, z, nw, sb, b, ctx.cu_q, ctx.ctx_before, ctx.slots, 4, H, dk, dv, tau, 1e-5, 1.1, scratch=scratch,
                       state_scratch=states, max_q=max(lens))
    assert rel_err(b, a) < 1e-2 and rel_err(sb, sa) < 1e-4


# ------------------------------------------------------------------------------------------ latent attention's kernels
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rq,rkv,rot,ng,half", [(20, 24, 4, 18, False), (16, 56, 8, 64, False), (6, 6, 0, 6, False),
                                                (80, 112, 16, 200, False), (7, 6, 6, 10, True)])
def test_latent_rows_with_a_rotated_key_part(dtype, rq, rkv, rot, ng, half):
    T, ps, before = 37, 8, 21
    rp = -(-(rkv + rot) // 16) * 16
    x = _x((T, rq + rkv + rot + ng), dtype, scale=2.0)
    wq, wkv = (1 + 0.2 * torch.randn(rq)).to(DEV), (1 + 0.2 * torch.randn(rkv)).to(DEV)
    inv = (500.0 ** (-2.0 * torch.arange(rot // 2, dtype=F64) / max(rot, 1))).float().to(DEV) if rot else None
    pages, _, table = _pages(before + T, ps, 1, rp, 0, 0, dtype)
    ctx = make_ctx([T], [before], [0], dtype=dtype)
    cq, gate = torch.empty(T, rq, dtype=dtype, device=DEV), torch.empty(T, ng, device=DEV)
    pr, cqr, gr = pages.cpu().clone(), cq.cpu().clone(), gate.cpu().clone()
    ops().latent_prep(x, wq, wkv, cq, pages, gate, table, ctx.positions, ctx.row_entry, ng, 1e-5, ctx.status, rot=rot,
                      inv_freq=inv, half_pairing=half)
    refs.latent_prep(x.cpu(), wq.cpu(), wkv.cpu(), cqr, pr, gr, table.cpu(), ctx.positions.cpu(), ctx.row_entry.cpu(), ng, 1e-5,
                     None, rot=rot, inv_freq=inv.cpu() if rot else None, half_pairing=half)
    assert rel_err(cq, cqr) < TOL[dtype] and rel_err(gate, gr) < 1e-5 and rel_err(pages, pr) < TOL[dtype]
    # a reader of another layer's latents: no c, no key part, no page is touched
    before_pages = pages.clone()
    xr = _x((T, rq + ng), dtype, seed=9)
    ops().latent_prep(xr, wq, None, cq, None, gate, table, ctx.positions, ctx.row_entry, ng, 1e-5, ctx.status)
    refs.latent_prep(xr.cpu(), wq.cpu(), None, cqr, None, gr, table.cpu(), ctx.positions.cpu(), ctx.row_entry.cpu(), ng, 1e-5, None)
    assert rel_err(cq, cqr) < TOL[dtype] and rel_err(gate, gr) < 1e-5 and torch.equal(pages, before_pages)
    if rot:
        H = 3
        q = _x((T, H * rp), dtype, seed=11)
        qr = q.cpu().clone()
        ops().latent_rope_q(q, ctx.positions, ctx.row_entry, inv, H, rkv, half)
        refs.latent_rope_q(qr, ctx.positions.cpu(), ctx.row_entry.cpu(), inv.cpu(), H, rkv, half)
        assert rel_err(q, qr) < TOL[dtype] and torch.equal(q.view(T, H, rp)[:, :, :rkv].cpu(), qr.view(T, H, rp)[:, :, :rkv])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n,H,rp,rank,dv", [(1, 3, 32, 24, 6), (37, 5, 64, 56, 24), (16, 2, 16, 6, 5), (130, 7, 144, 120, 40)])
def test_heads_expanded_and_gated(dtype, n, H, rp, rank, dv):
    o, w = _x((n, H * rp), dtype, seed=1), _x((H, dv, rank), dtype, seed=2, scale=0.3)
    gate = torch.rand(n, H * dv).to(DEV)
    wide = torch.zeros(n, H * dv + 9, dtype=dtype, device=DEV)
    want = torch.empty(n, H * dv, dtype=F64)
    ops().head_up_gate(o, w, gate, wide[:, 4:4 + H * dv])
    refs.head_up_gate(o.cpu(), w.cpu(), gate.cpu(), want)
    assert rel_err(wide[:, 4:4 + H * dv], want) < TOL[dtype] and float(wide[:, :4].abs().max()) == 0


@pytest.mark.parametrize("H,rp", [(8, 64), (3, 32), (5, 128), (16, 64)])
@pytest.mark.parametrize("window", [None, 37, 1])
def test_latent_core_on_tensor_cores_with_two_rows_a_tile(H, rp, window):
    """Models of up to eight heads put two neighbouring query rows into one tile; rows that are no neighbours (another
    request, a padding row, an odd row at the end) run one after the other.  A ragged step against the plain statement."""
    dtype = torch.bfloat16
    lens, before = [1, 5, 1, 2, 70, 3, 1], [40, 0, 99, 7, 30, 200, 0]
    re, pos = [], []
    for e, (n, b) in enumerate(zip(lens, before)):
        re += [e] * n
        pos += list(range(b, b + n))
    re, pos = re + [-1, -1, len(lens) - 1], pos + [0, 0, 1]          # padding rows, then the last request's next token
    n, ps = len(re), 16
    g = torch.Generator().manual_seed(H)
    pages = _x((64, 1, ps, rp), dtype, seed=3)
    table = torch.stack([torch.randperm(64, generator=g)[:16] for _ in lens]).to(torch.int32).to(DEV)
    q = _x((n, H * rp), dtype, seed=5, scale=0.3)
    gate = torch.rand(n, H, generator=g).to(DEV)
    out = torch.full((n, H * rp), 7.0, dtype=dtype, device=DEV)
    want = torch.zeros(n, H * rp, dtype=F64)
    ops().latent_core_mma(q, pages, table, _i32(pos), _i32(re), gate, out, H, window, 0.11)
    refs.latent_core(q.cpu(), pages.cpu(), table.cpu(), torch.tensor(pos), torch.tensor(re), gate.cpu(), want, H, window, 0.11)
    assert rel_err(out, want) < TOL[dtype]
    assert float(out[-3:-1].abs().max()) == 0                        # rows of no entry get zeros


# ------------------------------------------------------------------------------------------ routed experts
@pytest.mark.parametrize("E,top,groups,keep,scale", [(8, 3, 4, 2, 2.25), (6, 2, 3, 1, 1.7), (4, 1, 1, 1, 1.0), (16, 4, 4, 2, 0.5),
                                                     (3, 3, 3, 3, 1.0)])
def test_router_with_softmax_scores_and_groups_by_their_best(E, top, groups, keep, scale):
    n, H = 50, 40
    x = _x((n, H), torch.float32, seed=E)
    wr = (3.0 * torch.randn(E, H) / H ** 0.5).to(DEV)
    wsg = torch.randn(H).to(DEV)
    weights, want = torch.empty(n, E + 1, device=DEV), torch.empty(n, E + 1)
    ops().moe_router_sigmoid(x, wr, None, wsg, weights, top, groups, keep, softmax_scores=True, group_max=True, route_scale=scale)
    refs.moe_router_sigmoid(x.cpu(), wr.cpu(), None, wsg.cpu(), want, top, groups, keep, softmax_scores=True, group_max=True,
                            route_scale=scale)
    assert rel_err(weights, want) < 1e-5
    assert ((weights[:, :E] > 0).sum(1) == top).all() and rel_err(weights[:, :E].sum(1), torch.full((n,), scale)) < 1e-5
    if keep < groups and top > keep:                                 # the limit bites: other experts than the largest scores
        free = torch.empty(n, E + 1)
        refs.moe_router_sigmoid(x.cpu(), wr.cpu(), None, wsg.cpu(), free, top, 1, 1, softmax_scores=True, route_scale=scale)
        assert ((free[:, :E] > 0) != (want[:, :E] > 0)).any()


@pytest.mark.parametrize("dtype", DTYPES)
def test_experts_activation_with_a_gated_shared_expert(dtype):
    n, E, ff, sff = 9, 4, 16, 24
    I = E * ff + sff
    gu = _x((n, 2 * I), dtype, scale=1.5)
    weights = torch.rand(n, E + 1).to(DEV)
    out, want = torch.empty(n, I, dtype=dtype, device=DEV), torch.empty(n, I, dtype=F64)
    ops().moe_swiglu_scaled(gu, weights, out, ff, shared_gated=True)
    refs.moe_swiglu_scaled(gu.cpu(), weights.cpu(), want, ff, shared_gated=True)
    assert rel_err(out, want) < TOL[dtype]
    act = _x((n, I), dtype, seed=4)
    a2 = act.clone()
    ops().moe_scale(a2, weights, ff, shared_gated=True)
    w = torch.cat([weights[:, :E].repeat_interleave(ff, dim=1), weights[:, E:].expand(n, sff)], 1)
    assert rel_err(a2, act.double() * w.double()) < TOL[dtype]


# ------------------------------------------------------------------------------------------ whole models
LENS = {"A": [1, 9, 40, 131, 64, 23, 77], "B": [3, 50, 97, 30, 64], "B0": [2, 41, 90], "C": [2, 17, 150, 33, 210],
        "D": [1, 45, 20, 100]}


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
def plain_logits(dodilix_dirs):
    out = {}
    for name in LENS:
        for key in (name, name + "_calm"):
            cfg, w = dm.load_plain(dodilix_dirs[key])
            reqs = scenarios.make_requests(LENS[name], cfg["vocab"], seed=7)
            out[key] = (reqs, {r: plain.forward(cfg, w, t) for r, t in reqs.items()})
    return out


def test_stream_after_every_layer(dodilix_dirs):
    """float32, layer by layer: the sum of the stream's copies after every layer."""
    cfg, w = dm.load_plain(dodilix_dirs["A"])
    toks = scenarios.make_requests([37], cfg["vocab"], seed=1)["r0"]
    _, after = plain.forward(cfg, w, toks, return_layers=True)
    runner = make_runner(dodilix_dirs["A"], dtype=torch.float32, device="cuda", page_size=8, num_pages=16)
    seen = []
    model = runner.model
    run_entries, S = model.run_entries, cfg["streams"]

    def spy(ctx, caches, entries, h, pending):
        for e in entries:                              # one layer at a time; the update not yet written is folded in for the record
            pending = run_entries(ctx, caches, [e], h, pending)
            X = h.double().view(h.shape[0], S, -1)
            y = (pending.y.sum(0) if pending.y.dim() == 3 else pending.y).double()
            X = torch.einsum("st,nsh->nth", pending.mix.double(), X) + pending.out_w.double()[None, :, None] * y[:, None, :]
            seen.append(X.sum(1)[: len(toks)].cpu())
        return pending

    model.run_entries = spy
    runner.step([StepEntry("x", toks, [len(toks) - 1])])
    assert len(seen) == len(after) == 4
    for i, s in enumerate(seen):
        assert rel_err(s, after[i]) < 1e-4, i


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "B0", "C", "D"])
@pytest.mark.parametrize("cut", ["whole", "tail_decode", "portions", "mixed"])
def test_cuts_against_plain(dodilix_dirs, plain_logits, name, dtype, cut):
    key = name if dtype == torch.float32 else name + "_calm"
    reqs, want = plain_logits[key]
    ps = dm.PAGE_SIZE[name]
    cap = 256 if cut == "mixed" else 512                     # tokens; mixed: pages and slots are used again
    runner = make_runner(dodilix_dirs[key], dtype=dtype, device="cuda", page_size=ps, num_pages=cap // ps,
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
@pytest.mark.parametrize("name", ["A", "C"])
def test_first_tokens_and_long_decode(dodilix_dirs, name, dtype):
    """The first tokens one by one (an empty state, chunks of one key, the sink beside a lone key), then decoding across
    many chunks and page edges, with graphs replayed and the pages behind the chunks given back."""
    folder = _dir(dodilix_dirs, name, dtype)
    cfg, w = dm.load_plain(folder)
    toks = scenarios.make_requests([230], cfg["vocab"], seed=11)["r0"]
    want = plain.forward(cfg, w, toks)
    runner = make_runner(folder, dtype=dtype, device="cuda", page_size=8, num_pages=32, max_seq_len=256)
    got = torch.cat([runner.step([StepEntry("x", [t], [0])]).clone() for t in toks])
    runner.check_status()
    assert _close(got, want, dtype), rel_err(got, want)
    if dtype == torch.float32:
        assert rel_err(got[:14], want[:14]) < TOL[dtype]
    assert runner.graph_replays > 100
    held = runner.cache.pages_held("x")
    assert max(held) == 29 and min(held) <= (10 if name == "C" else 3)      # latents stay; chunked keys come back


@pytest.mark.parametrize("name", ["A", "C"])
def test_float32_cuts_agree_closely(dodilix_dirs, name):
    cfg, _ = dm.load_plain(dodilix_dirs[name])
    reqs = scenarios.make_requests([120], cfg["vocab"], seed=3)
    runner = make_runner(dodilix_dirs[name], dtype=torch.float32, device="cuda", num_pages=64, page_size=8)
    a = _replay(runner, scenarios.whole(reqs))["r0"]
    b = _replay(runner, scenarios.portions(reqs))["r0"]
    c = _replay(runner, scenarios.tail_decode(reqs))["r0"]
    assert rel_err(a, b) < 2e-5 and rel_err(a, c) < 2e-5


@pytest.mark.parametrize("dtype", DTYPES)
def test_batch_of_unequal_requests_equals_each_alone(dodilix_dirs, dtype):
    folder = _dir(dodilix_dirs, "A", dtype)
    cfg, _ = dm.load_plain(folder)
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


def test_greedy_generation_through_the_engine(dodilix_dirs):
    """Engine.generate (scheduler, portions, decode graphs, device sampler) against greedy decoding with the oracle."""
    from neurogrid_b200 import Engine
    cfg, w = dm.load_plain(dodilix_dirs["C"])
    prompts = list(scenarios.make_requests([12, 30, 5], cfg["vocab"], seed=9).values())
    eng = Engine(dodilix_dirs["C"], dtype="float32", max_seq_len=128, page_size=8, max_requests=2,
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
def test_trace_replay_program(dodilix_dirs, tmp_path, dtype):
    folder = dodilix_dirs["A" if dtype == "float32" else "A_calm"]
    cfg, w = dm.load_plain(folder)
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
