"""Attention with float32 scores and weights, one or two score maps per head, a window that keeps the first tokens."""
from __future__ import annotations

import math

import torch

from ..cache.manager import PagedNeed
from ..csrc import ops
from ..weights.decl import TensorDecl
from . import registry
from .base import PositionArgs
from .registry import register


@register("mixer", "mapped_attention")
class MappedAttention:
    """q, k, v projections (stacked into one product when bound, biases added there) -> per-map RMS norm of q and
    k (or one norm over the whole of q and one over the whole of k) -> q times its temperature -> rotation -> k, v into the layer's pages -> per head and map softmax(cap(scale q.k)) v over the visible
    keys -> one map: that; two maps: a_0 - lambda a_1, over its root mean square, times (1 - diff) -> output
    projection.  Keys lie in the pages as G * n_maps heads of key_dim, values as G heads of value_dim.  Scores,
    softmax weights, their sums with the values, norms, angles and lambda are float32 in both compute dtypes.

    ``owns_cache`` False builds a layer that reads another layer's keys and values: it has no k/v tensors.
    Steps of few rows (and the float32 path) run a kernel with a block per row and head and cut every row's keys
    into runs so that the GPU is filled; longer bfloat16 steps run the tensor-core kernel (the float32 weights as
    three bfloat16 terms) when the head sizes are multiples of 16 up to 128, and so do bfloat16 steps of single
    tokens, with the heads of a KV group as the rows of a tile and every row's keys cut into runs.
    """

    graph_safe = True      # launches depend on device data and on launch-time constants only
    GROUP_MAX_ROWS = 256   # decode-only steps of up to this many rows run the heads of a KV group as a tensor-core tile
    GROUP_MAX_RUNS = 512   # ... with rows * runs a row bounded by this
    SPLIT_MAX_ROWS = 32    # steps of up to this many rows may cut each row's keys into runs
    SPLIT_MIN_KEYS = 128   # ... of at least this many keys (one tile of the kernel)
    MAX_SPLITS = 16

    def __init__(self, spec, *, dtype, device, owns_cache=True):
        self.spec, self.dtype, self.device, self.owns_cache = spec, dtype, device, owns_cache
        self.position = registry.build("position", spec.position, device=device)
        self.w_qkv = self.b_qkv = self.w_o = self.b_o = self.q_norm = self.k_norm = self.sinks = None
        self.lam = 0.0
        self.whole = getattr(spec, "norm_scope", "head") == "projection"      # one norm over all of q, one over all of k

    def _proj(self):
        """The stacked projection's parts in order: q, k, v (a layer that reads another's cache: q only), then the
        output gate's logits if the mixer has one."""
        s = self.spec
        rows = {"q": s.n_heads * s.n_maps * s.key_dim, "k": s.n_kv_heads * s.n_maps * s.key_dim,
                "v": s.n_kv_heads * s.value_dim, "out_gate": s.n_heads * s.value_dim}
        parts = ("q", "k", "v") if self.owns_cache else ("q",)
        return {p: rows[p] for p in parts + (("out_gate",) if getattr(s, "out_gate", False) else ())}

    def tensors(self):
        s, n = self.spec, self.spec.names
        d = {n[p]: TensorDecl((rows, s.hidden)) for p, rows in self._proj().items()}
        d[n["o"]] = TensorDecl((s.hidden, s.n_heads * s.value_dim))
        if s.bias:
            for p, rows in self._proj().items():
                d[n[p + "_bias"]] = TensorDecl((rows,), "bias")
            d[n["o_bias"]] = TensorDecl((s.hidden,), "bias")
        if s.qk_norm and getattr(s, "norm_weight", True):
            rows = self._proj()
            d[n["q_norm"]] = TensorDecl((rows["q"] if self.whole else s.key_dim,), "norm")
            if self.owns_cache:
                d[n["k_norm"]] = TensorDecl((rows["k"] if self.whole else s.key_dim,), "norm")
        if s.n_maps == 2:
            for v in ("lq1", "lk1", "lq2", "lk2"):
                d[n[v]] = TensorDecl((s.key_dim,), "bias")
        if getattr(s, "sink", False):
            d[n["sink"]] = TensorDecl((s.n_heads,), "bias")
        return d

    def bind(self, t):
        s, n = self.spec, self.spec.names
        kw = dict(device=self.device, dtype=self.dtype)
        f32 = dict(device=self.device, dtype=torch.float32)
        self.w_qkv = torch.cat([t[n[p]].to(**kw) for p in self._proj()]).contiguous()
        self.w_o = t[n["o"]].to(**kw).contiguous()
        if s.bias:
            self.b_qkv = torch.cat([t[n[p + "_bias"]].to(**kw) for p in self._proj()]).contiguous()
            self.b_o = t[n["o_bias"]].to(**kw).contiguous()
        if s.qk_norm and getattr(s, "norm_weight", True):
            self.q_norm = t[n["q_norm"]].to(**f32).contiguous()
            if self.owns_cache:
                self.k_norm = t[n["k_norm"]].to(**f32).contiguous()
        if getattr(s, "sink", False):
            self.sinks = t[n["sink"]].to(**f32).contiguous()
        if s.n_maps == 2:            # one number per layer, formed in float32 as the stored vectors' products
            v = {k: t[n[k]].to(torch.float32) for k in ("lq1", "lk1", "lq2", "lk2")}
            self.lam = float(torch.exp((v["lq1"] * v["lk1"]).sum()) - torch.exp((v["lq2"] * v["lk2"]).sum())) + float(s.diff)

    def cache_need(self):
        s = self.spec
        return PagedNeed(s.n_kv_heads * s.n_maps, s.key_dim, s.cache_window, True, v_heads=s.n_kv_heads, v_dim=s.value_dim,
                         keep_first=s.cache_keep_first if s.cache_window else 0)

    def kernels(self):
        s = self.spec
        jobs = [("gemm_sm100" if self.dtype == torch.bfloat16 else "gemm_f32", None), ("mapped_attention", None)]
        if ops.mapped_attention_mma_takes(s.key_dim, s.value_dim, self.dtype):
            jobs.append(("mapped_attention_mma", {"NG_MA_D": s.key_dim, "NG_MA_DV": s.value_dim}))
        return jobs

    def scratch_bytes_per_row(self):
        s = self.spec
        return 4 * ops.mapped_attention_partial_floats(1, s.n_heads, s.n_maps, s.value_dim, self.MAX_SPLITS)

    def _longest(self, cache):
        s = self.spec
        longest = cache.table.shape[1] * cache.k_pages.shape[2]
        if getattr(s, "chunk", None):
            return min(longest, s.chunk)
        return min(longest, s.window + s.keep_first) if s.window else longest

    def _group_splits(self, n_rows, cache):
        """Runs a row's keys are cut into when single tokens run as tiles of a KV group's heads (tiles of 64 keys)."""
        s = self.spec
        want = -(-3 * ops.sm_count(self.device) // max(1, n_rows * s.n_kv_heads))
        return max(1, min(self.MAX_SPLITS, want, self._longest(cache) // 64, self.GROUP_MAX_RUNS // n_rows))

    # a block arrangement that ends mixer and feed-forward with ONE product calls ``core`` and multiplies itself
    def inner_width(self):
        return self.spec.n_heads * self.spec.value_dim

    def out_weight(self):
        return self.w_o, self.b_o

    def drop_out_weight(self):
        """The caller keeps a stacked copy of the output matrix and will not call ``forward``."""
        self.w_o = None

    def _splits(self, n_rows, cache):
        """Runs a row's keys are cut into: from the step's rows and the layer's constants only (a graph's launches)."""
        s = self.spec
        if n_rows > self.SPLIT_MAX_ROWS:
            return 1
        longest = self._longest(cache)
        most = min(self.MAX_SPLITS, longest // self.SPLIT_MIN_KEYS)
        if most <= 1 or torch.device(self.device).type != "cuda":       # (the host-side tests step the parts without a GPU)
            return 1
        return max(1, min(most, -(-6 * ops.sm_count(self.device) // max(1, n_rows * s.n_heads))))

    def core(self, x, ctx, cache, out, out_scale=1.0):
        """out[N, n_heads * value_dim] (may be a block of columns of a wider buffer): the heads' outputs (gated, if the
        mixer has an output gate), times ``out_scale``."""
        s = self.spec
        n = x.shape[0]
        if cache.writes and not self.owns_cache:
            raise RuntimeError("an attention layer without k/v weights cannot write a cache")
        writes = cache.writes
        n_q = s.n_heads * s.n_maps
        n_k, n_v = (s.n_kv_heads * s.n_maps, s.n_kv_heads) if self.owns_cache else (0, 0)
        qkv = ctx.ws.buf("mattn_qkv", n, self.w_qkv.shape[0], self.dtype)
        ops.linear(x, self.w_qkv, self.b_qkv, qkv)
        gated = getattr(s, "out_gate", False)
        gate = qkv[:, qkv.shape[1] - s.n_heads * s.value_dim:] if gated else None        # the gate's logits: the last columns
        if self.owns_cache and not writes:       # has k/v weights but this run reads another cache: the q columns only
            q_only = ctx.ws.buf("mattn_qonly", n, n_q * s.key_dim, self.dtype)
            q_only.copy_(qkv[:, : n_q * s.key_dim])
            qkv, n_k, n_v = q_only, 0, 0
        q = ctx.ws.buf("mattn_q", n, n_q * s.key_dim, self.dtype)
        pa = PositionArgs.of(self.position.kernel_args())
        ops.qkv_prep(qkv, q, self.q_norm, self.k_norm if n_k else None, pa.inv_freq, cache.k_pages if n_k else None,
                     cache.v_pages if n_v else None, cache.table, ctx.positions, ctx.row_entry, n_q, n_k, n_v,
                     s.key_dim, s.value_dim, s.eps, ctx.status, whole=self.whole,
                     q_temp_coef=getattr(s, "q_temp_coef", 0.0), q_temp_every=getattr(s, "q_temp_every", 1),
                     half_pairing=bool(pa.inv_freq is not None and pa.half_pairing),
                     unit_norm=bool(s.qk_norm and not getattr(s, "norm_weight", True)))
        self.attend(q, cache, ctx, out, pa.score_slopes)
        if gated or out_scale != 1.0:
            ops.gate_mul(out, gate, "sigmoid", out_scale)

    def attend(self, q, cache, ctx, out, slopes=None):
        """The attention core over the pages: q [N, n_heads * n_maps * key_dim] as the preparation left it.
        ``slopes``: the position encoding's score bias per head, if it has one."""
        s = self.spec
        n = q.shape[0]
        extra = dict(slopes=slopes, sinks=self.sinks, chunk=getattr(s, "chunk", None) or 0)
        if ctx.max_q == 1 and n <= self.GROUP_MAX_ROWS and not ctx.fixed_launches and \
                ops.mapped_attention_group_takes(s.key_dim, s.value_dim, s.n_heads, s.n_kv_heads, self.dtype):
            n_splits = self._group_splits(n, cache)
            per_run = ops.mapped_attention_partial_floats(1, s.n_heads, s.n_maps, s.value_dim, 2) // 2
            # (scratch whose bound follows from the layer's sizes is named after them: a layer of other sizes has its own)
            partial = ctx.ws.flat(f"mattn_group_partial_{s.n_heads}x{s.n_maps}x{s.value_dim}", n * n_splits * per_run,
                                  torch.float32,
                                  reserve=max(self.GROUP_MAX_RUNS, min(ctx.ws.max_rows, self.GROUP_MAX_ROWS)) * per_run)
            ops.mapped_attention_group(q, cache.k_pages, cache.v_pages, cache.table, ctx.cu_q, ctx.ctx_before, ctx.row_entry,
                                       out, partial, ctx.n_entries, s.n_heads, s.n_maps, s.window, s.keep_first,
                                       s.softmax_scale, s.softcap or 0.0, self.lam, s.n_maps == 2, 1.0 - s.diff, s.eps, n_splits,
                                       **extra)
            return
        if n > self.SPLIT_MAX_ROWS and ops.mapped_attention_mma_takes(s.key_dim, s.value_dim, self.dtype):
            ops.mapped_attention_mma(q, cache.k_pages, cache.v_pages, cache.table, ctx.cu_q, ctx.ctx_before, out,
                                     ctx.n_entries, ctx.max_q, s.n_heads, s.n_maps, s.window, s.keep_first,
                                     s.softmax_scale, s.softcap or 0.0, self.lam, s.n_maps == 2, 1.0 - s.diff, s.eps, **extra)
            return
        n_splits = self._splits(n, cache)
        partial = None
        if n_splits > 1 or ctx.ws.fixed:
            bound = ops.mapped_attention_partial_floats(min(ctx.ws.max_rows, self.SPLIT_MAX_ROWS), s.n_heads, s.n_maps,
                                                        s.value_dim, self.MAX_SPLITS)
            need = ops.mapped_attention_partial_floats(n, s.n_heads, s.n_maps, s.value_dim, n_splits)
            partial = ctx.ws.flat(f"mattn_partial_{s.n_heads}x{s.n_maps}x{s.value_dim}", need, torch.float32, reserve=bound)
        ops.mapped_attention(q, cache.k_pages, cache.v_pages, cache.table, ctx.positions, ctx.row_entry, out, s.n_heads,
                             s.n_maps, s.window, s.keep_first, s.softmax_scale, s.softcap or 0.0, self.lam,
                             s.n_maps == 2, 1.0 - s.diff, s.eps, n_splits, partial, **extra)

    def forward(self, x, ctx, cache, out_name="mixer_out"):
        """``out_name``: the workspace buffer of the result (a caller that runs two mixers on one input names two)."""
        a = ctx.ws.buf("mattn_out", x.shape[0], self.inner_width(), self.dtype)
        self.core(x, ctx, cache, a)
        return ops.linear_to_residual(a, self.w_o, self.b_o, ctx.ws, out_name, residual=ctx.residual)
