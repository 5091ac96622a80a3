"""Gated linear attention: a linear-attention recurrence whose float32 state decays per key channel and token."""
from __future__ import annotations

import torch

from ..cache.manager import SlotNeed
from ..csrc import ops
from ..weights.decl import TensorDecl
from .registry import register


@register("mixer", "gated_linear_attention")
class GatedLinearAttention:
    """q, k, v and gate projections (stacked into one product when bound) and the decay's logits through their
    low-rank pair z = W_a2 (W_a1 x) + b -> per head S <- diag(alpha) S + k v^T with alpha = sigmoid(z)^(1/tau) per key
    channel, o = S^T (q key_dim^(-1/2)) -> each head's o RMS-normed with a weight shared by the heads, times
    silu(gate) -> output projection.

    Everything that enters the recurrence besides the projections (the decay with its logarithm and exponential, the
    state, the read-out, the head's norm, the gate) is float32 in both compute dtypes.  State per request:
    S [heads, key_dim, value_dim] float32, zero at admission.  float32 steps and steps of short portions walk the
    tokens one by one (a token's arithmetic is then the same however its request is cut); bfloat16 steps with a long
    portion regroup the sums chunk by chunk."""

    graph_safe = True      # launches depend on device data and on launch-time constants only
    CHUNKED_MIN_ROWS = 64  # a bfloat16 step whose longest portion has this many tokens runs the chunk-by-chunk kernels

    def __init__(self, spec, *, dtype, device):
        self.spec, self.dtype, self.device = spec, dtype, device
        self.w_in = self.w_a1 = self.w_a2 = self.b_a2 = self.w_o = self.norm = None

    def tensors(self):
        s, n = self.spec, self.spec.names
        qk, vg = s.n_heads * s.key_dim, s.n_heads * s.value_dim
        return {n["q"]: TensorDecl((qk, s.hidden)), n["k"]: TensorDecl((qk, s.hidden)), n["v"]: TensorDecl((vg, s.hidden)),
                n["gate"]: TensorDecl((vg, s.hidden)), n["o"]: TensorDecl((s.hidden, vg)),
                n["norm"]: TensorDecl((s.value_dim,), "norm"),
                n["decay_down"]: TensorDecl((s.decay_rank, s.hidden)), n["decay_up"]: TensorDecl((qk, s.decay_rank)),
                n["decay_bias"]: TensorDecl((qk,), "bias")}

    def bind(self, t):
        n = self.spec.names
        kw = dict(device=self.device, dtype=self.dtype)
        self.w_in = torch.cat([t[n[p]].to(**kw) for p in ("q", "k", "v", "gate")]).contiguous()
        self.w_a1 = t[n["decay_down"]].to(**kw).contiguous()
        self.w_a2 = t[n["decay_up"]].to(**kw).contiguous()
        self.b_a2 = t[n["decay_bias"]].to(**kw).contiguous()
        self.w_o = t[n["o"]].to(**kw).contiguous()
        self.norm = t[n["norm"]].to(device=self.device, dtype=torch.float32).contiguous()

    def cache_need(self):
        s = self.spec
        return SlotNeed((s.n_heads, s.key_dim, s.value_dim))

    def kernels(self):
        return [("gemm_sm100" if self.dtype == torch.bfloat16 else "gemm_f32", None), ("gated_linear", None)]

    def _chunked(self, ctx):
        s = self.spec
        return self.dtype == torch.bfloat16 and ctx.max_q >= self.CHUNKED_MIN_ROWS and \
            ops.gated_linear_chunked_takes(s.key_dim, s.value_dim)

    def scratch_bytes_per_row(self):
        s = self.spec
        if self.dtype != torch.bfloat16:
            return 0
        return 4 * s.n_heads * s.value_dim + 4 * s.n_heads * (s.key_dim * s.value_dim + s.key_dim) // ops.GATED_LINEAR_CHUNK

    # a caller that ends two mixers with ONE product calls ``core`` and multiplies itself
    def inner_width(self):
        return self.spec.n_heads * self.spec.value_dim

    def out_weight(self):
        return self.w_o, None

    def drop_out_weight(self):
        """The caller keeps a stacked copy of the output matrix and will not call ``forward``."""
        self.w_o = None

    def core(self, x, ctx, cache, out, out_scale=1.0):
        """out[N, n_heads * value_dim] (may be a block of columns of a wider buffer): the normed, gated heads times
        ``out_scale``."""
        s = self.spec
        n = x.shape[0]
        p = ctx.ws.buf("gla_in", n, self.w_in.shape[0], self.dtype)
        ops.linear(x, self.w_in, None, p)
        low = ctx.ws.buf("gla_low", n, s.decay_rank, self.dtype)
        ops.linear(x, self.w_a1, None, low)
        z = ctx.ws.buf("gla_z", n, s.n_heads * s.key_dim, self.dtype)
        ops.linear(low, self.w_a2, self.b_a2, z)
        scratch = states = None
        if self._chunked(ctx):
            scratch = ctx.ws.buf("gla_raw", n, s.n_heads * s.value_dim, torch.float32)
            need = ops.gated_linear_chunked_scratch(n, ctx.n_entries, s.n_heads, s.key_dim, s.value_dim)
            bound = ops.gated_linear_chunked_scratch(ctx.ws.max_rows, ctx.ws.max_rows // self.CHUNKED_MIN_ROWS + 64,
                                                     s.n_heads, s.key_dim, s.value_dim)
            states = ctx.ws.flat(f"gla_states_{s.n_heads}x{s.key_dim}x{s.value_dim}", need, torch.float32,
                                 reserve=max(need, bound))
        ops.gated_linear(p, z, self.norm, cache.state, out, ctx.cu_q, ctx.ctx_before, ctx.slots, ctx.n_entries, s.n_heads,
                         s.key_dim, s.value_dim, s.tau, s.eps, out_scale, scratch=scratch, state_scratch=states,
                         max_q=ctx.max_q)

    def forward(self, x, ctx, cache, out_name="mixer_out"):
        o = ctx.ws.buf("gla_out", x.shape[0], self.inner_width(), self.dtype)
        self.core(x, ctx, cache, o)
        return ops.linear_to_residual(o, self.w_o, None, ctx.ws, out_name, residual=ctx.residual)
