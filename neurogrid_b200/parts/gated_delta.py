"""The gated delta rule mixer: a recurrence with a float32 state per head behind short convolutions of q, k and v."""
from __future__ import annotations

import torch

from ..cache.manager import SlotNeed
from ..csrc import ops
from ..weights.decl import TensorDecl
from .registry import register


@register("mixer", "gated_delta")
class GatedDelta:
    """q, k, v, gate, decay and beta projections (stacked into one product when bound) -> causal convolution per
    channel and silu on q, k, v -> q, k unit vectors per head, q times key_dim^(-1/2) -> per value head
    S <- g S, u = beta (v - S^T k), S <- S + k u^T, o = S^T q -> each head's o over its root mean square, times a
    weight and silu(gate) -> output projection.

    Everything that enters the recurrence besides the projections (the convolution's sum and silu, unit norms, beta,
    the decay with its softplus and exponentials, S, the head's norm, the gate) is float32 in both compute dtypes.
    State per request: S [heads, key_dim, value_dim] float32 (zero at admission) and the convolution's last
    taps - 1 inputs [taps - 1, channels] float32; the mixer declares the two needs and is handed the two views."""

    graph_safe = True      # launches depend on device data and on launch-time constants only
    CHUNKED_MIN_ROWS = 64  # a bfloat16 step whose longest portion has this many tokens runs the chunk-by-chunk kernels

    def __init__(self, spec, *, dtype, device):
        self.spec, self.dtype, self.device = spec, dtype, device
        self.channels = 2 * spec.n_qk_heads * spec.key_dim + spec.n_heads * spec.value_dim
        self.taps = max(spec.taps, 2)          # a single tap runs as two, the older one zero
        self.w_in = self.w_o = self.w_conv = self.a_log = self.dt_bias = self.norm = None

    def tensors(self):
        s, n = self.spec, self.spec.names
        qk, vg = s.n_qk_heads * s.key_dim, s.n_heads * s.value_dim
        return {n["q"]: TensorDecl((qk, s.hidden)), n["k"]: TensorDecl((qk, s.hidden)), n["v"]: TensorDecl((vg, s.hidden)),
                n["q_conv"]: TensorDecl((qk, s.taps), "conv"), n["k_conv"]: TensorDecl((qk, s.taps), "conv"),
                n["v_conv"]: TensorDecl((vg, s.taps), "conv"),
                n["beta"]: TensorDecl((s.n_heads, s.hidden)), n["decay"]: TensorDecl((s.n_heads, s.hidden)),
                n["a_log"]: TensorDecl((s.n_heads,), "bias"), n["dt_bias"]: TensorDecl((s.n_heads,), "bias"),
                n["norm"]: TensorDecl((s.value_dim,), "norm"), n["gate"]: TensorDecl((vg, s.hidden)),
                n["o"]: TensorDecl((s.hidden, vg))}

    def bind(self, t):
        s, n = self.spec, self.spec.names
        kw = dict(device=self.device, dtype=self.dtype)
        f32 = dict(device=self.device, dtype=torch.float32)
        self.w_in = torch.cat([t[n[p]].to(**kw) for p in ("q", "k", "v", "gate", "decay", "beta")]).contiguous()
        self.w_o = t[n["o"]].to(**kw).contiguous()
        w = torch.cat([t[n[p]].to(**f32) for p in ("q_conv", "k_conv", "v_conv")])
        if s.taps == 1:
            w = torch.cat([torch.zeros_like(w), w], dim=1)
        self.w_conv = w.contiguous()
        self.a_log = t[n["a_log"]].to(**f32).contiguous()
        self.dt_bias = t[n["dt_bias"]].to(**f32).contiguous()
        self.norm = t[n["norm"]].to(**f32).contiguous()

    def cache_need(self):
        s = self.spec
        return (SlotNeed((s.n_heads, s.key_dim, s.value_dim)), SlotNeed((self.taps - 1, self.channels)))

    def kernels(self):
        return [("gemm_sm100" if self.dtype == torch.bfloat16 else "gemm_f32", None), ("gated_delta", None)]

    def _chunked(self):
        s = self.spec
        # the head sizes the chunked kernels take: key rows in fours, at most 256; value columns in sixteens
        return self.dtype == torch.bfloat16 and s.key_dim % 4 == 0 and s.key_dim <= 256 and s.value_dim % 16 == 0

    def scratch_bytes_per_row(self):
        s = self.spec
        per_row = 4 * (self.channels + s.n_heads * s.value_dim)
        if self._chunked():
            per_row += 4 * s.n_heads * (64 * s.key_dim + 32 + s.key_dim * s.value_dim) // 32
        return per_row

    def forward(self, x, ctx, cache, out_name="mixer_out"):
        s = self.spec
        n = x.shape[0]
        state, conv_state = cache
        p = ctx.ws.buf("gd_in", n, self.w_in.shape[0], self.dtype)
        ops.linear(x, self.w_in, None, p)
        conv = ctx.ws.buf("gd_conv", n, self.channels, torch.float32)
        o_raw = ctx.ws.buf("gd_raw", n, s.n_heads * s.value_dim, torch.float32)
        o = ctx.ws.buf("gd_out", n, s.n_heads * s.value_dim, self.dtype)
        # float32 keeps the token-by-token kernel for every step: there a token's arithmetic is the same however its
        # request is cut.  bfloat16 steps with a long portion regroup the recurrence chunk by chunk (still float32).
        chunks = None
        if ctx.max_q >= self.CHUNKED_MIN_ROWS and self._chunked():
            need = ops.gated_delta_chunked_scratch(n, ctx.n_entries, s.n_heads, s.key_dim, s.value_dim)
            bound = ops.gated_delta_chunked_scratch(ctx.ws.max_rows, ctx.ws.max_rows // self.CHUNKED_MIN_ROWS + 64,
                                                    s.n_heads, s.key_dim, s.value_dim)
            chunks = ctx.ws.flat(f"gd_chunks_{s.n_heads}x{s.key_dim}x{s.value_dim}", need, torch.float32, reserve=max(need, bound))
        ops.gated_delta(p, self.w_conv, self.a_log, self.dt_bias, self.norm, conv_state.state, state.state, conv, o_raw, o,
                        ctx.cu_q, ctx.ctx_before, ctx.slots, ctx.row_entry, ctx.n_entries, ctx.max_q, s.n_heads,
                        s.n_qk_heads, s.key_dim, s.value_dim, s.eps, chunk_scratch=chunks)
        return ops.linear_to_residual(o, self.w_o, None, ctx.ws, out_name, residual=ctx.residual)
