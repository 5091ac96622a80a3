"""The retention mixer: linear attention with a fixed decay per head and a float32 state per request."""
from __future__ import annotations

import torch

from ..cache.manager import SlotNeed
from ..csrc import ops
from ..weights.decl import TensorDecl
from . import registry
from .base import PositionArgs
from .registry import register


@register("mixer", "retention")
class Retention:
    """q, k, v and gate projections (stacked into one product at bind time) -> rotation of q and k ->
    per head S_t = decay S_(t-1) + k_t v_t^T, o_t = S_t^T q_t -> each head's o over its root mean square
    -> times silu(gate) -> output projection.  No softmax and no denominator.

    Everything that enters the recurrence (angles, rotation, the key's scaling, decays, S, the head's
    norm, the gate) is float32 in both compute dtypes; the projections are products of the compute dtype.
    State per request: S [heads, key_dim, value_dim], float32, zero at admission."""

    graph_safe = True      # launches depend on device data and on launch-time constants only
    CHUNKED_MIN_ROWS = 16  # a step whose longest portion has this many tokens runs the chunk-by-chunk kernel

    def __init__(self, spec, *, dtype, device):
        self.spec, self.dtype, self.device = spec, dtype, device
        self.position = registry.build("position", spec.position, device=device)
        self.decay = torch.tensor(spec.decay, dtype=torch.float64).to(torch.float32).to(device)
        self.w_in = self.w_o = None

    def tensors(self):
        s, n = self.spec, self.spec.names
        qk, vg = s.n_heads * s.key_dim, s.n_heads * s.value_dim
        return {n["q"]: TensorDecl((qk, s.hidden)), n["k"]: TensorDecl((qk, s.hidden)),
                n["v"]: TensorDecl((vg, s.hidden)), n["gate"]: TensorDecl((vg, s.hidden)),
                n["o"]: TensorDecl((s.hidden, vg))}

    def bind(self, t):
        n = self.spec.names
        kw = dict(device=self.device, dtype=self.dtype)
        self.w_in = torch.cat([t[n[p]].to(**kw) for p in ("q", "k", "v", "gate")]).contiguous()
        self.w_o = t[n["o"]].to(**kw).contiguous()

    def cache_need(self):
        s = self.spec
        return SlotNeed((s.n_heads, s.key_dim, s.value_dim))

    def kernels(self):
        return [("gemm_sm100" if self.dtype == torch.bfloat16 else "gemm_f32", None), ("retention", None)]

    def scratch_bytes_per_row(self):
        """Workspace per row besides the products' outputs: the heads' outputs before their norm and the chunks' states."""
        s = self.spec
        if self.dtype != torch.bfloat16:
            return 0
        return 4 * s.n_heads * s.value_dim + 4 * s.n_heads * s.key_dim * s.value_dim // 32

    def forward(self, x, ctx, cache):
        s = self.spec
        n = x.shape[0]
        p = ctx.ws.buf("ret_in", n, self.w_in.shape[0], self.dtype)
        ops.linear(x, self.w_in, None, p)
        pa = PositionArgs.of(self.position.kernel_args())
        if pa.inv_freq is not None and (not pa.half_pairing or pa.pos_scale != 1.0):
            raise NotImplementedError("the retention kernel rotates pairs (i, i + dims/2) of unscaled positions")
        rot = 0 if pa.inv_freq is None else (s.key_dim if pa.rotary_dims is None else pa.rotary_dims)
        o = ctx.ws.buf("ret_out", n, s.n_heads * s.value_dim, self.dtype)
        # float32 keeps the token-by-token kernel for every step: there a token's arithmetic is the same however
        # its request is cut.  bfloat16 steps with a long portion regroup the sums chunk by chunk.
        chunked = (self.dtype == torch.bfloat16 and ctx.max_q >= self.CHUNKED_MIN_ROWS
                   and ops.retention_chunked_takes(s.key_dim, s.value_dim))
        scratch = states = None
        if chunked:
            scratch = ctx.ws.buf("ret_scratch", n, s.n_heads * s.value_dim, torch.float32)
            need = ops.retention_chunked_scratch(n, ctx.n_entries, s.n_heads, s.key_dim, s.value_dim)
            bound = ops.retention_chunked_scratch(ctx.ws.max_rows, ctx.ws.max_rows // self.CHUNKED_MIN_ROWS + 64,
                                                  s.n_heads, s.key_dim, s.value_dim)
            states = ctx.ws.flat(f"ret_states_{s.n_heads}x{s.key_dim}x{s.value_dim}", need, torch.float32, reserve=max(need, bound))
        ops.retention(p, pa.inv_freq if rot else None, rot, self.decay, cache.state, o, ctx.cu_q, ctx.ctx_before,
                      ctx.slots, ctx.n_entries, s.n_heads, s.key_dim, s.value_dim, s.eps, scratch=scratch,
                      state_scratch=states, max_q=ctx.max_q)
        return ops.linear_to_residual(o, self.w_o, None, ctx.ws, "mixer_out", residual=ctx.residual)
