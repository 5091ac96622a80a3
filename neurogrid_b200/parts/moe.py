"""Routed experts with a shared expert."""
from __future__ import annotations

import torch

from ..csrc import ops
from ..weights.decl import TensorDecl
from .registry import register


@register("ffn", "moe")
class MoE:
    """Router logits in float32 (with a bias) -> the top_k experts of each token, weighted by the softmax
    over the chosen logits -> sum of the chosen SwiGLU experts' outputs, plus a shared expert's.  With sigmoid
    scoring the experts are chosen by score plus a stored correction among the best groups of experts and weighted
    by their scores over the scores' sum (the scores may also be a softmax over all experts, a group's score its
    largest, the weights scaled); the clamped activation and the shared expert's gate are applied in the
    same pass as the routing weights.

    Laid out as two products over ALL experts side by side: gate and up rows of every expert (and of
    the shared expert behind them) are stacked when the weights are bound, the activations of expert e
    are multiplied by the token's routing weight for e (zero where it is not chosen, one for the shared
    expert), and one product with the down projections side by side is then the weighted sum itself.
    The shapes do not depend on the routing, so a step is the same launches whatever the router decides."""

    graph_safe = True      # launches depend on device data and on launch-time constants only

    def __init__(self, spec, *, dtype, device):
        self.spec, self.dtype, self.device = spec, dtype, device
        self.width = spec.n_experts * spec.expert_ff + spec.shared_ff
        self.w_gate_up = self.w_down = self.w_router = self.b_router = self.correction = self.w_shared_gate = None
        self.sigmoid = getattr(spec, "scoring", "softmax") in ("sigmoid", "softmax_all")    # the router kernel with groups
        self.clamped = getattr(spec, "activation", "swiglu") == "clamped_glu"

    def _expert_names(self):
        s, n = self.spec, self.spec.names
        pres = [n["expert"].format(e) + "." for e in range(s.n_experts)]
        return pres + ([n["shared"] + "."] if s.shared_ff else [])

    def tensors(self):
        s, n = self.spec, self.spec.names
        d = {n["router"]: TensorDecl((s.n_experts, s.hidden))}
        if not self.sigmoid:
            d[n["router_bias"]] = TensorDecl((s.n_experts,), "bias")
        if getattr(s, "correction", False):
            d[n["correction"]] = TensorDecl((s.n_experts,), "bias")
        if getattr(s, "shared_gate", False):
            d[n["shared_gate"]] = TensorDecl((1, s.hidden))
        for i, pre in enumerate(self._expert_names()):
            ff = s.expert_ff if i < s.n_experts else s.shared_ff
            d[pre + n["gate"]] = TensorDecl((ff, s.hidden))
            d[pre + n["up"]] = TensorDecl((ff, s.hidden))
            d[pre + n["down"]] = TensorDecl((s.hidden, ff))
        return d

    def bind(self, t):
        n = self.spec.names
        kw = dict(device=self.device, dtype=self.dtype)
        f32 = dict(device=self.device, dtype=torch.float32)
        pres = self._expert_names()
        self.w_gate_up = torch.cat([t[p + n["gate"]].to(**kw) for p in pres]
                                   + [t[p + n["up"]].to(**kw) for p in pres]).contiguous()
        self.w_down = torch.cat([t[p + n["down"]].to(**kw) for p in pres], dim=1).contiguous()
        self.w_router = t[n["router"]].to(**f32).contiguous()
        if not self.sigmoid:
            self.b_router = t[n["router_bias"]].to(**f32).contiguous()
        if getattr(self.spec, "correction", False):
            self.correction = t[n["correction"]].to(**f32).contiguous()
        if getattr(self.spec, "shared_gate", False):
            self.w_shared_gate = t[n["shared_gate"]].to(**f32).reshape(-1).contiguous()

    def kernels(self):
        return [("gemm_sm100" if self.dtype == torch.bfloat16 else "gemm_f32", None), ("elementwise", None), ("moe", None)]

    def forward(self, x, ctx):
        s = self.spec
        n, I = x.shape[0], self.width
        weights = ctx.ws.buf("moe_weights", n, s.n_experts + (self.w_shared_gate is not None), torch.float32)
        if self.sigmoid:
            ops.moe_router_sigmoid(x, self.w_router, self.correction, self.w_shared_gate, weights, s.top_k, s.n_groups,
                                   s.keep_groups, softmax_scores=s.scoring == "softmax_all",
                                   group_max=getattr(s, "group_score", "top2") == "max",
                                   route_scale=getattr(s, "route_scale", 1.0))
        else:
            ops.moe_router(x, self.w_router, self.b_router, weights, s.top_k)
        act = ctx.ws.buf("moe_act", n, I, self.dtype)
        if self.clamped:
            gu = ctx.ws.buf("moe_gate_up", n, 2 * I, self.dtype)
            ops.linear(x, self.w_gate_up, None, gu)
            ops.moe_clamped_glu_scaled(gu, weights, act, s.n_experts, s.expert_ff, s.limit, s.shared_limit, s.glu_alpha,
                                       self.w_shared_gate is not None)
        elif ops.gemm_sm100_ok(x, self.w_gate_up):
            ops.gemm_swiglu_sm100(x, self.w_gate_up, act)          # the gate rides in the epilogue
            ops.moe_scale(act, weights, s.expert_ff, shared_gated=self.w_shared_gate is not None)
        else:
            gu = ctx.ws.buf("moe_gate_up", n, 2 * I, self.dtype)
            ops.linear(x, self.w_gate_up, None, gu)
            ops.moe_swiglu_scaled(gu, weights, act, s.expert_ff,   # gate and routing weight in one pass
                                  shared_gated=self.w_shared_gate is not None)
        return ops.linear_to_residual(act, self.w_down, None, ctx.ws, "ffn_out", residual=ctx.residual)
