"""An ungated feed-forward: down(act(up x + b)) + b."""
from __future__ import annotations

import torch

from ..csrc import ops
from ..weights.decl import TensorDecl
from .registry import register


@register("ffn", "mlp")
class MLP:
    """y = W_down act(W_up x + b_up) + b_down with act the square of relu; the biases ride in the products, and in a
    step of few rows so does the activation."""

    graph_safe = True      # launches depend on device data and on launch-time constants only

    def __init__(self, spec, *, dtype, device):
        self.spec, self.dtype, self.device = spec, dtype, device
        self.w_up = self.w_down = self.b_up = self.b_down = None

    def tensors(self):
        s, n = self.spec, self.spec.names
        d = {n["up"]: TensorDecl((s.intermediate, s.hidden)), n["down"]: TensorDecl((s.hidden, s.intermediate))}
        if s.bias:
            d[n["up_bias"]] = TensorDecl((s.intermediate,), "bias")
            d[n["down_bias"]] = TensorDecl((s.hidden,), "bias")
        return d

    def bind(self, t):
        s, n = self.spec, self.spec.names
        kw = dict(device=self.device, dtype=self.dtype)
        self.w_up = t[n["up"]].to(**kw).contiguous()
        self.w_down = t[n["down"]].to(**kw).contiguous()
        if s.bias:
            self.b_up = t[n["up_bias"]].to(**kw).contiguous()
            self.b_down = t[n["down_bias"]].to(**kw).contiguous()

    def kernels(self):
        return [("gemm_sm100" if self.dtype == torch.bfloat16 else "gemm_f32", None), ("elementwise", None)]

    def forward(self, x, ctx):
        s = self.spec
        act = ctx.ws.buf("ffn_act", x.shape[0], s.intermediate, self.dtype)
        ops.linear_relu_squared(x, self.w_up, self.b_up, act)
        return ops.linear_to_residual(act, self.w_down, self.b_down, ctx.ws, "ffn_out", residual=ctx.residual)
