"""RMSNorm with the residual sum fused in front of it."""
from __future__ import annotations

import torch

from ..csrc import ops
from ..weights.decl import TensorDecl
from .registry import register


@register("norm", "rmsnorm")
class RMSNorm:
    """y = x * rsqrt(mean(x^2) + eps) * w, everything float32 until the one rounding of y.

    Reference: gpu/cuda/bf16_utils.cu:57-93 (norm), gpu/cuda/kernels.cu:196-262 (fused add).
    """

    graph_safe = True      # launches depend on device data and on launch-time constants only

    def __init__(self, spec, *, dtype, device):
        self.spec, self.dtype, self.device = spec, dtype, device
        self.weight = None

    def tensors(self):
        return {getattr(self.spec, "tensor", "weight"): TensorDecl((self.spec.size,), "norm")}

    def bind(self, t):
        self.weight = t[getattr(self.spec, "tensor", "weight")].to(device=self.device, dtype=torch.float32).contiguous()

    def kernels(self):
        return [("elementwise", None)]

    def forward(self, h, delta, out, rows=None):
        ops.add_rmsnorm(h, delta, self.weight, out, self.spec.eps, rows)
        return out


@register("norm", "rmsnorm_scalar")
class ScalarRMSNorm(RMSNorm):
    """y = x * rsqrt(mean(x^2) + eps) * g with one gain g for all coordinates.  The gain's tensor has no
    dimensions and the relative name "": it is stored under the norm's own name.  It is spread to a
    vector when bound, so the kernel of :class:`RMSNorm` (residual sum in front, float32 throughout) serves."""

    def tensors(self):
        return {"": TensorDecl((), "norm")}

    def bind(self, t):
        g = t[""].to(device=self.device, dtype=torch.float32).reshape(1)
        self.weight = g.expand(self.spec.size).contiguous()


@register("norm", "layernorm")
class LayerNorm(RMSNorm):
    """y = (x - mean(x)) * rsqrt(var(x) + eps) * w with the variance as the mean of the squared deviations, a weight
    and no bias; float32 until the one rounding of y, the residual sum in front as for :class:`RMSNorm`.
    ``post`` (float32 [H]) is added to the stream after the norm has read it."""

    takes_post = True

    def tensors(self):
        return {self.spec.tensor: TensorDecl((self.spec.size,), "norm")}

    def bind(self, t):
        self.weight = t[self.spec.tensor].to(device=self.device, dtype=torch.float32).contiguous()

    def forward(self, h, delta, out, rows=None, post=None):
        ops.add_layernorm(h, delta, self.weight, out, self.spec.eps, rows, post)
        return out
