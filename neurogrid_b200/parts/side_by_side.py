"""Two mixers on one input: their normed outputs averaged, or their outputs in a weighted sum."""
from __future__ import annotations

import torch

from ..csrc import ops
from ..weights.decl import TensorDecl
from . import registry
from .registry import register


@register("mixer", "side_by_side")
class SideBySide:
    """y = 0.5 * (rmsnorm(left(x)) * w_left + rmsnorm(right(x)) * w_right): both mixers read the same x, each output is
    divided by its root mean square over the model width and multiplied by a plain weight; sums and norms float32.
    The mixer's cache needs are its parts' needs one after the other (left's, then right's), and it is handed the views
    in that order.  In a step of few rows the result is added into the float32 stream here.

    ``spec.combine`` "weighted": y = left_scale * left(x) + right_scale * right(x).  Both mixers end with a projection
    into the stream, so their inner activations (each times its scale, in float32, before its one rounding) lie side
    by side in one buffer and ONE product with the two output matrices side by side along the contraction (stacked
    when bound) is the weighted sum; both parts must offer ``core``, ``inner_width`` and ``out_weight``."""

    def __init__(self, spec, *, dtype, device, owns_cache=True):
        self.spec, self.dtype, self.device = spec, dtype, device
        kw = dict(dtype=dtype, device=device)
        self.left = registry.build("mixer", spec.left, **kw)
        self.right = registry.build("mixer", spec.right, **kw)
        self.w_left = self.w_right = self.w_out = None
        self.weighted = getattr(spec, "combine", "norm_mean") == "weighted"
        if self.weighted:
            for part in (self.left, self.right):
                if not all(hasattr(part, a) for a in ("core", "inner_width", "out_weight")):
                    raise ValueError(f"side by side: a weighted sum needs the inner activations of {type(part).__name__}")

    def _sides(self):
        n = self.spec.names
        return ((n["left"], self.left), (n["right"], self.right))

    def tensors(self):
        s, n = self.spec, self.spec.names
        out = {} if self.weighted else {n["left_out"]: TensorDecl((s.hidden,), "norm"),
                                        n["right_out"]: TensorDecl((s.hidden,), "norm")}
        for sub, part in self._sides():
            for name, decl in part.tensors().items():
                out[f"{sub}.{name}"] = decl
        return out

    def bind(self, t):
        n = self.spec.names
        f32 = dict(device=self.device, dtype=torch.float32)
        own = ()
        if not self.weighted:
            self.w_left = t[n["left_out"]].to(**f32).contiguous()
            self.w_right = t[n["right_out"]].to(**f32).contiguous()
            own = (n["left_out"], n["right_out"])
        for sub, part in self._sides():
            pre = sub + "."
            part.bind({k[len(pre):]: v for k, v in t.items() if k.startswith(pre) and k not in own})
        if self.weighted:
            (wl, bl), (wr, br) = self.left.out_weight(), self.right.out_weight()
            if bl is not None or br is not None:
                raise ValueError("side by side: a weighted sum takes output projections without biases")
            self.w_out = torch.cat([wl, wr], dim=1).contiguous()
            for part in (self.left, self.right):             # the stacked matrix serves; the parts' own copies go
                if hasattr(part, "drop_out_weight"):
                    part.drop_out_weight()

    @staticmethod
    def _flat(need):
        return () if need is None else tuple(need) if isinstance(need, tuple) else (need,)

    def cache_need(self):
        return self._flat(self.left.cache_need()) + self._flat(self.right.cache_need())

    @staticmethod
    def _views(need, views):
        """The views a part expects for its need: none, one, or a tuple."""
        if need is None:
            return None
        return tuple(views) if isinstance(need, tuple) else views[0]

    def kernels(self):
        return [("elementwise", None)] + self.left.kernels() + self.right.kernels()

    def scratch_bytes_per_row(self):
        return sum(getattr(p, "scratch_bytes_per_row", lambda: 0)() for p in (self.left, self.right)) + 4 * self.spec.hidden

    @property
    def graph_safe(self):
        return bool(getattr(self.left, "graph_safe", False) and getattr(self.right, "graph_safe", False))

    def forward(self, x, ctx, cache):
        s = self.spec
        views = list(cache)
        n_left = len(self._flat(self.left.cache_need()))
        if self.weighted:
            ka = self.left.inner_width()
            inner = ctx.ws.buf("side_inner", x.shape[0], self.w_out.shape[1], self.dtype)
            self.left.core(x, ctx, self._views(self.left.cache_need(), views[:n_left]), inner[:, :ka], out_scale=s.left_scale)
            self.right.core(x, ctx, self._views(self.right.cache_need(), views[n_left:]), inner[:, ka:], out_scale=s.right_scale)
            return ops.linear_to_residual(inner, self.w_out, None, ctx.ws, "mixer_out", residual=ctx.residual)
        residual, ctx.residual = ctx.residual, None        # the parts hand their outputs over; the sum is formed here
        try:
            a = self.left.forward(x, ctx, self._views(self.left.cache_need(), views[:n_left]), out_name="side_left")
            b = self.right.forward(x, ctx, self._views(self.right.cache_need(), views[n_left:]), out_name="side_right")
        finally:
            ctx.residual = residual
        if residual is not None:
            ops.pair_norm_mean(a, b, self.w_left, self.w_right, residual, s.eps, self.dtype, accumulate=True)
            return None
        y = ctx.ws.buf("side_mean", x.shape[0], s.hidden, torch.float32)
        ops.pair_norm_mean(a, b, self.w_left, self.w_right, y, s.eps, self.dtype)
        return y.unsqueeze(0)               # a float32 stack of one: the norm that follows adds it in float32
