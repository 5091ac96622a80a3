"""Block arrangements: how norms, mixer and feed-forward sit around the residual stream."""
from __future__ import annotations

from . import registry
from .registry import register


@register("block", "prenorm")
class PreNormBlock:
    """r = x + mixer(norm1(x));  y = r + ffn(norm2(r)).

    The residual stream ``h`` is float32.  A block receives the previous block's
    feed-forward output as ``pending`` (not yet added) so that each residual sum rides in the
    norm kernel that follows it; it returns its own feed-forward output the same way.
    ``spec.ffn`` None: the layer has no feed-forward (and no second norm).  A part's tensor with the relative
    name "" is stored under the part's own name.
    Reference: gpu/engine/conv_layer.cu:220,328-341 and gpu/engine/layer.cu:1662-1765.
    """

    def __init__(self, spec, *, dtype, device, owns_cache=True):
        self.spec, self.dtype = spec, dtype
        kw = dict(dtype=dtype, device=device)
        mixer_kw = dict(kw)
        if not owns_cache:
            mixer_kw["owns_cache"] = False
        self.mixer = registry.build("mixer", spec.mixer, **mixer_kw)
        self.ffn = registry.build("ffn", spec.ffn, **kw) if spec.ffn is not None else None
        self.mixer_norm = registry.build("norm", spec.mixer_norm, **kw)
        self.ffn_norm = registry.build("norm", spec.ffn_norm, **kw) if spec.ffn is not None else None

    def parts(self):
        n = self.spec.names
        roles = {"mixer": self.mixer, "ffn": self.ffn, "mixer_norm": self.mixer_norm, "ffn_norm": self.ffn_norm}
        return {n[r]: p for r, p in roles.items() if p is not None}

    def tensors(self):
        out = {}
        for sub, part in self.parts().items():
            for name, decl in part.tensors().items():
                out[f"{sub}.{name}" if name else sub] = decl
        return out

    def bind(self, t):
        for sub, part in self.parts().items():
            pre = sub + "."
            own = {k[len(pre):]: v for k, v in t.items() if k.startswith(pre)}
            if sub in t:
                own[""] = t[sub]
            part.bind(own)

    def cache_need(self):
        return self.mixer.cache_need()

    def kernels(self):
        return [job for p in self.parts().values() for job in getattr(p, "kernels", list)()]

    @property
    def graph_safe(self):
        return all(getattr(p, "graph_safe", False) for p in self.parts().values())

    def forward(self, h, pending, ctx, cache):
        n, H = h.shape
        buf = ctx.ws.buf("normed", n, H, self.dtype)
        ctx.residual = h if ctx.fuse_residual else None      # parts may add their output into it and return None
        x = self.mixer_norm.forward(h, pending, buf)
        m = self.mixer.forward(x, ctx, cache)
        if self.ffn is None:
            return m
        x = self.ffn_norm.forward(h, m, buf)
        return self.ffn.forward(x, ctx)


@register("block", "prenorm_conv_side")
class PreNormConvSideBlock:
    """Pre-norm with an input convolution in front of each sublayer and a token input behind the layer:

        u = norm1(x);  x += mixer(u + conv1(u));  u = norm2(x);  x += ffn(u + conv2(u));  x += side(x, token)

    ``spec.options``: ``input_conv`` (an InputConvSpec, or None: sublayers read the norm's output) and
    ``token_side`` (a TokenSideSpec or None).  ``spec.ffn`` None: the layer has no feed-forward (and no second
    norm or convolution).  The block keeps, per request, the mixer's cache and each convolution's last inputs:
    it declares a tuple of needs and is handed the views in the same order (mixer, conv1, conv2)."""

    def __init__(self, spec, *, dtype, device, owns_cache=True):
        from .input_conv import InputConv, TokenSide
        self.spec, self.dtype = spec, dtype
        kw = dict(dtype=dtype, device=device)
        opt = spec.options
        self.mixer = registry.build("mixer", spec.mixer, **kw)
        self.mixer_norm = registry.build("norm", spec.mixer_norm, **kw)
        self.ffn = registry.build("ffn", spec.ffn, **kw) if spec.ffn is not None else None
        self.ffn_norm = registry.build("norm", spec.ffn_norm, **kw) if spec.ffn is not None else None
        conv = opt.get("input_conv")
        self.mixer_conv = InputConv(conv, **kw) if conv is not None else None
        self.ffn_conv = InputConv(conv, **kw) if conv is not None and self.ffn is not None else None
        self.side = TokenSide(opt["token_side"], **kw) if opt.get("token_side") is not None else None

    def parts(self):
        n = self.spec.names
        roles = {"mixer": self.mixer, "ffn": self.ffn, "mixer_norm": self.mixer_norm, "ffn_norm": self.ffn_norm,
                 "mixer_conv": self.mixer_conv, "ffn_conv": self.ffn_conv, "side": self.side}
        return {n[r]: p for r, p in roles.items() if p is not None}

    def tensors(self):
        out = {}
        for sub, part in self.parts().items():
            for name, decl in part.tensors().items():
                out[f"{sub}.{name}" if name else sub] = decl
        return out

    def shared_tensors(self):
        return self.side.shared_tensors() if self.side is not None else {}

    def bind(self, t):
        for sub, part in self.parts().items():
            pre = sub + "."
            own = {k[len(pre):]: v for k, v in t.items() if k.startswith(pre)}
            if sub in t:
                own[""] = t[sub]
            part.bind(own)

    def bind_shared(self, weights):
        if self.side is not None:
            self.side.bind_shared(weights)

    def cache_need(self):
        needs = [self.mixer.cache_need()]
        needs += [c.cache_need() for c in (self.mixer_conv, self.ffn_conv) if c is not None]
        return tuple(needs)

    def kernels(self):
        return [job for p in self.parts().values() for job in getattr(p, "kernels", list)()]

    @property
    def graph_safe(self):
        return all(getattr(p, "graph_safe", False) for p in self.parts().values())

    def forward(self, h, pending, ctx, cache):
        from ..csrc import ops
        n, H = h.shape
        views = list(cache)
        mixer_cache = views.pop(0)
        buf = ctx.ws.buf("normed", n, H, self.dtype)
        ctx.residual = h if ctx.fuse_residual else None
        x = self.mixer_norm.forward(h, pending, buf)
        if self.mixer_conv is not None:
            x = self.mixer_conv.forward(x, ctx, views.pop(0), ctx.ws.buf("conv_out", n, H, self.dtype))
        out = self.mixer.forward(x, ctx, mixer_cache)
        if self.ffn is not None:
            x = self.ffn_norm.forward(h, out, buf)
            if self.ffn_conv is not None:
                x = self.ffn_conv.forward(x, ctx, views.pop(0), ctx.ws.buf("conv_out", n, H, self.dtype))
            out = self.ffn.forward(x, ctx)
        if self.side is None:
            return out
        if out is not None:
            ops.residual_add(h, out)              # the token input reads the complete stream
        self.side.forward(h, ctx)
        return None


@register("block", "parallel")
class ParallelBlock:
    """One norm, both sublayers read it:  u = norm(x);  x += mixer(u) + ffn(u).

    When the mixer and the feed-forward both offer their inner activations (``inner_width()``, ``out_weight()`` and
    ``core`` / ``gated``), the two output projections are ONE product: the activations lie side by side in one buffer
    and the two matrices side by side along the contraction (stacked when bound), so the layer adds to the stream
    once.  In a step of few rows that product adds straight into the float32 stream; a bias of the mixer's
    projection is then added by the norm kernel, after it has read the stream.  Otherwise the sublayers run one
    after the other.  ``spec.ffn`` None: the layer has no feed-forward."""

    def __init__(self, spec, *, dtype, device, owns_cache=True):
        self.spec, self.dtype, self.device = spec, dtype, device
        kw = dict(dtype=dtype, device=device)
        mixer_kw = dict(kw)
        if not owns_cache:
            mixer_kw["owns_cache"] = False
        self.mixer = registry.build("mixer", spec.mixer, **mixer_kw)
        self.ffn = registry.build("ffn", spec.ffn, **kw) if spec.ffn is not None else None
        self.norm = registry.build("norm", spec.mixer_norm, **kw)
        self.joint = all(hasattr(self.mixer, a) for a in ("inner_width", "out_weight", "core")) and \
            (self.ffn is None or all(hasattr(self.ffn, a) for a in ("inner_width", "out_weight", "gated")))
        self.w_out = self.b_out = self.b_out_f32 = None

    def parts(self):
        n = self.spec.names
        roles = {"mixer": self.mixer, "ffn": self.ffn, "mixer_norm": self.norm}
        return {n[r]: p for r, p in roles.items() if p is not None}

    def tensors(self):
        out = {}
        for sub, part in self.parts().items():
            for name, decl in part.tensors().items():
                out[f"{sub}.{name}" if name else sub] = decl
        return out

    def bind(self, t):
        import torch
        for sub, part in self.parts().items():
            pre = sub + "."
            own = {k[len(pre):]: v for k, v in t.items() if k.startswith(pre)}
            if sub in t:
                own[""] = t[sub]
            part.bind(own)
        if self.joint:
            w, b = self.mixer.out_weight()
            if self.ffn is not None:
                w2, b2 = self.ffn.out_weight()
                w = torch.cat([w, w2], dim=1).contiguous()
                b = b if b2 is None else (b2 if b is None else b + b2)
            self.w_out, self.b_out = w, b
            self.b_out_f32 = b.to(torch.float32).contiguous() if b is not None else None
            for part in (self.mixer, self.ffn):              # the stacked matrix serves; the parts' own copies go
                if part is not None and self.ffn is not None and hasattr(part, "drop_out_weight"):
                    part.drop_out_weight()

    def cache_need(self):
        return self.mixer.cache_need()

    def kernels(self):
        return [job for p in self.parts().values() for job in getattr(p, "kernels", list)()]

    @property
    def graph_safe(self):
        return all(getattr(p, "graph_safe", False) for p in self.parts().values())

    def forward(self, h, pending, ctx, cache):
        from ..csrc import ops
        n, H = h.shape
        buf = ctx.ws.buf("normed", n, H, self.dtype)
        if not self.joint:
            ctx.residual = h if ctx.fuse_residual else None
            x = self.norm.forward(h, pending, buf)
            m = self.mixer.forward(x, ctx, cache)
            if m is not None:
                ops.residual_add(h, m)
            return self.ffn.forward(x, ctx) if self.ffn is not None else None
        ka = self.mixer.inner_width()
        inner = ctx.ws.buf("parallel_inner", n, self.w_out.shape[1], self.dtype)
        fused = ctx.fuse_residual and ops.residual_add_fusable(inner, self.w_out) and \
            (self.b_out is None or getattr(self.norm, "takes_post", False))
        if fused and self.b_out is not None:
            x = self.norm.forward(h, pending, buf, post=self.b_out_f32)
        else:
            x = self.norm.forward(h, pending, buf)
        self.mixer.core(x, ctx, cache, inner[:, :ka])
        if self.ffn is not None:
            self.ffn.gated(x, ctx, inner[:, ka:])
        if fused:
            return ops.linear_to_residual(inner, self.w_out, None, ctx.ws, "parallel_out", residual=h)
        return ops.linear_to_residual(inner, self.w_out, self.b_out, ctx.ws, "parallel_out")


class HyperPending:
    """What a hyper block leaves for the kernel after it: its last sublayer's output (not yet written into the copies of
    the stream) with the mixing matrix and output weights that write it."""

    def __init__(self, y, mix, out_w, eps):
        self.y, self.mix, self.out_w, self.eps = y, mix, out_w, eps


@register("block", "hyper")
class HyperBlock:
    """Pre-norm with hyper-connections: the residual stream is S copies x_1..x_S (``spec.options["streams"]``).  For
    sublayer q (the mixer, then the feed-forward if there is one), with vectors in_q, out_q [S] and a matrix mix_q [S,S]:

        u = sum_s in_q[s] x_s;   y = sublayer(norm_q(u));   x_t <- sum_s mix_q[s, t] x_s + out_q[t] y   (all t at once)

    The copies are float32 [N, S * H] (the buffer the model hands over as its stream).  One kernel does what lies
    between two sublayers: the update by the sublayer before (also the last one of the layer before, handed over as
    ``pending``), the read-out u and its norm.  The first block of a model receives the embedding output as
    ``pending.x0``: every copy starts as that.  Sublayers hand their outputs over (an activation tensor or a stack of
    float32 partial sums); they never add into the stream themselves, since every copy takes the output times a
    weight of its own."""

    def __init__(self, spec, *, dtype, device, owns_cache=True):
        self.spec, self.dtype, self.device = spec, dtype, device
        self.streams = int(spec.options["streams"])
        kw = dict(dtype=dtype, device=device)
        mixer_kw = dict(kw)
        if not owns_cache:
            mixer_kw["owns_cache"] = False
        self.mixer = registry.build("mixer", spec.mixer, **mixer_kw)
        self.ffn = registry.build("ffn", spec.ffn, **kw) if spec.ffn is not None else None
        self.mixer_norm = registry.build("norm", spec.mixer_norm, **kw)
        self.ffn_norm = registry.build("norm", spec.ffn_norm, **kw) if spec.ffn is not None else None
        self.hc = {}

    def parts(self):
        n = self.spec.names
        roles = {"mixer": self.mixer, "ffn": self.ffn, "mixer_norm": self.mixer_norm, "ffn_norm": self.ffn_norm}
        return {n[r]: p for r, p in roles.items() if p is not None}

    def _hc_names(self):
        n = self.spec.names
        return [n["mixer_hc"]] + ([n["ffn_hc"]] if self.ffn is not None else [])

    def tensors(self):
        from ..weights.decl import TensorDecl
        out, S = {}, self.streams
        for sub, part in self.parts().items():
            for name, decl in part.tensors().items():
                out[f"{sub}.{name}" if name else sub] = decl
        for hc in self._hc_names():
            out[hc + ".in"] = TensorDecl((S,), "share")
            out[hc + ".out"] = TensorDecl((S,), "norm")
            out[hc + ".mix"] = TensorDecl((S, S), "eye")
        return out

    def bind(self, t):
        import torch
        for sub, part in self.parts().items():
            pre = sub + "."
            own = {k[len(pre):]: v for k, v in t.items() if k.startswith(pre)}
            if sub in t:
                own[""] = t[sub]
            part.bind(own)
        f32 = dict(device=self.device, dtype=torch.float32)
        for hc in self._hc_names():
            self.hc[hc] = tuple(t[f"{hc}.{k}"].to(**f32).contiguous() for k in ("in", "out", "mix"))

    def cache_need(self):
        return self.mixer.cache_need()

    def kernels(self):
        return [("hyper", None)] + [job for p in self.parts().values() for job in getattr(p, "kernels", list)()]

    @property
    def graph_safe(self):
        return all(getattr(p, "graph_safe", False) for p in self.parts().values())

    def _between(self, X, pending, hc, norm, buf):
        """The update by the sublayer before, then the read-out through ``hc``'s weights and ``norm``."""
        from ..csrc import ops
        w_in = self.hc[hc][0]
        kw = dict(in_w=w_in, norm_w=norm.weight, out=buf, eps=norm.spec.eps)
        if isinstance(pending, HyperStart):
            ops.hc_step(X, self.streams, x0=pending.x0, **kw)
        elif pending is None:
            ops.hc_step(X, self.streams, **kw)
        else:
            ops.hc_step(X, self.streams, delta=pending.y, mix=pending.mix, out_w=pending.out_w, **kw)
        return buf

    def forward(self, X, pending, ctx, cache):
        n = X.shape[0]
        H = X.shape[1] // self.streams
        buf = ctx.ws.buf("normed", n, H, self.dtype)
        ctx.residual = None                                  # sublayers hand their outputs over
        names = self._hc_names()
        x = self._between(X, pending, names[0], self.mixer_norm, buf)
        y = self.mixer.forward(x, ctx, cache)
        pending = HyperPending(y, self.hc[names[0]][2], self.hc[names[0]][1], self.spec.mixer_norm.eps)
        if self.ffn is not None:
            x = self._between(X, pending, names[1], self.ffn_norm, buf)
            y = self.ffn.forward(x, ctx)
            pending = HyperPending(y, self.hc[names[1]][2], self.hc[names[1]][1], self.spec.ffn_norm.eps)
        return pending


class HyperStart:
    """Handed to a model's first hyper block: every copy of the stream starts as ``x0`` [N, H] float32."""

    def __init__(self, x0):
        self.x0 = x0
