"""Position encodings, as parameters of the q/k kernel."""
from __future__ import annotations

import math

import torch

from .base import PositionArgs
from .registry import register


@register("position", "rope")
class Rope:
    """angle(pos, i) = (pos / scale) * theta^(-2i/dims); pairs (2i, 2i+1) or (i, i+dims/2), dims = the head's
    size or, for a partial rotation, ``rotary_dims`` (the frequency table then has rotary_dims/2 entries).

    Reference: gpu/cuda/bf16_utils.cu:330-378.  The frequencies are formed in float64 on the
    host and rounded once; the angle and its sine and cosine are float32 on the device.
    """

    def __init__(self, spec, *, device):
        self.spec = spec
        dims = spec.head_dim if spec.rotary_dims is None else spec.rotary_dims
        i = torch.arange(dims // 2, dtype=torch.float64)
        f = float(spec.theta) ** (-2.0 * i / max(dims, 1))
        if spec.freq_scaling is not None:                  # by wavelength: short ones stay, long ones are divided, a blend between
            factor, low, high, original = (float(v) for v in spec.freq_scaling)
            wavelength = 2.0 * math.pi / f
            s = (original / wavelength - low) / (high - low) if high != low else torch.ones_like(f)
            blend = (1.0 - s) * f / factor + s * f
            f = torch.where(wavelength < original / high, f, torch.where(wavelength > original / low, f / factor, blend))
        self.inv_freq = f.to(torch.float32).to(device)

    def kernel_args(self):
        return PositionArgs(self.inv_freq, self.spec.pairing == "half", float(self.spec.scale),
                            rotary_dims=self.spec.rotary_dims)


@register("position", "distance_bias")
class DistanceBias:
    """No rotation; slope_h * (query position - key position) is taken off head h's scores,
    slope_h = 2^(-exponent * (h + 1) / n_heads) (formed in float64, rounded once)."""

    def __init__(self, spec, *, device):
        self.spec = spec
        h = torch.arange(1, spec.n_heads + 1, dtype=torch.float64)
        self.slopes = torch.pow(2.0, -float(spec.exponent) * h / spec.n_heads).to(torch.float32).to(device)

    def kernel_args(self):
        return PositionArgs(score_slopes=self.slopes)


@register("position", "none")
class NoPosition:
    def __init__(self, spec, *, device):
        self.spec = spec

    def kernel_args(self):
        return PositionArgs()
