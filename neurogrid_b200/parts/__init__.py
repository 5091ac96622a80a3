from . import attention, block, gated_delta, gated_linear, input_conv, mlp, side_by_side, latent_attention, mapped_attention, moe, norm, position, retention, shortconv, swiglu  # noqa: F401  (registers the parts)
from .base import PagedView, PositionArgs, SlotView, StepContext, Workspace
from .registry import build, register, registered
