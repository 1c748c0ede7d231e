"""Short causal convolutions over a request's time axis."""

from __future__ import annotations

import torch

from ..kernels import api as K
from .base import Part, StateNeed, StepContext, register_part


class ResidualShortConv(Part):
    """h <- h + conv(h): a causal convolution on each channel alone, ``weight`` [D, taps], no bias:
    conv(h)_t = sum_j weight[:, j] * h_(t - taps + 1 + j), with h = 0 at negative times.  The last taps - 1
    inputs of a request are its state (float32), so a sequence may come in portions of any size.  Input and sums are
    float32; the output has the activations' type."""

    kernel_libraries = ("group_norm",)

    def __init__(self, weight: torch.Tensor):
        self.weight = weight.to(torch.float32).contiguous()
        self.width, self.taps = weight.shape

    def state_need(self) -> StateNeed | None:
        return StateNeed((self.taps - 1, self.width), torch.float32) if self.taps > 1 else None

    def forward(self, ctx: StepContext, h32: torch.Tensor, state: torch.Tensor | None) -> torch.Tensor:
        out = torch.empty(h32.shape, dtype=ctx.runtime.dtype, device=h32.device)
        K.short_conv(h32, self.weight, state, ctx.cu_q, ctx.q_start, ctx.slot_ids, ctx.req_of_token, ctx.positions, out)
        return out


register_part("conv", "residual_short", ResidualShortConv)
