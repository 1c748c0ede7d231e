"""Mixers that carry a fixed-size state from token to token instead of keys and values."""

from __future__ import annotations

import torch

import numpy as np

from ..kernels import api as K
from ..tracing import scope
from .base import LayerCache, Mixer, StateNeed, StepContext, StepShape, as_rows, register_part
from .conv import ResidualShortConv
from .linear import linear


class InputConvMixer(Mixer):
    """Base of mixers whose input may first pass a short convolution (``input_conv``): they take the normed rows
    unrounded, and the convolution's state is the first of their states."""

    needs_f32_input = True
    input_conv: ResidualShortConv | None = None

    def own_state_needs(self) -> tuple:
        return ()

    def state_needs(self) -> tuple:
        conv = self.input_conv.state_need() if self.input_conv is not None else None
        return (() if conv is None else (conv,)) + tuple(self.own_state_needs())

    def sub_parts(self):
        return () if self.input_conv is None else (self.input_conv,)

    def read_input(self, ctx: StepContext, h32: torch.Tensor, cache: LayerCache):
        """(rows in the activations' type, the mixer's own state slabs)."""
        states = cache.states
        if self.input_conv is None:
            return h32.to(ctx.runtime.dtype), states
        if self.input_conv.state_need() is None:
            return self.input_conv.forward(ctx, h32, None), states
        return self.input_conv.forward(ctx, h32, states[0]), states[1:]


SEGMENT_TOKENS = 256  # tokens of a long portion that one block of the recurrence kernel walks


def plan_scan_segments(shape: StepShape) -> dict:
    """The step planner of the recurrences: when a request brings a long portion (at least two segments), the step's
    tokens cut into segments of SEGMENT_TOKENS, int32 [n, 4] = (request, first row, end row, flags: 1 = the request's
    first segment, 2 = the request has several).  A recurrence over time gives the GPU only its state's parallelism;
    segments scanned at once from a zero state, and corrected afterwards, multiply it by their number.  Steps of short
    portions and single tokens get no list (their tokens are walked in order, one block per request and head)."""
    if max(shape.q_lens) < 2 * SEGMENT_TOKENS:
        return {}
    segs, n0 = [], 0
    for r, T in enumerate(shape.q_lens):
        if T >= 2 * SEGMENT_TOKENS:
            for c in range(0, T, SEGMENT_TOKENS):
                segs.append((r, n0 + c, n0 + min(T, c + SEGMENT_TOKENS), (1 if c == 0 else 0) | 2))
        else:
            segs.append((r, n0, n0 + T, 1))
        n0 += T
    return {"scan_segments": np.array(segs, dtype=np.int32).reshape(-1, 4)}


class HGRN2(InputConvMixer):
    """Gated linear recurrence with a matrix state per head, whose forget gate f doubles as the write gate 1 - f
    (keys do not exist in this form):  q = silu(W_q h), v = W_v h, f = lower + (1 - lower) * sigmoid(W_f h + b_f);
    S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T;  o_t = S_t^T q_t;  each head's o is RMS-normed over its value size with
    one weight shared by the heads, and the heads go through W_o.  Gates, state and norm are float32.

    ``w_qfv``: [2 H dk + H dv, D], the q, f and v projections stacked in that order."""

    kernel_libraries = ("recurrent", "gemm_simt")
    kernel_libraries_bf16 = ("gemm_stream",)

    def __init__(self, w_qfv: torch.Tensor, f_bias: torch.Tensor, lower: torch.Tensor, norm_weight: torch.Tensor,
                 w_o: torch.Tensor, heads: int, dim: int, vdim: int, eps: float, input_conv: ResidualShortConv | None = None):
        if w_qfv.shape[0] != heads * (2 * dim + vdim) or w_o.shape[1] != heads * vdim or f_bias.numel() != heads * dim \
                or lower.numel() != heads * dim or norm_weight.numel() != vdim:
            raise ValueError(f"HGRN2 weights do not fit {heads} heads of {dim} x {vdim}: qfv {tuple(w_qfv.shape)}, o {tuple(w_o.shape)}")
        self.w_qfv, self.w_o = w_qfv, w_o
        self.f_bias, self.lower = f_bias.to(torch.float32).contiguous(), lower.to(torch.float32).contiguous()
        self.norm_weight = norm_weight.to(torch.float32).contiguous()
        self.heads, self.dim, self.vdim, self.eps = heads, dim, vdim, float(eps)
        self.input_conv = input_conv

    def own_state_needs(self):
        return (StateNeed((self.heads, self.dim, self.vdim), torch.float32),)

    def step_planners(self):
        return (plan_scan_segments,)

    def forward(self, ctx: StepContext, h, cache: LayerCache, h32: torch.Tensor | None = None):
        a, (state,) = self.read_input(ctx, h32, cache)
        with scope("qkv_matmul"):
            qfv = as_rows(linear(ctx, a, self.w_qfv, torch.float32, partials=True))
        o = torch.empty((a.shape[0], self.heads * self.vdim), dtype=ctx.runtime.dtype, device=a.device)
        with scope("attention"):
            segs = ctx.arrays.get("scan_segments")
            n_seg = 0 if segs is None else segs.numel() // 4
            need = K.hgrn2_scan_scratch(a.shape[0], self.heads, self.dim, self.vdim, n_seg)
            scratch = ctx.workspace.get("hgrn2_scan", need, torch.float32) if ctx.workspace else None
            K.hgrn2_scan(qfv.data, qfv.splits, self.f_bias, self.lower, state, ctx.cu_q, ctx.slot_ids, self.norm_weight,
                         self.eps, o, self.heads, self.dim, self.vdim, scratch, segs if n_seg else None, n_seg, SEGMENT_TOKENS)
        with scope("projection"):
            return linear(ctx, o, self.w_o, torch.float32, partials=True)


register_part("mixer", "hgrn2", HGRN2)
