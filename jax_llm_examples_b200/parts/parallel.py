"""Several mixers side by side on the same input, their outputs added with a weight each."""

from __future__ import annotations

import torch

from ..tracing import scope
from .base import LayerCache, Mixer, ProjectedMixer, StepContext, as_rows, register_part
from .linear import linear


class ParallelMixers(Mixer):
    """out = sum_i scale_i * mixer_i(h) for mixers of the form W_o core(W_in h) (:class:`ProjectedMixer`).

    The mixers' W_in are stacked into one product over h, every core writes scale_i times its rows into its own column
    range of one buffer, and the W_o laid side by side turn that buffer into the weighted sum: two products for the
    whole layer, and no kernel that adds.  At most one of the mixers may keep keys and values in pages; their
    per-request states follow one another in the order of the mixers.

    Between the two products the mixers do not depend on one another: with ``overlap``, in steps of few rows (decoding)
    the first runs on the step's own stream and the others on the workspace's second stream (a branch of a captured
    graph), so that the step's chain of dependent launches is as long as the longest mixer's, not their sum (decode
    at batch 8: 0.97 -> 0.88 ms for eight layers at width 2048).  Prompt portions run them one after the other:
    side by side, a persistent attention kernel and a recurrence that walks its tokens in order slowed each other
    down (a 2048-token prompt step 6.7 -> 7.6 ms)."""

    OVERLAP_MAX_ROWS = 256

    def __init__(self, mixers: list[ProjectedMixer], scales: list[float], overlap: bool = True):
        if len(mixers) != len(scales) or not mixers:
            raise ValueError("one scale per mixer is needed")
        if sum(m.kv_need() is not None for m in mixers) > 1:
            raise ValueError("at most one of the mixers side by side may keep keys and values")
        self.mixers, self.scales, self.overlap = list(mixers), [float(s) for s in scales], bool(overlap)
        self.sizes = [(m.in_features, m.out_features) for m in mixers]
        self.w_in = torch.cat([m.w_in for m in mixers], dim=0).contiguous()
        self.w_o = torch.cat([m.w_o for m in mixers], dim=1).contiguous()
        for m in mixers:  # the stacked copies are the ones in use
            m.w_in = m.w_o = None

    def sub_parts(self):
        return tuple(self.mixers)

    def kv_need(self):
        for m in self.mixers:
            if m.kv_need() is not None:
                return m.kv_need()
        return None

    def state_needs(self):
        return tuple(s for m in self.mixers for s in m.state_needs())

    def forward(self, ctx: StepContext, h: torch.Tensor, cache: LayerCache):
        with scope("qkv_matmul"):
            proj = as_rows(linear(ctx, h, self.w_in, torch.float32, partials=True))
        out = torch.empty((h.shape[0], self.w_o.shape[1]), dtype=ctx.runtime.dtype, device=h.device)
        col_in = col_out = at_state = 0
        calls = []
        for m, scale, (f_in, f_out) in zip(self.mixers, self.scales, self.sizes):
            n_state = len(m.state_needs())
            states = tuple(cache.states[at_state:at_state + n_state])
            has_kv = m.kv_need() is not None
            sub = LayerCache(cache.pages if has_kv else None, cache.block_table if has_kv else None, cache.writes and has_kv,
                             states[0] if states else None, states)
            calls.append((m, col_in, sub, out[:, col_out:col_out + f_out], scale))
            col_in, col_out, at_state = col_in + f_in, col_out + f_out, at_state + n_state
        side = None
        if self.overlap and len(calls) > 1 and ctx.workspace is not None and h.is_cuda and h.shape[0] <= self.OVERLAP_MAX_ROWS:
            main, side = torch.cuda.current_stream(), ctx.workspace.side_stream()
            side.wait_stream(main)  # the stacked projection is there
            with torch.cuda.stream(side):
                for m, col, sub, view, scale in calls[1:]:
                    m.core(ctx, h, proj, col, sub, view, scale)
            calls = calls[:1]
        for m, col, sub, view, scale in calls:
            m.core(ctx, h, proj, col, sub, view, scale)
        if side is not None:
            torch.cuda.current_stream().wait_stream(side)
        with scope("projection"):
            return linear(ctx, out, self.w_o, torch.float32, partials=True)


register_part("mixer", "parallel", ParallelMixers)
