"""Attention over one cached latent per token, from which every head's keys and values are made."""

from __future__ import annotations

import functools

import numpy as np
import torch

from ..cache.manager import Retention
from ..kernels import api as K
from ..tracing import scope
from .attention import plan_attention_tiles
from .base import KVNeed, LayerCache, StepContext, StepShape, as_rows, register_part
from .conv import ResidualShortConv
from .linear import grouped_linear, linear
from .recurrent import InputConvMixer


def rotary_frequencies(base: float, dims: int) -> torch.Tensor:
    """f_i = base^(-2i / dims), i < dims / 2, evaluated in float64 and rounded once to float32."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    return (float(base) ** (-2.0 * i / dims)).to(torch.float32)


@functools.lru_cache(maxsize=None)
def plan_head_groups(heads: int):
    """The step planner for per-head products over head-major rows [H, N, ...]: the row offsets h * N of the heads'
    groups (one planner per head count; mixers with the same count share it)."""
    name = f"head_group_offsets_{heads}"

    def planner(shape: StepShape) -> dict[str, np.ndarray]:
        n = int(sum(shape.q_lens))
        return {name: np.arange(heads + 1, dtype=np.int32) * n}

    planner.array_name = name
    return planner


class LatentAttention(InputConvMixer):
    """Causal attention with low-rank queries and ONE cached latent per token.

    c_q = RMSnorm(W_dq h) * w_qn;  q = W_uq c_q, per head [dn unrotated | dr rotated].
    W_dkv h = [c_pre (rank) | k_rot (dr)];  c = RMSnorm(c_pre) * w_kvn;  k_rot is rotated and shared by all heads.
    Per head: k_nope = W_uk c, v = W_uv c;  score = (q_nope . k_nope + q_rot . k_rot) * scale;  the softmax's
    denominator also holds exp(sink_h) (no key, no value);  out = W_o [heads' weighted values].

    Only [c | k_rot] is cached (``planes`` = 1, one "head" of rank + dr).  The kernels work in the latent space:
    q_lat = W_uk[h]^T q_nope (a product per head), scores and weighted sums against the cached rows, then
    v = W_uv[h] out_lat (a product per head).  Rotation: the first ``rot_dims`` entries of the rotated part, in pairs
    (2i, 2i+1), by position * rot_base^(-2i / rot_dims).

    ``w_down``: [q_rank + rank + dr, D] = W_dq over W_dkv.  ``w_uk``: [H dn, rank]; ``w_uv``: [H dv, rank]."""

    kernel_libraries = ("attention_latent", "gemm_simt")
    kernel_libraries_bf16 = ("gemm_stream",)

    def __init__(self, w_down: torch.Tensor, q_norm_weight: torch.Tensor, w_uq: torch.Tensor, kv_norm_weight: torch.Tensor,
                 w_uk: torch.Tensor, w_uv: torch.Tensor, w_o: torch.Tensor, sink: torch.Tensor | None, heads: int, dim: int,
                 rot_dim: int, vdim: int, q_rank: int, kv_rank: int, scale: float, rot_base: float, rot_dims: int, eps: float,
                 input_conv: ResidualShortConv | None = None):
        H, dn, dr, dv = heads, dim, rot_dim, vdim
        ok = (w_down.shape[0] == q_rank + kv_rank + dr and tuple(w_uq.shape) == (H * (dn + dr), q_rank)
              and tuple(w_uk.shape) == (H * dn, kv_rank) and tuple(w_uv.shape) == (H * dv, kv_rank)
              and w_o.shape[1] == H * dv and q_norm_weight.numel() == q_rank and kv_norm_weight.numel() == kv_rank
              and (sink is None or sink.numel() == H))
        if not ok:
            raise ValueError(f"latent attention weights do not fit {H} heads of {dn}+{dr}/{dv}, ranks {q_rank}/{kv_rank}")
        if rot_dims % 2 or not 0 <= rot_dims <= dr:
            raise ValueError(f"{rot_dims} rotated entries of a rotated part of {dr}")
        self.w_down, self.w_uq, self.w_o = w_down, w_uq, w_o
        self.q_norm_weight = q_norm_weight.to(torch.float32).contiguous()
        self.kv_norm_weight = kv_norm_weight.to(torch.float32).contiguous()
        # per head: q_lat = W_uk[h]^T q_nope needs [rank, dn] as the product's [out, in]; v = W_uv[h] out_lat has it already
        self.w_uk_t = w_uk.reshape(H, dn, kv_rank).transpose(1, 2).contiguous()
        self.w_uv = w_uv.reshape(H, dv, kv_rank).contiguous()
        # prompt portions (bfloat16) up-project keys and values of all heads in one product
        self.w_ukv = torch.cat([w_uk, w_uv], dim=0).contiguous() if w_uk.dtype == torch.bfloat16 else None
        self.sink = None if sink is None else sink.to(torch.float32).contiguous()
        self.heads, self.dim, self.rot_dim, self.vdim = H, dn, dr, dv
        self.q_rank, self.kv_rank, self.scale, self.eps = q_rank, kv_rank, float(scale), float(eps)
        self.rot_dims = rot_dims
        self.inv_freq = rotary_frequencies(rot_base, rot_dims).to(w_down.device) if rot_dims else \
            torch.zeros(1, dtype=torch.float32, device=w_down.device)
        self.input_conv = input_conv
        self._planner = plan_head_groups(H)

    def kv_need(self) -> KVNeed:
        return KVNeed(1, self.kv_rank + self.rot_dim, Retention.all(), planes=1)

    def step_planners(self):
        # the attention part's planner gives the rows of the single decoded tokens of a mixed step
        return (self._planner, plan_attention_tiles)

    # Scores of a prompt portion are made as one [H, T, L] float32 tensor per query tile; this bounds its size.
    SCORE_TILE_BYTES = 1 << 30
    QUERY_TILE = 512  # query rows of a portion per score product
    MIN_SPLIT_KEYS = 64
    SPLIT_ROUNDS = 2  # blocks per multiprocessor that the key ranges of a decode step aim at

    def _latent_space(self, ctx: StepContext, q_lat, q_rot, cache: LayerCache, out_lat, rows=None, n_rows: int = 0) -> None:
        """The latent-space kernel for all token rows, or the listed ones.  Few rows (decoding): the keys are cut into
        ranges so that about two rounds of blocks fill the GPU; a second kernel adds the ranges."""
        H = self.heads
        served = n_rows if rows is not None else q_rot.shape[0]
        per_block = 8 * (2 if self.kv_rank > 512 else 4)  # heads a block of the kernel serves (csrc/attention_latent.cu)
        blocks = served * -(-H // per_block)
        want = max(1, (self.SPLIT_ROUNDS * K.sm_count()) // max(blocks, 1))
        tile = K.LATENT_KEY_TILE
        per_split = -(-ctx.max_kv_len // want)  # keys each range would hold, rounded up to whole tiles below
        split_keys = max(self.MIN_SPLIT_KEYS, -(-per_split // tile) * tile)
        splits = -(-ctx.max_kv_len // split_keys)
        part_acc = part_ml = None
        if splits > 1:
            part_acc = ctx.workspace.get("latent_part_acc", served * H * splits * self.kv_rank, torch.float32)
            part_ml = ctx.workspace.get("latent_part_ml", served * H * splits * 2, torch.float32)
        K.attention_latent(q_lat, q_rot, cache.pages, cache.block_table, ctx.req_of_token, ctx.positions, self.sink, out_lat,
                           self.scale, ctx.status, rows, n_rows, splits, split_keys, part_acc, part_ml)

    def _portion(self, ctx: StepContext, cache: LayerCache, r: int, n0: int, T: int, start: int, q_full, rows_out) -> None:
        """One request's prompt portion (rows n0 .. n0 + T, positions start ..) on the tensor cores: the request's cached
        rows gathered, every head's keys and values up-projected from them (the library's product), scores and weighted
        sums as per-head products (the library's, bfloat16 in, 32-bit sums), and between them this package's softmax
        with the causal edge and the sink, in 32-bit."""
        dt, dev = q_full.dtype, q_full.device
        H, dn, dr, dv = self.heads, self.dim, self.rot_dim, self.vdim
        keys = start + T
        L = -(-keys // 8) * 8  # rows in multiples of 8 for the products; the padding is zero and no query sees it
        c = torch.empty((L, self.kv_rank), dtype=dt, device=dev)
        kr = torch.empty((L, dr), dtype=dt, device=dev)
        c[keys:].zero_()
        kr[keys:].zero_()
        K.latent_gather(cache.pages, cache.block_table[r], c[:keys], kr[:keys], ctx.status)
        kv_up = linear(ctx, c, self.w_ukv, dt)  # [L, H dn + H dv]
        k = torch.empty((H, L, dn + dr), dtype=dt, device=dev)
        K.latent_key_assemble(kv_up, kr, k, H, dn)
        v = kv_up[:, H * dn:].unflatten(1, (H, dv)).permute(1, 0, 2)  # [H, L, dv], a view
        # query tiles: each sees the keys up to its own last row only (the rest of the causal triangle is not computed)
        tile = max(16, min(self.QUERY_TILE, self.SCORE_TILE_BYTES // (4 * H * L)))
        for t0 in range(0, T, tile):
            t1 = min(T, t0 + tile)
            Lt = min(L, -(-(start + t1) // 8) * 8)
            scores = torch.bmm(q_full[:, n0 + t0:n0 + t1], k[:, :Lt].transpose(1, 2), out_dtype=torch.float32)  # [H, t, Lt]
            probs = torch.empty(scores.shape, dtype=dt, device=dev)
            K.causal_sink_softmax(scores, self.sink, self.scale, start + t0, probs)
            o = torch.bmm(probs, v[:, :Lt])  # [H, t, dv]
            K.heads_to_rows(o, rows_out[n0 + t0:n0 + t1])

    def forward(self, ctx: StepContext, h, cache: LayerCache, h32: torch.Tensor | None = None):
        dt, dev = ctx.runtime.dtype, h32.device
        a, _ = self.read_input(ctx, h32, cache)
        n, H = a.shape[0], self.heads
        offsets = ctx.arrays[self._planner.array_name]
        # prompt portions in bfloat16 go to the tensor cores, request by request (their sizes are read on the host: such
        # a step is never captured in a graph, only steps of single tokens are)
        portions = dt == torch.bfloat16 and ctx.max_q_len > 1 and self.w_ukv is not None
        with scope("qkv_matmul"):
            down = as_rows(linear(ctx, a, self.w_down, torch.float32, partials=True))
        cq = torch.empty((n, self.q_rank), dtype=dt, device=dev)
        with scope("rope"):  # both latents' norms, the shared key part's rotation and the page write in one kernel
            K.latent_kv_prep(down.data, down.splits, self.q_norm_weight, self.kv_norm_weight, self.eps, self.inv_freq,
                             self.rot_dims, cq, cache.pages if cache.writes else None, cache.block_table if cache.writes else None,
                             ctx.req_of_token, ctx.positions, self.q_rank, self.kv_rank, self.rot_dim, ctx.status)
        with scope("qkv_matmul"):
            q = as_rows(linear(ctx, cq, self.w_uq, torch.float32, partials=True))
        q_nope = torch.empty((H, n, self.dim), dtype=dt, device=dev)
        q_rot = torch.empty((n, H, self.rot_dim), dtype=torch.float32, device=dev)
        q_full = torch.empty((H, n, self.dim + self.rot_dim), dtype=dt, device=dev) if portions else None
        with scope("rope"):
            K.latent_q_prep(q.data, q.splits, self.inv_freq, self.rot_dims, ctx.positions, q_nope, q_rot, H, self.dim,
                            self.rot_dim, q_full)
        rows = torch.empty((n, H * self.vdim), dtype=dt, device=dev)
        with scope("attention"):
            singles = len(ctx.host_arrays["attn_single_rows"]) if portions else n
            if singles:
                q_lat = grouped_linear(ctx, q_nope.view(H * n, self.dim), self.w_uk_t, offsets, torch.float32, largest_group=n)
                out_lat = torch.empty((H, n, self.kv_rank), dtype=dt, device=dev)
                if portions:  # only the single tokens' rows mean anything; the portions' rows are overwritten below
                    out_lat.zero_()
                    self._latent_space(ctx, q_lat.view(H, n, self.kv_rank), q_rot, cache, out_lat, ctx.arrays["attn_single_rows"], singles)
                else:
                    self._latent_space(ctx, q_lat.view(H, n, self.kv_rank), q_rot, cache, out_lat)
                v = grouped_linear(ctx, out_lat.view(H * n, self.kv_rank), self.w_uv, offsets, dt, largest_group=n)
                K.heads_to_rows(v.view(H, n, self.vdim), rows)
            if portions:
                n0 = 0
                for r, (T, start) in enumerate(zip(ctx.host_q_lens, ctx.host_q_start)):
                    if T > 1:
                        self._portion(ctx, cache, r, n0, T, start, q_full, rows)
                    n0 += T
        with scope("projection"):
            return linear(ctx, rows, self.w_o, torch.float32, partials=True)


register_part("mixer", "latent_attention", LatentAttention)
