"""Makisun: its tensors by name and how its layers are put together from parts.

Tensor names: ``embed``, ``head``, ``final.norm`` and per layer ``l<i>.``: ``norm1``, ``norm2`` (norm weights stored
as offsets from one), ``ls1``, ``ls2`` (the scale vectors on the sublayers' outputs), ``mix.*`` and ``mlp.*``.  Linear
weights are [out, in].

* ``wkv`` mixer: ``mix.mu.{r,k,v,g,w}``, ``mix.{r,k,v,g}``, ``mix.w1``, ``mix.w2``, ``mix.w0``, ``mix.u``, ``mix.norm``, ``mix.o``.
* ``parallel`` mixer: ``mix.left.{q,k,v,g,o}``, ``mix.left.q.norm``, ``mix.left.k.norm``; ``mix.right.{q,k,v,g,o}``,
  ``mix.right.norm``, ``mix.right.a1``, ``mix.right.a2``, ``mix.right.a2.b``.
* dense feed-forward: ``mlp.up``, ``mlp.down``; mixture of experts: ``mlp.e<j>.up``, ``mlp.e<j>.down``, ``mlp.router``,
  ``mlp.router.b``, and ``mlp.shared.up``, ``mlp.shared.down`` if it has a shared expert.

Layer rules (config: :class:`..config.makisun.MakisunConfig`): x += ls1 * mixer(norm1(x)); x += ls2 * ff(norm2(x));
norm(x) = x / sqrt(mean(x^2) + eps) * (1 + w).  The model's norm has the same form; the head is a tensor of its own.
"""

from __future__ import annotations

from typing import Mapping

import torch

from ..config.makisun import MakisunConfig, ParallelSpec, WKVSpec
from ..config.registry import Architecture, register_architecture
from ..parts import DecoderModel, GatedPagedAttention, Runtime, make_part, rotary_frequencies
from ..weights.loader import TensorSpec

BLENDS = ("r", "k", "v", "g", "w")  # the order of the time-mix blends in the stacked ``mu``


def _rank(r: int | None) -> int:
    return -1 if r is None else r  # -1: whatever the stored tensor has


def tensor_specs(cfg: MakisunConfig) -> dict[str, TensorSpec]:
    D, V = cfg.width, cfg.vocab
    specs: list[TensorSpec] = [TensorSpec("embed", (V, D))]
    for i, L in enumerate(cfg.layers):
        p, m = f"l{i}.", L.mixer
        specs += [TensorSpec(p + "norm1", (D,), "bias"), TensorSpec(p + "ls1", (D,), "norm")]
        if isinstance(m, WKVSpec):
            F, q = m.heads * m.dim, p + "mix."
            specs += [TensorSpec(q + "mu." + s, (D,), "unit") for s in BLENDS]
            specs += [TensorSpec(q + s, (F, D)) for s in ("r", "k", "v", "g")]
            specs += [TensorSpec(q + "w1", (_rank(m.decay_rank), D)), TensorSpec(q + "w2", (F, _rank(m.decay_rank))),
                      TensorSpec(q + "w0", (F,), "bias"), TensorSpec(q + "u", (m.heads, m.dim), "bias"),
                      TensorSpec(q + "norm", (F,), "norm"), TensorSpec(q + "o", (D, F))]
        else:
            assert isinstance(m, ParallelSpec)
            a, g, q = m.left, m.right, p + "mix.left."
            specs += [TensorSpec(q + "q", (a.heads * a.dim, D)), TensorSpec(q + "k", (a.kv_heads * a.dim, D)),
                      TensorSpec(q + "v", (a.kv_heads * a.vdim, D)), TensorSpec(q + "q.norm", (a.dim,), "norm"),
                      TensorSpec(q + "k.norm", (a.dim,), "norm"), TensorSpec(q + "g", (a.heads, D)),
                      TensorSpec(q + "o", (D, a.heads * a.vdim))]
            q = p + "mix.right."
            specs += [TensorSpec(q + "q", (g.heads * g.dim, D)), TensorSpec(q + "k", (g.heads * g.dim, D)),
                      TensorSpec(q + "v", (g.heads * g.vdim, D)), TensorSpec(q + "g", (g.heads * g.vdim, D)),
                      TensorSpec(q + "o", (D, g.heads * g.vdim)), TensorSpec(q + "norm", (g.vdim,), "norm"),
                      TensorSpec(q + "a1", (_rank(g.decay_rank), D)), TensorSpec(q + "a2", (g.heads * g.dim, _rank(g.decay_rank))),
                      TensorSpec(q + "a2.b", (g.heads * g.dim,), "bias")]
        if L.mlp is not None:
            q = p + "mlp."
            specs += [TensorSpec(p + "norm2", (D,), "bias"), TensorSpec(p + "ls2", (D,), "norm")]
            if L.mlp.kind == "dense":
                specs += [TensorSpec(q + "up", (L.mlp.ff, D)), TensorSpec(q + "down", (D, L.mlp.ff))]
            else:
                for e in range(L.mlp.experts):
                    specs += [TensorSpec(f"{q}e{e}.up", (L.mlp.ff, D)), TensorSpec(f"{q}e{e}.down", (D, L.mlp.ff))]
                specs += [TensorSpec(q + "router", (L.mlp.experts, D)), TensorSpec(q + "router.b", (L.mlp.experts,), "bias")]
                if L.mlp.shared_ff is not None:
                    specs += [TensorSpec(q + "shared.up", (L.mlp.shared_ff, D)), TensorSpec(q + "shared.down", (D, L.mlp.shared_ff))]
    specs += [TensorSpec("final.norm", (D,), "bias"), TensorSpec("head", (V, D))]
    return {s.name: s for s in specs}


def build(cfg: MakisunConfig, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> DecoderModel:
    """Puts the decoder together.  ``tensors`` (by spec name) is consumed as the weights are stacked into the layouts
    the kernels read."""
    t = dict(tensors) if not isinstance(tensors, dict) else tensors
    dev, eps = runtime.device, cfg.norm_eps

    def take(name: str) -> torch.Tensor:
        return t.pop(name).to(dev)

    def norm(name: str):
        # the stored weight is an offset from one; 1 + w is exact in float32
        return make_part("norm", "group_rms", weight=1.0 + take(name).to(torch.float32), eps=eps, groups=1)

    blocks = []
    for i, L in enumerate(cfg.layers):
        p, m = f"l{i}.", L.mixer
        if isinstance(m, WKVSpec):
            q = p + "mix."
            mixer = make_part(
                "mixer", "time_mix_wkv", mu=torch.stack([take(q + "mu." + s) for s in BLENDS]),
                w_rkvg=torch.stack([take(q + s) for s in ("r", "k", "v", "g")]), w_w1=take(q + "w1"), w_w2=take(q + "w2"),
                w0=take(q + "w0"), bonus=take(q + "u"), norm_weight=take(q + "norm"), w_o=take(q + "o").contiguous(),
                heads=m.heads, dim=m.dim, eps=eps)
        else:
            a, g, q = m.left, m.right, p + "mix.left."
            left = make_part(
                "mixer", "gated_paged_attention",
                w_in=torch.cat([take(q + "q"), take(q + "k"), take(q + "v"), take(q + "g")], dim=0).contiguous(),
                w_o=take(q + "o").contiguous(), n_heads=a.heads, n_kv_heads=a.kv_heads, head_dim=a.dim, value_dim=a.vdim,
                scale=a.scale, eps=eps, q_norm_weight=take(q + "q.norm"), k_norm_weight=take(q + "k.norm"),
                inv_freq=rotary_frequencies(a.rot_base, a.rot_dims).to(dev) if a.rot_dims else None, rot_dims=a.rot_dims,
                window=a.window, gated=True, padded_dim=GatedPagedAttention.padded_size(a.dim, a.vdim, runtime.dtype))
            q = p + "mix.right."
            right = make_part(
                "mixer", "gated_linear_attention",
                w_in=torch.cat([take(q + "q"), take(q + "k"), take(q + "v"), take(q + "g")], dim=0).contiguous(),
                w_a1=take(q + "a1"), w_a2=take(q + "a2"), a_bias=take(q + "a2.b"), norm_weight=take(q + "norm"),
                w_o=take(q + "o").contiguous(), heads=g.heads, dim=g.dim, vdim=g.vdim, tau=g.tau, eps=eps)
            mixer = make_part("mixer", "parallel", mixers=[left, right], scales=[m.left_scale, m.right_scale])
        norm1, ls1 = norm(p + "norm1"), take(p + "ls1")
        if L.mlp is None:
            blocks.append(make_part("block", "scaled_pre_norm", norm1=norm1, mixer=mixer, scale1=ls1))
            continue
        q = p + "mlp."
        if L.mlp.kind == "dense":
            ff = make_part("feed_forward", "dense_biased", w_up=take(q + "up").contiguous(), b_up=None,
                           w_down=take(q + "down").contiguous(), b_down=None, activation="gelu")
        else:
            shared = None
            if L.mlp.shared_ff is not None:
                shared = make_part("feed_forward", "dense_biased", w_up=take(q + "shared.up").contiguous(), b_up=None,
                                   w_down=take(q + "shared.down").contiguous(), b_down=None, activation="relu2")
            ff = make_part(
                "feed_forward", "softmax_routed_mlp", w_router=take(q + "router"), router_bias=take(q + "router.b"),
                we_up=torch.stack([take(f"{q}e{e}.up") for e in range(L.mlp.experts)]),
                we_down=torch.stack([take(f"{q}e{e}.down") for e in range(L.mlp.experts)]), top_k=L.mlp.top, activation="relu2",
                shared=shared)
        blocks.append(make_part("block", "scaled_pre_norm", norm1=norm1, mixer=mixer, scale1=ls1, norm2=norm(p + "norm2"),
                                feed_forward=ff, scale2=take(p + "ls2")))
    embedding = take("embed").contiguous()
    final_norm = norm("final.norm")
    return DecoderModel(runtime, embedding, blocks, final_norm, take("head").contiguous(), config=cfg,
                        embedding_scale=cfg.embedding_scale)


MAKISUN = Architecture(name="Makisun", parse_config=MakisunConfig.from_dict, tensor_specs=tensor_specs, build=build)
register_architecture(MAKISUN)
