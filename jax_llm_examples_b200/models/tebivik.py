"""Tebivik: its tensors by name and how its layers are put together from parts.

Tensor names: ``embed`` (also the output head, unscaled), ``final.norm``, ``loop.in`` / ``loop.step`` (with a loop),
and per layer ``l<i>.``: ``norm1``, ``norm1b`` (around the mixer), ``norm2``, ``norm2b`` (around the feed-forward, if
the layer has one), ``canon1`` (the short convolution on the mixer's input), ``mix.*`` and ``mlp.*``.  Linear weights
are [out, in].

Layer rules (config: :class:`..config.tebivik.TebivikConfig`): every layer is a sandwich-norm block
(x += m * norm_b(sublayer(norm(x)))) with grouped RMS norms; its mixer is an HGRN2 recurrence or latent attention,
both behind a residual short convolution; its feed-forward, if any, is a biased MLP with squared-relu.  A stretch of
layers may run several times with the same weights: every pass opens with a re-injection of the embedding's output
(one shared matrix, one step vector per pass) and has caches and states of its own.
"""

from __future__ import annotations

from typing import Mapping

import torch

from ..config.registry import Architecture, register_architecture
from ..config.tebivik import HGRN2Spec, LatentAttentionSpec, TebivikConfig
from ..parts import DecoderModel, Runtime, make_part
from ..weights.loader import TensorSpec


def _mixer_specs(p: str, spec, D: int) -> list[TensorSpec]:
    m = spec.mixer
    if isinstance(m, HGRN2Spec):
        hk, hv = m.heads * m.dim, m.heads * m.vdim
        return [TensorSpec(p + "q", (hk, D)), TensorSpec(p + "f", (hk, D)), TensorSpec(p + "f.b", (hk,), "bias"),
                TensorSpec(p + "lower", (hk,), "unit"), TensorSpec(p + "v", (hv, D)), TensorSpec(p + "norm", (m.vdim,), "norm"),
                TensorSpec(p + "o", (D, hv))]
    assert isinstance(m, LatentAttentionSpec)
    H = m.heads
    return [TensorSpec(p + "dq", (m.q_rank, D)), TensorSpec(p + "dq.norm", (m.q_rank,), "norm"),
            TensorSpec(p + "uq", (H * (m.dim + m.rot_dim), m.q_rank)), TensorSpec(p + "dkv", (m.kv_rank + m.rot_dim, D)),
            TensorSpec(p + "dkv.norm", (m.kv_rank,), "norm"), TensorSpec(p + "uk", (H * m.dim, m.kv_rank)),
            TensorSpec(p + "uv", (H * m.vdim, m.kv_rank)), TensorSpec(p + "sink", (H,), "bias"),
            TensorSpec(p + "o", (D, H * m.vdim))]


def tensor_specs(cfg: TebivikConfig) -> dict[str, TensorSpec]:
    D, V = cfg.width, cfg.vocab
    specs: list[TensorSpec] = [TensorSpec("embed", (V, D))]
    if cfg.loop is not None:
        specs += [TensorSpec("loop.in", (D, 2 * D)), TensorSpec("loop.step", (cfg.loop.times, D), "bias")]
    for i, L in enumerate(cfg.layers):
        p = f"l{i}."
        specs += [TensorSpec(p + "norm1", (D,), "norm"), TensorSpec(p + "norm1b", (D,), "norm"),
                  TensorSpec(p + "canon1", (D, cfg.canon_taps), "bias")]
        specs += _mixer_specs(p + "mix.", L, D)
        if L.mlp is not None:
            specs += [TensorSpec(p + "norm2", (D,), "norm"), TensorSpec(p + "norm2b", (D,), "norm"),
                      TensorSpec(p + "mlp.up", (L.mlp.ff, D)), TensorSpec(p + "mlp.up.b", (L.mlp.ff,), "bias"),
                      TensorSpec(p + "mlp.down", (D, L.mlp.ff)), TensorSpec(p + "mlp.down.b", (D,), "bias")]
    specs.append(TensorSpec("final.norm", (D,), "norm"))
    return {s.name: s for s in specs}


def build(cfg: TebivikConfig, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> DecoderModel:
    """Puts the decoder together.  ``tensors`` (by spec name) is consumed as the weights are fused into the layouts
    the kernels read."""
    t = dict(tensors) if not isinstance(tensors, dict) else tensors
    dev = runtime.device

    def take(name: str) -> torch.Tensor:
        return t.pop(name).to(dev)

    def norm(name: str):
        return make_part("norm", "group_rms", weight=take(name), eps=cfg.norm_eps, groups=cfg.norm_groups)

    blocks = []
    for i, L in enumerate(cfg.layers):
        p, m = f"l{i}.", L.mixer
        conv = make_part("conv", "residual_short", weight=take(p + "canon1"))
        if isinstance(m, HGRN2Spec):
            mixer = make_part(
                "mixer", "hgrn2",
                w_qfv=torch.cat([take(p + "mix.q"), take(p + "mix.f"), take(p + "mix.v")], dim=0).contiguous(),
                f_bias=take(p + "mix.f.b"), lower=take(p + "mix.lower"), norm_weight=take(p + "mix.norm"),
                w_o=take(p + "mix.o").contiguous(), heads=m.heads, dim=m.dim, vdim=m.vdim, eps=cfg.norm_eps, input_conv=conv)
        else:
            mixer = make_part(
                "mixer", "latent_attention",
                w_down=torch.cat([take(p + "mix.dq"), take(p + "mix.dkv")], dim=0).contiguous(),
                q_norm_weight=take(p + "mix.dq.norm"), w_uq=take(p + "mix.uq").contiguous(),
                kv_norm_weight=take(p + "mix.dkv.norm"), w_uk=take(p + "mix.uk"), w_uv=take(p + "mix.uv"),
                w_o=take(p + "mix.o").contiguous(), sink=take(p + "mix.sink"), heads=m.heads, dim=m.dim, rot_dim=m.rot_dim,
                vdim=m.vdim, q_rank=m.q_rank, kv_rank=m.kv_rank, scale=m.scale, rot_base=m.rot_base, rot_dims=m.rot_dims,
                eps=cfg.norm_eps, input_conv=conv)
        norm1, norm1b = norm(p + "norm1"), norm(p + "norm1b")
        if L.mlp is None:
            blocks.append(make_part("block", "sandwich_norm", norm1=norm1, mixer=mixer, norm1b=norm1b, mult=cfg.residual_mult))
            continue
        ff = make_part("feed_forward", "dense_biased", w_up=take(p + "mlp.up").contiguous(), b_up=take(p + "mlp.up.b"),
                       w_down=take(p + "mlp.down").contiguous(), b_down=take(p + "mlp.down.b"), activation="relu2")
        blocks.append(make_part("block", "sandwich_norm", norm1=norm1, mixer=mixer, norm1b=norm1b, norm2=norm(p + "norm2"),
                                feed_forward=ff, norm2b=norm(p + "norm2b"), mult=cfg.residual_mult))
    # the order of execution: every pass of the loop opens with a re-injection block of its own (one shared matrix)
    order: list[tuple[int]] = []
    if cfg.loop is not None:
        w_in, steps = take("loop.in"), take("loop.step")
        entries = []
        for k in range(cfg.loop.times):
            e = make_part("block", "reinjection", w_in=w_in, step=steps[k])
            if entries:
                e.share_weights(entries[0])
            entries.append(e)
        first_entry = len(blocks)
        blocks += entries
    for i, opens_pass in cfg.layer_order():
        if opens_pass is not None:
            order.append((first_entry + opens_pass,))
        order.append((i,))
    embedding = take("embed").contiguous()
    final_norm = norm("final.norm")
    return DecoderModel(runtime, embedding, blocks, final_norm, embedding, schedule=DecoderModel.schedule_of(order, blocks),
                        config=cfg, embedding_scale=cfg.embedding_scale)


TEBIVIK = Architecture(name="Tebivik", parse_config=TebivikConfig.from_dict, tensor_specs=tensor_specs, build=build)
register_architecture(TEBIVIK)
