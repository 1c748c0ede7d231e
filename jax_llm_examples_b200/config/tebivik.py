"""Typed configuration of the Tebivik decoder, read from config.json's own keys.

A Tebivik model is a list of layers, each with one mixer (``hgrn2``: a gated linear recurrence; ``latent_attention``:
attention over a cached latent) and an optional dense feed-forward, a loop that runs a stretch of the layers several
times with the same weights, grouped RMS norms before and after every sublayer, and a short causal convolution on
every mixer's input.  Every size and every constant that can differ between two models is a key of the file.
"""

from __future__ import annotations

import dataclasses
from typing import Any, Mapping

from .base import ConfigError, read_key, require


@dataclasses.dataclass(frozen=True)
class HGRN2Spec:
    heads: int
    dim: int  # rows of a head's state (query channels)
    vdim: int  # columns of a head's state (value channels)


@dataclasses.dataclass(frozen=True)
class LatentAttentionSpec:
    heads: int
    dim: int  # unrotated query/key entries per head
    rot_dim: int  # rotated query/key entries per head (the key's are shared by all heads)
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    rot_base: float
    rot_dims: int  # how many of the rotated part's entries are rotated (in pairs)


@dataclasses.dataclass(frozen=True)
class MlpSpec:
    kind: str
    ff: int


@dataclasses.dataclass(frozen=True)
class LayerSpec:
    type: str
    mixer: "HGRN2Spec | LatentAttentionSpec"
    mlp: MlpSpec | None


@dataclasses.dataclass(frozen=True)
class LoopSpec:
    start: int
    stop: int
    times: int


@dataclasses.dataclass(frozen=True)
class TebivikConfig:
    vocab: int
    width: int
    layers: tuple[LayerSpec, ...]
    loop: LoopSpec | None
    norm_eps: float
    norm_groups: int
    residual_mult: float
    embedding_scale: float
    canon_taps: int

    # the names the rest of the framework asks a configuration for
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    def layer_order(self) -> list[tuple[int, int | None]]:
        """(layer, number of the pass that it opens or None) in the order of execution: the layers before the loop,
        the looped stretch ``times`` times, the layers after it."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, None) for i in range(n)]
        lp = self.loop
        order: list[tuple[int, int | None]] = [(i, None) for i in range(lp.start)]
        for t in range(lp.times):
            order += [(i, t if i == lp.start else None) for i in range(lp.start, lp.stop)]
        return order + [(i, None) for i in range(lp.stop, n)]

    @staticmethod
    def from_dict(d: Mapping[str, Any]) -> "TebivikConfig":
        width = read_key(d, "width", int)
        norm = read_key(d, "norm", dict)
        layers = []
        raw_layers = read_key(d, "layers", list)
        require(len(raw_layers) > 0, "'layers' is empty")
        for i, L in enumerate(raw_layers):
            require(isinstance(L, dict), f"layers[{i}] must be an object")
            kind = read_key(L, "type", str)
            m = read_key(L, "mixer", dict)
            if kind == "hgrn2":
                mixer: Any = HGRN2Spec(read_key(m, "heads", int), read_key(m, "dim", int), read_key(m, "vdim", int))
            elif kind == "latent_attention":
                rot = read_key(m, "rot", dict)
                mixer = LatentAttentionSpec(
                    heads=read_key(m, "heads", int), dim=read_key(m, "dim", int), rot_dim=read_key(m, "rot_dim", int),
                    vdim=read_key(m, "vdim", int), q_rank=read_key(m, "q_rank", int), kv_rank=read_key(m, "kv_rank", int),
                    scale=read_key(m, "scale", float), rot_base=read_key(rot, "base", float), rot_dims=read_key(rot, "dims", int))
                require(mixer.rot_dims % 2 == 0 and 0 <= mixer.rot_dims <= mixer.rot_dim,
                        f"layers[{i}]: rot.dims = {mixer.rot_dims} must be even and at most rot_dim = {mixer.rot_dim}")
            else:
                raise ConfigError(f"config.json: layers[{i}].type = {kind!r} is no mixer of this architecture (hgrn2, latent_attention)")
            require(all(v > 0 for v in (mixer.heads, mixer.dim, mixer.vdim)), f"layers[{i}]: sizes must be positive")
            mlp = None
            if L.get("mlp") is not None:
                ml = read_key(L, "mlp", dict)
                mlp = MlpSpec(read_key(ml, "kind", str), read_key(ml, "ff", int))
                require(mlp.kind == "dense", f"layers[{i}].mlp.kind = {mlp.kind!r}; this architecture has 'dense'")
                require(mlp.ff > 0, f"layers[{i}].mlp.ff must be positive")
            layers.append(LayerSpec(kind, mixer, mlp))
        loop = None
        if d.get("loop") is not None:
            lp = read_key(d, "loop", dict)
            loop = LoopSpec(read_key(lp, "start", int), read_key(lp, "stop", int), read_key(lp, "times", int))
            require(0 <= loop.start < loop.stop <= len(layers), f"loop [{loop.start}, {loop.stop}) does not lie within the {len(layers)} layers")
            require(loop.times >= 1, "loop.times must be at least 1")
        cfg = TebivikConfig(
            vocab=read_key(d, "vocab", int), width=width, layers=tuple(layers), loop=loop,
            norm_eps=read_key(norm, "eps", float), norm_groups=read_key(norm, "groups", int),
            residual_mult=read_key(d, "residual_mult", float),
            embedding_scale=read_key(read_key(d, "embedding", dict), "scale", float),
            canon_taps=read_key(read_key(d, "canon", dict), "taps", int))
        require(cfg.vocab > 0 and cfg.width > 0, "vocab and width must be positive")
        require(cfg.norm_groups >= 1 and cfg.width % cfg.norm_groups == 0, f"norm.groups = {cfg.norm_groups} does not divide the width {cfg.width}")
        require(cfg.norm_eps > 0, "norm.eps must be positive")
        require(cfg.canon_taps >= 1, "canon.taps must be at least 1")
        return cfg
