"""Typed configuration of the Makisun decoder, read from config.json's own keys.

A Makisun model is a list of pre-norm layers with a scale vector on each sublayer's output.  A layer's mixer is either
``wkv`` (RWKV-style time mixing with a data-dependent decay) or ``parallel`` (windowed softmax attention with a gate
per head beside gated linear attention, both on the same input, their outputs added with a weight each); its
feed-forward is dense (exact gelu), a mixture of experts (squared relu, softmax over the chosen experts' logits, an
optional shared expert) or missing.  Every size and constant that can differ between two models is a key of the file;
the ranks of the decays' small products are the stored tensors' own (``decay_rank`` names them only where weights are
made at random).
"""

from __future__ import annotations

import dataclasses
from typing import Any, Mapping

from .base import ConfigError, read_key, require


@dataclasses.dataclass(frozen=True)
class WKVSpec:
    heads: int
    dim: int
    decay_rank: int | None = None


@dataclasses.dataclass(frozen=True)
class WindowAttentionSpec:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    window: int
    rot_base: float
    rot_dims: int
    scale: float


@dataclasses.dataclass(frozen=True)
class GLASpec:
    heads: int
    dim: int
    vdim: int
    tau: float
    decay_rank: int | None = None


@dataclasses.dataclass(frozen=True)
class ParallelSpec:
    left: WindowAttentionSpec
    right: GLASpec
    left_scale: float
    right_scale: float


@dataclasses.dataclass(frozen=True)
class MlpSpec:
    kind: str  # "dense" or "moe"
    ff: int  # dense: the hidden size; moe: an expert's
    experts: int = 0
    top: int = 0
    shared_ff: int | None = None


@dataclasses.dataclass(frozen=True)
class LayerSpec:
    type: str
    mixer: "WKVSpec | ParallelSpec"
    mlp: MlpSpec | None


@dataclasses.dataclass(frozen=True)
class MakisunConfig:
    vocab: int
    width: int
    layers: tuple[LayerSpec, ...]
    norm_eps: float
    embedding_scale: float

    # the names the rest of the framework asks a configuration for
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @staticmethod
    def from_dict(d: Mapping[str, Any]) -> "MakisunConfig":
        raw_layers = read_key(d, "layers", list)
        require(len(raw_layers) > 0, "'layers' is empty")
        layers = []
        for i, L in enumerate(raw_layers):
            require(isinstance(L, dict), f"layers[{i}] must be an object")
            kind = read_key(L, "type", str)
            m = read_key(L, "mixer", dict)
            if kind == "wkv":
                mixer: Any = WKVSpec(read_key(m, "heads", int), read_key(m, "dim", int), read_key(m, "decay_rank", int, None))
                require(mixer.heads > 0 and mixer.dim > 0, f"layers[{i}]: sizes must be positive")
            elif kind == "parallel":
                lm, rm = read_key(m, "left", dict), read_key(m, "right", dict)
                rot = read_key(lm, "rot", dict)
                left = WindowAttentionSpec(
                    heads=read_key(lm, "heads", int), kv_heads=read_key(lm, "kv_heads", int), dim=read_key(lm, "dim", int),
                    vdim=read_key(lm, "vdim", int), window=read_key(read_key(lm, "mask", dict), "size", int),
                    rot_base=read_key(rot, "base", float), rot_dims=read_key(rot, "dims", int), scale=read_key(lm, "scale", float))
                require(all(v > 0 for v in (left.heads, left.kv_heads, left.dim, left.vdim, left.window)),
                        f"layers[{i}].mixer.left: sizes must be positive")
                require(left.heads % left.kv_heads == 0, f"layers[{i}].mixer.left: {left.heads} heads are no multiple of {left.kv_heads} kv_heads")
                require(left.rot_dims % 2 == 0 and 0 <= left.rot_dims <= left.dim,
                        f"layers[{i}].mixer.left: rot.dims = {left.rot_dims} must be even and at most dim = {left.dim}")
                right = GLASpec(heads=read_key(rm, "heads", int), dim=read_key(rm, "dim", int), vdim=read_key(rm, "vdim", int),
                                tau=read_key(rm, "tau", float), decay_rank=read_key(rm, "decay_rank", int, None))
                require(all(v > 0 for v in (right.heads, right.dim, right.vdim)) and right.tau > 0,
                        f"layers[{i}].mixer.right: sizes and tau must be positive")
                mixer = ParallelSpec(left, right, read_key(m, "left_scale", float), read_key(m, "right_scale", float))
            else:
                raise ConfigError(f"config.json: layers[{i}].type = {kind!r} is no mixer of this architecture (wkv, parallel)")
            mlp = None
            if L.get("mlp") is not None:
                ml = read_key(L, "mlp", dict)
                mk = read_key(ml, "kind", str)
                if mk == "dense":
                    mlp = MlpSpec("dense", read_key(ml, "ff", int))
                elif mk == "moe":
                    router = read_key(ml, "router", dict)
                    shared = ml.get("shared")
                    mlp = MlpSpec("moe", read_key(read_key(ml, "expert", dict), "ff", int), read_key(router, "experts", int),
                                  read_key(router, "top", int), None if shared is None else read_key(shared, "ff", int))
                    require(1 <= mlp.top <= mlp.experts, f"layers[{i}].mlp.router: top = {mlp.top} of {mlp.experts} experts")
                    require(mlp.shared_ff is None or mlp.shared_ff > 0, f"layers[{i}].mlp.shared.ff must be positive")
                else:
                    raise ConfigError(f"config.json: layers[{i}].mlp.kind = {mk!r}; this architecture has 'dense' and 'moe'")
                require(mlp.ff > 0, f"layers[{i}].mlp: ff must be positive")
            layers.append(LayerSpec(kind, mixer, mlp))
        cfg = MakisunConfig(
            vocab=read_key(d, "vocab", int), width=read_key(d, "width", int), layers=tuple(layers),
            norm_eps=read_key(read_key(d, "norm", dict), "eps", float),
            embedding_scale=read_key(read_key(d, "embedding", dict), "scale", float))
        require(cfg.vocab > 0 and cfg.width > 0, "vocab and width must be positive")
        require(cfg.norm_eps > 0, "norm.eps must be positive")
        return cfg
