"""Shared by the Tebivik tests: small configurations of their own, model folders from a seed, the plain
implementation's logits."""

from __future__ import annotations

import copy
import functools

import numpy as np
import torch

from tests.plain import tebivik_plain as plain


def _hgrn2(heads, dim, vdim, ff=None):
    return {"type": "hgrn2", "mixer": {"heads": heads, "dim": dim, "vdim": vdim},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def _latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, base, dims, ff=None):
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
                      "scale": scale, "rot": {"base": base, "dims": dims}},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


CONFIGS = {
    # every size small and odd (no size is a multiple of 8, so every product runs on the 32-bit FMA kernel in both
    # precisions); the loop lies in the middle and runs three times; only part of the rotated entries is rotated;
    # the layers with a feed-forward are not the first ones; one layer of each mixer has a single head
    "small": {
        "architecture": "Tebivik", "vocab": 50, "width": 36, "residual_mult": 0.4, "embedding": {"scale": 1.7},
        "norm": {"eps": 1e-5, "groups": 3}, "canon": {"taps": 4}, "loop": {"start": 1, "stop": 3, "times": 3},
        "layers": [_hgrn2(3, 5, 7), _latent(3, 5, 6, 4, 9, 10, 0.31, 3000.0, 4, ff=20), _hgrn2(1, 12, 9, ff=44),
                   _latent(1, 8, 2, 8, 6, 7, 0.5, 10.0, 2)],
    },
    # sizes in multiples of 8 (bfloat16 products run on the tcgen05 streaming kernel); one pass only; two taps;
    # one norm group; attention first
    "wide": {
        "architecture": "Tebivik", "vocab": 96, "width": 128, "residual_mult": 1.0, "embedding": {"scale": 1.0},
        "norm": {"eps": 1e-6, "groups": 1}, "canon": {"taps": 2}, "loop": {"start": 0, "stop": 2, "times": 1},
        "layers": [_latent(4, 16, 16, 24, 48, 40, 0.2, 10000.0, 16, ff=256), _hgrn2(2, 40, 64)],
    },
    # no loop at all, one tap (a convolution without state), recurrences only: a model without a page of cache
    "plainest": {
        "architecture": "Tebivik", "vocab": 40, "width": 32, "residual_mult": 0.8, "embedding": {"scale": 0.5},
        "norm": {"eps": 1e-6, "groups": 2}, "canon": {"taps": 1}, "loop": None,
        "layers": [_hgrn2(2, 8, 16, ff=48), _hgrn2(4, 4, 8)],
    },
}


def config(name: str, **overrides) -> dict:
    c = copy.deepcopy(CONFIGS[name])
    c.update(overrides)
    return c


def make_dir(path, name: str, seed: int, **overrides):
    from jax_llm_examples_b200 import write_random_model

    return write_random_model(path, config(name, **overrides), seed, norm_noise=0.1, std=0.15)


@functools.lru_cache(maxsize=32)
def _plain_model(folder: str):
    return plain.load_config(folder), plain.load_weights(folder, torch.float64)


@functools.lru_cache(maxsize=256)
def _plain_logits(folder: str, tokens: tuple) -> np.ndarray:
    cfg, w = _plain_model(folder)
    with torch.no_grad():
        return plain.forward(cfg, w, list(tokens)).numpy()


def plain_logits(folder, tokens) -> np.ndarray:
    return _plain_logits(str(folder), tuple(tokens))


# float32: a few thousand roundings of 6e-8 per logit.  bfloat16: activations are rounded (4e-3) several times per layer
# run, and a tiny model's logits are sums of few terms, so single rows scatter: the mean over all rows is held tight and a
# single row is capped where a fault (a lost state, a key off by one) would still stand out by a factor of ten.
TOL = {"float32": 3e-5, "bfloat16": 1.2e-1}
TOL_MEAN = {"float32": 1e-5, "bfloat16": 3e-2}


def row_err(got: np.ndarray, ref: np.ndarray) -> float:
    """Difference of two logit rows, each with its mean taken off, relative to the reference row's spread."""
    d = (got - got.mean()) - (ref - ref.mean())
    return float(np.sqrt((d ** 2).mean()) / max(np.sqrt(((ref - ref.mean()) ** 2).mean()), 1e-9))


def compare(folder, requests: dict, got: dict, dtype: str) -> float:
    """Every logit row a trace produced against the plain implementation's row at that place."""
    errs = []
    for rid, toks in requests.items():
        ref = plain_logits(folder, toks)
        for pos in range(len(toks)):
            if (rid, pos) in got:
                err = row_err(got[(rid, pos)], ref[pos])
                assert err < TOL[dtype], f"{dtype}: request {rid} position {pos}: relative error {err:.3e}"
                errs.append(err)
    mean = float(np.mean(errs))
    assert mean < TOL_MEAN[dtype], f"{dtype}: mean relative error {mean:.3e} over {len(errs)} rows"
    return max(errs)


def greedy_checked(folder, prompt, got, dtype: str) -> None:
    """``got`` must be the plain implementation's greedy continuation, except where its two best logits are closer
    than the precision tells apart; after such a step the comparison follows the engine's choice."""
    toks = list(prompt)
    tol = 1e-4 if dtype == "float32" else 5e-2
    for step, g in enumerate(got):
        logits = plain_logits(folder, toks)[-1]
        best = int(np.argmax(logits))
        if g != best:
            gap = float(logits[best] - logits[g]) / float(np.abs(logits - logits.mean()).max())
            assert gap < tol, f"{dtype}: step {step}: engine chose {g}, plain {best}, relative logit gap {gap:.2e}"
        toks.append(g)
