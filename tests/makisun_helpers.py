"""Shared by the Makisun tests: small configurations of their own, model folders from a seed, the plain
implementation's logits (with the engine's expert choices, where the test hands them over)."""

from __future__ import annotations

import copy
import functools
import json
from pathlib import Path

import numpy as np
import torch

from tests.plain import makisun_plain as plain


def wkv(heads, dim, rank, mlp=None):
    return {"type": "wkv", "mixer": {"heads": heads, "dim": dim, "decay_rank": rank}, "mlp": mlp}


def parallel(left, right, left_scale, right_scale, mlp=None):
    heads, kv, dim, vdim, window, base, dims, scale = left
    rheads, rdim, rvdim, tau, rank = right
    return {"type": "parallel", "mlp": mlp,
            "mixer": {"left": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "mask": {"size": window},
                               "rot": {"base": base, "dims": dims}, "scale": scale},
                      "right": {"heads": rheads, "dim": rdim, "vdim": rvdim, "tau": tau, "decay_rank": rank},
                      "left_scale": left_scale, "right_scale": right_scale}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, shared=None):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared is not None:
        m["shared"] = {"ff": shared}
    return m


CONFIGS = {
    # every size small and odd (no size is a multiple of 8: every product runs on the 32-bit FMA kernel in both
    # precisions); a window shorter than a page; values of another size than keys; three query heads per key head;
    # a layer without a feed-forward; experts with and without a shared one, top-1 routing; part of the head rotated
    "small": {
        "architecture": "Makisun", "vocab": 61, "width": 36, "embedding": {"scale": 2.5}, "norm": {"eps": 1e-5},
        "layers": [wkv(3, 5, 3, moe(5, 2, 12, shared=9)),
                   parallel((6, 2, 10, 6, 7, 100.0, 4, 0.4), (2, 7, 9, 3.5, 5), 1.3, 0.6, dense(30)),
                   wkv(1, 12, 2),
                   parallel((2, 2, 9, 11, 100, 5000.0, 8, 0.33), (1, 6, 6, 1.0, 3), 0.5, 1.0, moe(3, 1, 10))],
    },
    # sizes in multiples of 8 (bfloat16 products on the tcgen05 streaming kernel, attention on the tensor-core kernels at
    # head size 64); one key head for four query heads; a window that straddles page borders; the whole head rotated
    "wide": {
        "architecture": "Makisun", "vocab": 96, "width": 128, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6},
        "layers": [parallel((4, 1, 64, 64, 40, 10000.0, 64, 0.1), (2, 32, 64, 8.0, 8), 1.0, 1.0, moe(8, 3, 64, shared=32)),
                   wkv(2, 64, 16, dense(256))],
    },
    # keys shorter than values and both padded in the cache (to 64 in bfloat16); no rotation at all; a window of one
    # token (a query sees itself only); as many experts chosen as there are; equal numbers of query and key heads
    "padded": {
        "architecture": "Makisun", "vocab": 50, "width": 48, "embedding": {"scale": 0.7}, "norm": {"eps": 1e-6},
        "layers": [parallel((3, 3, 24, 40, 1, 10.0, 0, 0.2), (3, 16, 8, 20.0, 8), 0.9, 1.1, moe(2, 2, 16)),
                   parallel((2, 1, 24, 16, 33, 300.0, 24, 0.25), (2, 8, 24, 2.0, 16), 1.0, 0.7, dense(40))],
    },
    # recurrences only: a model without a page of cache
    "recurrent": {
        "architecture": "Makisun", "vocab": 40, "width": 32, "embedding": {"scale": 4.0}, "norm": {"eps": 1e-6},
        "layers": [wkv(2, 16, 8, dense(48)), wkv(4, 4, 4, moe(4, 2, 8, shared=8))],
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
def plain_model(folder: str):
    folder = Path(folder)
    return json.loads((folder / "config.json").read_text()), plain.read_safetensors(folder / "model.safetensors")


def routed_layers(folder) -> int:
    cfg, _ = plain_model(str(folder))
    return sum(1 for L in cfg["layers"] if L.get("mlp") and L["mlp"]["kind"] == "moe")


def plain_logits(folder, tokens, forced=None):
    """(logits [T, V], the largest shortfall of a forced expert's logit below the logit it needed, relative to the
    layer's typical logit)."""
    cfg, P = plain_model(str(folder))
    with torch.no_grad():
        logits, _, routers = plain.forward(cfg, P, list(tokens), forced)
    worst = 0.0
    for z, chosen in routers:
        top = chosen.shape[1]
        needed = torch.topk(z, top, dim=-1).values[:, -1:]
        short = (needed - torch.gather(z, 1, chosen)).clamp_min(0.0).max()
        worst = max(worst, float(short / z.pow(2).mean().sqrt().clamp_min(1e-9)))
    return logits.numpy(), worst


# float32: a few thousand roundings of 6e-8 per logit.  bfloat16: activations are rounded (4e-3) several times per layer,
# and a tiny model's logits are sums of few terms, so single rows scatter: the mean over all rows is held tight and a
# single row is capped where a fault (a lost state, a key off by one) would still stand out by a factor of ten.
TOL = {"float32": 3e-5, "bfloat16": 1.2e-1}
TOL_MEAN = {"float32": 1e-5, "bfloat16": 3e-2}
TIE = {"float32": 2e-5, "bfloat16": 6e-2}  # how far below the needed logit a chosen expert's may lie (a tie either way)


def row_err(got: np.ndarray, ref: np.ndarray) -> float:
    """Difference of two logit rows, each with its mean taken off, relative to the reference row's spread."""
    d = (got - got.mean()) - (ref - ref.mean())
    return float(np.sqrt((d ** 2).mean()) / max(np.sqrt(((ref - ref.mean()) ** 2).mean()), 1e-9))


def compare(folder, requests: dict, got: dict, routing: dict | None, dtype: str) -> float:
    """Every logit row a trace produced against the plain implementation's row at that place.  With ``routing`` (the
    engine's expert choices by (request, position)) the plain implementation takes those experts; they must be its own
    choice too, except where two router logits tie within the precision."""
    errs = []
    n_routed = routed_layers(folder)
    for rid, toks in requests.items():
        forced = None
        if routing is not None and n_routed:
            forced = [torch.as_tensor(np.stack([routing[(rid, p)][j] for p in range(len(toks))])) for j in range(n_routed)]
        ref, shortfall = plain_logits(folder, toks, forced)
        assert shortfall < TIE[dtype], f"{dtype}: request {rid}: an expert was chosen whose logit is too low by {shortfall:.2e}"
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
    tol = 1e-4 if dtype == "float32" else 8e-2
    for step, g in enumerate(got):
        logits = plain_logits(folder, toks)[0][-1]
        best = int(np.argmax(logits))
        if g != best:
            gap = float(logits[best] - logits[g]) / float(np.abs(logits - logits.mean()).max())
            assert gap < tol, f"{dtype}: step {step}: engine chose {g}, plain {best}, relative logit gap {gap:.2e}"
        toks.append(g)
