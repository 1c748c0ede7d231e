"""Makisun on the GPU against the plain implementation: each mechanism alone (kernel or part against the plain
function of the same name), inputs made so that a fault shows (a far token, a window's edge), then whole models through
the engine's step function under every kind of cut, batches against requests alone, pages and slots that are used
again, long decoding, and greedy generation through the scheduler.  All configurations are this file's own
(``tests/makisun_helpers.py``)."""

import json
import os
import random
import subprocess
import sys

import numpy as np
import pytest
import torch

from tests import helpers as H
from tests import makisun_helpers as MH
from tests.plain import makisun_plain as plain
from tests.test_tebivik_gpu import _close, _ctx

pytestmark = pytest.mark.gpu
DEV = "cuda"
DTYPES = [("float32", torch.float32, 2e-5), ("bfloat16", torch.bfloat16, 3e-2)]


def _run_in_cuts(rt, seqs, cuts, slots, forward, n_steps):
    """Feeds each sequence in its own portions, the live ones of a step as one batch; returns the outputs per sequence."""
    at, got = [0] * len(seqs), [[] for _ in seqs]
    for step in range(n_steps):
        live = [r for r in range(len(seqs)) if step < len(cuts[r])]
        if not live:
            break
        lens = [cuts[r][step] for r in live]
        rows = torch.cat([seqs[r][at[r]:at[r] + n] for r, n in zip(live, lens)])
        ctx = _ctx(rt, lens, [at[r] for r in live], [slots[r] for r in live])
        out = forward(ctx, rows)
        o = 0
        for r, n in zip(live, lens):
            got[r].append(out[o:o + n])
            o += n
            at[r] += n
    return [torch.cat(g) for g in got]


# ------------------------------------------------------------------------------------- kernels alone
@pytest.mark.parametrize("D, splits", [(36, 1), (200, 3), (30, 2)])
def test_layer_scale_rides_in_the_norm_kernel(D, splits):
    """x += scale * (sum of partials), channel by channel, then the norm with a weight: one kernel."""
    from jax_llm_examples_b200.kernels import api as K

    torch.manual_seed(D)
    N, eps = 5, 1e-5
    x, part = torch.randn(N, D, device=DEV), torch.randn(splits, N, D, device=DEV)
    ls, w = torch.randn(D, device=DEV), torch.randn(D, device=DEV)
    x2, out32 = x.clone(), torch.empty(N, D, device=DEV)
    K.group_norm(x2, part, splits, None, ls, 1, 1.0, w, 1, True, eps, None, out32, post_norm=False)
    x_ref = x.double().cpu() + ls.double().cpu() * part.sum(0).double().cpu()
    _close(x2, x_ref, 3e-6, "residual")
    _close(out32, plain.rms_divide(x_ref, eps) * w.double().cpu(), 3e-6, "normed rows")


@pytest.mark.parametrize("act, ref", [("gelu", plain.gelu_erf), ("tanh", torch.tanh), ("relu2", plain.relu_squared)])
def test_activations_on_partial_sums(act, ref):
    from jax_llm_examples_b200.kernels import api as K

    torch.manual_seed(0)
    rows = torch.randn(2, 7, 20, device=DEV) * 2
    out = torch.empty(7, 20, device=DEV)
    K.bias_act(rows, out, None, None, act, 2)
    _close(out, ref(rows.sum(0).double().cpu()), 2e-6, act)


@pytest.mark.parametrize("dk, dv, rot, dpad", [(10, 6, 4, 10), (24, 40, 0, 64), (64, 64, 64, 64), (9, 11, 8, 16)])
def test_norm_then_rotate_half_then_padded_cache_rows(dk, dv, rot, dpad):
    """q and k: weighted RMS norm over the head, THEN the rotation of entry i with i + rot / 2 (i < rot / 2), the rest
    unchanged; v copied; all three padded with zeros to the cache's head size; large positions."""
    from jax_llm_examples_b200.kernels import api as K
    from jax_llm_examples_b200.parts import rotary_frequencies

    torch.manual_seed(dk)
    Hq, Hkv, N, page, eps, base = 4, 2, 6, 4, 1e-5, 300.0
    F = (Hq + Hkv) * dk + Hkv * dv
    proj = torch.randn(2, N, F + 3, device=DEV)  # two partials; three columns in front belong to something else
    qw, kw = torch.rand(dk, device=DEV) + 0.5, torch.rand(dk, device=DEV) + 0.5
    positions = torch.tensor([0, 1, 2, 3, 70001, 5], device=DEV, dtype=torch.int32)
    pages = torch.full((3, 2, Hkv, page, dpad), 7.0, device=DEV)
    table = torch.tensor([[2, 0]], device=DEV, dtype=torch.int32)
    # tokens at positions 0..3 and 5 land in pages 2 and 0; position 70001 would be far outside the table: keep it a query only
    req = torch.zeros(N, device=DEV, dtype=torch.int32)
    q_out = torch.full((N, Hq, dpad), 7.0, device=DEV)
    status = torch.zeros(1, device=DEV, dtype=torch.int32)
    inv = rotary_frequencies(base, rot).to(DEV) if rot else None
    keep = [0, 1, 2, 3, 5]
    sub = torch.tensor(keep, device=DEV)
    K.rope_half_kv_store(K.rows_view(proj[:, sub].contiguous(), 2, 3), Hq * dk, (Hq + Hkv) * dk, q_out[:5], pages, table, req[:5].contiguous(),
                         positions[sub].contiguous(), qw, kw, eps, inv, rot, Hq, Hkv, dk, dv, status)
    assert int(status) == 0
    s = proj.sum(0).double().cpu()[:, 3:]
    pos = positions.cpu()
    q = plain.rotate_half(plain.rms_divide(s[:, :Hq * dk].view(N, Hq, dk), eps) * qw.double().cpu(), pos, base, rot)
    k = plain.rotate_half(plain.rms_divide(s[:, Hq * dk:(Hq + Hkv) * dk].view(N, Hkv, dk), eps) * kw.double().cpu(), pos, base, rot)
    v = s[:, (Hq + Hkv) * dk:].view(N, Hkv, dv)
    _close(q_out[:5, :, :dk], q[keep], 3e-6, "q")
    assert float(q_out[:5, :, dk:].abs().max()) == 0.0 if dpad > dk else True
    for i, p in enumerate([0, 1, 2, 3, 5]):
        pg, slot = int(table[0, p // page]), p % page
        _close(pages[pg, 0, :, slot, :dk], k[keep[i]], 3e-6, f"k at {p}")
        _close(pages[pg, 1, :, slot, :dv], v[keep[i]], 3e-6, f"v at {p}")
        assert float(pages[pg, 0, :, slot, dk:].abs().max() if dpad > dk else 0.0) == 0.0
        assert float(pages[pg, 1, :, slot, dv:].abs().max() if dpad > dv else 0.0) == 0.0
    # a query alone (no cache write) at a large position: the angle is position * frequency in 32-bit
    q2 = torch.empty(1, Hq, dpad, device=DEV)
    K.rope_half_kv_store(K.rows_view(proj[:, 4:5].contiguous(), 2, 3), Hq * dk, (Hq + Hkv) * dk, q2, None, None, req[:1], positions[4:5].contiguous(),
                         qw, kw, eps, inv, rot, Hq, Hkv, dk, dv, status)
    _close(q2[0, :, :dk], q[4], 8e-3 if rot else 3e-6, "q far out")  # 70001 * f rounded to 32 bits: 4e-3 rad at most


@pytest.mark.parametrize("read_after", [True, False])
def test_decay_scan_keeps_a_far_token_and_reads_the_current_one_the_right_way(read_after):
    """Made so that a fault shows.  Channel 0 of head 1 never decays and is written ONCE, at token 3, with a marker value;
    700 tokens later a query on that channel must read the marker exactly, through portions of many sizes and a state
    carried across steps.  Channel 1 decays by 1/2 per token: a token written d steps ago counts 2^-d.  Read after the
    update, the current token counts undecayed; read before it, it counts only through the bonus."""
    from jax_llm_examples_b200.kernels import api as K

    torch.manual_seed(0)
    H_, dk, dv, T = 2, 5, 37, 704
    q, k = torch.zeros(T, H_, dk, device=DEV), torch.zeros(T, H_, dk, device=DEV)
    d = torch.rand(T, H_, dk, device=DEV) * 0.5 + 0.2
    v = torch.randn(T, H_, dv, device=DEV)
    k[:, 0], q[:, 0] = torch.randn(T, dk, device=DEV), torch.randn(T, dk, device=DEV)  # head 0: ordinary traffic
    d[:, 1, 0], d[:, 1, 1] = 1.0, 0.5
    k[3, 1, 0] = 1.0
    q[703, 1, 0] = 1.0  # reads the marker v[3, 1] from 700 tokens back
    k[690, 1, 1], k[700, 1, 1] = 1.0, 1.0
    q[700, 1, 1] = 1.0
    bonus = torch.full((H_, dk), 3.0, device=DEV)
    state = torch.zeros(4, H_, dk, dv, device=DEV)
    state[2] = 99.0  # another request's slot: must stay as it is
    o = torch.empty(T, H_, dv, device=DEV)
    cuts = [1, 2, 1, 16, 17, 33, 2, 255, 300, 1, 1, 70, 3, 2]
    assert sum(cuts) == T
    at = 0
    for n in cuts:
        sl = slice(at, at + n)
        cu = torch.tensor([0, n], device=DEV, dtype=torch.int32)
        K.decay_scan(q[sl].contiguous(), k[sl].contiguous(), d[sl].contiguous(), v[sl].contiguous(), None if read_after else bonus,
                     state, cu, torch.tensor([1], device=DEV, dtype=torch.int32), o[sl], read_after)
        at += n
    assert torch.equal(state[2], torch.full_like(state[2], 99.0)) and float(state[0].abs().max()) == 0.0
    _close(o[703, 1], v[3, 1], 1e-6, "the far token")
    # token 700 on channel 1: itself and token 690, ten decays later (nine when the state is read before this token's decay)
    if read_after:
        ref = v[700, 1] + 0.5 ** 10 * v[690, 1]
    else:
        ref = 3.0 * v[700, 1] + 0.5 ** 9 * v[690, 1]
    _close(o[700, 1], ref, 1e-6, "the current token and a decayed one")
    # everything against the recurrence in float64
    S = torch.zeros(H_, dk, dv, dtype=torch.float64)
    q64, k64, d64, v64 = (t.double().cpu() for t in (q, k, d, v))
    want = torch.zeros(T, H_, dv, dtype=torch.float64)
    for t in range(T):
        kv = k64[t][:, :, None] * v64[t][:, None, :]
        if read_after:
            S = d64[t][:, :, None] * S + kv
            want[t] = torch.einsum("hkv,hk->hv", S, q64[t])
        else:
            want[t] = torch.einsum("hkv,hk->hv", S + 3.0 * kv, q64[t])
            S = d64[t][:, :, None] * S + kv
    _close(o, want, 1e-5, "all tokens")
    _close(state[1], S, 1e-5, "the state at the end")


@pytest.mark.parametrize("dk, dv", [(1, 1), (16, 8), (33, 70), (128, 64), (200, 40), (300, 33)])
def test_decay_scan_sizes_and_a_batch_of_unequal_requests(dk, dv):
    """Other sizes (one channel; more rows than one warp's registers; no multiple of anything) and three requests of
    unequal length in one launch against each alone."""
    from jax_llm_examples_b200.kernels import api as K

    torch.manual_seed(dk)
    H_, lens = 2, [19, 1, 40]
    N = sum(lens)
    q, k, v = torch.randn(N, H_, dk, device=DEV), torch.randn(N, H_, dk, device=DEV) * dk ** -0.5, torch.randn(N, H_, dv, device=DEV)
    d = torch.rand(N, H_, dk, device=DEV)
    cu = torch.tensor([0, 19, 20, 60], device=DEV, dtype=torch.int32)
    slots = torch.tensor([2, 0, 1], device=DEV, dtype=torch.int32)
    state, o = torch.zeros(3, H_, dk, dv, device=DEV), torch.empty(N, H_, dv, device=DEV)
    K.decay_scan(q, k, d, v, None, state, cu, slots, o, True)
    at = 0
    for r, n in enumerate(lens):
        S = torch.zeros(H_, dk, dv, dtype=torch.float64)
        for t in range(at, at + n):
            S = d[t].double().cpu()[:, :, None] * S + k[t].double().cpu()[:, :, None] * v[t].double().cpu()[:, None, :]
            _close(o[t], torch.einsum("hkv,hk->hv", S, q[t].double().cpu()), 2e-5, f"request {r} token {t - at}")
        _close(state[int(slots[r])], S, 2e-5, f"state of request {r}")
        at += n


def test_decay_forms():
    """exp(-exp(z + b)) and sigmoid(z + b)^(1 / tau) in 32-bit, also far out in both tails; q is scaled, k and v pass."""
    from jax_llm_examples_b200.kernels import api as K

    H_, dk, dv, N = 2, 6, 3, 4
    z = torch.tensor([-60.0, -9.0, -1.0, 0.0, 0.3, 2.0, 7.0, 11.0, 30.0, 80.0, -0.2, 1.0], device=DEV).repeat(N, 1) \
        + torch.arange(N, device=DEV)[:, None] * 0.01
    proj = torch.randn(N, 2 * H_ * dk + H_ * dv, device=DEV)
    bias = torch.randn(H_ * dk, device=DEV) * 0.1
    outs = [torch.empty(N, H_, dk, device=DEV) for _ in range(3)] + [torch.empty(N, H_, dv, device=DEV)]
    view = lambda c: K.rows_view(proj, 1, c)
    for form, tau, ref in (("double_exp", 1.0, lambda x: torch.exp(-torch.exp(x))),
                           ("sigmoid_power", 7.0, lambda x: torch.sigmoid(x) ** (1 / 7.0)), ("sigmoid_power", 0.5, lambda x: torch.sigmoid(x) ** 2.0)):
        K.decay_prep(view(0), view(H_ * dk), view(2 * H_ * dk), K.rows_view(z.contiguous(), 1), bias, form, tau, 0.25, *outs, H_, dk, dv)
        want = ref((z + bias).double().cpu()).view(N, H_, dk)
        assert float((outs[2].double().cpu() - want).abs().max()) < 2e-6, form
        _close(outs[0], 0.25 * proj[:, :H_ * dk].reshape(N, H_, dk), 1e-6, "q")
        assert torch.equal(outs[1], proj[:, H_ * dk:2 * H_ * dk].reshape(N, H_, dk)) and torch.equal(outs[3], proj[:, 2 * H_ * dk:].reshape(N, H_, dv))


def test_router_with_a_bias_and_the_softmax_over_the_chosen():
    from jax_llm_examples_b200.kernels import api as K

    torch.manual_seed(4)
    for N, D, E, k, many in ((7, 36, 5, 2, False), (40, 64, 12, 4, True), (3, 20, 3, 3, False), (9, 16, 6, 1, False)):
        h, w, b = torch.randn(N, D, device=DEV), torch.randn(E, D, device=DEV), torch.randn(E, device=DEV) * 3
        idx, wt = torch.empty(N, k, dtype=torch.int32, device=DEV), torch.empty(N, k, device=DEV)
        K.router(h, w, idx, wt, many_rows=many, bias=b, weight_form="softmax_of_chosen")
        z = h.double().cpu() @ w.double().cpu().T + b.double().cpu()
        top = torch.topk(z, k, dim=-1)
        assert torch.equal(idx.cpu().long(), top.indices)
        _close(wt, torch.softmax(top.values, dim=-1), 1e-5, "weights")
        assert torch.allclose(wt.sum(-1), torch.ones(N, device=DEV), atol=1e-6)


# ------------------------------------------------------------------------------------- parts alone
def _wkv_weights(D, H_, dk, rank):
    g = lambda *s: torch.randn(*s) * 0.3
    F = H_ * dk
    w = {"mu." + s: torch.rand(D) for s in "rkvgw"}
    w.update({s: g(F, D) for s in "rkvg"})
    w.update({"w1": g(rank, D), "w2": g(F, rank), "w0": g(F) - 1.0, "u": g(H_, dk), "norm": 1 + 0.2 * torch.randn(F), "o": g(D, F)})
    return w


@pytest.mark.parametrize("name, dtype, tol", DTYPES)
@pytest.mark.parametrize("H_, dk, D, rank", [(3, 5, 36, 3), (1, 40, 64, 8), (2, 128, 48, 16), (5, 33, 24, 1)])
def test_time_mix_part_in_portions_and_token_by_token(name, dtype, tol, H_, dk, D, rank):
    """The plain mixer over whole sequences against the part fed with a long portion, portions of two and three tokens
    and single tokens, for two requests with their own states (the previous input and the matrix state)."""
    from jax_llm_examples_b200.parts import LayerCache, Runtime, TimeMixWKV

    torch.manual_seed(dk)
    rt = Runtime(dtype, torch.device(DEV))
    wd = {k: v.to(dtype) for k, v in _wkv_weights(D, H_, dk, rank).items()}
    d = lambda k: wd[k].to(DEV)
    mixer = TimeMixWKV(torch.stack([d("mu." + s) for s in "rkvgw"]), torch.stack([d(s) for s in "rkvg"]), d("w1"), d("w2"), d("w0"),
                       d("u"), d("norm"), d("o"), H_, dk, 1e-5)
    states = tuple(torch.zeros(3, *n.shape, device=DEV) for n in mixer.state_needs())
    assert [tuple(s.shape[1:]) for s in states] == [(D,), (H_, dk, dk)]
    seqs = [torch.randn(n, D).to(dtype).float() for n in (37, 12)]
    ref = [plain.wkv_mixer(s.double(), {"m." + k: v.double() for k, v in wd.items()}, "m.", {"heads": H_, "dim": dk}, 1e-5) for s in seqs]
    fwd = lambda ctx, rows: H.as_rows_sum(mixer.forward(ctx, None, LayerCache(None, None, False, states[0], states), h32=rows.to(DEV)))
    got = _run_in_cuts(rt, seqs, [[20, 2, 1, 3, 1, 1, 9], [1, 1, 2, 5, 3]], [2, 1], fwd, 7)
    for r in range(2):
        _close(got[r], ref[r], tol, f"{name} request {r}")


@pytest.mark.parametrize("name, dtype, tol", DTYPES)
@pytest.mark.parametrize("H_, dk, dv, D, rank, tau", [(2, 7, 9, 36, 5, 3.5), (1, 32, 64, 64, 8, 16.0), (4, 16, 16, 40, 3, 1.0)])
def test_gated_linear_attention_part_in_portions(name, dtype, tol, H_, dk, dv, D, rank, tau):
    from jax_llm_examples_b200.parts import GatedLinearAttention, LayerCache, Runtime

    torch.manual_seed(dk)
    rt = Runtime(dtype, torch.device(DEV))
    g = lambda *s: torch.randn(*s) * 0.3
    w = {"q": g(H_ * dk, D), "k": g(H_ * dk, D), "v": g(H_ * dv, D), "g": g(H_ * dv, D), "a1": g(rank, D), "a2": g(H_ * dk, rank),
         "a2.b": g(H_ * dk) + 2.0, "norm": 1 + 0.2 * torch.randn(dv), "o": g(D, H_ * dv)}
    wd = {k: v.to(dtype) for k, v in w.items()}
    d = lambda k: wd[k].to(DEV)
    mixer = GatedLinearAttention(torch.cat([d("q"), d("k"), d("v"), d("g")]), d("a1"), d("a2"), d("a2.b"), d("norm"), d("o"), H_, dk, dv, tau, 1e-5)
    state = torch.zeros(3, H_, dk, dv, device=DEV)
    seqs = [torch.randn(n, D).to(dtype) for n in (41, 10)]
    m = {"heads": H_, "dim": dk, "vdim": dv, "tau": tau}
    ref = [plain.gated_linear_attention(s.double(), {"m." + k: v.double() for k, v in wd.items()}, "m.", m, 1e-5) for s in seqs]
    fwd = lambda ctx, rows: H.as_rows_sum(mixer.forward(ctx, rows.to(DEV), LayerCache(None, None, False, state, (state,))))
    got = _run_in_cuts(rt, seqs, [[24, 2, 1, 3, 1, 1, 9], [1, 1, 2, 6]], [0, 2], fwd, 7)
    for r in range(2):
        _close(got[r], ref[r], tol, f"{name} request {r}")


def _attention_part(wd, m, eps, dtype):
    from jax_llm_examples_b200.parts import GatedPagedAttention, rotary_frequencies

    d = lambda k: wd[k].to(DEV)
    return GatedPagedAttention(
        torch.cat([d("q"), d("k"), d("v"), d("g")]), d("o"), m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["scale"], eps,
        d("q.norm"), d("k.norm"), rotary_frequencies(m["rot"]["base"], m["rot"]["dims"]).to(DEV) if m["rot"]["dims"] else None,
        m["rot"]["dims"], window=m["mask"]["size"], padded_dim=GatedPagedAttention.padded_size(m["dim"], m["vdim"], dtype))


@pytest.mark.parametrize("name, dtype, tol", DTYPES)
@pytest.mark.parametrize("m", [
    {"heads": 6, "kv_heads": 2, "dim": 10, "vdim": 6, "mask": {"size": 7}, "rot": {"base": 100.0, "dims": 4}, "scale": 0.4},
    {"heads": 4, "kv_heads": 1, "dim": 64, "vdim": 64, "mask": {"size": 20}, "rot": {"base": 1e4, "dims": 64}, "scale": 0.1},
    {"heads": 2, "kv_heads": 2, "dim": 24, "vdim": 40, "mask": {"size": 1000}, "rot": {"base": 10.0, "dims": 0}, "scale": 0.2},
    {"heads": 3, "kv_heads": 3, "dim": 128, "vdim": 32, "mask": {"size": 1}, "rot": {"base": 5e5, "dims": 32}, "scale": 0.05},
])
def test_windowed_gated_attention_part_over_scattered_pages(name, dtype, tol, m):
    """A prompt portion, a portion that starts in the middle of a page, and single tokens, against the plain function:
    the window's edge crosses page borders; keys and values of unequal size share the padded pages."""
    from jax_llm_examples_b200.parts import LayerCache, Runtime

    torch.manual_seed(m["heads"])
    D, eps, T = 48, 1e-5, 45
    rt = Runtime(dtype, torch.device(DEV))
    g = lambda *s: torch.randn(*s) * 0.3
    Hq, Hkv, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    w = {"q": g(Hq * dk, D), "k": g(Hkv * dk, D), "v": g(Hkv * dv, D), "g": g(Hq, D), "q.norm": 1 + 0.2 * torch.randn(dk),
         "k.norm": 1 + 0.2 * torch.randn(dk), "o": g(D, Hq * dv)}
    wd = {k: v.to(dtype) for k, v in w.items()}
    mixer = _attention_part(wd, m, eps, dtype)
    need = mixer.kv_need()
    assert (need.planes, need.num_kv_heads) == (2, Hkv) and need.head_dim >= max(dk, dv)
    pages = torch.zeros(40, 2, Hkv, 16, need.head_dim, device=DEV, dtype=dtype)
    table = torch.randperm(40)[:3].reshape(1, 3).to(torch.int32).to(DEV)
    hs = torch.randn(T, D).to(dtype)
    outs = []
    for lo, hi in ((0, 21), (21, 43), (43, 44), (44, 45)):
        ctx = _ctx(rt, [hi - lo], [lo], planners=mixer.step_planners())
        outs.append(H.as_rows_sum(mixer.forward(ctx, hs[lo:hi].to(DEV), LayerCache(pages, table, True, None))))
        assert int(ctx.status) == 0
    ref = plain.window_attention(hs.double(), {"m." + k: v.double() for k, v in wd.items()}, "m.", m, eps)
    _close(torch.cat(outs), ref, tol, name)


@pytest.mark.parametrize("name, dtype, tol", DTYPES)
def test_two_mixers_side_by_side_share_their_products(name, dtype, tol):
    """left_scale * attention + right_scale * linear attention through ONE input product and ONE output product, against
    the plain sum of the two plain mixers: a portion of more than 256 rows (the mixers run one after the other), a short
    portion and single tokens (the second mixer runs on another stream), states and pages carried between them."""
    from jax_llm_examples_b200.parts import GatedLinearAttention, LayerCache, ParallelMixers, Runtime

    torch.manual_seed(9)
    D, eps, T = 40, 1e-5, 300
    rt = Runtime(dtype, torch.device(DEV))
    g = lambda *s: torch.randn(*s) * 0.3
    m = {"left": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 12, "mask": {"size": 37}, "rot": {"base": 1000.0, "dims": 6}, "scale": 0.3},
         "right": {"heads": 3, "dim": 8, "vdim": 5, "tau": 4.0}, "left_scale": 1.3, "right_scale": 0.6}
    a, r = m["left"], m["right"]
    w = {"left.q": g(32, D), "left.k": g(16, D), "left.v": g(24, D), "left.g": g(4, D), "left.q.norm": 1 + 0.2 * torch.randn(8),
         "left.k.norm": 1 + 0.2 * torch.randn(8), "left.o": g(D, 48),
         "right.q": g(24, D), "right.k": g(24, D), "right.v": g(15, D), "right.g": g(15, D), "right.a1": g(4, D), "right.a2": g(24, 4),
         "right.a2.b": g(24) + 2.0, "right.norm": 1 + 0.2 * torch.randn(5), "right.o": g(D, 15)}
    wd = {k: v.to(dtype) for k, v in w.items()}
    d = lambda k: wd[k].to(DEV)
    left = _attention_part({k[5:]: v for k, v in wd.items() if k.startswith("left.")}, a, eps, dtype)
    right = GatedLinearAttention(torch.cat([d("right.q"), d("right.k"), d("right.v"), d("right.g")]), d("right.a1"), d("right.a2"),
                                 d("right.a2.b"), d("right.norm"), d("right.o"), 3, 8, 5, 4.0, eps)
    both = ParallelMixers([left, right], [1.3, 0.6])
    assert both.kv_need() == left.kv_need() and len(both.state_needs()) == 1 and both.w_in.shape[0] == 76 + 78 and both.w_o.shape == (D, 63)
    pages = torch.zeros(40, 2, 2, 16, both.kv_need().head_dim, device=DEV, dtype=dtype)
    table = torch.randperm(40)[:19].reshape(1, 19).to(torch.int32).to(DEV)
    state = torch.zeros(2, 3, 8, 5, device=DEV)
    hs = torch.randn(T, D).to(dtype)
    outs = []
    for lo, hi in ((0, 270), (270, 298), (298, 299), (299, 300)):
        ctx = _ctx(rt, [hi - lo], [lo], [1], planners=both.step_planners() or left.step_planners())
        outs.append(H.as_rows_sum(both.forward(ctx, hs[lo:hi].to(DEV), LayerCache(pages, table, True, state, (state,)))))
        assert int(ctx.status) == 0
    ref = plain.parallel_mixer(hs.double(), {"m." + k: v.double() for k, v in wd.items()}, "m.", m, eps)
    _close(torch.cat(outs), ref, tol, name)
    assert float(state[0].abs().max()) == 0.0 and float(state[1].abs().max()) > 0.0


@pytest.mark.parametrize("name, dtype, tol", DTYPES)
@pytest.mark.parametrize("size", [16, 128])  # padded to 64 in bfloat16 (the mma.sync kernels), and the tcgen05 kernel's size
@pytest.mark.parametrize("window", [5, 16, 21, 64])
def test_a_key_just_inside_and_just_outside_the_window(name, dtype, tol, window, size):
    """Made so that a fault shows: queries and keys are the (normed) hidden state itself, and ONE earlier token points
    where the query points, with a score that outweighs everything; its value is a marker.  Placed window - 1 tokens
    back it must be all the query sees; placed window tokens back it must be gone.  In a prompt portion and for a
    token decoded alone; edges at and across page borders (pages of 16)."""
    from jax_llm_examples_b200.parts import GatedPagedAttention, LayerCache, Runtime

    torch.manual_seed(window)
    D = dk = dv = size
    rt = Runtime(dtype, torch.device(DEV))
    eye = torch.eye(D)
    w_in = torch.cat([eye, eye, eye, torch.zeros(1, D)]).to(dtype).to(DEV)  # q = k = v = h; gate logit 0: a half
    mixer = GatedPagedAttention(w_in, eye.to(dtype).to(DEV), 1, 1, dk, dv, 8.0, 1e-6, None, None, None, 0, window=window,
                                padded_dim=GatedPagedAttention.padded_size(dk, dv, dtype))
    T = 100
    for qpos, decoded in ((99, False), (99, True), (70, False), (window - 1, False), (window, True)):
        for back, seen in ((window - 1, True), (window, False)):
            if qpos - back < 0:
                continue
            hs = torch.randn(T, D) * 0.05
            direction = torch.zeros(D)
            direction[3] = 4.0
            hs[qpos] = direction
            hs[qpos - back] = direction + torch.nn.functional.one_hot(torch.tensor(8), D).float()  # the marker: entry 8
            hs = hs.to(dtype)
            page = 64 if size == 128 else 16  # pages of 64: long portions of head size 128 go to the tcgen05 kernel
            pages = torch.zeros(12, 2, 1, page, mixer.head_dim, device=DEV, dtype=dtype)
            table = torch.randperm(12)[:7].reshape(1, 7).to(torch.int32).to(DEV)
            cuts = [(0, qpos), (qpos, qpos + 1)] if decoded else [(0, qpos + 1)]
            out = None
            for lo, hi in cuts:
                if hi > lo:
                    ctx = _ctx(rt, [hi - lo], [lo], planners=mixer.step_planners(), page_size=page)
                    out = H.as_rows_sum(mixer.forward(ctx, hs[lo:hi].to(DEV), LayerCache(pages, table, True, None)))
            if size == 128 and dtype == torch.bfloat16 and not decoded and qpos >= 63:
                assert any("tc" in kinds for kinds in ctx.scratch.get("attention_kernels", ())), "the tcgen05 kernel did not run"
            marker = 2.0 * float(out[-1, 8])  # the gate halves
            # seen: the needle shares the weight with the query itself (equal scores up to the marker's part): about a half
            assert (marker > 0.4) == seen and (seen or abs(marker) < 0.05), \
                f"{name} window {window}: query {qpos} ({'decoded' if decoded else 'prompt'}), key {back} back: marker {marker:.3f}"


@pytest.mark.parametrize("name, dtype, tol", DTYPES)
@pytest.mark.parametrize("E, k, D, F, shared", [(5, 2, 36, 12, 9), (8, 3, 128, 64, 32), (2, 2, 48, 16, None), (3, 1, 40, 8, None)])
def test_softmax_routed_experts_part(name, dtype, tol, E, k, D, F, shared):
    """The part against the plain mixture with the part's own choices forced (they must be the plain choice unless two
    logits tie): weights over the chosen only, outputs weighted, the shared expert added unweighted."""
    from jax_llm_examples_b200.parts import DenseBiasedMLP, Runtime, SoftmaxRoutedMLPExperts

    torch.manual_seed(E)
    rt = Runtime(dtype, torch.device(DEV))
    g = lambda *s: torch.randn(*s) * 0.3
    w = {"router": g(E, D), "router.b": torch.randn(E)}
    for e in range(E):
        w[f"e{e}.up"], w[f"e{e}.down"] = g(F, D), g(D, F)
    if shared:
        w["shared.up"], w["shared.down"] = g(shared, D), g(D, shared)
    wd = {n: v.to(dtype) for n, v in w.items()}
    d = lambda n: wd[n].to(DEV)
    sh = DenseBiasedMLP(d("shared.up"), None, d("shared.down"), None, "relu2") if shared else None
    ff = SoftmaxRoutedMLPExperts(d("router"), d("router.b"), torch.stack([d(f"e{e}.up") for e in range(E)]),
                                 torch.stack([d(f"e{e}.down") for e in range(E)]), k, "relu2", sh)
    N = 23
    h32 = torch.randn(N, D)
    ctx = _ctx(rt, [N], [0])
    ctx.scratch["record_routing"] = []
    got = H.as_rows_sum(ff.forward(ctx, h32.to(dtype).to(DEV), h32.to(DEV)))
    chosen = ctx.scratch["record_routing"][0].cpu()
    mlp = {"router": {"experts": E, "top": k}, "shared": {"ff": shared} if shared else None}
    P = {"m." + n: v.double() for n, v in wd.items()}
    # the router reads the unrounded rows, the experts their rounding to the activations' type
    z = plain.router_logits(h32.double(), P, "m.")
    assert torch.equal(torch.sort(chosen.long(), dim=-1).values, torch.sort(torch.topk(z, k, dim=-1).indices, dim=-1).values)
    hr = h32.to(dtype).double()
    wts = torch.softmax(torch.gather(z, 1, chosen.long()), dim=-1)
    ref = torch.zeros(N, D, dtype=torch.float64)
    for t in range(N):
        for j in range(k):
            ref[t] += wts[t, j] * plain.expert(hr[t:t + 1], P, f"m.e{int(chosen[t, j])}.")[0]
    if shared:
        ref += plain.expert(hr, P, "m.shared.")
    _close(got, ref, tol, name)
    full, _, _ = plain.mixture_of_experts(hr, P, "m.", mlp, chosen)  # the plain function itself, fed the rounded rows
    assert float((full - ref).abs().max()) < 0.1 * float(ref.abs().max()) + 1e-9


# --------------------------------------------------------------------------------------- whole models, by traces
@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("makisun")
    return {n: MH.make_dir(root / n, n, seed=i + 1) for i, n in enumerate(MH.CONFIGS)}


def _engine(folder, dtype, max_tokens=512, page_size=16, max_slots=4, **kw):
    import jax_llm_examples_b200 as J

    return J.Engine(J.load_model(folder, dtype, DEV), max_tokens=max_tokens, page_size=page_size, max_slots=max_slots, **kw)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(MH.CONFIGS))
def test_every_kind_of_cut_against_the_plain_implementation(folders, name, dtype):
    """Whole prompts; most of a prompt and then 40 tokens one by one; portions down to two tokens; up to four live
    requests mixed, in a pool too small for all of them, so that pages and slots are used again.  Every position's
    logits are compared, the first tokens of a sequence included; the plain implementation takes the engine's experts."""
    vocab = MH.config(name)["vocab"]
    rng = random.Random(7)
    requests = H.random_requests(rng, vocab, [61, 1, 2, 33, 17, 90, 5])
    engine = _engine(folders[name], dtype, max_tokens=16 * 16)
    for steps in (H.trace_whole(requests), H.trace_tail_decode(requests, tail=40), H.trace_portions(requests, rng),
                  H.trace_mixed(requests, rng, max_live=4)):
        got, routing = H.run_trace(engine, steps, record_routing=True)
        assert len(got) == sum(len(t) for t in requests.values())
        MH.compare(folders[name], requests, got, routing, dtype)
        assert engine.manager.free_slots() == 4 and all(engine.manager.free_pages(g) == engine.num_pages for g in range(len(engine.manager.groups)))


@pytest.mark.parametrize("name", ["small", "wide", "padded"])
def test_logits_do_not_depend_on_the_cut_or_on_the_batch(folders, name):
    """float32: the same request whole, token by token, in portions, and beside three other requests gives the same
    logits to within rounding of a sum's order (far below the tolerance against the plain implementation)."""
    vocab = MH.config(name)["vocab"]
    rng = random.Random(11)
    requests = H.random_requests(rng, vocab, [70, 23, 41, 9])
    engine = _engine(folders[name], "float32")
    whole, _ = H.run_trace(engine, H.trace_whole(requests), record_routing=False)
    for steps in (H.trace_tail_decode(requests, tail=70), H.trace_portions(requests, rng), H.trace_mixed(requests, rng)):
        got, _ = H.run_trace(engine, steps, record_routing=False)
        worst = max(MH.row_err(got[k], whole[k]) for k in whole)
        assert worst < 2e-6, f"{name}: logits moved by {worst:.2e} with the cut"


@pytest.mark.parametrize("name", ["small", "wide", "recurrent"])
def test_decoding_through_replayed_graphs_equals_decoding_without(folders, name):
    """bfloat16: decode-only steps are captured in CUDA graphs and replayed; states and pages are found by slot and table
    on the device, so the replayed steps must give what the same steps give launched one kernel at a time."""
    vocab = MH.config(name)["vocab"]
    rng = random.Random(5)
    requests = H.random_requests(rng, vocab, [50, 37])
    outs = []
    for graphs in (True, False):
        engine = _engine(folders[name], "bfloat16", use_graphs=graphs)
        got, _ = H.run_trace(engine, H.trace_tail_decode(requests, tail=30), record_routing=False)
        assert (engine.graph_replays > 0) == graphs
        outs.append(got)
    worst = max(MH.row_err(outs[0][k], outs[1][k]) for k in outs[0])
    # a replayed step's attention is planned for a rounded-up length: other splits, sums in another order
    assert worst < (1e-6 if name == "recurrent" else 2e-2), f"{name}: replayed steps differ by {worst:.2e}"


def test_long_decoding_and_slots_used_again(folders):
    """300 tokens one by one after a short prompt, in both precisions: the recurrent states and the window's pages are
    carried over hundreds of steps (the window's old pages are given back on the way); then the same slot serves
    another request, which must not see what the first left."""
    name = "small"
    vocab = MH.config(name)["vocab"]
    toks = [random.Random(3).randrange(vocab) for _ in range(320)]
    other = [random.Random(4).randrange(vocab) for _ in range(25)]
    for dtype in ("float32", "bfloat16"):
        engine = _engine(folders[name], dtype, max_tokens=320, max_slots=1)
        for req in ({"a": toks}, {"b": other}):
            got, routing = H.run_trace(engine, H.trace_tail_decode(req, tail=300), record_routing=True)
            MH.compare(folders[name], req, got, routing, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_long_prompt_whole_and_in_portions(folders, dtype):
    """560 tokens in one step beside a short request, and the same in two portions: against the plain implementation at
    places near the start, in the middle and at the end, and against each other."""
    import jax_llm_examples_b200 as J

    name = "wide"
    vocab = MH.config(name)["vocab"]
    rng = random.Random(5)
    toks, other = [rng.randrange(vocab) for _ in range(560)], [rng.randrange(vocab) for _ in range(30)]
    want = [0, 1, 2, 39, 40, 41, 255, 256, 300, 511, 512, 558, 559]
    engine = _engine(folders[name], dtype, max_tokens=1024)
    engine.record_routing = True
    a, b = engine.new_request(), engine.new_request()
    whole = engine.step([J.StepEntry(a, toks, want), J.StepEntry(b, other, [29])]).cpu().numpy().copy()
    forced = [c.cpu()[:560] for c in engine.last_routing]
    engine.finish(a), engine.finish(b)
    a = engine.new_request()
    first = engine.step([J.StepEntry(a, toks[:300], [w for w in want if w < 300])]).cpu().numpy().copy()
    second = engine.step([J.StepEntry(a, toks[300:], [w - 300 for w in want if w >= 300])]).cpu().numpy().copy()
    engine.check_status()
    engine.finish(a)
    parts = np.concatenate([first, second])
    ref, shortfall = MH.plain_logits(folders[name], toks, forced)
    assert shortfall < MH.TIE[dtype]
    for k, w in enumerate(want):
        assert MH.row_err(whole[k], ref[w]) < MH.TOL[dtype], f"{dtype}: position {w} of the whole prompt"
        if dtype == "float32":  # in bfloat16 the portions may choose other experts where two logits tie
            assert MH.row_err(parts[k], ref[w]) < MH.TOL[dtype], f"{dtype}: position {w} of the prompt in portions"
            assert MH.row_err(whole[k], parts[k]) < 1e-5


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["small", "wide", "recurrent"])
def test_greedy_generation_through_the_scheduler(folders, name, dtype):
    """The framework's own entry point: prompts of unequal length under a small token budget per step, so that
    prompt portions run beside decoded tokens."""
    import jax_llm_examples_b200 as J

    vocab = MH.config(name)["vocab"]
    prompts = [[(7 * i + 3 * j) % vocab for i in range(n)] for j, n in enumerate((29, 3, 12))]
    model = J.load_model(folders[name], dtype, DEV)
    got = J.generate(model, prompts, J.SamplingParams(max_new_tokens=10), page_size=16, max_tokens_per_step=16)
    for p, g in zip(prompts, got):
        assert len(g) == 10
        MH.greedy_checked(folders[name], p, g, dtype)


def test_command_line_generates_from_a_preset_and_from_a_folder(folders, capsys):
    from jax_llm_examples_b200.main import main

    assert main(["--preset", "makisun_tiny", "--random-prompts", "2", "--prompt-len", "9", "--max-new-tokens", "4"]) == 0
    assert capsys.readouterr().out.count("-" * 80) == 2
    assert main(["--model", str(folders["recurrent"]), "--dtype", "float32", "--prompt-ids", "1,2,3,4,5", "--max-new-tokens", "5",
                 "--page-size", "16"]) == 0
    ids = [int(t) for t in capsys.readouterr().out.splitlines()[1].split()]
    MH.greedy_checked(folders["recurrent"], [1, 2, 3, 4, 5], ids, "float32")


def test_trace_replay_program_on_a_makisun_folder(folders, tmp_path):
    """bin/trace_run picks the model class by config.json and writes the wanted logits."""
    name, dtype = "padded", "float32"
    vocab = MH.config(name)["vocab"]
    toks = [(5 * i + 2) % vocab for i in range(21)]
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": toks[:13], "want": [0, 12]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": toks[13:20], "want": []}, {"id": "b", "tokens": toks[:2], "want": [1]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": toks[20:], "want": [0]}], "end": ["a"]}]
    out = tmp_path / "out"
    p = subprocess.run([sys.executable, os.path.join(H.ROOT, "bin", "trace_run"), "--model", str(folders[name]), "--dtype", dtype,
                        "--out", str(out), "--max-tokens", "128"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    ref = MH.plain_logits(folders[name], toks)[0]
    rows = {0: [0, 12], 1: [1], 2: [20]}
    for step, places in rows.items():
        got = np.fromfile(out / f"{step}.f32", dtype="<f4").reshape(len(places), vocab)
        for g, pl in zip(got, places):
            assert MH.row_err(g, ref[pl]) < MH.TOL[dtype]
