"""Tebivik on the GPU against the plain implementation: each mechanism alone (kernel or part against the plain
function of the same name), then whole models through the engine's step function under every kind of cut, batches
against requests alone, pages and slots that are used again, long decoding, and greedy generation through the
scheduler.  All configurations are this file's own (``tests/tebivik_helpers.py``)."""

import random
import subprocess
import sys

import numpy as np
import pytest
import torch

from tests import helpers as H
from tests import tebivik_helpers as TH
from tests.plain import tebivik_plain as plain

pytestmark = pytest.mark.gpu
DEV = "cuda"
DTYPES = [("float32", torch.float32, 2e-5), ("bfloat16", torch.bfloat16, 3e-2)]


def _ctx(runtime, q_lens, starts, slots=None, planners=(), page_size=16, n_pages=64):
    """A step context for a hand-made batch (what Engine.step builds) and a block table over scattered pages."""
    from jax_llm_examples_b200.parts import StepContext, Workspace

    pos = [s + i for n, s in zip(q_lens, starts) for i in range(n)]
    req = [r for r, n in enumerate(q_lens) for _ in range(n)]
    slots = list(range(len(q_lens))) if slots is None else slots
    t = lambda v: torch.tensor(v, device=DEV, dtype=torch.int32)
    N = sum(q_lens)
    ctx = StepContext(runtime=runtime, n_tokens=N, n_requests=len(q_lens), token_ids=t([0] * N), positions=t(pos),
                      req_of_token=t(req), cu_q=t(list(np.concatenate([[0], np.cumsum(q_lens)]))), q_start=t(starts),
                      kv_len=t([s + n for n, s in zip(q_lens, starts)]), slot_ids=t(slots), logit_rows=t([]), n_logit_rows=0,
                      status=torch.zeros(1, device=DEV, dtype=torch.int32), host_q_lens=list(q_lens), host_q_start=list(starts),
                      host_slot_ids=slots, max_q_len=max(q_lens), max_kv_len=max(s + n for n, s in zip(q_lens, starts)),
                      workspace=Workspace(torch.device(DEV)))
    ctx.plan_with(planners, page_size)
    return ctx


def _close(got: torch.Tensor, ref: torch.Tensor, tol: float, what: str = ""):
    got, ref = got.double().cpu(), ref.double().cpu()
    err = float((got - ref).abs().max() / ref.abs().max().clamp_min(1e-9))
    assert err < tol, f"{what}: relative error {err:.3e} (allowed {tol:.1e})"


# ------------------------------------------------------------------------------------- kernels and parts alone
@pytest.mark.parametrize("D, groups, splits", [(36, 3, 1), (200, 1, 3), (1024, 8, 2), (30, 30, 1)])
def test_group_norm_kernel_closes_one_sublayer_and_opens_the_next(D, groups, splits):
    """x += mult * w_b * groupnorm(sum of partials + bias); out = w * groupnorm(x): one kernel, against the plain norm."""
    from jax_llm_examples_b200.kernels import api as K

    torch.manual_seed(D)
    N, mult, eps = 5, 0.6, 1e-5
    x, part = torch.randn(N, D, device=DEV), torch.randn(splits, N, D, device=DEV)
    bias, wb, w = (torch.randn(D, device=DEV) for _ in range(3))
    x2 = x.clone()
    out, out32 = torch.empty(N, D, device=DEV, dtype=torch.bfloat16), torch.empty(N, D, device=DEV)
    K.group_norm(x2, part, splits, bias, wb, groups, mult, w, groups, True, eps, out, out32)
    x_ref = x.double().cpu() + mult * plain.group_rms_norm((part.sum(0) + bias).double().cpu(), wb.double().cpu(), eps, groups)
    _close(x2, x_ref, 3e-6, "residual")
    _close(out32, plain.group_rms_norm(x_ref, w.double().cpu(), eps, groups), 3e-6, "normed rows")
    _close(out.float(), out32, 1e-2, "rounded rows")
    # gathered rows (the final norm of a step that wants few logits): x stays as it was
    rows = torch.tensor([3, 0], device=DEV, dtype=torch.int32)
    x3, o3 = x.clone(), torch.empty(2, D, device=DEV)
    K.group_norm(x3, part, splits, bias, wb, groups, mult, w, groups, True, eps, None, o3, rows)
    assert torch.equal(x3, x)
    _close(o3, plain.group_rms_norm(x_ref[[3, 0]], w.double().cpu(), eps, groups), 3e-6, "gathered rows")
    # a plain delta, no closing norm, no opening norm: the sum itself in the activations' type
    x4, o4 = x.clone(), torch.empty(N, D, device=DEV)
    K.group_norm(x4, part, splits, pre_norm=False, out=o4)
    _close(o4, (x + part.sum(0)), 3e-6, "plain sum")


@pytest.mark.parametrize("D", [40, 38])  # four channels per thread, and one
@pytest.mark.parametrize("taps", [1, 2, 4])
def test_short_conv_carries_its_last_inputs_across_portions_of_any_size(taps, D):
    """Three requests of unequal length in portions down to one token, interleaved in one batch; state slots given
    in another order than the requests; a slot used again after it was cleared."""
    from jax_llm_examples_b200.parts import ResidualShortConv, Runtime

    torch.manual_seed(taps)
    rt = Runtime(torch.float32, torch.device(DEV))
    conv = ResidualShortConv(torch.randn(D, taps, device=DEV))
    need = conv.state_need()
    assert (need is None) == (taps == 1)
    state = None if need is None else torch.zeros(6, *need.shape, device=DEV)
    seqs = [torch.randn(n, D, device=DEV) for n in (23, 9, 14)]
    slots = [4, 1, 5]
    want = [s.double().cpu() + plain.causal_conv(s.double().cpu(), conv.weight.double().cpu()) for s in seqs]
    cuts = [[1, 1, 2, 5, 1, 3, 2, 8], [2, 1, 1, 1, 4], [3, 1, 2, 2, 1, 1, 4]]
    at, got = [0, 0, 0], [[], [], []]
    for step in range(8):
        live = [r for r in range(3) if step < len(cuts[r])]
        lens = [cuts[r][step] for r in live]
        h = torch.cat([seqs[r][at[r]:at[r] + n] for r, n in zip(live, lens)])
        ctx = _ctx(rt, lens, [at[r] for r in live], [slots[r] for r in live])
        out = conv.forward(ctx, h.contiguous(), state)
        o = 0
        for r, n in zip(live, lens):
            got[r].append(out[o:o + n])
            o += n
            at[r] += n
    for r in range(3):
        _close(torch.cat(got[r]), want[r], 2e-6, f"request {r}")
    if state is not None:  # the slot of request 1 goes to a new request: cleared, it must not remember
        state[1].zero_()
        ctx = _ctx(rt, [5], [0], [1])
        _close(conv.forward(ctx, seqs[0][:5].contiguous(), state), want[0][:5], 2e-6, "slot used again")


def _hgrn2_weights(D, H, dk, dv, dev="cpu"):
    g = lambda *s: torch.randn(*s) * 0.3
    return {"q": g(H * dk, D), "f": g(H * dk, D), "f.b": g(H * dk), "lower": torch.rand(H * dk), "v": g(H * dv, D),
            "norm": 1 + 0.2 * torch.randn(dv), "o": g(D, H * dv)}


@pytest.mark.parametrize("name, dtype, tol", DTYPES)
@pytest.mark.parametrize("H_, dk, dv, D", [(3, 5, 7, 36), (1, 40, 64, 64), (2, 128, 96, 48), (5, 33, 1, 24)])
def test_hgrn2_part_in_portions_and_token_by_token(name, dtype, tol, H_, dk, dv, D):
    """The recurrence over a whole sequence in the plain way against the part fed with a long portion, portions of
    two and three tokens and single tokens, for two requests with their own states."""
    from jax_llm_examples_b200.parts import HGRN2, LayerCache, Runtime

    torch.manual_seed(dk)
    rt = Runtime(dtype, torch.device(DEV))
    w = _hgrn2_weights(D, H_, dk, dv)
    wd = {k: v.to(dtype) for k, v in w.items()}  # stored precision
    mixer = HGRN2(torch.cat([wd["q"], wd["f"], wd["v"]]).to(DEV), wd["f.b"].to(DEV), wd["lower"].to(DEV), wd["norm"].to(DEV),
                  wd["o"].to(DEV), H_, dk, dv, 1e-5)
    (need,) = mixer.state_needs()
    state = torch.zeros(3, *need.shape, device=DEV)
    seqs = [torch.randn(n, D).to(dtype) for n in (37, 12)]
    ref = [plain.hgrn2(s.double(), {"m." + k: v.double() for k, v in wd.items()}, "m.", {"heads": H_, "dim": dk, "vdim": dv}, 1e-5)
           for s in seqs]
    cuts = [[20, 2, 1, 3, 1, 1, 9], [1, 1, 2, 5, 3]]
    at, got = [0, 0], [[], []]
    for step in range(7):
        live = [r for r in range(2) if step < len(cuts[r])]
        lens = [cuts[r][step] for r in live]
        h = torch.cat([seqs[r][at[r]:at[r] + n] for r, n in zip(live, lens)]).float().to(DEV)
        ctx = _ctx(rt, lens, [at[r] for r in live], [2 - r for r in live])
        out = H.as_rows_sum(mixer.forward(ctx, None, LayerCache(None, None, False, state, (state,)), h32=h))
        o = 0
        for r, n in zip(live, lens):
            got[r].append(out[o:o + n])
            o += n
            at[r] += n
    for r in range(2):
        _close(torch.cat(got[r]), ref[r], tol, f"{name} request {r}")


@pytest.mark.parametrize("name, dtype, tol", DTYPES)
def test_hgrn2_long_portions_are_scanned_in_segments(name, dtype, tol):
    """Portions of at least two segments are scanned segment by segment at once (each but the first from a zero state,
    then chained and corrected): a request of 700 tokens beside a short one and one that decodes, then a second long
    portion that goes on from the carried state, against the plain recurrence over the whole sequences; and against the
    same tokens walked in order (no segments), to within rounding."""
    from jax_llm_examples_b200.parts import HGRN2, LayerCache, Runtime
    from jax_llm_examples_b200.parts.recurrent import SEGMENT_TOKENS, plan_scan_segments

    torch.manual_seed(3)
    H_, dk, dv, D = 3, 12, 20, 32
    rt = Runtime(dtype, torch.device(DEV))
    wd = {k: v.to(dtype) for k, v in _hgrn2_weights(D, H_, dk, dv).items()}
    wd["lower"] = (0.05 + 0.9 * torch.rand(H_ * dk)).to(dtype)
    mixer = HGRN2(torch.cat([wd["q"], wd["f"], wd["v"]]).to(DEV), wd["f.b"].to(DEV), wd["lower"].to(DEV), wd["norm"].to(DEV),
                  wd["o"].to(DEV), H_, dk, dv, 1e-5)
    assert mixer.step_planners() == (plan_scan_segments,)
    lens = (2 * SEGMENT_TOKENS + 188 + 2 * SEGMENT_TOKENS + 5, 40, 9)
    seqs = [torch.randn(n, D).to(dtype) for n in lens]
    ref = [plain.hgrn2(s.double(), {"m." + k: v.double() for k, v in wd.items()}, "m.", {"heads": H_, "dim": dk, "vdim": dv}, 1e-5)
           for s in seqs]
    first = 2 * SEGMENT_TOKENS + 188
    steps = [[(0, 0, first), (1, 0, 40), (2, 0, 1)], [(2, 1, 2), (0, first, lens[0])], [(2, 2, 9)]]
    results = {}
    for planned in (True, False):
        state = torch.zeros(3, H_, dk, dv, device=DEV)
        got = [[], [], []]
        for step in steps:
            h = torch.cat([seqs[r][lo:hi] for r, lo, hi in step]).float().to(DEV)
            ctx = _ctx(rt, [hi - lo for _, lo, hi in step], [lo for _, lo, _ in step], [r for r, _, _ in step],
                       planners=mixer.step_planners() if planned else ())
            assert ("scan_segments" in ctx.arrays) == (planned and max(hi - lo for _, lo, hi in step) >= 2 * SEGMENT_TOKENS)
            out = H.as_rows_sum(mixer.forward(ctx, None, LayerCache(None, None, False, state, (state,)), h32=h))
            o = 0
            for r, lo, hi in step:
                got[r].append(out[o:o + hi - lo])
                o += hi - lo
        results[planned] = [torch.cat(g) for g in got]
        for r in range(3):
            _close(results[planned][r], ref[r], tol, f"{name} request {r} segments={planned}")
    for r in range(3):
        _close(results[True][r], results[False][r], 1e-5 if dtype == torch.float32 else 2e-2, f"{name} request {r}: segments against in order")


def _latent_weights(D, m):
    H_, dn, dr, dv, qr, kr = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["q_rank"], m["kv_rank"]
    g = lambda *s: torch.randn(*s) * 0.3
    return {"dq": g(qr, D), "dq.norm": 1 + 0.2 * torch.randn(qr), "uq": g(H_ * (dn + dr), qr), "dkv": g(kr + dr, D),
            "dkv.norm": 1 + 0.2 * torch.randn(kr), "uk": g(H_ * dn, kr), "uv": g(H_ * dv, kr), "sink": torch.randn(H_), "o": g(D, H_ * dv)}


def _latent_part(wd, m, eps, conv=None):
    from jax_llm_examples_b200.parts import LatentAttention

    d = lambda k: wd[k].to(DEV)
    return LatentAttention(torch.cat([wd["dq"], wd["dkv"]]).to(DEV), d("dq.norm"), d("uq"), d("dkv.norm"), d("uk"), d("uv"), d("o"),
                           d("sink"), m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["q_rank"], m["kv_rank"], m["scale"],
                           m["rot"]["base"], m["rot"]["dims"], eps, conv)


@pytest.mark.parametrize("name, dtype, tol", DTYPES)
@pytest.mark.parametrize("m", [
    {"heads": 3, "dim": 5, "rot_dim": 6, "vdim": 4, "q_rank": 9, "kv_rank": 10, "scale": 0.31, "rot": {"base": 3000.0, "dims": 4}},
    {"heads": 10, "dim": 16, "rot_dim": 8, "vdim": 24, "q_rank": 48, "kv_rank": 40, "scale": 0.2, "rot": {"base": 1e4, "dims": 8}},
    {"heads": 1, "dim": 8, "rot_dim": 0, "vdim": 8, "q_rank": 8, "kv_rank": 72, "scale": 0.5, "rot": {"base": 10.0, "dims": 0}},
])
def test_latent_attention_part_over_scattered_pages(name, dtype, tol, m):
    """A prompt portion, a portion that starts in the middle of a page, and single tokens, against the plain function
    (which up-projects keys and values per head; the part works in the latent space)."""
    from jax_llm_examples_b200.parts import LayerCache, Runtime

    torch.manual_seed(m["heads"])
    D, eps, T = 48, 1e-5, 45
    rt = Runtime(dtype, torch.device(DEV))
    wd = {k: v.to(dtype) for k, v in _latent_weights(D, m).items()}
    mixer = _latent_part(wd, m, eps)
    need = mixer.kv_need()
    assert (need.planes, need.num_kv_heads, need.head_dim) == (1, 1, m["kv_rank"] + m["rot_dim"])
    pages = torch.zeros(40, 1, 1, 16, need.head_dim, device=DEV, dtype=dtype)
    table = torch.randperm(40)[:3].reshape(1, 3).to(torch.int32).to(DEV)
    hs = torch.randn(T, D).to(dtype)
    outs = []
    for lo, hi in ((0, 21), (21, 43), (43, 44), (44, 45)):
        ctx = _ctx(rt, [hi - lo], [lo], planners=mixer.step_planners())
        outs.append(H.as_rows_sum(mixer.forward(ctx, None, LayerCache(pages, table, True, None), h32=hs[lo:hi].float().to(DEV))))
        assert int(ctx.status) == 0
    ref = plain.latent_attention(hs.double(), {"m." + k: v.double() for k, v in wd.items()}, "m.", m, eps)
    _close(torch.cat(outs), ref, tol, name)


def test_latent_attention_kernel_sees_a_far_key_and_nothing_beyond_the_query():
    """Made so that a fault shows: among 700 keys of random latents, ONE far back is aligned with the query, and so
    is the key right AFTER the query (already in the cache: the step wrote the whole portion).  The output must be the
    far key's latent; the later key must count for nothing; with a huge sink everything shrinks towards zero.
    Query positions at a page's last and first row, and at the kernel's key-tile edges."""
    from jax_llm_examples_b200.kernels import api as K

    torch.manual_seed(0)
    H_, rank, dr, T, page = 2, 24, 4, 700, 16
    rows = torch.randn(T, rank + dr, device=DEV) * 0.1
    n_pages = -(-T // page)
    order = torch.randperm(n_pages, device=DEV)
    pages = torch.zeros(n_pages, 1, 1, page, rank + dr, device=DEV)
    pages[order, 0, 0] = torch.nn.functional.pad(rows, (0, 0, 0, n_pages * page - T)).reshape(n_pages, page, -1)
    table = order.to(torch.int32).reshape(1, -1).contiguous()
    status = torch.zeros(1, device=DEV, dtype=torch.int32)
    for far, qpos in ((3, 698), (0, 31), (15, 32), (16, 63), (31, 64), (64, 65), (200, 415), (7, 7)):
        direction = torch.randn(rank + dr, device=DEV)
        direction /= direction.norm()
        cache = pages.clone()
        flat = lambda p: (order[p // page], 0, 0, p % page)
        cache[flat(far)] = 30 * direction
        if qpos + 1 < T:
            cache[flat(qpos + 1)] = 60 * direction  # the future: twice as well aligned, and invisible
        q_lat = direction[:rank].repeat(H_, 1, 1).contiguous()  # [H, 1, rank]
        q_rot = direction[rank:].repeat(1, H_, 1).contiguous()  # [1, H, dr]
        pos = torch.tensor([qpos], device=DEV, dtype=torch.int32)
        req = torch.zeros(1, device=DEV, dtype=torch.int32)
        out = torch.empty(H_, 1, rank, device=DEV)
        K.attention_latent(q_lat, q_rot, cache, table, req, pos, None, out, 1.0, status)
        _close(out[0, 0], 30 * direction[:rank], 1e-4, f"far key {far} seen from {qpos}")
        # the plain softmax over the visible keys, with a sink per head
        sink = torch.tensor([2.0, 40.0], device=DEV)
        K.attention_latent(q_lat, q_rot, cache, table, req, pos, sink, out, 1.0, status)
        vis = torch.stack([cache[flat(p)] for p in range(qpos + 1)]).double()
        s = vis @ direction.double()
        for h in range(H_):
            big = max(float(s.max()), float(sink[h]))
            e = torch.exp(s - big)
            ref = (e[:, None] * vis[:, :rank]).sum(0) / (e.sum() + np.exp(float(sink[h]) - big))
            _close(out[h, 0], ref, 1e-4, f"sink of head {h} at {qpos}")
        assert float(out[1, 0].norm()) < 0.01 * float(out[0, 0].norm())  # exp(40 - 30) outweighs every key
    assert int(status) == 0


@pytest.mark.parametrize("T, L, start", [(5, 12, 7), (16, 64, 48), (3, 37, 0), (9, 203, 150)])
def test_prompt_softmax_stops_at_the_causal_edge_and_counts_the_sink_once(T, L, start):
    """The softmax between the two products of a prompt portion: query row i (position start + i) weighs the keys up to
    its own position.  The key right behind the edge gets by far the largest score; it must weigh nothing.  The sink
    adds exp(sink) to the denominator, unscaled, once."""
    from jax_llm_examples_b200.kernels import api as K

    torch.manual_seed(L)
    H_, scale = 3, 0.37
    s = torch.randn(H_, T, L, device=DEV)
    for i in range(T):
        if start + i + 1 < L:
            s[:, i, start + i + 1] = 80.0  # just outside
        s[:, i, start + i] += 3.0  # just inside: the query's own position
    sink = torch.tensor([-1.0, 0.5, 6.0], device=DEV)
    for out_dtype, tol in ((torch.float32, 2e-6), (torch.bfloat16, 5e-3)):
        p = torch.full((H_, T, L), 7.0, device=DEV, dtype=out_dtype)
        K.causal_sink_softmax(s, sink, scale, start, p)
        ref = torch.zeros(H_, T, L, dtype=torch.float64)
        for i in range(T):
            vis = min(L, start + i + 1)
            z = s[:, i, :vis].double().cpu() * scale
            e = torch.exp(z - z.max(dim=-1, keepdim=True).values)
            ref[:, i, :vis] = e / (e.sum(-1, keepdim=True) + torch.exp(sink.double().cpu()[:, None] - z.max(dim=-1, keepdim=True).values))
        assert float((p.double().cpu() - ref).abs().max()) < tol
        assert float(p[:, 0, min(L - 1, start + 1):].float().abs().max()) == 0.0 or start + 1 >= L
    p0 = torch.empty(H_, T, L, device=DEV)
    K.causal_sink_softmax(s, None, scale, start, p0)  # without a sink the visible weights sum to one
    assert torch.allclose(p0.sum(-1), torch.ones(H_, T, device=DEV), atol=1e-5)


@pytest.mark.parametrize("name, dtype, tol", DTYPES)
@pytest.mark.parametrize("D, F", [(40, 72), (38, 70)])  # four values per access, and one
def test_biased_mlp_and_reinjection_block(name, dtype, tol, D, F):
    from jax_llm_examples_b200.parts import DenseBiasedMLP, ReinjectionBlock, Rows, Runtime

    torch.manual_seed(1)
    rt = Runtime(dtype, torch.device(DEV))
    N = 6
    w = {"up": torch.randn(F, D) * 0.3, "up.b": torch.randn(F) * 0.5, "down": torch.randn(D, F) * 0.3, "down.b": torch.randn(D)}
    wd = {k: v.to(dtype) for k, v in w.items()}
    ff = DenseBiasedMLP(wd["up"].to(DEV), wd["up.b"].to(DEV), wd["down"].to(DEV), wd["down.b"].to(DEV), "relu2")
    ctx = _ctx(rt, [N], [0])
    h = torch.randn(N, D).to(dtype)
    got = H.as_rows_sum(ff.forward(ctx, h.to(DEV), None)) + ff.bias_out
    _close(got, plain.dense_ff(h.double(), {"m." + k: v.double() for k, v in wd.items()}, "m."), tol, name)
    # x <- W [x + pending; x0] + step, twice with one W (the product with x0 is made once)
    w_in, steps = (torch.randn(D, 2 * D) * 0.2).to(dtype), torch.randn(2, D).to(dtype)
    a, b = ReinjectionBlock(w_in.to(DEV), steps[0].to(DEV)), ReinjectionBlock(w_in.to(DEV), steps[1].to(DEV))
    b.share_weights(a)
    x, x0, pend = torch.randn(N, D), torch.randn(N, D), torch.randn(2, N, D)
    ctx.scratch["embedding_output"] = x0.to(DEV)
    xg = x.to(DEV).clone()
    assert a.forward(ctx, xg, Rows(pend.to(DEV), 2), None) is None
    ref = torch.cat([x + pend.sum(0), x0], dim=-1).double() @ w_in.double().T + steps[0].double()
    _close(xg, ref, tol, f"{name} first pass")
    assert b.forward(ctx, xg, None, None) is None
    ref = torch.cat([ref, x0.double()], dim=-1) @ w_in.double().T + steps[1].double()
    _close(xg, ref, 3 * tol, f"{name} second pass")


# --------------------------------------------------------------------------------------- whole models, by traces
@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("tebivik")
    return {n: TH.make_dir(root / n, n, seed=i + 1) for i, n in enumerate(TH.CONFIGS)}


def _engine(folder, dtype, max_tokens=512, page_size=16, max_slots=4, **kw):
    import jax_llm_examples_b200 as J

    return J.Engine(J.load_model(folder, dtype, DEV), max_tokens=max_tokens, page_size=page_size, max_slots=max_slots, **kw)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(TH.CONFIGS))
def test_every_kind_of_cut_against_the_plain_implementation(folders, name, dtype):
    """Whole prompts; most of a prompt and then 40 tokens one by one (decoding through replayed graphs in bfloat16);
    portions down to two tokens; up to four live requests mixed, in a pool too small for all of them, so that pages
    and slots are used again.  Every position's logits are compared, the first tokens of a sequence included."""
    vocab = TH.config(name)["vocab"]
    rng = random.Random(7)
    requests = H.random_requests(rng, vocab, [61, 1, 2, 33, 17, 90, 5])
    engine = _engine(folders[name], dtype, max_tokens=16 * 16)
    for steps in (H.trace_whole(requests), H.trace_tail_decode(requests, tail=40), H.trace_portions(requests, rng),
                  H.trace_mixed(requests, rng, max_live=4)):
        got, _ = H.run_trace(engine, steps, record_routing=False)
        assert len(got) == sum(len(t) for t in requests.values())
        TH.compare(folders[name], requests, got, dtype)
        assert engine.manager.free_slots() == 4 and all(engine.manager.free_pages(g) == engine.num_pages for g in range(len(engine.manager.groups)))
    if dtype == "bfloat16":
        assert engine.graph_replays > 0  # decode steps ran as replayed graphs, states and pages found by slot and table


@pytest.mark.parametrize("name", ["small", "wide"])
def test_logits_do_not_depend_on_the_cut_or_on_the_batch(folders, name):
    """float32: the same request whole, token by token, in portions, and beside three other requests gives the same
    logits to within rounding of a sum's order (far below the tolerance against the plain implementation)."""
    vocab = TH.config(name)["vocab"]
    rng = random.Random(11)
    requests = H.random_requests(rng, vocab, [70, 23, 41, 9])
    engine = _engine(folders[name], "float32")
    whole, _ = H.run_trace(engine, H.trace_whole(requests), record_routing=False)
    for steps in (H.trace_tail_decode(requests, tail=70), H.trace_portions(requests, rng), H.trace_mixed(requests, rng)):
        got, _ = H.run_trace(engine, steps, record_routing=False)
        worst = max(TH.row_err(got[k], whole[k]) for k in whole)
        assert worst < 2e-6, f"{name}: logits moved by {worst:.2e} with the cut"


def test_long_decoding_and_a_far_token(folders):
    """300 tokens one by one after a short prompt, in bfloat16 through replayed graphs and in float32: the recurrent
    state and the cache are carried over hundreds of steps and several pages."""
    name = "small"
    vocab = TH.config(name)["vocab"]
    toks = [random.Random(3).randrange(vocab) for _ in range(320)]
    for dtype in ("float32", "bfloat16"):
        engine = _engine(folders[name], dtype, max_tokens=320)
        got, _ = H.run_trace(engine, H.trace_tail_decode({"a": toks}, tail=300), record_routing=False)
        TH.compare(folders[name], {"a": toks}, got, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_long_prompt_whole_and_in_portions(folders, dtype):
    """560 tokens in one step (the recurrences scan it in segments; attention sees keys 500 tokens back), the same in two
    portions that are walked in order, and beside a short request: against the plain implementation at places near
    the start, around the segments' edges and at the end, and against each other."""
    import jax_llm_examples_b200 as J

    name = "small"
    vocab = TH.config(name)["vocab"]
    rng = random.Random(5)
    toks, other = [rng.randrange(vocab) for _ in range(560)], [rng.randrange(vocab) for _ in range(30)]
    want = [0, 1, 2, 254, 255, 256, 257, 300, 511, 512, 513, 558, 559]
    engine = _engine(folders[name], dtype, max_tokens=1024)
    a, b = engine.new_request(), engine.new_request()
    whole = engine.step([J.StepEntry(a, toks, want), J.StepEntry(b, other, [29])]).cpu().numpy().copy()
    engine.finish(a), engine.finish(b)
    a = engine.new_request()
    first = engine.step([J.StepEntry(a, toks[:300], [w for w in want if w < 300])]).cpu().numpy().copy()
    second = engine.step([J.StepEntry(a, toks[300:], [w - 300 for w in want if w >= 300])]).cpu().numpy().copy()
    engine.check_status()
    engine.finish(a)
    parts = np.concatenate([first, second])
    ref = TH.plain_logits(folders[name], toks)
    for k, w in enumerate(want):
        assert TH.row_err(whole[k], ref[w]) < TH.TOL[dtype], f"{dtype}: position {w} of the whole prompt"
        assert TH.row_err(parts[k], ref[w]) < TH.TOL[dtype], f"{dtype}: position {w} of the prompt in portions"
        assert TH.row_err(whole[k], parts[k]) < (1e-5 if dtype == "float32" else TH.TOL[dtype])
    assert TH.row_err(whole[len(want)], TH.plain_logits(folders[name], other)[29]) < TH.TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["small", "wide", "plainest"])
def test_greedy_generation_through_the_scheduler(folders, name, dtype):
    """The framework's own entry point: prompts of unequal length under a small token budget per step, so that
    prompt portions run beside decoded tokens."""
    import jax_llm_examples_b200 as J

    vocab = TH.config(name)["vocab"]
    prompts = [[(7 * i + 3 * j) % vocab for i in range(n)] for j, n in enumerate((29, 3, 12))]
    model = J.load_model(folders[name], dtype, DEV)
    got = J.generate(model, prompts, J.SamplingParams(max_new_tokens=10), page_size=16, max_tokens_per_step=16)
    for p, g in zip(prompts, got):
        assert len(g) == 10
        TH.greedy_checked(folders[name], p, g, dtype)


def test_command_line_generates_with_a_preset_and_with_a_folder(folders, capsys):
    from jax_llm_examples_b200.main import main

    assert main(["--preset", "tebivik_tiny", "--random-prompts", "2", "--prompt-len", "9", "--max-new-tokens", "4"]) == 0
    out = capsys.readouterr().out
    assert out.count("-" * 80) == 2
    assert main(["--model", str(folders["small"]), "--dtype", "float32", "--prompt-ids", "1,2,3,4,5", "--max-new-tokens", "5",
                 "--page-size", "16"]) == 0
    ids = [int(t) for t in capsys.readouterr().out.splitlines()[1].split()]
    TH.greedy_checked(folders["small"], [1, 2, 3, 4, 5], ids, "float32")


def test_trace_replay_program_on_a_tebivik_folder(folders, tmp_path):
    """bin/trace_run picks the model class by config.json and writes the wanted logits."""
    import json
    import os

    name, dtype = "wide", "float32"
    vocab = TH.config(name)["vocab"]
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
    ref = TH.plain_logits(folders[name], toks)
    rows = {0: [0, 12], 1: [1], 2: [20]}
    assert not (out / "1.f32.tmp").exists()
    for step, places in rows.items():
        got = np.fromfile(out / f"{step}.f32", dtype="<f4").reshape(len(places), vocab)
        for g, pl in zip(got, places):
            assert TH.row_err(g, ref[pl]) < TH.TOL[dtype]
