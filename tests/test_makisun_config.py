"""Makisun without a GPU: the configuration reader, the tensor list, random model folders, and the plain
implementation against other ways of writing the same mathematics."""

import copy
import json

import pytest
import torch

from tests import makisun_helpers as MH
from tests.plain import makisun_plain as plain


def test_config_is_read_from_the_files_own_keys():
    from jax_llm_examples_b200.config.makisun import MakisunConfig, ParallelSpec, WKVSpec
    from jax_llm_examples_b200.config.registry import resolve

    cj = MH.config("small")
    arch = resolve(cj)
    assert arch.name == "Makisun"
    cfg = arch.parse_config(cj)
    assert isinstance(cfg, MakisunConfig) and (cfg.vocab_size, cfg.hidden_size, cfg.norm_eps, cfg.embedding_scale) == (61, 36, 1e-5, 2.5)
    assert [type(L.mixer) for L in cfg.layers] == [WKVSpec, ParallelSpec, WKVSpec, ParallelSpec]
    a = cfg.layers[1].mixer
    assert (a.left.heads, a.left.kv_heads, a.left.dim, a.left.vdim, a.left.window, a.left.rot_dims, a.left.scale) == (6, 2, 10, 6, 7, 4, 0.4)
    assert (a.right.heads, a.right.dim, a.right.vdim, a.right.tau, a.left_scale, a.right_scale) == (2, 7, 9, 3.5, 1.3, 0.6)
    assert cfg.layers[2].mlp is None and cfg.layers[1].mlp.kind == "dense" and cfg.layers[1].mlp.ff == 30
    m = cfg.layers[0].mlp
    assert (m.kind, m.experts, m.top, m.ff, m.shared_ff) == ("moe", 5, 2, 12, 9) and cfg.layers[3].mlp.shared_ff is None


@pytest.mark.parametrize("path, value, word", [
    (("layers", 0, "type"), "mamba", "no mixer"),
    (("layers", 1, "mixer", "left", "kv_heads"), 4, "no multiple"),
    (("layers", 1, "mixer", "left", "rot", "dims"), 5, "even"),
    (("layers", 1, "mixer", "left", "rot", "dims"), 12, "at most"),
    (("layers", 0, "mlp", "router", "top"), 6, "top"),
    (("layers", 1, "mlp", "kind"), "glu", "dense"),
    (("norm", "eps"), 0.0, "eps"),
    (("layers", 1, "mixer", "right", "tau"), 0.0, "tau"),
])
def test_config_errors_name_the_key(path, value, word):
    from jax_llm_examples_b200.config.base import ConfigError
    from jax_llm_examples_b200.config.makisun import MakisunConfig

    cj = MH.config("small")
    d = cj
    for k in path[:-1]:
        d = d[k]
    d[path[-1]] = value
    with pytest.raises(ConfigError, match=word):
        MakisunConfig.from_dict(cj)
    cj = MH.config("small")
    del cj["layers"][1]["mixer"]["left"]["mask"]
    with pytest.raises(ConfigError, match="mask"):
        MakisunConfig.from_dict(cj)


def test_tensor_list_random_folder_and_ranks_that_only_the_file_gives(tmp_path):
    """A folder written from a configuration holds exactly the architecture's tensors; a configuration that does not
    name the decays' ranks takes them from the stored tensors, and cannot be drawn at random."""
    from jax_llm_examples_b200.config.registry import resolve
    from jax_llm_examples_b200.weights.loader import WeightError, load_tensors

    folder = MH.make_dir(tmp_path / "m", "small", seed=3)
    cj = json.loads((folder / "config.json").read_text())
    arch = resolve(cj)
    specs = arch.tensor_specs(arch.parse_config(cj))
    P = plain.read_safetensors(folder / "model.safetensors")
    assert set(P) == set(specs)
    assert P["l0.mix.w1"].shape == (3, 36) and P["l1.mix.right.a2"].shape == (14, 5) and P["l0.mix.u"].shape == (3, 5)
    assert P["l0.mlp.e4.down"].shape == (36, 12) and "l3.mlp.shared.up" not in P and "l2.norm2" not in P
    # without the ranks in the configuration any rank fits, and the tensors still load
    bare = copy.deepcopy(cj)
    for L in bare["layers"]:
        (L["mixer"] if L["type"] == "wkv" else L["mixer"]["right"]).pop("decay_rank")
    specs2 = arch.tensor_specs(arch.parse_config(bare))
    assert specs2["l0.mix.w1"].shape == (-1, 36)
    got = load_tensors(folder, specs2, None, torch.float32)
    assert got["l0.mix.w2"].shape == (15, 3)
    from jax_llm_examples_b200 import write_random_model
    with pytest.raises(ValueError, match="only a stored tensor"):
        write_random_model(tmp_path / "n", bare, 0)
    # a wrong size is still reported
    wrong = copy.deepcopy(cj)
    wrong["layers"][0]["mixer"]["heads"] = 4
    with pytest.raises(WeightError, match="wrong shapes"):
        load_tensors(folder, arch.tensor_specs(arch.parse_config(wrong)), None, torch.float32)


def test_plain_recurrences_equal_their_sums_over_the_past():
    """The two recurrences of the plain implementation against the same outputs written as explicit sums over all
    earlier tokens (products of decays), and the windowed attention against a dense masked softmax."""
    torch.manual_seed(0)
    T, D, eps = 9, 12, 1e-5
    h = torch.randn(T, D, dtype=torch.float64)
    m = {"heads": 2, "dim": 3, "vdim": 4, "tau": 2.5}
    P = {"q": torch.randn(6, D), "k": torch.randn(6, D), "v": torch.randn(8, D), "g": torch.randn(8, D), "a1": torch.randn(2, D),
         "a2": torch.randn(6, 2), "a2.b": torch.randn(6), "norm": torch.rand(4) + 0.5, "o": torch.randn(D, 8)}
    P = {"m." + k: v.double() for k, v in P.items()}
    got = plain.gated_linear_attention(h, P, "m.", m, eps)
    q = (h @ P["m.q"].T).view(T, 2, 3) * 3 ** -0.5
    k, v = (h @ P["m.k"].T).view(T, 2, 3), (h @ P["m.v"].T).view(T, 2, 4)
    alpha = torch.sigmoid((h @ P["m.a1"].T) @ P["m.a2"].T + P["m.a2.b"]).pow(1 / 2.5).view(T, 2, 3)
    o = torch.zeros(T, 2, 4, dtype=torch.float64)
    for t in range(T):
        for s in range(t + 1):
            decay = alpha[s + 1:t + 1].prod(0)  # the decays applied after token s was written
            o[t] += torch.einsum("hk,hv->hv", q[t] * decay * k[s], v[s])
    o = o / (o.pow(2).mean(-1, keepdim=True) + eps).sqrt() * P["m.norm"]
    g = h @ P["m.g"].T
    ref = (o.reshape(T, 8) * g * torch.sigmoid(g)) @ P["m.o"].T
    assert torch.allclose(got, ref, atol=1e-10)

    w = {"heads": 2, "dim": 3}
    Q = {"mu." + s: torch.rand(D) for s in "rkvgw"}
    Q.update({s: torch.randn(6, D) for s in "rkvg"})
    Q.update({"w1": torch.randn(2, D), "w2": torch.randn(6, 2), "w0": torch.randn(6), "u": torch.randn(2, 3), "norm": torch.rand(6) + 0.5,
              "o": torch.randn(D, 6)})
    Q = {"m." + k: v.double() for k, v in Q.items()}
    got = plain.wkv_mixer(h, Q, "m.", w, eps)
    prev = torch.cat([torch.zeros(1, D, dtype=torch.float64), h[:-1]])
    mix = lambda s: h + (prev - h) * Q["m.mu." + s]
    r, k, v = ((mix(s) @ Q["m." + s].T).view(T, 2, 3) for s in "rkv")
    dec = torch.exp(-torch.exp(torch.tanh(mix("w") @ Q["m.w1"].T) @ Q["m.w2"].T + Q["m.w0"])).view(T, 2, 3)
    o = torch.zeros(T, 2, 3, dtype=torch.float64)
    for t in range(T):
        o[t] += torch.einsum("hk,hv->hv", r[t] * Q["m.u"] * k[t], v[t])  # the token itself: through the bonus, undecayed
        for s in range(t):
            o[t] += torch.einsum("hk,hv->hv", r[t] * dec[s + 1:t].prod(0) * k[s], v[s])
    o = (o / (o.pow(2).mean(-1, keepdim=True) + eps).sqrt()).reshape(T, 6) * Q["m.norm"]
    gg = mix("g") @ Q["m.g"].T
    assert torch.allclose(got, (o * gg * torch.sigmoid(gg)) @ Q["m.o"].T, atol=1e-10)


def test_plain_window_and_rotation():
    """A query sees itself and window - 1 tokens before it; rotated scores depend on the distance only; entries beyond
    the rotated ones pass unchanged."""
    torch.manual_seed(1)
    x = torch.randn(7, 2, 10, dtype=torch.float64)
    pos = torch.arange(7)
    y = plain.rotate_half(x, pos, 100.0, 6)
    assert torch.equal(y[..., 6:], x[..., 6:]) and torch.allclose(y[0], x[0])
    same = x[:1].expand(7, 2, 10).contiguous()
    r = plain.rotate_half(same, pos, 100.0, 6)
    s = torch.einsum("ihd,jhd->hij", r, r)
    assert torch.allclose(s[:, 2, 0], s[:, 5, 3]) and torch.allclose(s[:, 6, 5], s[:, 1, 0])
    # window: with values that name their position, position 5 of a window of 3 mixes positions 3, 4, 5 only
    D = 8
    m = {"heads": 1, "kv_heads": 1, "dim": 4, "vdim": 8, "mask": {"size": 3}, "rot": {"base": 10.0, "dims": 0}, "scale": 0.0}
    P = {"m.q": torch.zeros(4, D), "m.k": torch.zeros(4, D), "m.v": torch.eye(8), "m.g": torch.zeros(1, D), "m.q.norm": torch.ones(4),
         "m.k.norm": torch.ones(4), "m.o": torch.eye(8)}
    P = {k: v.double() for k, v in P.items()}
    h = torch.eye(8, dtype=torch.float64)
    out = plain.window_attention(h, P, "m.", m, 1e-6)  # scale 0: uniform weights; gate sigmoid(0) = 1/2
    assert torch.allclose(out[5], 0.5 * torch.tensor([0, 0, 0, 1, 1, 1, 0, 0], dtype=torch.float64) / 3)
    assert torch.allclose(out[1], 0.5 * torch.tensor([1, 1, 0, 0, 0, 0, 0, 0], dtype=torch.float64) / 2)


def test_plain_router_takes_the_softmax_over_the_chosen_only():
    torch.manual_seed(2)
    D, E = 6, 5
    P = {"m.router": torch.randn(E, D), "m.router.b": torch.tensor([0.0, 0.0, 5.0, 0.0, -5.0])}
    for e in range(E):
        P[f"m.e{e}.up"], P[f"m.e{e}.down"] = torch.randn(4, D), torch.randn(D, 4)
    P = {k: v.double() for k, v in P.items()}
    h = torch.randn(3, D, dtype=torch.float64) * 0.1
    out, z, chosen = plain.mixture_of_experts(h, P, "m.", {"router": {"experts": E, "top": 2}})
    assert (chosen[:, 0] == 2).all() and (chosen != 4).all()  # the bias decides
    for t in range(3):
        zz = z[t, chosen[t]]
        wgt = torch.exp(zz) / torch.exp(zz).sum()
        ref = sum(wgt[j] * plain.expert(h[t:t + 1], P, f"m.e{int(chosen[t, j])}.")[0] for j in range(2))
        assert torch.allclose(out[t], ref)
