"""Tebivik without a GPU: the configuration reader, the tensor list, the order of execution, the registry, a model
folder written from a seed, and the plain implementation's own consistency."""

import copy

import pytest
import torch

from tests import tebivik_helpers as TH
from tests.plain import tebivik_plain as plain


def test_config_is_read_from_its_own_keys():
    from jax_llm_examples_b200.config import ConfigError, TebivikConfig, resolve

    cj = TH.config("small")
    cfg = resolve(cj).parse_config(cj)
    assert isinstance(cfg, TebivikConfig)
    assert (cfg.vocab, cfg.width, cfg.norm_groups, cfg.canon_taps) == (cj["vocab"], cj["width"], cj["norm"]["groups"], cj["canon"]["taps"])
    assert [L.type for L in cfg.layers] == [L["type"] for L in cj["layers"]]
    assert cfg.layers[0].mlp is None and cfg.layers[1].mlp.ff == cj["layers"][1]["mlp"]["ff"]
    att = next(L.mixer for L in cfg.layers if L.type == "latent_attention")
    assert att.rot_base == 3000.0 and att.rot_dims == 4 and att.rot_dim == 6
    for path, bad in ((("width",), None), (("norm", "groups"), 5), (("layers", 0, "type"), "mamba"), (("loop", "stop"), 9),
                      (("layers", 1, "mlp", "kind"), "moe"), (("canon", "taps"), 0)):
        broken = copy.deepcopy(cj)
        d = broken
        for k in path[:-1]:
            d = d[k]
        if bad is None:
            del d[path[-1]]
        else:
            d[path[-1]] = bad
        with pytest.raises(ConfigError):
            resolve(broken).parse_config(broken)


def test_the_order_of_execution_repeats_the_looped_stretch():
    from jax_llm_examples_b200.config import TebivikConfig

    cj = TH.config("small")
    cfg = TebivikConfig.from_dict(cj)  # 4 layers, loop over [1, 3) three times
    assert cfg.layer_order() == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (1, 2), (2, None), (3, None)]
    assert plain.layer_order(cj) == cfg.layer_order()
    cj["loop"] = None
    assert TebivikConfig.from_dict(cj).layer_order() == [(i, None) for i in range(4)]


def test_registry_takes_a_single_architecture_name_or_a_list():
    from jax_llm_examples_b200.config import ConfigError, resolve

    cj = TH.config("small")
    assert resolve(cj).name == "Tebivik"
    listed = {k: v for k, v in cj.items() if k != "architecture"}
    listed["architectures"] = ["Tebivik"]
    assert resolve(listed).name == "Tebivik"
    with pytest.raises(ConfigError):
        resolve({k: v for k, v in cj.items() if k != "architecture"})


def test_a_folder_written_from_a_seed_holds_exactly_the_tensors_of_the_list(tmp_path):
    import jax_llm_examples_b200 as J
    from jax_llm_examples_b200.config import resolve
    from jax_llm_examples_b200.weights.loader import WeightError, load_tensors

    cj = TH.config("small")
    folder = J.write_random_model(tmp_path / "m", cj, seed=3, norm_noise=0.1)
    arch = resolve(cj)
    specs = arch.tensor_specs(arch.parse_config(cj))
    tensors = load_tensors(folder, specs, None, torch.bfloat16, "cpu")
    assert set(tensors) == set(specs)
    w = plain.load_weights(folder, torch.float32)  # the plain implementation's own reader sees the same file
    assert set(w) == set(specs) and all(tuple(w[n].shape) == tuple(specs[n].shape) for n in specs)
    assert 0 < float(w["l0.mix.lower"].min()) and float(w["l0.mix.lower"].max()) < 1
    assert "l0.mlp.up" not in specs and "l1.mlp.up.b" in specs and "loop.step" in specs
    no_loop = dict(cj, loop=None)
    with pytest.raises(WeightError) as e:
        load_tensors(folder, resolve(no_loop).tensor_specs(resolve(no_loop).parse_config(no_loop)), None, torch.bfloat16, "cpu")
    assert sorted(e.value.unexpected) == ["loop.in", "loop.step"]


def test_plain_implementation_is_causal_and_its_parts_reduce_as_they_should(tmp_path):
    import jax_llm_examples_b200 as J

    cj = TH.config("small")
    folder = J.write_random_model(tmp_path / "m", cj, seed=5, norm_noise=0.1)
    w = plain.load_weights(folder, torch.float64)
    toks = [(5 * i + 1) % cj["vocab"] for i in range(19)]
    with torch.no_grad():
        full = plain.forward(cj, w, toks)
        part = plain.forward(cj, w, toks[:11])
    assert torch.allclose(full[:11], part, atol=1e-10)  # later tokens change nothing earlier
    x = torch.randn(5, 24, dtype=torch.float64)
    g = torch.rand(24, dtype=torch.float64) + 0.5
    assert torch.allclose(plain.group_rms_norm(x, g, 1e-6, 1), plain.rms_norm(x, g, 1e-6))
    by_hand = torch.cat([plain.rms_norm(x[:, :12], g[:12], 1e-6), plain.rms_norm(x[:, 12:], g[12:], 1e-6)], dim=-1)
    assert torch.allclose(plain.group_rms_norm(x, g, 1e-6, 2), by_hand)
    # a convolution of one tap scales the token itself; of three taps reaches two tokens back and no further
    assert torch.allclose(plain.causal_conv(x, g[:, None]), x * g)
    w3 = torch.randn(24, 3, dtype=torch.float64)
    y = plain.causal_conv(x, w3)
    assert torch.allclose(y[0], w3[:, 2] * x[0]) and torch.allclose(y[3], w3[:, 0] * x[1] + w3[:, 1] * x[2] + w3[:, 2] * x[3])
    # rotating by position 0 changes nothing; a rotation keeps each pair's length
    v = torch.randn(4, 3, 8, dtype=torch.float64)
    r = plain.rotate_pairs(v, torch.tensor([0, 1, 2, 3]), 100.0, 6)
    assert torch.allclose(r[0], v[0]) and torch.allclose(r[..., 6:], v[..., 6:])
    assert torch.allclose(r[..., 0:2].norm(dim=-1), v[..., 0:2].norm(dim=-1))
