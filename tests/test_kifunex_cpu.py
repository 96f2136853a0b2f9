"""Kifunex without a GPU: its configuration and errors, the model as data (tensor names against the plain
implementation's table, layers that run with another layer's tensors, cache entries and page groups), and the rotary
frequencies with wavelength scaling."""
import copy

import pytest
import torch

import plain_kifunex as pk
from nano_vllm_cpp_b200.config import ConfigError, get_architecture
from nano_vllm_cpp_b200.parts import Model
from nano_vllm_cpp_b200.parts.rotary import RotaryNeoX

SCALING = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}
CFG = pk.model_config(
    [pk.attention_layer(dim=32, heads=4, kv_heads=2, window=24, rot_dims=16, scaling=SCALING, scale=0.2, mlp=pk.moe()),
     pk.attention_layer(dim=48, heads=3, kv_heads=3, window=17, rot_dims=48, mlp=None),
     pk.attention_layer(dim=32, heads=4, kv_heads=2, window=24, rot_dims=16, scaling=SCALING, scale=0.2, mlp=pk.moe(),
                        weights_of=0),
     pk.attention_layer(dim=48, heads=3, kv_heads=3, window=17, rot_dims=48, mlp=None, weights_of=1)],
    width=96, vocab=210, streams=3)


def build(cfg):
    arch = get_architecture("Kifunex")
    typed = arch.config_from_dict(cfg)
    return typed, Model(arch.build_model(typed))


def test_tensor_names_and_shapes_are_the_plain_table():
    _, model = build(CFG)
    specs = model.tensor_specs()
    table = pk.tensor_table(CFG)
    assert set(specs) == set(table)
    for name, (shape, _) in table.items():
        assert tuple(specs[name].shape) == tuple(shape), name


def test_layers_that_run_with_another_layers_tensors():
    typed, model = build(CFG)
    assert len(model.layers) == 2 and [c.layer for c in model.calls] == [0, 1, 0, 1]
    assert all(c.cache_of is None for c in model.calls)              # every call keeps its own keys and values
    specs = model.cache_specs()
    assert [s.window for s in specs] == [24, 17, 24, 17] and [s.head_dim for s in specs] == [32, 48, 32, 48]
    assert typed.weight_owner(3) == 1
    chain = copy.deepcopy(CFG)
    chain["layers"][3]["weights_of"] = 2                             # through layer 2 to layer 0
    chain["layers"][3]["mixer"] = chain["layers"][0]["mixer"]
    chain["layers"][3]["mlp"] = chain["layers"][0]["mlp"]
    typed, model = build(chain)
    assert [c.layer for c in model.calls] == [0, 1, 0, 0]


def test_configuration_errors_name_the_key():
    def broken(path, value, drop=False):
        d = copy.deepcopy(CFG)
        node = d
        for k in path[:-1]:
            node = node[k]
        if drop:
            del node[path[-1]]
        else:
            node[path[-1]] = value
        return d
    arch = get_architecture("Kifunex")
    for path, value, drop, word in [
            (("layers", 0, "mixer", "heads"), 5, False, "kv_heads"),
            (("layers", 0, "mixer", "vdim"), 16, False, "vdim"),
            (("layers", 0, "mixer", "scale"), None, True, "scale"),
            (("layers", 0, "mixer", "rot", "dims"), 34, False, "rot.dims"),
            (("layers", 0, "mixer", "rot", "scaling", "low"), 4.0, False, "scaling"),
            (("layers", 0, "mlp", "router", "top"), 7, False, "router.top"),
            (("layers", 0, "mlp", "kind"), "dense", False, "mlp.kind"),
            (("layers", 1, "type"), "conv", False, "type"),
            (("layers", 2, "weights_of"), 2, False, "weights_of"),
            (("layers", 2, "weights_of"), 9, False, "weights_of"),
            (("width",), None, True, "width"),
            (("streams",), 0, False, "streams")]:
        with pytest.raises(ConfigError) as e:
            arch.config_from_dict(broken(path, value, drop))
        assert word in str(e.value), (path, str(e.value))
    loop = copy.deepcopy(CFG)
    loop["layers"][0]["weights_of"] = 2
    with pytest.raises(ConfigError):
        arch.config_from_dict(loop)


def test_parts_a_file_leaves_out_are_switched_off():
    d = copy.deepcopy(CFG)
    del d["logit_softcap"], d["logit_scale"], d["streams"]
    d["layers"][1]["mixer"]["mask"] = None
    d["layers"][3]["mixer"]["mask"] = None
    d["layers"][1]["mixer"]["rot"] = None
    d["layers"][3]["mixer"]["rot"] = None
    d["layers"][0]["mlp"]["shared"] = None
    d["layers"][2]["mlp"]["shared"] = None
    typed, model = build(d)
    assert typed.streams == 1 and typed.logit_softcap == 0.0 and typed.logit_scale == 1.0
    assert model.cache_specs()[1].window == 0 and model.layers[1].mixer.position.rotary_dim == 0
    assert "l0.mlp.shared.up" not in model.tensor_specs()


@pytest.mark.parametrize("rot", [{"dims": 16, "base": 10000.0, "scaling": SCALING},
                                 {"dims": 80, "base": 120000.0, "scaling": {"factor": 6.0, "low": 1.5, "high": 5.0, "original": 300}},
                                 {"dims": 32, "base": 500.0, "scaling": {"factor": 2.0, "low": 2.0, "high": 3.0, "original": 40}},
                                 {"dims": 48, "base": 500.0, "scaling": None}])
def test_rotary_frequencies(rot):
    part = RotaryNeoX(rot["dims"], rot["base"], rot["scaling"])
    got = torch.tensor(part.frequencies(), dtype=torch.float64)
    want = pk.rotary_frequencies(rot)
    assert torch.allclose(got, want, rtol=1e-12, atol=0)
    if rot["scaling"]:
        plain = pk.rotary_frequencies(dict(rot, scaling=None))
        ratio = want / plain
        sc = rot["scaling"]
        # the three regimes are all there: untouched, divided by the factor, and in between
        assert float(ratio.max()) == 1.0 and abs(float(ratio.min()) - 1.0 / sc["factor"]) < 1e-12
        assert bool(((ratio < 1.0) & (ratio > 1.0 / sc["factor"] + 1e-9)).any())
