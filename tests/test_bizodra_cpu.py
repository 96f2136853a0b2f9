"""Host side of the Bizodra decoder: reading its configuration, the tensors its model asks for, what its mixers
keep per request, and the rotation's frequencies, against the plain implementation's own tables."""
import copy

import pytest
import torch

import plain_bizodra as pb
from test_bizodra_gpu import CONFIGS, ROT_A, ROT_B


def build(cfg):
    from nano_vllm_cpp_b200.config.registry import get_architecture, architecture_name
    from nano_vllm_cpp_b200.parts import Model
    arch = get_architecture(architecture_name(cfg))
    return arch, arch.config_from_dict(cfg), Model(arch.build_model(arch.config_from_dict(cfg)))


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_model_asks_for_the_tensors_of_the_format(name):
    _, typed, model = build(CONFIGS[name])
    want = {n: tuple(s) for n, (s, _) in pb.tensor_shapes(CONFIGS[name]).items()}
    got = {n: tuple(s.shape) for n, s in model.tensor_specs().items()}
    assert got == want
    assert typed.num_hidden_layers == len(CONFIGS[name]["layers"]) and typed.vocab_size == CONFIGS[name]["vocab"]


def test_architecture_is_found_by_either_key():
    from nano_vllm_cpp_b200.config.registry import architecture_name, known_architectures
    from nano_vllm_cpp_b200.config import ConfigError
    assert architecture_name({"architecture": "Bizodra"}) == "Bizodra"
    assert architecture_name({"architectures": ["Qwen2MoeForCausalLM"], "architecture": "x"}) == "Qwen2MoeForCausalLM"
    assert {"Bizodra", "Qwen2MoeForCausalLM"} <= set(known_architectures())
    with pytest.raises(ConfigError):
        architecture_name({})


@pytest.mark.parametrize("path,value,word", [
    (("layers", 0, "type"), "lstm", "type"), (("layers", 1, "mixer", "heads"), 0, "heads"),
    (("layers", 0, "mixer", "left", "kv_heads"), 3, "kv_heads"), (("layers", 0, "mixer", "right", "conv"), 0, "conv"),
    (("layers", 0, "mlp", "kind"), "moe", "kind"), (("norm", "eps"), -1.0, "eps"), (("width",), "wide", "width"),
    (("layers", 0, "mixer", "left", "rot", "dims"), 34, "dims"), (("token_side", "dim"), 0, "dim"),
    (("layers", 0, "mixer", "left", "rot", "scaling", "factor"), None, "factor"),
])
def test_config_errors_name_the_key(path, value, word):
    from nano_vllm_cpp_b200.config import ConfigError, BizodraConfig
    cfg = copy.deepcopy(CONFIGS["P"])
    d = cfg
    for k in path[:-1]:
        d = d[k]
    d[path[-1]] = value
    with pytest.raises(ConfigError, match=word):
        BizodraConfig.from_dict(cfg)


def test_layer_types_with_numeric_suffixes_name_the_same_kinds():
    from nano_vllm_cpp_b200.config import BizodraConfig, ConfigError
    from nano_vllm_cpp_b200.config.bizodra_config import MatrixLstmConfig, ParallelConfig
    cfg = copy.deepcopy(CONFIGS["Q"])
    cfg["layers"][0]["type"], cfg["layers"][1]["type"], cfg["layers"][2]["type"] = "mlstm_3", "parallel", "parallel_2"
    typed = BizodraConfig.from_dict(cfg)
    assert [type(L.mixer) for L in typed.layers] == [MatrixLstmConfig, ParallelConfig, ParallelConfig]
    for bad in ("mlstm_", "_2", "mlstm_x", "parallel2"):
        cfg["layers"][0]["type"] = bad
        with pytest.raises(ConfigError, match="type"):
            BizodraConfig.from_dict(cfg)
    del cfg["layers"][1]["mixer"]["left"]["rot"]            # without 'rot' nothing is turned
    cfg["layers"][0]["type"] = "mlstm"
    assert BizodraConfig.from_dict(cfg).layers[1].mixer.left.rot.dims == 0


def test_what_the_mixers_keep_per_request():
    from nano_vllm_cpp_b200.parts import KVCacheSpec, StateCacheSpec, CompositeCacheSpec
    _, _, model = build(CONFIGS["P"])
    par, lstm, _ = model.cache_specs()
    left, right = par.parts
    assert left == KVCacheSpec(1, 32, 0, 48)
    assert right == CompositeCacheSpec((StateCacheSpec((4, 24, 40)), StateCacheSpec((2, 2 * 2 * 24 + 4 * 40))))
    assert lstm == CompositeCacheSpec((StateCacheSpec((3, 16, 24)), StateCacheSpec((3, 16)), StateCacheSpec((3,))))
    # one tap: no inputs are kept
    _, _, one = build({"architecture": "Bizodra", "vocab": 9, "width": 16, "norm": {"eps": 1e-6}, "layers": [
        {"type": "parallel", "mlp": None, "mixer": {"left": dict(CONFIGS["Q"]["layers"][1]["mixer"]["left"]),
                                                    "right": {"heads": 2, "kv_heads": 1, "dim": 8, "vdim": 8, "conv": 1}}}]})
    assert one.cache_specs()[0].parts[1] == CompositeCacheSpec((StateCacheSpec((2, 8, 8)),))


def test_device_cache_places_every_state_in_one_buffer_per_slot():
    from nano_vllm_cpp_b200.cache import DeviceCache
    _, _, model = build(CONFIGS["P"])
    cache = DeviceCache(model.cache_specs(), 16, 3, "cpu", torch.float32)
    cache.allocate(5, 4)
    assert cache.has_state and cache.windows == [0]
    buf = cache.state_buffers[torch.float32]
    views = [cache.views[0].parts[1].parts[0], cache.views[0].parts[1].parts[1]] + cache.views[1].parts + cache.views[2].parts
    assert [tuple(v.state.shape) for v in views] == [(3, 4, 24, 40), (3, 2, 256), (3, 3, 16, 24), (3, 3, 16), (3, 3),
                                                     (3, 1, 40, 64), (3, 1, 40), (3, 1)]
    spans = sorted((v.state[0].data_ptr(), v.state[0].numel() * 4) for v in views)
    assert spans[0][0] == buf.data_ptr() and all(a % 16 == 0 for a, _ in spans)
    assert all(a + n <= b for (a, n), (b, _) in zip(spans, spans[1:]))            # no two arrays overlap
    assert spans[-1][0] + spans[-1][1] <= buf.data_ptr() + buf.shape[1] * 4
    views[3].state[1].fill_(7.0)                                                   # a view writes into the buffer
    assert float(buf[1].sum()) == 7.0 * 48 and float(buf[0].sum()) == 0.0
    k, v = cache.views[0].parts[0].k, cache.views[0].parts[0].v
    assert tuple(k.shape) == (5, 1, 16, 32) and tuple(v.shape) == (5, 1, 16, 48)
    assert cache.bytes_per_page() == [16 * (32 + 48) * 4]


@pytest.mark.parametrize("rot", [ROT_A, ROT_B, {"dims": 0, "base": 10.0}])
def test_rotation_frequencies(rot):
    from nano_vllm_cpp_b200.parts.rotary import RotaryInterleaved
    part = RotaryInterleaved(rot["dims"], rot["base"], rot.get("scaling"))
    f, amp = pb.rotary_frequencies(rot)
    assert part.pairing == "interleaved" and abs(part.amplitude - amp) < 1e-15
    assert torch.allclose(torch.tensor(part.frequencies(), dtype=torch.float64), f, rtol=1e-14, atol=0)
    if rot.get("scaling"):                  # the scaling changes some pairs and not others
        plain = torch.tensor(RotaryInterleaved(rot["dims"], rot["base"]).frequencies(), dtype=torch.float64)
        assert bool((f == plain).any()) and bool((f < plain).any())
