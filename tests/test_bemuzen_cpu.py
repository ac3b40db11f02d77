"""What can be checked of the Bemuzen design without a GPU: the configuration reads and writes
back, the description names the checkpoint's tensors, the cache gives every part what it asked for,
and the plain implementation gives the same rows however a prompt is cut."""

from __future__ import annotations

import json
import math

import pytest
import torch

import bemuzen_configs
import plain_bemuzen


def typed(raw):
    import vllm_from_scratch_b200 as engine
    return engine.load_model_config(raw)


@pytest.mark.parametrize("name", list(bemuzen_configs.CONFIGS))
def test_configuration_round_trip_and_tensor_names(name):
    raw, _ = bemuzen_configs.CONFIGS[name]
    entry, config = typed(raw)
    assert entry.name == "Bemuzen"
    again = entry.config_class.from_dict(json.loads(json.dumps(config.to_dict())))
    assert again == config
    from vllm_from_scratch_b200.parts.model import DecoderModel
    model = DecoderModel(entry.build_spec(config), torch.float32, "cpu")
    weights = entry.random_weights(config, 1)
    expected = model.expected_weights()
    assert set(expected) == set(weights)
    for key, info in expected.items():
        assert tuple(weights[key].shape) == tuple(info.shape), key
    # layers without a feed-forward bring two norms, the others four
    for index, layer in enumerate(raw["layers"]):
        assert (f"l{index}.norm2" in expected) == (layer["mlp"] is not None)


def test_configuration_refuses_what_the_design_has_not():
    from vllm_from_scratch_b200.config import ConfigError
    raw = json.loads(json.dumps(bemuzen_configs.BZ_A))
    raw["layers"][0]["type"] = "convolution"
    with pytest.raises(ConfigError):
        typed(raw)
    raw = json.loads(json.dumps(bemuzen_configs.BZ_A))
    raw["layers"][0]["mixer"]["right"]["decay"] = [0.5]
    with pytest.raises(ConfigError):
        typed(raw)
    raw = json.loads(json.dumps(bemuzen_configs.BZ_A))
    raw["layers"][1]["mlp"] = {"kind": "experts", "ff": 8}
    with pytest.raises(ConfigError):
        typed(raw)
    raw = json.loads(json.dumps(bemuzen_configs.BZ_A))
    del raw["norm"]
    with pytest.raises(ConfigError):
        typed(raw)


def test_cache_gives_pages_and_named_states_together():
    from vllm_from_scratch_b200.cache import CacheManager, CacheStorage
    from vllm_from_scratch_b200.parts.model import DecoderModel
    entry, config = typed(bemuzen_configs.BZ_A)
    spec = entry.build_spec(config)
    model = DecoderModel(spec, torch.float32, "cpu")
    storage = CacheStorage(model.cache_needs(), [None] * len(spec.schedule), 16, 6, 3, torch.float32, "cpu",
                           embedding_need=model.embedding.cache_need())
    # two paired layers with different key/value sizes: two groups, values in slabs of their own
    assert len(storage.groups) == 2
    first, scan, third = storage.views
    assert first.kind == "pages" and first.keys.shape == (6, 2, 16, 16) and first.values.shape == (6, 2, 16, 24)
    assert set(first.states) == {"right.state"} and first.states["right.state"].shape == (4, 2, 8, 16)
    assert scan.kind == "state" and set(scan.states) == {"state", "conv"}
    assert scan.states["conv"].shape == (4, 3, 2 * 16 + 2 * 8) and scan.states["state"].shape == (4, 2, 8, 16)
    assert third.values.shape == (6, 2, 16, 8)
    assert storage.embedding_view.state.dtype == torch.int32 and storage.embedding_view.state.shape == (4, 1)
    assert storage.has_state and len(storage.states) == 5
    # a slot that is handed out again starts from zeros in every state tensor
    for tensor in storage.states.values():
        tensor.fill_(7)
    storage.zero_slots([1])
    for tensor in storage.states.values():
        assert not tensor[1].any() and tensor[0].eq(7).all() and tensor[2].eq(7).all()
    manager = CacheManager(storage.group_windows, 16, 6, 3, True, has_state=storage.has_state)
    assert not manager.prefix_caching          # a published prefix cannot stand for a recurrent state
    assert storage.bytes_per_token() == 2 * (16 + 24) * 4 + 2 * (24 + 8) * 4      # heads * (key + value) * float32


def test_paired_mixers_refuse_two_sets_of_pages():
    from vllm_from_scratch_b200.parts import MIXERS, PartEnv, PartSpec, POSITION_ENCODINGS
    env = PartEnv(32, torch.float32, torch.device("cpu"), "mix")
    attention = {"num_heads": 2, "num_kv_heads": 1, "head_dim": 8, "scale": 1.0}
    pair = MIXERS.get("paired_mixers")(
        {"branches": (PartSpec("biased_attention", attention, name="x"), PartSpec("biased_attention", attention, name="y")),
         "eps": 1e-5}, env, POSITION_ENCODINGS.get("none")({}, env))
    with pytest.raises(ValueError):
        pair.cache_need()


@pytest.mark.parametrize("name", ["A", "B"])
def test_plain_implementation_does_not_depend_on_the_cut(name):
    raw, _ = bemuzen_configs.CONFIGS[name]
    entry, config = typed(raw)
    weights = entry.random_weights(config, 5, dtype=torch.float32)
    model = plain_bemuzen.PlainBemuzen(raw, weights, torch.float64)
    tokens = torch.randint(0, raw["vocab"], (23,), generator=torch.Generator().manual_seed(2)).tolist()
    whole, trail = model.step({}, tokens)
    state, rows, done = {}, [], 0
    for size in (1, 2, 5, 1, 1, 7, 6):
        rows.append(model.step(state, tokens[done:done + size])[0])
        done += size
    cut = torch.cat(rows)
    assert cut.shape == whole.shape and trail.shape[:2] == (len(raw["layers"]), len(tokens))
    assert float((cut - whole).abs().max()) < 1e-9


def test_query_temperature_steps_where_the_design_says():
    assert plain_bemuzen.query_temperature(0, 0.5, 4) == 1.0
    assert plain_bemuzen.query_temperature(2, 0.5, 4) == 1.0
    assert math.isclose(plain_bemuzen.query_temperature(3, 0.5, 4), 1.0 + 0.5 * math.log(2.0))
    assert math.isclose(plain_bemuzen.query_temperature(11, 0.5, 4), 1.0 + 0.5 * math.log(4.0))
