"""The Lobuzen design without a GPU: its configuration reads and writes back, its description names the
tensors of a model folder, the cache groups follow the windows of the layers that read them, and the plain
implementation itself gives the same rows however a prompt is fed."""

from __future__ import annotations

import copy

import pytest
import torch

import lobuzen_configs
import plain_lobuzen as plain


@pytest.mark.parametrize("name", list(lobuzen_configs.CONFIGS))
def test_config_round_trip_and_names(name):
    import vllm_from_scratch_b200 as engine
    from vllm_from_scratch_b200.parts.model import DecoderModel
    raw = lobuzen_configs.CONFIGS[name][0]
    entry, typed = engine.load_model_config(raw)
    assert entry.name == "Lobuzen"
    assert entry.config_class.from_dict(typed.to_dict()) == typed
    model = DecoderModel(entry.build_spec(typed), torch.float32, "cpu")
    weights = entry.random_weights(typed, 3)
    expected = model.expected_weights()
    assert set(weights) == set(expected)
    for key, info in expected.items():
        assert tuple(weights[key].shape) == tuple(info.shape), key
    assert model.graph_safe()


def test_cache_follows_the_longest_window_that_reads_it():
    import vllm_from_scratch_b200 as engine
    from vllm_from_scratch_b200.parts.model import DecoderModel
    entry, typed = engine.load_model_config(lobuzen_configs.LZ_A)
    needs = DecoderModel(entry.build_spec(typed), torch.float32, "cpu").cache_needs()
    assert needs[0].window == 33 and needs[0].value_dim == 0 and needs[0].head_dim == 32
    assert needs[2] is None and needs[4] is None            # they read layer 0's rows
    assert needs[1].window == 12 and needs[3].window is None
    # a reader without a window keeps every row of the owner
    raw = copy.deepcopy(lobuzen_configs.LZ_A)
    del raw["layers"][2]["mixer"]["mask"]
    entry, typed = engine.load_model_config(raw)
    assert DecoderModel(entry.build_spec(typed), torch.float32, "cpu").cache_needs()[0].window is None


@pytest.mark.parametrize("change, message", [
    (lambda raw: raw["layers"][2]["mixer"].update(kv_from=1), "caches no latent rows"),
    (lambda raw: raw["layers"][2]["mixer"].update(kv_from=2), "earlier layer"),
    (lambda raw: raw["layers"][2]["mixer"].update(kv_rank=16), "kv_rank"),
    (lambda raw: raw["layers"][0]["mlp"]["router"].update(top=5), "cannot come from"),
    (lambda raw: raw["layers"][1]["mlp"].update(kind="other"), "part of the design"),
    (lambda raw: raw["layers"][1].update(type="mamba2"), "not a mixer of this design"),
])
def test_config_errors(change, message):
    import vllm_from_scratch_b200 as engine
    raw = copy.deepcopy(lobuzen_configs.LZ_A)
    change(raw)
    with pytest.raises(Exception, match=message):
        engine.load_model_config(raw)


def test_plain_routing():
    router = {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 1}}
    h = torch.tensor([1.0], dtype=torch.float64)
    # scores rise with the expert's index; the correction lifts group 0 above the others for the choice only
    w = {"router": torch.tensor([[-2.0], [-1.0], [0.0], [0.5], [1.0], [2.0]], dtype=torch.float64),
         "correction": torch.tensor([5.0, 4.0, 0.0, 0.0, 0.0, 0.0], dtype=torch.float64)}
    chosen, weights = plain.route(w, router, h)
    assert chosen == [0, 1]
    assert torch.allclose(torch.stack(weights), torch.sigmoid(torch.tensor([-2.0, -1.0], dtype=torch.float64)))
    # negative choice scores: an excluded expert must not win with a score of zero
    w["correction"] = torch.tensor([-9.0, -9.5, -20.0, -20.0, -20.0, -20.0], dtype=torch.float64)
    assert plain.route(w, router, h)[0] == [0, 1]
    # a group's mark is the sum of its two best, not its best
    router = {"experts": 4, "top": 1, "groups": {"count": 2, "keep": 1}}
    w = {"router": torch.zeros(4, 1, dtype=torch.float64),
         "correction": torch.tensor([0.9, -5.0, 0.5, 0.4], dtype=torch.float64)}
    assert plain.route(w, router, h)[0] == [2]


def test_plain_rows_do_not_depend_on_the_portions():
    import vllm_from_scratch_b200 as engine
    raw = lobuzen_configs.LZ_C
    entry, typed = engine.load_model_config(raw)
    weights = entry.random_weights(typed, 5, std=0.2, dtype=torch.float32)
    tokens = torch.randint(0, raw["vocab"], (30,), generator=torch.Generator().manual_seed(1)).tolist()
    model = plain.PlainLobuzen(raw, weights)
    whole = model.run("x", tokens)
    again = torch.cat([model.run("y", tokens[:7]), model.run("y", tokens[7:9]), model.run("y", tokens[9:])])
    assert torch.equal(whole, again)
    # a window of one position sees itself only: the first layers of this model mix no tokens at all
    assert not torch.allclose(whole[5], model.run("z", tokens[4:6])[1])
