"""Farorax without a GPU: configuration, the order of calls, the weight contract, and the
engine's bookkeeping (pages of windows, state slots, the loop's passes, the factor on the parts'
outputs) run with the plain kernel set against the plain model."""

import copy
import json

import pytest
import torch

from farorax_models import CONFIGS, F1, F3, F5, assert_rows_close, make_model_dir
from plain_farorax import PlainModel, layer_runs
from plain_ops import PlainOps
from tiny_models import cut, mixed_schedule, prompts, replay


def engine(folder, page_size, capacity, max_requests=4):
    from mlx_one_b200.cache import CacheManager
    from mlx_one_b200.engine.loading import load_model
    from mlx_one_b200.engine.runner import Runner

    loaded = load_model(folder, "float32", "cpu", PlainOps())
    cache = CacheManager(loaded.model.cache_needs, page_size=page_size, capacity_tokens=capacity,
                         max_requests=max_requests, dtype=torch.float32, device="cpu")
    return Runner(loaded.model, cache), cache


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("farorax_cpu")
    return {name: make_model_dir(name, root) for name in CONFIGS}


# ------------------------------------------------------------------ configuration


def test_config_round_trip_and_registry(tmp_path):
    from mlx_one_b200.config import FaroraxConfig, read_config

    for name, (config, _, _) in CONFIGS.items():
        typed = FaroraxConfig.from_dict(config)
        again = FaroraxConfig.from_dict(typed.to_dict())
        assert again == typed, name
    (tmp_path / "config.json").write_text(json.dumps(F1))
    entry, typed = read_config(tmp_path)
    assert entry.name == "farorax" and typed.width == F1["width"] and typed.loop.times == 2
    assert typed.residual_mult == 0.5 and typed.logit_softcap == 20.0
    assert typed.layers[0].mixer.window == 24 and typed.layers[0].mixer.rot.scaling.high == 3.0
    assert typed.layers[1].mlp.groups == 3 and typed.layers[1].mlp.keep == 2
    assert typed.layers[1].mlp.shared_ff == 40 and typed.layers[2].mlp is None
    assert typed.layers[1].mixer.decay == (0.9, 0.5)
    five = FaroraxConfig.from_dict(F5)
    assert five.layers[0].mixer.window is None and five.layers[2].mixer.rot is None
    assert five.layers[0].mlp.groups == 1 and five.layers[0].mlp.keep == 1


@pytest.mark.parametrize("path, value, text", [
    (("layers", 0, "type"), "parallel", "type"),
    (("layers", 0, "mixer", "kv_heads"), 3, "kv_heads"),
    (("layers", 0, "mixer", "rot", "dims"), 7, "dims"),
    (("layers", 0, "mixer", "rot", "dims"), 64, "dims"),
    (("layers", 0, "mixer", "mask", "size"), 0, "mask.size"),
    (("layers", 0, "mlp", "kind"), "plain", "kind"),
    (("layers", 1, "mixer", "decay"), [0.5], "decay"),
    (("layers", 1, "mixer", "decay"), [0.5, 1.5], "decay"),
    (("layers", 1, "mlp", "router", "top"), 5, "top"),
    (("layers", 1, "mlp", "router", "groups", "count"), 4, "groups"),
    (("layers", 1, "mlp", "router", "groups", "keep"), 4, "keep"),
    (("loop", "stop"), 9, "loop"),
    (("loop", "times"), 0, "times"),
    (("norm", "eps"), -1.0, "eps"),
    (("residual_mult",), 0.0, "residual_mult"),
    (("logit_softcap",), -3.0, "logit_softcap"),
])
def test_config_rejections(path, value, text):
    from mlx_one_b200.config import ConfigError, FaroraxConfig

    config = copy.deepcopy(F1)
    at = config
    for key in path[:-1]:
        at = at[key]
    at[path[-1]] = value
    with pytest.raises(ConfigError, match=text):
        FaroraxConfig.from_dict(config)


def test_missing_key_is_named():
    from mlx_one_b200.config import ConfigError, FaroraxConfig

    config = copy.deepcopy(F1)
    del config["layers"][1]["mlp"]["expert"]["ff"]
    with pytest.raises(ConfigError, match=r"layers\[1\]\.mlp\.expert\.ff"):
        FaroraxConfig.from_dict(config)
    config = copy.deepcopy(F1)
    del config["layers"][0]["mixer"]["rot"]["scaling"]["low"]
    with pytest.raises(ConfigError, match=r"layers\[0\]\.mixer\.rot\.scaling\.low"):
        FaroraxConfig.from_dict(config)


def test_order_of_calls_and_weight_contract():
    from mlx_one_b200.architectures.farorax import describe
    from mlx_one_b200.config import FaroraxConfig
    from mlx_one_b200.parts import FixedState, PagedKeyValues, cache_entries, expected_tensors

    spec = describe(FaroraxConfig.from_dict(F3))
    assert [call.layer for call in spec.order] == [index for index, _ in layer_runs(F3)] == \
        [0, 1, 1, 1, 2, 3]
    passes = [(call.inject.row, call.inject.mix) for call in spec.order if call.inject is not None]
    assert passes == [(0, "loop.in"), (1, "loop.in"), (2, "loop.in")]
    needs = cache_entries(spec)
    assert len(needs) == 6                                  # every call keeps something of its own
    assert needs[1] == PagedKeyValues(1, 64, 100) and needs[0] == FixedState((4 * 128 * 32,), "float32")
    names = expected_tensors(spec)
    assert names["loop.in"].shape == (128, 256) and names["loop.step"].shape == (3, 128)
    assert names["l1.mix.sink"].shape == (8,) and names["l1.mix.o"].shape == (128, 8 * 64)
    assert names["l2.mlp.router"].shape == (8, 128) and names["l2.mlp.e7.down"].shape == (128, 48)
    assert names["l2.mlp.shared.gate"].shape == (64, 128) and names["l0.mix.norm"].shape == (128,)
    assert "l0.mix.sink" not in names and "l3.mlp.router" not in names
    five = expected_tensors(describe(FaroraxConfig.from_dict(F5)))
    assert five["l0.mix.v"].shape == (40, 72) and five["l0.mix.k"].shape == (24, 72)
    assert "l2.norm2" not in five and "l0.mlp.shared.up" in five


def test_a_wrong_tensor_is_one_error(folders, tmp_path):
    from mlx_one_b200.engine.loading import load_model
    from mlx_one_b200.weights import WeightError
    from mlx_one_b200.weights.safetensors_io import write_safetensors
    from plain_farorax import read_tensors

    tensors = read_tensors(folders["F1"] / "model.safetensors")
    del tensors["l0.mix.sink"]
    tensors["l1.mlp.router"] = tensors["l1.mlp.router"][:3]
    tensors["extra.one"] = torch.zeros(2, dtype=torch.bfloat16)
    write_safetensors(tmp_path / "model.safetensors", tensors, {"format": "pt"})
    (tmp_path / "config.json").write_text(json.dumps(F1))
    with pytest.raises(WeightError) as caught:
        load_model(tmp_path, "float32", "cpu", PlainOps())
    text = str(caught.value)
    assert "l0.mix.sink" in text and "l1.mlp.router" in text and "extra.one" in text


# ------------------------------------------------------------------ the engine's bookkeeping


@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_portions_and_single_tokens(folders, name):
    config, _, page = CONFIGS[name]
    plain = PlainModel(folders[name])
    runner, cache = engine(folders[name], page, 256)
    (tokens,) = prompts(config["vocab"], (90,), seed=4)
    want = plain.logits(tokens)
    got = replay(runner, cache, [([("w", tokens)], ["w"])])["w"]
    assert_rows_close(got, want, torch.float32, f"{name} whole")
    for sizes in ((7, 2, 13, 1, 1, 3), (2,)):
        steps = [([("r", part)], []) for part in cut(tokens, sizes)]
        steps[-1] = (steps[-1][0], ["r"])
        assert_rows_close(replay(runner, cache, steps)["r"], want, torch.float32, f"{name} {sizes}")
    assert not cache.requests()


@pytest.mark.parametrize("name", ["F1", "F4", "F5"])
def test_mixed_batches_with_pages_and_slots_used_again(folders, name):
    config, _, page = CONFIGS[name]
    plain = PlainModel(folders[name])
    lengths = (40, 30, 23, 50, 17, 9, 2, 1)
    requests = dict(enumerate(prompts(config["vocab"], lengths, seed=5)))
    runner, cache = engine(folders[name], page, 4 * 64, max_requests=4)
    got = replay(runner, cache, mixed_schedule(requests))
    for request_id, tokens in requests.items():
        assert_rows_close(got[request_id], plain.logits(tokens), torch.float32,
                          f"{name} mixed request {request_id}")
    assert not cache.requests()


def test_pages_behind_a_window_come_back(folders):
    """A request far longer than the pool: the attention layers' pages that have left every
    window are handed out again, and the logits stay those of the plain model."""
    config, _, page = CONFIGS["F2"]                         # windows of 7, pages of 8
    runner, cache = engine(folders["F2"], page, 64, max_requests=1)
    (tokens,) = prompts(config["vocab"], (200,), seed=6)
    steps = [([("r", part)], []) for part in cut(tokens, (5, 1, 9, 2))]
    steps[-1] = (steps[-1][0], ["r"])
    got = replay(runner, cache, steps)["r"]
    assert_rows_close(got, PlainModel(folders["F2"]).logits(tokens), torch.float32, "a long request")


def test_greedy_generation_through_the_entry_point(folders):
    """The engine's own entry point and scheduler: prompts in portions of eight tokens, three
    requests at a time, greedy tokens against the plain model's."""
    from mlx_one_b200 import BatchingConfig, CacheConfig, Engine, TextGenerationOptions

    config, _, page = CONFIGS["F1"]
    plain = PlainModel(folders["F1"])
    batch = prompts(config["vocab"], (7, 30, 3, 19), seed=8)
    engine_ = Engine(folders["F1"], execution_dtype="float32", ops=PlainOps(), device="cpu",
                     cache_config=CacheConfig(block_size_tokens=page, capacity_tokens=256),
                     batching_config=BatchingConfig(max_sequences=3, prefill_chunk_size=8))
    results = engine_.generate_batch_ids(batch, TextGenerationOptions(max_tokens=6, ignore_eos=True))
    for prompt, result in zip(batch, results):
        assert list(result.token_ids) == plain.greedy(prompt, 6)
    engine_.close()
