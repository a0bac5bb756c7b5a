"""Galarax without a GPU: configuration, the order of calls, the weight contract, and the
engine's bookkeeping (cache entries under names, slots, the loop's passes) run with the plain
kernel set against the plain model."""

import copy
import json

import pytest
import torch

from galarax_models import CONFIGS, G1, G3, make_model_dir
from plain_galarax import PlainModel, layer_runs, rotary_frequencies
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


def close(got, want, what):
    assert torch.allclose(got, want, atol=2e-4, rtol=2e-4), \
        f"{what}: differs by {(got - want).abs().max().item():.3e}"


# ------------------------------------------------------------------ configuration


def test_config_round_trip_and_registry(tmp_path):
    from mlx_one_b200.config import GalaraxConfig, read_config

    for name, (config, _, _) in CONFIGS.items():
        typed = GalaraxConfig.from_dict(config)
        again = GalaraxConfig.from_dict(typed.to_dict())
        assert again == typed, name
    (tmp_path / "config.json").write_text(json.dumps(G1))
    entry, typed = read_config(tmp_path)
    assert entry.name == "galarax" and typed.width == G1["width"] and typed.loop.times == 2
    assert typed.layers[1].ff is None and typed.layers[2].left.rot is None
    assert typed.layers[0].left.rot.scaling.factor == 4.0


@pytest.mark.parametrize("path, value, text", [
    (("layers", 0, "type"), "serial", "type"),
    (("layers", 0, "mixer", "left", "kv_heads"), 3, "kv_heads"),
    (("layers", 0, "mixer", "left", "rot", "dims"), 7, "dims"),
    (("layers", 0, "mixer", "left", "rot", "dims"), 64, "dims"),
    (("layers", 0, "mlp", "kind"), "gated", "kind"),
    (("loop", "stop"), 9, "loop"),
    (("loop", "times"), 0, "times"),
    (("norm", "eps"), -1.0, "eps"),
])
def test_config_rejections(path, value, text):
    from mlx_one_b200.config import ConfigError, GalaraxConfig

    config = copy.deepcopy(G1)
    at = config
    for key in path[:-1]:
        at = at[key]
    at[path[-1]] = value
    with pytest.raises(ConfigError, match=text):
        GalaraxConfig.from_dict(config)


def test_missing_key_is_named():
    from mlx_one_b200.config import ConfigError, GalaraxConfig

    config = copy.deepcopy(G1)
    del config["layers"][2]["mixer"]["right"]["conv"]
    with pytest.raises(ConfigError, match=r"layers\[2\]\.mixer\.right\.conv"):
        GalaraxConfig.from_dict(config)


# ------------------------------------------------------------------ description in parts


def test_order_of_calls_and_what_enters_the_stream():
    from mlx_one_b200.architectures.galarax import describe
    from mlx_one_b200.config import GalaraxConfig

    for name, (config, _, _) in CONFIGS.items():
        spec = describe(GalaraxConfig.from_dict(config))
        want = layer_runs(config)
        assert [call.layer for call in spec.order] == [layer for layer, _ in want], name
        for call, (_, turn) in zip(spec.order, want):
            if turn is None:
                assert call.inject is None
            else:
                assert call.inject.row == turn and call.inject.embedding == (turn > 0)
    spec = describe(GalaraxConfig.from_dict(G3))
    assert [call.layer for call in spec.order] == [0, 1, 1, 1, 2, 3]


def test_weight_contract_and_cache_entries():
    from mlx_one_b200.architectures.galarax import describe
    from mlx_one_b200.config import GalaraxConfig
    from mlx_one_b200.parts import FixedState, PagedKeyValues, cache_entries, expected_tensors

    spec = describe(GalaraxConfig.from_dict(G1))
    names = expected_tensors(spec)
    assert names["embed"].shape == (300, 64) and names["head"].shape == (300, 64)
    assert names["loop.step"].shape == (2, 64) and names["final.norm"].shape == (64,)
    assert names["l0.mix.left.q"].shape == (128, 64) and names["l0.mix.left.q.b"].shape == (128,)
    assert names["l0.mix.left.v"].shape == (32, 64) and names["l0.mix.left.o"].shape == (64, 64)
    assert names["l0.mix.right.q"].shape == (32, 64) and names["l0.mix.right.q.conv"].shape == (32, 4)
    assert names["l0.mix.right.v.conv"].shape == (96, 4) and names["l0.mix.right.b"].shape == (4, 64)
    assert names["l0.mix.right.A_log"].shape == (4,) and names["l0.mix.right.norm"].shape == (24,)
    assert names["l0.mix.right.o"].shape == (64, 96) and names["l0.mix.left.out"].shape == (64,)
    assert names["l0.mlp.up"].shape == (96, 64) and "l1.mlp.up" not in names
    assert "l1.norm2" not in names and names["l2.norm2"].shape == (64,)
    needs = cache_entries(spec)
    # five calls (two passes of two layers, then the last layer), two things each
    assert len(needs) == 10
    assert needs[(0, "left")] == PagedKeyValues(2, 32, None)       # rows of max(32, 16)
    assert needs[(4, "left")] == PagedKeyValues(1, 16, None)
    assert needs[(0, "right")] == FixedState((4 * 16 * 24 + 4 * (2 * 32 + 96),), "float32")


def test_stretched_frequencies():
    from mlx_one_b200.parts import POSITIONS, PartSpec, Runtime

    rot = G3["layers"][0]["mixer"]["left"]["rot"]
    want, amplitude = rotary_frequencies(rot, torch.float64)
    sc = rot["scaling"]
    part = POSITIONS.get("yarn")(PartSpec("yarn", {
        "theta": rot["base"], "rotary_dim": rot["dims"], "factor": sc["factor"],
        "original": sc["original"], "fast": sc["fast"], "slow": sc["slow"]}), {},
        Runtime(torch.float32, torch.device("cpu"), None))
    table, dims = part.rotary_table()
    assert dims == rot["dims"] and abs(part.amplitude() - amplitude) < 1e-12
    assert torch.allclose(table.double(), want, rtol=1e-6, atol=0)
    # the fastest pair keeps its frequency, the slowest is divided by the factor
    plain = rot["base"] ** (-2 * torch.arange(dims // 2, dtype=torch.float64) / dims)
    assert torch.isclose(want[0], plain[0]) and torch.isclose(want[-1], plain[-1] / sc["factor"])
    assert ((want <= plain * (1 + 1e-12)) & (want >= plain / sc["factor"] * (1 - 1e-12))).all()


# ------------------------------------------------------------------ the engine's bookkeeping


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("galarax")
    return {name: make_model_dir(name, root) for name in ("G1", "G2", "G4", "G5")}


@pytest.mark.parametrize("name", ["G1", "G2", "G4", "G5"])
def test_whole_and_portions_against_the_plain_model(folders, name):
    config, _, page = CONFIGS[name]
    runner, cache = engine(folders[name], page, 128)
    plain = PlainModel(folders[name])
    (tokens,) = prompts(config["vocab"], (29,), seed=2)
    want = plain.logits(tokens)
    close(replay(runner, cache, [([("w", tokens)], ["w"])])["w"], want, f"{name} whole")
    for sizes in ((5, 2, 1, 7), (2,), (1,)):
        steps = [([("r", part)], []) for part in cut(tokens, sizes)]
        steps[-1] = (steps[-1][0], ["r"])
        close(replay(runner, cache, steps)["r"], want, f"{name} portions {sizes}")


def test_hidden_states_after_every_run(folders):
    config, _, page = CONFIGS["G1"]
    runner, cache = engine(folders["G1"], page, 64)
    (tokens,) = prompts(config["vocab"], (9,), seed=6)
    seen = []
    runner.model.observer = lambda place, residual, delta: seen.append(
        (place, (residual if delta is None else residual + delta.float()).clone()))
    replay(runner, cache, [([("w", tokens)], ["w"])])
    want = []
    PlainModel(folders["G1"]).logits(tokens, want)
    assert [place for place, _ in seen] == [-1, 0, 1, 2, 3, 4]
    for (place, got), state in zip(seen[1:], want):
        close(got, state.float(), f"stream after run {place}")


def test_mixed_batches_with_slots_and_pages_used_again(folders):
    config, _, page = CONFIGS["G1"]
    lengths = (20, 31, 12, 26, 9, 33, 5, 17)
    requests = dict(enumerate(prompts(config["vocab"], lengths, seed=5)))
    runner, cache = engine(folders["G1"], page, 4 * 36, max_requests=4)
    got = replay(runner, cache, mixed_schedule(requests, decode_tail=4))
    plain = PlainModel(folders["G1"])
    assert cache.stats().slots_total == (4, 4)          # eight requests through four slots
    for request_id, tokens in requests.items():
        close(got[request_id], plain.logits(tokens), f"mixed request {request_id}")
    assert not cache.requests()


def test_greedy_generation_through_the_entry_point(folders):
    from mlx_one_b200 import BatchingConfig, CacheConfig, Engine, TextGenerationOptions
    from mlx_one_b200.engine.loading import load_model

    config, _, page = CONFIGS["G2"]
    loaded = load_model(folders["G2"], "float32", "cpu", PlainOps())
    engine_ = Engine(loaded, cache_config=CacheConfig(block_size_tokens=page, capacity_tokens=256),
                     batching_config=BatchingConfig(max_sequences=3, prefill_chunk_size=5))
    plain = PlainModel(folders["G2"])
    batch = prompts(config["vocab"], (7, 12, 3, 9), seed=8)
    results = engine_.generate_batch_ids(batch, TextGenerationOptions(max_tokens=6, ignore_eos=True))
    for prompt, result in zip(batch, results):
        assert list(result.token_ids) == plain.greedy(prompt, 6)
    engine_.close()


def test_command_line_writes_a_random_model(tmp_path):
    import subprocess
    import sys
    from pathlib import Path

    from plain_galarax import read_tensors

    root = Path(__file__).resolve().parent.parent
    (tmp_path / "config.json").write_text(json.dumps(G1))
    done = subprocess.run([sys.executable, str(root / "bin" / "mlx-one"), "random-model",
                           str(tmp_path / "config.json"), str(tmp_path / "model"), "--seed", "3"],
                          capture_output=True, text=True, timeout=300)
    assert done.returncode == 0, done.stderr
    stored = read_tensors(tmp_path / "model" / "model.safetensors")
    assert stored["l2.mix.right.v.conv"].shape == (16, 2) and stored["loop.step"].shape == (2, 64)
    assert json.loads((tmp_path / "model" / "config.json").read_text())["architecture"] == "Galarax"
    # norm weights stored around zero, plain weights around one
    assert stored["l0.norm1"].float().abs().mean() < 0.3 < stored["l0.mix.left.out"].float().mean()
