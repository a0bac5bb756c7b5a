"""Farorax models whose every size and constant is drawn at random (seeded): the 32-bit engine
against the plain model over whole requests, decoded tails, portions and mixed batches; the
bfloat16 engine over the same, up to each request's first position that is routed by a hair."""

import random

import pytest
import torch

from farorax_models import assert_rows_close, attention, dense, draw_tensors, lightning, routed
from plain_farorax import PlainModel
from tiny_models import cut, mixed_schedule, prompts, replay

pytestmark = pytest.mark.gpu
DEVICE = "cuda:0"


def random_config(seed: int) -> dict:
    rng = random.Random(seed)
    width = rng.choice([48, 64, 80, 96, 128, 160, 192, 256])

    def feed_forward():
        kind = rng.random()
        if kind < 0.15:
            return None
        if kind < 0.55:
            return dense(rng.choice([32, 40, 96, 200, 256, 384]))
        experts = rng.choice([2, 4, 6, 8, 12, 16])
        groups = rng.choice([g for g in (1, 2, 3, 4) if experts % g == 0])
        keep = rng.randint(1, groups)
        top = rng.randint(1, min(4, keep * (experts // groups)))
        if top == experts:
            top = max(top - 1, 1)
        return routed(rng.choice([8, 24, 40, 64, 128]), experts, top,
                      (groups, keep) if rng.random() < 0.8 else None if groups == 1 else (groups, keep),
                      rng.choice([None, 16, 48, 128]))

    def attention_layer():
        dim = rng.choice([8, 16, 24, 32, 40, 48, 64, 80, 96, 128])
        vdim = dim if rng.random() < 0.7 else rng.choice([8, 16, 32, 48, 64, 96])
        kv_heads = rng.choice([1, 2, 3, 4])
        heads = kv_heads * rng.choice([1, 2, 3, 4] if kv_heads > 1 else [1, 2, 4, 8, 10])
        rot = None
        if rng.random() < 0.85:
            rot = {"base": rng.choice([100.0, 10000.0, 500000.0]),
                   "dims": rng.choice([2, dim // 2 // 2 * 2 or 2, dim])}
            if rng.random() < 0.6:
                low = rng.choice([0.5, 1.0, 2.0])
                rot["scaling"] = {"factor": rng.choice([2.0, 4.0, 8.0, 32.0]), "low": low,
                                  "high": low * rng.choice([2.0, 4.0, 8.0]),
                                  "original": rng.choice([16, 64, 256, 4096])}
        window = rng.choice([1, 3, 8, 17, 33, 64, 96, 100, 200, 1000, None])
        return attention(heads, kv_heads, dim, vdim, rng.uniform(0.05, 0.3), window, rot, feed_forward())

    def lightning_layer():
        heads = rng.randint(1, 6)
        return lightning(heads, rng.choice([4, 8, 16, 32, 48, 64, 96, 128, 136, 200]),
                         rng.choice([4, 8, 16, 24, 32, 64, 100, 128]),
                         [rng.choice([0.3, 0.8, 0.95, 0.99, 0.999, 1.0]) for _ in range(heads)],
                         feed_forward())

    count = rng.randint(2, 6)
    kinds = [rng.choice("al") for _ in range(count)]
    kinds[rng.randrange(count)] = "a"
    kinds[(kinds.index("a") + 1) % count] = "l"
    config = {"architecture": "Farorax", "vocab": rng.randint(50, 700), "width": width,
              "norm": {"eps": rng.choice([1e-6, 1e-5])},
              "residual_mult": rng.choice([0.2, 0.3, 0.5, 0.8, 1.0, 1.3]),
              "layers": [attention_layer() if kind == "a" else lightning_layer() for kind in kinds]}
    if rng.random() < 0.85:
        config["logit_softcap"] = rng.choice([5.0, 15.0, 30.0, 60.0])
    if rng.random() < 0.7:
        start = rng.randrange(count)
        config["loop"] = {"start": start, "stop": rng.randint(start + 1, count),
                          "times": rng.randint(1, 3)}
    return config


def engine(folder, dtype, page_size, capacity, max_requests=4):
    from mlx_one_b200.cache import CacheManager
    from mlx_one_b200.engine.loading import load_model
    from mlx_one_b200.engine.runner import Runner

    loaded = load_model(folder, dtype, DEVICE)
    cache = CacheManager(loaded.model.cache_needs, page_size=page_size, capacity_tokens=capacity,
                         max_requests=max_requests, dtype=dtype, device=DEVICE)
    return Runner(loaded.model, cache), cache


@pytest.mark.parametrize("seed", range(10))
def test_a_model_drawn_at_random(tmp_path, seed):
    import json

    from mlx_one_b200.weights.safetensors_io import write_safetensors

    config = random_config(seed)
    write_safetensors(tmp_path / "model.safetensors", draw_tensors(config, 100 + seed), {"format": "pt"})
    (tmp_path / "config.json").write_text(json.dumps(config))
    plain = PlainModel(tmp_path)
    page = (16, 16, 8, 4)[seed % 4]
    lengths = (150, 64, 23, 50, 9, 2, 1)
    requests = dict(enumerate(prompts(config["vocab"], lengths, seed=seed)))
    want = {key: plain.logits(tokens) for key, tokens in requests.items()}
    for dtype in (torch.float32, torch.bfloat16):
        runner, cache = engine(tmp_path, dtype, page, 4 * 192, max_requests=4)
        tokens = requests[0]
        got = replay(runner, cache, [([("w", tokens)], ["w"])])["w"]
        assert_rows_close(got, want[0], dtype, f"seed {seed} whole")
        steps = [([("d", tokens[:110])], [])] + [([("d", [t])], []) for t in tokens[110:]]
        steps[-1] = (steps[-1][0], ["d"])
        assert_rows_close(replay(runner, cache, steps)["d"], want[0], dtype, f"seed {seed} decoded tail")
        steps = [([("p", part)], []) for part in cut(tokens, (7, 2, 40, 3, 1))]
        steps[-1] = (steps[-1][0], ["p"])
        assert_rows_close(replay(runner, cache, steps)["p"], want[0], dtype, f"seed {seed} portions")
        got = replay(runner, cache, mixed_schedule(requests))
        for key in requests:
            assert_rows_close(got[key], want[key], dtype, f"seed {seed} mixed request {key}")
        assert not cache.requests()
