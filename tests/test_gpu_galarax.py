"""Galarax on the GPU against the plain implementation: each new mechanism alone, then the
engine over whole requests, decoded tails, portions down to two tokens, mixed batches with
pages and slots used again, far keys and long memory, and greedy generation."""

import math

import pytest
import torch

from galarax_models import CONFIGS, assert_rows_close as assert_close, make_model_dir
from plain_galarax import (PlainModel, causal_conv, causal_softmax_attention, delta_recurrence,
                           rms, rotate, rotary_frequencies, silu)
from tiny_models import cut, mixed_schedule, prompts, replay

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]
DEVICE = "cuda:0"


@pytest.fixture(scope="module")
def ops():
    from mlx_one_b200.kernels import default_ops
    return default_ops(DEVICE)


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("galarax")
    return {name: make_model_dir(name, root) for name in CONFIGS}


@pytest.fixture(scope="module")
def plain(folders):
    return {name: PlainModel(folder) for name, folder in folders.items()}


def engine(folder, dtype, page_size, capacity, max_requests=4):
    from mlx_one_b200.cache import CacheManager
    from mlx_one_b200.engine.loading import load_model
    from mlx_one_b200.engine.runner import Runner

    loaded = load_model(folder, dtype, DEVICE)
    cache = CacheManager(loaded.model.cache_needs, page_size=page_size, capacity_tokens=capacity,
                         max_requests=max_requests, dtype=dtype, device=DEVICE)
    return Runner(loaded.model, cache), cache


def context(portions, histories):
    """A StepContext for requests that bring ``portions`` tokens after ``histories`` tokens."""
    from mlx_one_b200.parts import StepContext

    ints = lambda values: torch.tensor(values, dtype=torch.int32, device=DEVICE)
    positions, owner, starts = [], [], [0]
    for r, (n, before) in enumerate(zip(portions, histories)):
        positions += list(range(before, before + n))
        owner += [r] * n
        starts.append(starts[-1] + n)
    return StepContext(tokens=len(positions), requests=len(portions), token_ids=ints([0] * len(positions)),
                       positions=ints(positions), token_request=ints(owner),
                       request_start=ints(starts), history=ints(histories),
                       max_portion=max(portions), max_context=max(p + h for p, h in zip(portions, histories)))


def bound(dtype, tight=2e-5, loose=2e-2):
    return tight if dtype == torch.float32 else loose


# ------------------------------------------------------------------ mechanisms alone


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("dim, vdim, dims, amplitude_factor", [(32, 16, 16, 4.0), (16, 48, 16, None),
                                                               (64, 64, 32, 16.0), (24, 24, 2, 8.0)])
def test_rotation_norm_and_page_write(ops, dtype, dim, vdim, dims, amplitude_factor):
    """Queries and keys: partial rotation with stretched frequencies and scaled cosine and sine,
    then division by the root mean square; values untouched; all three padded to the pages' row
    size. Positions lie at the start, at page borders and far away; pages are out of order."""
    from mlx_one_b200.parts import POSITIONS, PagedKeyValues, PagedView, PartSpec, Runtime

    heads, kv_heads, page, eps = 4, 2, 8, 1e-5
    row = max(dim, vdim)
    rot = {"base": 777.0, "dims": dims}
    spec = {"theta": rot["base"], "rotary_dim": dims, "factor": None}
    if amplitude_factor:
        rot["scaling"] = {"factor": amplitude_factor, "original": 48, "fast": 6.0, "slow": 0.7}
        spec.update(factor=amplitude_factor, original=48, fast=6.0, slow=0.7)
    encoding = POSITIONS.get("yarn")(PartSpec("yarn", spec), {}, Runtime(dtype, torch.device(DEVICE), ops))
    histories, portions = [0, 7, 1530], [3, 10, 5]
    ctx = context(portions, histories)
    generator = torch.Generator().manual_seed(dim * 100 + vdim)
    width = (heads + kv_heads) * dim + kv_heads * vdim
    qkv = torch.randn(ctx.tokens, width, generator=generator).to(dtype)
    pages = 200
    table = torch.full((3, 200), -1, dtype=torch.int32)
    order = torch.randperm(pages - 1, generator=generator).tolist()
    for r, (n, before) in enumerate(zip(portions, histories)):
        for block in range(before // page, (before + n - 1) // page + 1):
            table[r, block] = order.pop()
    kv = torch.zeros(2, pages, kv_heads, page, row, dtype=dtype, device=DEVICE)
    view = PagedView(kv, table.to(DEVICE), page, PagedKeyValues(kv_heads, row, None))
    q = ops.qk_norm_rope_store(qkv.to(DEVICE), heads=heads, kv_heads=kv_heads, head_dim=dim,
                               q_weight=None, k_weight=None, eps=eps, rotary=encoding.rotary_table(),
                               ctx=ctx, view=view, write=True, value_dim=vdim,
                               amplitude=encoding.amplitude(), norm_after=True)
    ops.check_errors()
    x = qkv.double()
    positions = ctx.positions.cpu()
    want_q = rms(rotate(x[:, :heads * dim].view(-1, heads, dim), positions, rot), eps)
    want_k = rms(rotate(x[:, heads * dim:(heads + kv_heads) * dim].view(-1, kv_heads, dim), positions, rot), eps)
    want_v = x[:, (heads + kv_heads) * dim:].view(-1, kv_heads, vdim)
    # (32-bit angles: position * frequency is rounded to 1530 * 2^-24 at the far positions)
    tolerance = bound(dtype, 3e-4)
    got_q = q.cpu().double()
    assert (got_q[..., :dim] - want_q).abs().max() < tolerance and (got_q[..., dim:] == 0).all()
    for t in range(ctx.tokens):
        r, p = int(ctx.token_request[t]), int(positions[t])
        slot = kv[:, int(table[r, p // page]), :, p % page].cpu().double()
        assert (slot[0, :, :dim] - want_k[t]).abs().max() < tolerance, f"key of token {t}"
        assert (slot[1, :, :vdim] - want_v[t]).abs().max() < tolerance, f"value of token {t}"
        assert (slot[0, :, dim:] == 0).all() and (slot[1, :, vdim:] == 0).all()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("dim, vdim", [(32, 16), (96, 80), (72, 112), (128, 128), (24, 200)])
@pytest.mark.parametrize("portion", [1, 37])
def test_a_far_key_stands_out(ops, dtype, portion, dim, vdim):
    """One key hundreds of positions back (just after a page border) is the only one that matches
    the last queries: their output must be that key's value. Decoded alone and in a portion."""
    from mlx_one_b200.parts import PagedKeyValues, PagedView

    heads, kv_heads, page, eps, scale = 2, 1, 16, 1e-6, 32.0 / dim
    total, far, row = 600, 33, max(dim, vdim)
    generator = torch.Generator().manual_seed(5)
    q = torch.randn(total, heads, dim, generator=generator)
    k = torch.randn(total, kv_heads, dim, generator=generator)
    v = torch.randn(total, kv_heads, vdim, generator=generator)
    q[total - portion:] = 6.0 * k[far]          # (the norm keeps the direction only)
    qkv = torch.cat([q.flatten(1), k.flatten(1), v.flatten(1)], dim=1).to(dtype)
    want = causal_softmax_attention(rms(qkv[:, :heads * dim].double().view(total, heads, dim), eps),
                                    rms(qkv[:, heads * dim:(heads + 1) * dim].double().view(total, 1, dim), eps),
                                    qkv[:, (heads + 1) * dim:].double().view(total, 1, vdim), scale)
    assert (want[-1, 0] - qkv[far, (heads + 1) * dim:].double()).abs().max() < 0.05
    blocks = math.ceil(total / page)
    table = torch.arange(blocks, dtype=torch.int32).flip(0)[None].contiguous().to(DEVICE)
    kv = torch.zeros(2, blocks + 1, kv_heads, page, row, dtype=dtype, device=DEVICE)
    view = PagedView(kv, table, page, PagedKeyValues(kv_heads, row, None))
    common = dict(heads=heads, kv_heads=kv_heads, head_dim=dim, q_weight=None, k_weight=None, eps=eps,
                  rotary=None, scale=scale, window=None, view=view, write=True, value_dim=vdim,
                  amplitude=1.0, norm_after=True)
    first = total - portion
    ops.qkv_attention(qkv[:first].to(DEVICE), ctx=context([first], [0]), **common)
    got = ops.qkv_attention(qkv[first:].to(DEVICE), ctx=context([portion], [first]), **common)
    ops.check_errors()
    assert (got.view(portion, heads, row)[..., vdim:] == 0).all()
    got = got.view(portion, heads, row)[..., :vdim].cpu().double()
    assert (got - want[first:]).abs().max() < bound(dtype, 1e-4, 3e-2)


def delta_pieces(projected, conv, a_log, dt_bias, norm_weight, eps, sizes):
    """The mixer between its two products, from the plain functions, for one whole sequence."""
    H, G, D, V = sizes["heads"], sizes["kv_heads"], sizes["key_dim"], sizes["value_dim"]
    T, qk, inner = projected.shape[0], G * D, H * V
    mixed = silu(causal_conv(projected[:, :2 * qk + inner], conv))
    unit = lambda x: x / torch.sqrt((x * x).sum(-1, keepdim=True) + 1e-6)
    q = unit(mixed[:, :qk].view(T, G, D)) * D ** -0.5
    k = unit(mixed[:, qk:2 * qk].view(T, G, D))
    v = mixed[:, 2 * qk:].view(T, H, V)
    at = 2 * qk + inner
    gate = projected[:, at:at + inner].view(T, H, V)
    beta = torch.sigmoid(projected[:, at + inner:at + inner + H])
    g = torch.exp(-torch.exp(a_log) * torch.nn.functional.softplus(projected[:, at + inner + H:] + dt_bias))
    o = delta_recurrence(q, k, v, beta, g)
    return (rms(o, eps) * norm_weight * silu(gate)).reshape(T, inner)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("sizes", [dict(heads=4, kv_heads=2, key_dim=16, value_dim=24, taps=4),
                                   dict(heads=2, kv_heads=1, key_dim=40, value_dim=8, taps=2),
                                   dict(heads=3, kv_heads=3, key_dim=128, value_dim=40, taps=3),
                                   dict(heads=1, kv_heads=1, key_dim=200, value_dim=33, taps=1),
                                   dict(heads=2, kv_heads=2, key_dim=24, value_dim=160, taps=5)])
def test_gated_delta_rule_alone(ops, dtype, sizes):
    """Two requests side by side, each fed in portions of changing size (also single tokens and
    a portion shorter than the convolution), against one pass of the plain recurrence. The
    decay is slow, so what the first tokens wrote is still read at the end."""
    from mlx_one_b200.parts import FixedState, StateView
    from mlx_one_b200.parts.mixers import GatedDeltaRule

    H, G, D, V, taps = (sizes[key] for key in ("heads", "kv_heads", "key_dim", "value_dim", "taps"))
    channels, inner = 2 * G * D + H * V, H * V
    width = channels + inner + 2 * H
    generator = torch.Generator().manual_seed(D)
    lengths = (150, 61)
    projected = [(1.5 * torch.randn(n, width, generator=generator)).to(dtype) for n in lengths]
    conv = 0.5 * torch.randn(channels, taps, generator=generator)
    a_log = torch.full((H,), -5.0) + torch.randn(H, generator=generator)
    dt_bias, norm_weight, eps = torch.randn(H, generator=generator), 1 + 0.2 * torch.randn(V, generator=generator), 1e-5
    size = GatedDeltaRule.state_size({"heads": H, "kv_heads": G, "key_dim": D, "value_dim": V, "taps": taps})
    state = torch.zeros(5, size, device=DEVICE)
    state[:] = float("nan")                                   # stale contents of other slots must not matter
    state[[3, 1]] = 0
    slots = torch.tensor([3, 1], dtype=torch.int32, device=DEVICE)
    view = StateView(state, slots, FixedState((size,), "float32"))
    constants = dict(conv=conv.to(DEVICE), a_log=a_log.to(DEVICE), dt_bias=dt_bias.to(DEVICE),
                     norm_weight=norm_weight.to(DEVICE), eps=eps, unit_eps=1e-6, view=view, write=True, **sizes)
    cuts = [cut(list(range(lengths[0])), (40, 1, 2, 17, 1, 1, 64, 3)), cut(list(range(lengths[1])), (1, 2, 30, 1, 5))]
    got = [[], []]
    fed = [0, 0]
    while any(cuts):
        live = [r for r in (0, 1) if cuts[r]]
        parts = [cuts[r].pop(0) for r in live]
        rows = torch.cat([projected[r][part[0]:part[-1] + 1] for r, part in zip(live, parts)]).to(DEVICE)
        view.slots = slots[live].contiguous()
        out = ops.gated_delta_rule(rows, ctx=context([len(p) for p in parts], [fed[r] for r in live]), **constants)
        at = 0
        for r, part in zip(live, parts):
            got[r].append(out[at:at + len(part)].cpu())
            at += len(part)
            fed[r] += len(part)
    ops.check_errors()
    for r in (0, 1):
        want = delta_pieces(projected[r].double(), conv.double(), a_log.double(), dt_bias.double(),
                            norm_weight.double(), eps, sizes)
        difference = (torch.cat(got[r]).double() - want).abs().max()
        # (bfloat16: the output is rounded to 8 bits of mantissa at values of up to 8)
        assert difference < bound(dtype, 5e-5, 0.1), f"request {r}: {difference}"
    assert torch.isnan(state[[0, 2, 4]]).all() and torch.isfinite(state[[1, 3]]).all()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden", [200, 203, 4104])
def test_stream_operations(ops, dtype, hidden):
    generator = torch.Generator().manual_seed(3)
    tokens, vocab = 37, 50
    residual = torch.randn(tokens, hidden, generator=generator)
    delta = torch.randn(tokens, hidden, generator=generator).to(dtype)
    table = torch.randn(vocab, hidden, generator=generator).to(dtype)
    vector = torch.randn(hidden, generator=generator)
    ids = torch.randint(0, vocab, (tokens,), generator=generator, dtype=torch.int32)
    on = lambda t: t.to(DEVICE)
    got = on(residual.clone())
    ops.add_vectors(got, on(delta), on(ids), on(table), on(vector))
    want = residual.double() + delta.double() + table[ids.long()].double() + vector.double()
    assert (got.cpu().double() - want).abs().max() < 1e-5
    got = on(residual.clone())
    ops.add_vectors(got, None, on(ids), None, on(vector))
    assert (got.cpu().double() - (residual.double() + vector.double())).abs().max() < 1e-6
    # the mean of normed branches, in 32-bit
    a, b = (torch.randn(tokens, hidden, generator=generator) * s for s in (3.0, 0.01))
    a, b = a.to(dtype), b.to(dtype)
    wa, wb = torch.randn(hidden, generator=generator), torch.randn(hidden, generator=generator)
    got = on(residual.clone())
    ops.normed_mean_add(got, [on(a), on(b)], [on(wa), on(wb)], 1e-6)
    want = residual.double() + 0.5 * (rms(a.double(), 1e-6) * wa.double() + rms(b.double(), 1e-6) * wb.double())
    assert (got.cpu().double() - want).abs().max() < 2e-5
    # activations
    z = (3 * torch.randn(tokens, hidden, generator=generator)).to(dtype)
    for kind, plain in (("relu2", lambda x: torch.relu(x) ** 2), ("relu", torch.relu), ("silu", silu),
                        ("gelu_tanh", lambda x: 0.5 * x * (1 + torch.tanh(math.sqrt(2 / math.pi) * (x + 0.044715 * x ** 3))))):
        got = ops.activation(on(z), kind).cpu().double()
        want = plain(z.double())
        assert (got - want).abs().max() <= bound(dtype, 1e-5, 0.01 * float(want.abs().max())), kind


# ------------------------------------------------------------------ the engine


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_requests_and_first_tokens(folders, plain, name, dtype):
    config, _, page = CONFIGS[name]
    runner, cache = engine(folders[name], dtype, page, 256)
    for i, tokens in enumerate(prompts(config["vocab"], (1, 2, 3, 21, 100), seed=1)):
        got = replay(runner, cache, [([(i, tokens)], [i])])[i]
        assert_close(got, plain[name].logits(tokens), dtype, f"{name} whole request {i}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_prefill_against_token_by_token(folders, plain, name, dtype):
    """A prompt in one step and then 60 tokens decoded one by one; and the same request fed
    token by token from its first token on."""
    config, _, page = CONFIGS[name]
    runner, cache = engine(folders[name], dtype, page, 256)
    (tokens,) = prompts(config["vocab"], (101,), seed=3)
    want = plain[name].logits(tokens)
    steps = [([("r", tokens[:41])], [])] + [([("r", [t])], []) for t in tokens[41:]]
    steps[-1] = (steps[-1][0], ["r"])
    assert_close(replay(runner, cache, steps)["r"], want, dtype, f"{name} prompt then decode")
    steps = [([("s", [t])], []) for t in tokens[:50]]
    steps[-1] = (steps[-1][0], ["s"])
    assert_close(replay(runner, cache, steps)["s"], want[:50], dtype, f"{name} token by token")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_portions_of_changing_size(folders, plain, name, dtype):
    config, _, page = CONFIGS[name]
    runner, cache = engine(folders[name], dtype, page, 256)
    (tokens,) = prompts(config["vocab"], (131,), seed=4)
    want = plain[name].logits(tokens)
    for sizes in ((7, 2, 13, 3, 2, 5), (2,), (33, 1, 31), (64, 3)):
        steps = [([("r", part)], []) for part in cut(tokens, sizes)]
        steps[-1] = (steps[-1][0], ["r"])
        assert_close(replay(runner, cache, steps)["r"], want, dtype, f"{name} portions {sizes}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_mixed_batches_with_pages_and_slots_used_again(folders, plain, name, dtype):
    """Up to four live requests in a pool of four slots and few pages: portions of some beside
    decoded tokens of others, requests left out of steps, slots and pages of finished requests
    handed to later ones; every request must come out as it does alone."""
    config, _, page = CONFIGS[name]
    lengths = (40, 64, 23, 50, 17, 61, 9, 33, 2, 1)
    requests = dict(enumerate(prompts(config["vocab"], lengths, seed=5)))
    runner, cache = engine(folders[name], dtype, page, 4 * 64, max_requests=4)
    got = replay(runner, cache, mixed_schedule(requests))
    assert cache.stats().pages_low_water[0] < cache.stats().pages_total[0] // 2
    for request_id, tokens in requests.items():
        assert_close(got[request_id], plain[name].logits(tokens), dtype, f"{name} mixed request {request_id}")
    assert not cache.requests()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["G1", "G3"])
def test_steps_of_a_repeated_shape_are_replayed(folders, plain, name, dtype):
    """Pairs of requests whose steps have the same shape again and again: the later ones are
    replayed from CUDA graphs (other tokens, pages, slots and histories, fillers at the scratch
    slot) and must match the plain model like the first."""
    config, _, page = CONFIGS[name]
    runner, cache = engine(folders[name], dtype, page, 512)
    requests = dict(enumerate(prompts(config["vocab"], [42, 35] * 5, seed=9)))
    for pair in range(5):
        a, b = requests[2 * pair], requests[2 * pair + 1]
        first = (24, 17) if pair != 3 else (22, 19)
        steps = [([(2 * pair, a[:first[0]]), (2 * pair + 1, b[:first[1]])], []),
                 ([(2 * pair, a[first[0]:27]), (2 * pair + 1, b[first[1]:20])], [])]
        steps += [([(2 * pair, [a[27 + i]]), (2 * pair + 1, [b[20 + i]])], []) for i in range(15)]
        steps[-1] = (steps[-1][0], [2 * pair, 2 * pair + 1])
        got = replay(runner, cache, steps)
        assert_close(got[2 * pair], plain[name].logits(a), dtype, f"{name} pair {pair} a")
        assert_close(got[2 * pair + 1], plain[name].logits(b), dtype, f"{name} pair {pair} b")
    assert runner.use_graphs and runner.graph_replays >= 6


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_memory_and_a_long_prompt(tmp_path, dtype):
    """A model that forgets slowly, 700 tokens in portions that cut pages and convolutions, a
    decoded tail: the first tokens still move the last logits (the plain model says by how
    much), and the engine agrees with the plain model everywhere."""
    config, _, page = CONFIGS["G3"]
    folder = make_model_dir("G3", tmp_path, decay_bias=-7.0)
    model = PlainModel(folder)
    (tokens,) = prompts(config["vocab"], (700,), seed=21)
    want = model.logits(tokens)
    changed = list(tokens)
    changed[2] = (changed[2] + 1) % config["vocab"]
    moved = (model.logits(changed)[-1] - want[-1]).abs().max()
    runner, cache = engine(folder, dtype, page, 704, max_requests=2)
    sizes = [300, 129, 2, 200, 37] + [1] * 32
    assert sum(sizes) == len(tokens)
    steps, at = [], 0
    for size in sizes:
        steps.append(([("long", tokens[at:at + size])], []))
        at += size
    steps[-1] = (steps[-1][0], ["long"])
    got = replay(runner, cache, steps)["long"]
    assert_close(got, want, dtype, "long memory")
    if dtype == torch.float32:
        assert moved > 1e-2 and moved > 20 * (got[-1].cpu() - want[-1]).abs().max(), \
            "the first tokens no longer show at the end"


def test_greedy_generation_through_the_entry_point(folders, plain):
    from mlx_one_b200 import BatchingConfig, CacheConfig, Engine, TextGenerationOptions

    config, _, page = CONFIGS["G1"]
    engine_ = Engine(folders["G1"], execution_dtype="float32",
                     cache_config=CacheConfig(block_size_tokens=page, capacity_tokens=512),
                     batching_config=BatchingConfig(max_sequences=3, prefill_chunk_size=16))
    batch = prompts(config["vocab"], (7, 30, 3, 19, 12), seed=8)
    results = engine_.generate_batch_ids(batch, TextGenerationOptions(max_tokens=12, ignore_eos=True))
    for prompt, result in zip(batch, results):
        assert list(result.token_ids) == plain["G1"].greedy(prompt, 12)
    engine_.close()


def test_command_line_and_trace_replay(folders, plain, tmp_path):
    """`mlx-one generate` with token ids (greedy against the plain model, sampled with a seed) and
    `trace_run` as a process: steps on standard input, logits files out, requests ended and their
    slots used again."""
    import json
    import subprocess
    import sys
    from pathlib import Path

    import numpy as np

    root = Path(__file__).resolve().parent.parent
    folder = folders["G2"]
    run = lambda *args: subprocess.run([sys.executable, str(root / "bin" / "mlx-one"), *args],
                                       capture_output=True, text=True, timeout=600)
    greedy = run("generate", str(folder), "5 17 3 200", "--token-ids", "--max-tokens", "6",
                 "--dtype", "float32")
    assert greedy.returncode == 0, greedy.stderr
    assert [int(t) for t in greedy.stdout.split()] == plain["G2"].greedy([5, 17, 3, 200], 6)
    sampled = [run("generate", str(folder), "5 17 3", "--token-ids", "--max-tokens", "8",
                   "--temperature", "0.9", "--top-k", "30", "--seed", "11") for _ in range(2)]
    assert sampled[0].returncode == 0 and sampled[0].stdout == sampled[1].stdout
    assert len(sampled[0].stdout.split()) == 8

    vocab = CONFIGS["G2"][0]["vocab"]
    a, b, c = prompts(vocab, (21, 9, 30), seed=17)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:8], "want": [0, 7]},
                                     {"id": "b", "tokens": b, "want": [8]}], "end": ["b"]},
             {"step": 1, "entries": [{"id": "a", "tokens": a[8:20], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": a[20:], "want": [0]},
                                     {"id": "c", "tokens": c[:2], "want": [1]}], "end": ["a"]},
             {"step": 3, "entries": [{"id": "c", "tokens": c[2:], "want": [27]}], "end": ["c"]}]
    out = tmp_path / "logits"
    done = subprocess.run([sys.executable, str(root / "bin" / "trace_run"), "--model", str(folder),
                           "--dtype", "float32", "--out", str(out), "--max-tokens", "128",
                           "--max-requests", "2"],
                          input="".join(json.dumps(step) + "\n" for step in steps),
                          capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr
    assert [line for line in done.stdout.split("\n") if line.startswith("done")] == \
        [f"done {i}" for i in range(4)]
    read = lambda step, rows: torch.from_numpy(np.fromfile(out / f"{step}.f32", dtype="<f4")).view(rows, vocab)
    assert not (out / "1.f32").exists()
    wa, wb, wc = (plain["G2"].logits(t) for t in (a, b, c))
    assert_close(read(0, 3), torch.stack([wa[0], wa[7], wb[8]]), torch.float32, "step 0")
    assert_close(read(2, 2), torch.stack([wa[20], wc[1]]), torch.float32, "step 2")
    assert_close(read(3, 1), wc[29:30], torch.float32, "step 3")
