"""Farorax on the GPU against the plain implementation: each new mechanism alone, then the
engine over whole requests, decoded tails, portions down to two tokens, mixed batches with
pages and slots used again, keys at the edges of windows and far away, long decoding, replayed
graphs, and greedy generation through the entry point."""

import math

import pytest
import torch

from farorax_models import (CONFIGS, F1, assert_rows_close as assert_close, attention, dense,
                            lightning, make_model_dir, sliced)
from plain_farorax import (PlainModel, decayed_outer_product_state, gelu_tanh, pair_frequencies,
                           rms_norm, rotate_neighbours, routing, silu, windowed_attention_with_sink)
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
    root = tmp_path_factory.mktemp("farorax")
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


def context(portions, histories, leading_single=0):
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
                       max_portion=max(portions), max_context=max(p + h for p, h in zip(portions, histories)),
                       leading_single=leading_single)


def on(tensor):
    return tensor.to(DEVICE)


# ------------------------------------------------------------------ attention alone


def paged(keys, values, page, dtype, generator):
    """One request's keys and values [T, G, D] in pages handed out in a random order; what no
    token has written holds large numbers (a key or value read from there would show)."""
    T, G, D = keys.shape
    blocks = -(-T // page)
    pages = blocks + 3
    order = torch.randperm(pages - 1, generator=generator)[:blocks]
    kv = torch.full((2, pages, G, page, D), 100.0).to(dtype)
    for t in range(T):
        kv[0, order[t // page], :, t % page] = keys[t].to(dtype)
        kv[1, order[t // page], :, t % page] = values[t].to(dtype)
    return kv, order.to(torch.int32)[None, :].contiguous()


def edge_case(T, heads, kv_heads, dim, window, generator):
    """Queries, keys and values of one sequence in which, for the last queries, the key just
    outside the window matches the query of head 0 best by far, and the key just inside the
    window matches head 1 (of the same key head, where there are two): a window that is one
    token off shows as a wholly different output. Values are small but for those keys'."""
    q = 0.3 * torch.randn(T, heads, dim, generator=generator)
    k = 0.3 * torch.randn(T, kv_heads, dim, generator=generator)
    v = 0.1 * torch.randn(T, kv_heads, dim, generator=generator)
    second = 1 if heads // kv_heads > 1 else None
    for i in range(max(window, 1), T):
        if i % 3:
            continue
        outside, inside = i - window, i - window + 1
        # head 0 of query i points at key `outside`, head 1 at key `inside`
        k[outside, 0] = 0.05 * torch.randn(dim, generator=generator)
        k[outside, 0, 0] = 6.0
        q[i, 0, 0] = 8.0
        v[outside, 0] = 3.0
        if second is not None and inside != outside and inside < i:
            k[inside, 0, 1] = 6.0
            q[i, second, 1] = 8.0
            v[inside, 0] = -2.0
    return q, k, v


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, kv_heads, dim, window, page, T", [
    (4, 2, 32, 24, 4, 90), (6, 2, 96, 33, 16, 150), (3, 3, 40, 7, 8, 40), (8, 1, 64, 100, 16, 330),
    (2, 1, 16, 1, 2, 12), (4, 4, 128, 64, 8, 200), (10, 1, 48, 500, 16, 700)])
def test_window_edges_and_sinks_in_prompts_and_decoding(ops, dtype, heads, kv_heads, dim, window,
                                                        page, T):
    """softmax over the window with a sink per head: whole prompts, a prompt's second portion,
    and single tokens (several key splits where the window is long), against the plain function.
    The key just outside every third query's window would take all the weight if it were seen."""
    from mlx_one_b200.parts import PagedKeyValues, PagedView

    generator = torch.Generator().manual_seed(heads * 1000 + dim + window)
    q, k, v = edge_case(T, heads, kv_heads, dim, window, generator)
    sinks = 1.5 * torch.randn(heads, generator=generator)
    scale = 0.7 / math.sqrt(dim)
    round_trip = lambda x: x.to(dtype).double()
    want = windowed_attention_with_sink(round_trip(q), round_trip(k), round_trip(v), scale, window,
                                        sinks.double()).reshape(T, -1)
    kv, table = paged(k, v, page, dtype, generator)
    view = PagedView(on(kv), on(table), page, PagedKeyValues(kv_heads, dim, window))
    call = lambda queries, ctx: ops.paged_attention(
        on(queries.to(dtype)).contiguous(), heads=heads, kv_heads=kv_heads, head_dim=dim,
        scale=scale, window=window, ctx=ctx, view=view, sinks=on(sinks)).cpu().double()
    tolerance = 1e-4 if dtype == torch.float32 else 0.05
    # the whole prompt; its second part after the first; every token of the tail alone
    got = call(q, context([T], [0]))
    assert (got - want).abs().max() < tolerance, "whole prompt"
    half = T // 2 + 1
    got = call(q[half:], context([T - half], [half]))
    assert (got - want[half:]).abs().max() < tolerance, "second portion"
    for position in list(range(max(T - 40, 0), T)) + [0, min(window, T - 1)]:
        got = call(q[position:position + 1], context([1], [position]))
        assert (got - want[position]).abs().max() < tolerance, f"single token at {position}"
    ops.check_errors()
    # the sink takes its share: without it the output is another
    without = windowed_attention_with_sink(round_trip(q), round_trip(k), round_trip(v), scale,
                                           window, torch.full((heads,), -1e9).double()).reshape(T, -1)
    assert (without - want).abs().max() > 0.1


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_far_key_among_hundreds_without_a_window(ops, dtype):
    """No window: the last queries match one key near the start of 900; several requests decode
    side by side (key splits merged by clusters and by the merge kernel), the sink counted once."""
    from mlx_one_b200.parts import PagedKeyValues, PagedView

    heads, kv_heads, dim, page, T = 8, 2, 64, 16, 900
    generator = torch.Generator().manual_seed(5)
    q = 0.3 * torch.randn(T, heads, dim, generator=generator)
    k = 0.3 * torch.randn(T, kv_heads, dim, generator=generator)
    v = 0.1 * torch.randn(T, kv_heads, dim, generator=generator)
    k[3, :, 5], v[3] = 6.0, 2.0
    q[-30:, :, 5] = 8.0
    sinks = torch.linspace(-2, 6, heads)
    scale = 0.125
    round_trip = lambda x: x.to(dtype).double()
    want = windowed_attention_with_sink(round_trip(q), round_trip(k), round_trip(v), scale, T,
                                        sinks.double()).reshape(T, -1)
    assert want[-1].abs().max() > 0.5                     # the far key is what the output is
    kv, table = paged(k, v, page, dtype, generator)
    tolerance = 1e-4 if dtype == torch.float32 else 0.05
    for batch in (1, 3, 30):
        positions = [T - 1 - i for i in range(batch)]
        tables = on(table.repeat(batch, 1).contiguous())
        view = PagedView(on(kv), tables, page, PagedKeyValues(kv_heads, dim, None))
        got = ops.paged_attention(on(q[positions].to(dtype)).contiguous(), heads=heads,
                                  kv_heads=kv_heads, head_dim=dim, scale=scale, window=None,
                                  ctx=context([1] * batch, positions), view=view,
                                  sinks=on(sinks)).cpu().double()
        assert (got - want[positions]).abs().max() < tolerance, f"{batch} requests"
    ops.check_errors()


def test_neighbour_pairs_and_the_long_context_rule(ops):
    """The frequencies of the encoding against the plain rule, and the reordering of rows that
    turns pairs of neighbours into pairs of halves: scores stay what they are."""
    from mlx_one_b200.parts import POSITIONS, PartSpec, Runtime

    for rot in ({"base": 10000.0, "dims": 32, "scaling": {"factor": 8.0, "low": 1.0, "high": 3.0,
                                                         "original": 64}},
                {"base": 300.0, "dims": 6, "scaling": {"factor": 2.0, "low": 0.5, "high": 6.0,
                                                       "original": 40}},
                {"base": 1000.0, "dims": 8}):
        scaling = rot.get("scaling") or {}
        spec = PartSpec("rope_long", {"theta": rot["base"], "rotary_dim": rot["dims"],
                                      "layout": "neighbours", "factor": scaling.get("factor"),
                                      "original": scaling.get("original"), "low": scaling.get("low"),
                                      "high": scaling.get("high")})
        encoding = POSITIONS.get("rope_long")(spec, {}, Runtime(torch.float32, torch.device(DEVICE), ops))
        freq, dims = encoding.rotary_table()
        want = pair_frequencies(rot, torch.float64)
        assert dims == rot["dims"] and torch.allclose(freq.cpu().double(), want, rtol=1e-6, atol=0)
        if "scaling" in rot:
            plain = torch.tensor([rot["base"] ** (-2.0 * i / dims) for i in range(dims // 2)])
            ratio = want / plain.double()
            assert ratio.max() > 0.999 and ratio.min() < 1.001 / scaling["factor"] \
                and ((ratio > 1.01 / scaling["factor"]) & (ratio < 0.99)).any(), "all three regimes"
        head = dims + 4
        order = encoding.row_order(head)
        assert sorted(order.tolist()) == list(range(head))
        generator = torch.Generator().manual_seed(dims)
        x = torch.randn(5, 2, head, generator=generator, dtype=torch.float64)
        positions = torch.tensor([0, 1, 17, 300, 4000])
        turned = rotate_neighbours(x, positions, rot)
        # the same rotation on reordered rows, pairs (i, i + dims / 2)
        y = x[..., order]
        angle = positions.double()[:, None] * want[None, :]
        cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
        a, b = y[..., :dims // 2], y[..., dims // 2:dims]
        halves = torch.cat([a * cos - b * sin, b * cos + a * sin, y[..., dims:]], -1)
        assert torch.allclose(halves, turned[..., order], atol=1e-12)


# ------------------------------------------------------------------ lightning attention alone


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, key_dim, value_dim, decay", [
    (2, 16, 24, (0.9, 0.5)), (3, 40, 8, (1.0, 0.999, 0.0)), (4, 128, 32, (0.95, 0.9, 0.99, 0.7)),
    (1, 4, 4, (0.5,)), (2, 136, 20, (0.999, 0.9)), (2, 96, 130, (0.97, 0.8)), (1, 256, 64, (0.99,))])
def test_lightning_attention_in_portions(ops, dtype, heads, key_dim, value_dim, decay):
    """Two requests side by side whose tokens come in portions of 1 to 300 tokens (long ones are
    cut into segments that run side by side), on slots between slots full of NaN: outputs and
    the state carried from step to step against the plain recurrence."""
    from mlx_one_b200.parts import FixedState, StateView

    generator = torch.Generator().manual_seed(key_dim * 7 + value_dim)
    qk, inner = heads * key_dim, heads * value_dim
    lengths = (437, 390)
    eps = 1e-5
    projected = [torch.randn(n, 2 * qk + 2 * inner, generator=generator).to(dtype) for n in lengths]
    weight = 1 + 0.2 * torch.randn(inner, generator=generator)
    want = []
    for x in projected:
        x = x.double()
        n = x.shape[0]
        o = decayed_outer_product_state(silu(x[:, :qk]).view(n, heads, key_dim),
                                        silu(x[:, qk:2 * qk]).view(n, heads, key_dim),
                                        silu(x[:, 2 * qk:2 * qk + inner]).view(n, heads, value_dim),
                                        torch.tensor(decay, dtype=torch.float64))
        want.append(rms_norm(o.reshape(n, inner), weight.double(), eps)
                    * torch.sigmoid(x[:, 2 * qk + inner:]))
    state = torch.full((5, heads * key_dim * value_dim), float("nan"), device=DEVICE)
    slots = torch.tensor([3, 1], dtype=torch.int32, device=DEVICE)
    state[3] = 0
    state[1] = 0
    view = StateView(state, slots, FixedState((heads * key_dim * value_dim,), "float32"))
    portions = [(1, 2), (5, 1), (130, 64), (1, 1), (300, 200), (0, 122)]
    at = [0, 0]
    tolerance = 2e-4 if dtype == torch.float32 else 0.03
    for sizes in portions:
        live = [r for r in (0, 1) if sizes[r]]
        rows = torch.cat([projected[r][at[r]:at[r] + sizes[r]] for r in live])
        ctx = context([sizes[r] for r in live], [at[r] for r in live])
        step_view = StateView(state, slots[live].contiguous(), view.need)
        got = ops.lightning_attention(on(rows), decay=on(torch.tensor(decay, dtype=torch.float32)),
                                      norm_weight=on(weight), eps=eps, ctx=ctx, view=step_view,
                                      write=True, heads=heads, key_dim=key_dim,
                                      value_dim=value_dim).cpu().double()
        expect = torch.cat([want[r][at[r]:at[r] + sizes[r]] for r in live])
        assert (got - expect).abs().max() < tolerance, f"portions {sizes} after {at}"
        for r in live:
            at[r] += sizes[r]
    assert at == [437, 390] and torch.isnan(state[[0, 2, 4]]).all()
    ops.check_errors()


# ------------------------------------------------------------------ routing alone


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("experts, top, groups, keep", [(6, 2, 3, 2), (4, 1, 1, 1), (8, 3, 4, 2),
                                                        (5, 2, 1, 1), (64, 6, 8, 3), (12, 12, 3, 3),
                                                        (9, 2, 9, 4), (130, 4, 2, 1)])
def test_routing_weights(ops, dtype, experts, top, groups, keep):
    hidden, tokens = 72, 50
    generator = torch.Generator().manual_seed(experts)
    x = torch.randn(tokens, hidden, generator=generator).to(dtype)
    router = (3 * torch.randn(experts, hidden, generator=generator) / hidden ** 0.5).to(torch.bfloat16)
    margins = []
    want = routing(x.double(), router.double(), experts, top, groups, keep, margins)
    got = ops.route_experts(on(x), on(router.float()), experts=experts, top=top, groups=groups,
                            keep=keep, group_score=2).cpu().double()
    clear = margins[0] > 1e-4
    assert clear.float().mean() > 0.9
    assert (got[clear] - want[clear]).abs().max() < 1e-5
    assert ((got > 0).sum(-1) == top).all() and (got.sum(-1) - 1).abs().max() < 1e-5


@pytest.mark.parametrize("dtype", DTYPES)
def test_experts_as_columns_of_one_product(ops, dtype):
    """The routing weights multiplied into the experts' columns; the shared expert's stay."""
    generator = torch.Generator().manual_seed(3)
    tokens, experts, width, shared = 9, 5, 20, 24
    gated = torch.randn(tokens, experts * width + shared, generator=generator).to(dtype)
    weights = torch.rand(tokens, experts, generator=generator)
    weights[weights < 0.5] = 0
    got = on(gated.clone())
    ops.scale_expert_columns(got, on(weights), width)
    want = gated.double().clone()
    want[:, :experts * width] = (want[:, :experts * width].view(tokens, experts, width)
                                 * weights.double()[:, :, None]).view(tokens, -1)
    assert (got.cpu().double() - want).abs().max() <= (1e-6 if dtype == torch.float32 else 0.02)
    assert torch.equal(got.cpu()[:, experts * width:], gated[:, experts * width:])


@pytest.mark.parametrize("tokens, hidden, experts, width, top, shared", [
    (300, 128, 6, 72, 2, 40), (1000, 256, 8, 256, 3, None), (129, 64, 16, 8, 1, 8),
    (2048, 192, 4, 136, 3, 136), (1, 128, 8, 64, 2, 64), (3, 256, 64, 32, 6, None)])
def test_experts_over_sorted_tokens(ops, tokens, hidden, experts, width, top, shared):
    """Large steps in bfloat16, and steps so small that they use few of the experts: tokens sorted
    by expert and one grouped product per matrix over the stacked weights, against every expert
    applied to its tokens one by one. Some experts get no token at all, others more than a tile."""
    generator = torch.Generator().manual_seed(tokens + experts)
    x = torch.randn(tokens, hidden, generator=generator).bfloat16()
    stack = experts * width + (shared or 0)
    gate_up = (torch.randn(2 * stack, hidden, generator=generator) / hidden ** 0.5).bfloat16()
    down = (torch.randn(hidden, stack, generator=generator) / width ** 0.5).bfloat16()
    weights = torch.zeros(tokens, experts)
    busy = max(experts - 2, top)                          # the last experts are never chosen
    for t in range(tokens):
        chosen = torch.randperm(busy, generator=generator)[:top]
        weights[t, chosen] = torch.rand(top, generator=generator) + 0.1
    assert ops.sorts_experts(on(x), experts=experts, width=width, top=top, stack=stack)
    extra = {}
    if shared:
        at = experts * width
        extra = dict(shared_gate_up=on(torch.cat([gate_up[at:at + shared],
                                                  gate_up[stack + at:stack + at + shared]])),
                     shared_down=on(down[:, at:].contiguous()))
    got = ops.routed_experts_sorted(on(x), on(weights), on(gate_up), on(down), experts=experts,
                                    width=width, top=top, **extra).cpu().double()
    ops.check_errors()
    both = x.double() @ gate_up.double().T
    gated = (silu(both[:, :stack]) * both[:, stack:]).bfloat16().double()
    scale = torch.ones(tokens, stack, dtype=torch.float64)
    scale[:, :experts * width] = weights.double().repeat_interleave(width, dim=1)
    want = (gated * scale) @ down.double().T
    assert (got - want).abs().max() < 0.03 * want.abs().max()


# ------------------------------------------------------------------ the stream's operations


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tokens, hidden", [(1, 72), (5, 64), (40, 192), (1600, 128)])
def test_stream_operations_with_a_factor(ops, dtype, tokens, hidden):
    generator = torch.Generator().manual_seed(tokens)
    vocab, m = 50, 0.4
    residual = torch.randn(tokens, hidden, generator=generator)
    delta = torch.randn(tokens, hidden, generator=generator).to(dtype)
    table = torch.randn(vocab, hidden, generator=generator).to(dtype)
    weight = 1 + 0.2 * torch.randn(hidden, generator=generator)
    ids = torch.randint(0, vocab, (tokens,), generator=generator, dtype=torch.int32)
    loose = 1e-5 if dtype == torch.float32 else 0.03
    # add + norm with a factor on what is added
    stream = on(residual.clone())
    got = ops.add_rmsnorm(stream, on(delta), on(weight), 1e-5, dtype, delta_scale=m)
    summed = residual.double() + m * delta.double()
    assert (stream.cpu().double() - summed).abs().max() < 1e-6
    assert (got.cpu().double() - rms_norm(summed, weight.double(), 1e-5)).abs().max() < loose
    # vectors with a factor on the pending output
    stream = on(residual.clone())
    ops.add_vectors(stream, on(delta), on(ids), None, on(weight), delta_scale=m)
    assert (stream.cpu().double() - (summed + weight.double())).abs().max() < 1e-6
    # the stream beside the embeddings
    both = ops.concat_stream(on(residual), on(delta), on(ids), on(table), dtype, delta_scale=m)
    assert (both[:, :hidden].cpu().double() - summed).abs().max() < loose
    assert torch.equal(both[:, hidden:].cpu(), table[ids.long()])
    both = ops.concat_stream(on(residual), None, on(ids), on(table), dtype)
    assert (both[:, :hidden].cpu().double() - residual.double()).abs().max() < loose
    # the soft cap
    logits = 40 * torch.randn(tokens, 33, generator=generator)
    got = on(logits.clone())
    ops.softcap(got, 15.0)
    assert (got.cpu().double() - 15 * torch.tanh(logits.double() / 15)).abs().max() < 1e-5
    # a gate of another activation, and a product added into the stream with a factor
    if hidden % 8 == 0 and tokens <= 40:
        a = torch.randn(tokens, hidden, generator=generator).to(dtype)
        gate_up = (torch.randn(2 * 48, hidden, generator=generator) / hidden ** 0.5).to(dtype)
        got = ops.linear_gated(on(a), on(gate_up), "gelu_tanh").cpu().double()
        both = a.double() @ gate_up.double().T
        want = gelu_tanh(both[:, :48]) * both[:, 48:]
        assert (got - want).abs().max() < (1e-5 if dtype == torch.float32 else 0.06)
        down = (torch.randn(hidden, hidden, generator=generator) / hidden ** 0.5).to(dtype)
        stream = on(residual.clone())
        pending = ops.linear_add(on(a), on(down), None, stream, scale=m)
        total = stream.cpu().double() + (0 if pending is None else m * pending.cpu().double())
        assert (total - (residual.double() + m * (a.double() @ down.double().T))).abs().max() < loose


# ------------------------------------------------------------------ the engine


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_requests_and_first_tokens(folders, plain, name, dtype):
    config, _, page = CONFIGS[name]
    runner, cache = engine(folders[name], dtype, page, 256)
    for i, tokens in enumerate(prompts(config["vocab"], (1, 2, 3, 21, 150), seed=1)):
        got = replay(runner, cache, [([(i, tokens)], [i])])[i]
        assert_close(got, plain[name].logits(tokens), dtype, f"{name} whole request {i}")


def test_the_stream_after_every_layer(folders, plain):
    """The 32-bit engine's stream after each call of a layer (a looped layer counts each time)
    against the plain model's."""
    runner, cache = engine(folders["F1"], torch.float32, 4, 64)
    (tokens,) = prompts(F1["vocab"], (19,), seed=2)
    seen = []
    model = runner.model

    def watch(place, residual, delta):
        if place < 0:
            return
        scale = model.layers[model.order[place].layer].pending_scale
        # (a step's rows may be followed by fillers that round its shape up)
        seen.append((residual if delta is None else residual + scale * delta.float())[:len(tokens)].cpu())
    model.observer = watch
    replay(runner, cache, [([("r", tokens)], ["r"])])
    model.observer = None
    states = []
    plain["F1"].logits(tokens, states)
    assert len(seen) == len(states) == 5
    for place, (got, want) in enumerate(zip(seen, states)):
        assert (got.double() - want).abs().max() < 1e-4, f"after call {place}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_prefill_against_token_by_token(folders, plain, name, dtype):
    """A prompt in one step and then 60 tokens decoded one by one (the windows pass over decoded
    tokens); and the same request fed token by token from its first token on."""
    config, _, page = CONFIGS[name]
    runner, cache = engine(folders[name], dtype, page, 256)
    (tokens,) = prompts(config["vocab"], (101,), seed=3)
    want = plain[name].logits(tokens)
    steps = [([("r", tokens[:41])], [])] + [([("r", [t])], []) for t in tokens[41:]]
    steps[-1] = (steps[-1][0], ["r"])
    assert_close(replay(runner, cache, steps)["r"], want, dtype, f"{name} prompt then decode")
    steps = [([("s", [t])], []) for t in tokens[:50]]
    steps[-1] = (steps[-1][0], ["s"])
    assert_close(replay(runner, cache, steps)["s"], sliced(want, 50), dtype, f"{name} token by token")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_portions_of_changing_size(folders, plain, name, dtype):
    config, _, page = CONFIGS[name]
    runner, cache = engine(folders[name], dtype, page, 512)
    (tokens,) = prompts(config["vocab"], (331,), seed=4)
    want = plain[name].logits(tokens)
    for sizes in ((7, 2, 13, 3, 2, 5), (2,), (33, 1, 31), (64, 3), (200, 129, 2)):
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
    for request_id, tokens in requests.items():
        assert_close(got[request_id], plain[name].logits(tokens), dtype, f"{name} mixed request {request_id}")
    assert not cache.requests()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["F1", "F3"])
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
def test_long_decoding_with_long_memory(tmp_path, dtype):
    """A model whose lightning heads hardly forget and whose window is longer than a few pages:
    a prompt in portions that cut pages and segments, then 200 tokens decoded one by one. The
    third token still moves the last logits (the plain model says by how much), and the engine
    agrees with the plain model everywhere."""
    config = {"architecture": "Farorax", "vocab": 200, "width": 64, "norm": {"eps": 1e-5},
              "residual_mult": 0.6, "logit_softcap": 25.0,
              "layers": [lightning(2, 32, 32, (1.0, 0.9995), dense(128)),
                         attention(4, 2, 32, 32, 0.2, 150, {"base": 10000.0, "dims": 32}, dense(128)),
                         lightning(2, 32, 32, (0.999, 0.99), None)],
              "loop": {"start": 0, "stop": 3, "times": 2}}
    folder = make_model_dir("F1", tmp_path, config)
    model = PlainModel(folder)
    (tokens,) = prompts(config["vocab"], (700,), seed=21)
    want = model.logits(tokens)
    changed = list(tokens)
    changed[2] = (changed[2] + 1) % config["vocab"]
    moved = (model.logits(changed)[-1] - want[-1]).abs().max()
    runner, cache = engine(folder, dtype, 16, 704, max_requests=2)
    sizes = [269, 129, 2, 63, 37] + [1] * 200
    assert sum(sizes) == len(tokens)
    steps, at = [], 0
    for size in sizes:
        steps.append(([("long", tokens[at:at + size])], []))
        at += size
    steps[-1] = (steps[-1][0], ["long"])
    got = replay(runner, cache, steps)["long"]
    assert_close(got, want, dtype, "long memory")
    if dtype == torch.float32:
        assert moved > 1e-3 and moved > 20 * (got[-1].cpu() - want[-1]).abs().max(), \
            "the first tokens no longer show at the end"


def test_greedy_generation_through_the_entry_point(folders, plain):
    from mlx_one_b200 import BatchingConfig, CacheConfig, Engine, TextGenerationOptions

    config, _, page = CONFIGS["F1"]
    engine_ = Engine(folders["F1"], execution_dtype="float32",
                     cache_config=CacheConfig(block_size_tokens=page, capacity_tokens=512),
                     batching_config=BatchingConfig(max_sequences=3, prefill_chunk_size=16))
    batch = prompts(config["vocab"], (7, 30, 3, 19, 12), seed=8)
    results = engine_.generate_batch_ids(batch, TextGenerationOptions(max_tokens=12, ignore_eos=True))
    for prompt, result in zip(batch, results):
        assert list(result.token_ids) == plain["F1"].greedy(prompt, 12)
    engine_.close()


def test_command_line_and_trace_replay(folders, plain, tmp_path):
    """`mlx-one generate` with token ids (greedy against the plain model) and `trace_run` as a
    process: steps on standard input, logits files out, requests ended and their slots used
    again."""
    import json
    import subprocess
    import sys
    from pathlib import Path

    import numpy as np

    root = Path(__file__).resolve().parent.parent
    folder = folders["F2"]
    run = lambda *args: subprocess.run([sys.executable, str(root / "bin" / "mlx-one"), *args],
                                       capture_output=True, text=True, timeout=600)
    greedy = run("generate", str(folder), "5 17 3 200", "--token-ids", "--max-tokens", "6",
                 "--dtype", "float32")
    assert greedy.returncode == 0, greedy.stderr
    assert [int(t) for t in greedy.stdout.split()] == plain["F2"].greedy([5, 17, 3, 200], 6)

    vocab = CONFIGS["F2"][0]["vocab"]
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
    wa, wb, wc = (plain["F2"].logits(t) for t in (a, b, c))
    close = lambda got, want: (got - want).abs().max() < 2e-4
    assert close(read(0, 3), torch.stack([wa[0], wa[7], wb[8]]))
    assert close(read(2, 2), torch.stack([wa[20], wc[1]]))
    assert close(read(3, 1), wc[29:30])
