"""Farorax described in parts.

Every layer is a pre-norm block whose parts' outputs are multiplied by ``residual_mult`` before
they enter the 32-bit stream. The mixer of a layer is either grouped-query softmax attention
(no biases; rotary encoding of neighbouring pairs of the first dimensions of a head, with the
long-context rule for slow frequencies; a sliding window; a learned sink per head in the
softmax's denominator; keys and values of different sizes) or lightning attention (silu on
queries, keys and values; a 32-bit matrix state per head that decays by a constant per token;
the heads' outputs normed together and gated). The feed-forward is gated (gelu gate) or a
mixture of routed experts (sigmoid scores, groups of experts, a shared expert), or absent.

A run of layers may be executed several times with the same weights (``loop``): each pass has
cache entries of its own; before every pass the stream becomes ``loop.in`` applied to the
stream and the tokens' embeddings side by side, plus row t of ``loop.step`` (t the number of
the pass). The logits are soft-capped.

Stored names: ``embed``, ``head``, ``final.norm``, ``loop.in``, ``loop.step``, and per layer i
``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.{q,k,v,o}``, ``l<i>.mix.sink`` (attention),
``l<i>.mix.{g,norm}`` (lightning), ``l<i>.mlp.{gate,up,down}`` (dense) or ``l<i>.mlp.router``,
``l<i>.mlp.e<j>.{gate,up,down}``, ``l<i>.mlp.shared.{gate,up,down}`` (experts); matrices are
[out, in].
"""

from __future__ import annotations

from ..config.farorax import (AttentionMixer, DenseFeedForward, FaroraxConfig, LightningMixer,
                              RoutedFeedForward)
from ..config.registry import Architecture
from ..parts.spec import Injection, LayerCall, LayerSpec, ModelSpec, PartSpec, TensorSpec

LOOP_VECTORS = "loop.step"
LOOP_MATRIX = "loop.in"


def _attention(mixer: AttentionMixer, width: int) -> PartSpec:
    position = PartSpec("none")
    if mixer.rot is not None:
        scaling = mixer.rot.scaling
        position = PartSpec("rope_long", {
            "theta": mixer.rot.base, "rotary_dim": mixer.rot.dims, "layout": "neighbours",
            "factor": None if scaling is None else scaling.factor,
            "original": None if scaling is None else scaling.original,
            "low": None if scaling is None else scaling.low,
            "high": None if scaling is None else scaling.high})
    return PartSpec("attention", {
        "hidden": width, "heads": mixer.heads, "kv_heads": mixer.kv_heads, "head_dim": mixer.dim,
        "value_dim": mixer.vdim, "bias": False, "qk_norm_eps": None, "position": position,
        "scale": mixer.scale, "window": mixer.window, "sink": True,
    }, "mix.", {"q_proj.weight": "q", "k_proj.weight": "k", "v_proj.weight": "v",
                "out_proj.weight": "o"})


def _lightning(mixer: LightningMixer, width: int, eps: float) -> PartSpec:
    return PartSpec("lightning", {
        "hidden": width, "heads": mixer.heads, "key_dim": mixer.dim, "value_dim": mixer.vdim,
        "decay": mixer.decay, "eps": eps}, "mix.")


def _feed_forward(mlp, width: int) -> PartSpec:
    if isinstance(mlp, DenseFeedForward):
        return PartSpec("swiglu", {"hidden": width, "width": mlp.ff, "activation": "gelu_tanh"},
                        "mlp.", {"w1.weight": "gate", "w3.weight": "up", "w2.weight": "down"})
    assert isinstance(mlp, RoutedFeedForward)
    return PartSpec("routed", {
        "hidden": width, "width": mlp.ff, "experts": mlp.experts, "top": mlp.top,
        "groups": mlp.groups, "keep": mlp.keep, "shared_width": mlp.shared_ff,
        "activation": "silu", "scores": "sigmoid", "group_score": 2}, "mlp.")


def call_order(config: FaroraxConfig) -> tuple[LayerCall, ...]:
    """The layers in the order they run, a looped run unrolled, with what happens to the
    stream before each pass."""
    count, loop = len(config.layers), config.loop
    if loop is None:
        return tuple(LayerCall(index) for index in range(count))
    order = [LayerCall(index) for index in range(loop.start)]
    for turn in range(loop.times):
        for index in range(loop.start, loop.stop):
            inject = None
            if index == loop.start:
                inject = Injection(LOOP_VECTORS, turn, mix=LOOP_MATRIX)
            order.append(LayerCall(index, inject=inject))
    order += [LayerCall(index) for index in range(loop.stop, count)]
    return tuple(order)


def describe(config: FaroraxConfig) -> ModelSpec:
    width, eps = config.width, config.norm_eps
    norm = lambda name: PartSpec("rmsnorm", {"size": width, "eps": eps}, "", {"weight": name})
    layers = []
    for index, layer in enumerate(config.layers):
        if layer.type == "attention":
            mixer = _attention(layer.mixer, width)
        else:
            mixer = _lightning(layer.mixer, width, eps)
        feed_forward = feed_forward_norm = None
        if layer.mlp is not None:
            feed_forward = _feed_forward(layer.mlp, width)
            feed_forward_norm = norm("norm2")
        layers.append(LayerSpec(
            prefix=f"l{index}.",
            block=PartSpec("prenorm", {"residual_scale": config.residual_mult}), mixer=mixer,
            mixer_norm=norm("norm1"), feed_forward=feed_forward,
            feed_forward_norm=feed_forward_norm))
    vectors = {}
    if config.loop is not None:
        vectors[LOOP_VECTORS] = TensorSpec((config.loop.times, width))
        vectors[LOOP_MATRIX] = TensorSpec((width, 2 * width))
    return ModelSpec(
        architecture="farorax", vocab_size=config.vocab, hidden_size=width, embedding="embed",
        layers=tuple(layers), order=call_order(config), final_norm=norm("final.norm"),
        head="head", max_positions=1 << 30, vectors=vectors,
        logit_softcap=config.logit_softcap)


ARCHITECTURE = Architecture("farorax", FaroraxConfig, describe)
