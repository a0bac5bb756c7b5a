"""Galarax described in parts.

Every layer is a pre-norm block (norm weights stored around zero) whose mixer runs two mixers
side by side on the same input: grouped-query softmax attention (biased projections, rotary
encoding of the first dimensions of a head with stretched frequencies, queries and keys divided
by their root mean square after the rotation, a score scale of the configuration's) and a gated
delta rule (short convolutions, unit-length queries and keys, a 32-bit matrix state per head).
Each branch's output is normed over the model width and the two are averaged. The feed-forward,
where a layer has one, is down(relu(up x)^2).

A run of layers may be executed several times with the same weights (``loop``): each pass has
cache entries of its own; before every pass but the first the tokens' embeddings are added to
the stream again, and before every pass row t of ``loop.step`` is (t the number of the pass).

Stored names: ``embed``, ``head``, ``final.norm``, ``loop.step``, and per layer i ``l<i>.norm1``,
``l<i>.norm2``, ``l<i>.mix.left.{q,k,v}`` (+ ``.b``), ``l<i>.mix.left.o``, ``l<i>.mix.right.{q,k,v}``
(+ ``.conv``), ``l<i>.mix.right.{b,a,A_log,dt_bias,norm,g,o}``, ``l<i>.mix.{left,right}.out``,
``l<i>.mlp.{up,down}``; matrices are [out, in].
"""

from __future__ import annotations

from ..config.galarax import GalaraxConfig, GalaraxLayer
from ..config.registry import Architecture
from ..parts.spec import Injection, LayerCall, LayerSpec, ModelSpec, PartSpec, TensorSpec

LOOP_VECTORS = "loop.step"


def _left(layer: GalaraxLayer, width: int, eps: float) -> PartSpec:
    left = layer.left
    position = PartSpec("none")
    if left.rot is not None:
        scaling = left.rot.scaling
        position = PartSpec("yarn", {
            "theta": left.rot.base, "rotary_dim": left.rot.dims,
            "factor": None if scaling is None else scaling.factor,
            "original": None if scaling is None else scaling.original,
            "fast": None if scaling is None else scaling.fast,
            "slow": None if scaling is None else scaling.slow})
    return PartSpec("attention", {
        "hidden": width, "heads": left.heads, "kv_heads": left.kv_heads, "head_dim": left.dim,
        "value_dim": left.vdim, "bias": True, "qk_norm_eps": eps, "qk_norm": "plain_after",
        "position": position, "scale": left.scale, "window": None,
    }, "left.", {"q_proj.weight": "q", "q_proj.bias": "q.b", "k_proj.weight": "k",
                 "k_proj.bias": "k.b", "v_proj.weight": "v", "v_proj.bias": "v.b",
                 "out_proj.weight": "o"})


def _right(layer: GalaraxLayer, width: int, eps: float) -> PartSpec:
    right = layer.right
    return PartSpec("gated_delta", {
        "hidden": width, "heads": right.heads, "kv_heads": right.kv_heads,
        "key_dim": right.dim, "value_dim": right.vdim, "taps": right.conv, "eps": eps}, "right.")


def call_order(config: GalaraxConfig) -> tuple[LayerCall, ...]:
    """The layers in the order they run, a looped run unrolled, with what enters the stream
    before each pass."""
    count, loop = len(config.layers), config.loop
    if loop is None:
        return tuple(LayerCall(index) for index in range(count))
    order = [LayerCall(index) for index in range(loop.start)]
    for turn in range(loop.times):
        for index in range(loop.start, loop.stop):
            inject = None
            if index == loop.start:
                inject = Injection(LOOP_VECTORS, turn, embedding=turn > 0)
            order.append(LayerCall(index, inject=inject))
    order += [LayerCall(index) for index in range(loop.stop, count)]
    return tuple(order)


def describe(config: GalaraxConfig) -> ModelSpec:
    width, eps = config.width, config.norm_eps
    norm = lambda name: PartSpec("rmsnorm", {"size": width, "eps": eps, "offset": 1.0}, "",
                                 {"weight": name})
    layers = []
    for index, layer in enumerate(config.layers):
        mixer = PartSpec("parallel", {"hidden": width, "eps": eps, "branches": (
            ("left", _left(layer, width, eps), "left.out"),
            ("right", _right(layer, width, eps), "right.out"))}, "mix.")
        feed_forward = feed_forward_norm = None
        if layer.ff is not None:
            feed_forward = PartSpec("dense", {"hidden": width, "width": layer.ff,
                                              "activation": "relu2"}, "mlp.",
                                    {"up.weight": "up", "down.weight": "down"})
            feed_forward_norm = norm("norm2")
        layers.append(LayerSpec(prefix=f"l{index}.", block=PartSpec("prenorm"), mixer=mixer,
                                mixer_norm=norm("norm1"), feed_forward=feed_forward,
                                feed_forward_norm=feed_forward_norm))
    vectors = {}
    if config.loop is not None:
        vectors[LOOP_VECTORS] = TensorSpec((config.loop.times, width))
    return ModelSpec(
        architecture="galarax", vocab_size=config.vocab, hidden_size=width, embedding="embed",
        layers=tuple(layers), order=call_order(config), final_norm=norm("final.norm"),
        head="head", max_positions=1 << 30, vectors=vectors)


ARCHITECTURE = Architecture("galarax", GalaraxConfig, describe)
