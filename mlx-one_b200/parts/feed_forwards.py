"""Feed-forward parts."""

from __future__ import annotations

import torch

from .base import FeedForward
from .registry import FEED_FORWARDS
from .spec import TensorSpec


@FEED_FORWARDS.register("swiglu")
class SwiGLU(FeedForward):
    """w2(silu(w1 x) * w3 x), no biases. Parameters: ``hidden``, ``width``. The gate and
    up matrices are stacked at load time so that one matrix product feeds the gate kernel.
    Reference: src/mlx_one/models/language/lfm2/reference_math.py:114-135."""

    @classmethod
    def tensors(cls, spec):
        hidden, width = spec["hidden"], spec["width"]
        return {
            "w1.weight": TensorSpec((width, hidden)),
            "w3.weight": TensorSpec((width, hidden)),
            "w2.weight": TensorSpec((hidden, width)),
        }

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.width = spec["width"]
        self.gate_up = self.matrix(torch.cat([tensors["w1.weight"], tensors["w3.weight"]], dim=0))
        self.down = self.matrix(tensors["w2.weight"])

    fuses_residual = True
    accepts_normed_input = True

    def forward(self, x, ctx, residual=None):
        gated = self.ops.linear_swiglu(x, self.gate_up)
        if residual is None:
            return self.ops.linear(gated, self.down)
        return self.ops.linear_add(gated, self.down, None, residual)


@FEED_FORWARDS.register("dense")
class DenseFeedForward(FeedForward):
    """down(act(up x)), no gate, no biases. Parameters: ``hidden``, ``width``, ``activation``:
    ``relu2`` (the square of max(z, 0)), ``gelu_tanh`` (0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715
    z^3)))), ``silu`` or ``relu``. The activation is the up product's epilogue where the kernels
    have one."""

    ACTIVATIONS = ("relu2", "gelu_tanh", "silu", "relu")

    @classmethod
    def tensors(cls, spec):
        hidden, width = spec["hidden"], spec["width"]
        return {"up.weight": TensorSpec((width, hidden)),
                "down.weight": TensorSpec((hidden, width))}

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.activation = spec.get("activation", "relu2")
        if self.activation not in self.ACTIVATIONS:
            raise ValueError(f"unknown activation {self.activation!r}")
        self.up = self.matrix(tensors["up.weight"])
        self.down = self.matrix(tensors["down.weight"])

    fuses_residual = True
    accepts_normed_input = True

    def forward(self, x, ctx, residual=None):
        hidden = self.ops.linear_act(x, self.up, self.activation)
        if residual is None:
            return self.ops.linear(hidden, self.down)
        return self.ops.linear_add(hidden, self.down, None, residual)
