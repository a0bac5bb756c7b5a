"""Arrangements of a layer's parts."""

from __future__ import annotations

from .base import Block
from .registry import BLOCKS


@BLOCKS.register("prenorm")
class PreNormBlock(Block):
    """h = x + mixer(norm(x)); out = h + feed_forward(norm(h)). Each residual add is fused
    with the norm that follows it, so the block returns its last output unadded; a part that
    ``fuses_residual`` may instead add its output into the stream itself and return None.
    A layer without a feed-forward ends after the mixer. Parameter ``residual_scale`` (1): the
    factor m in h = x + m mixer(norm(x)); out = h + m feed_forward(norm(h)). The factor is
    applied where the output is added: by the part itself if it adds into the stream and
    ``scales_residual``, else by the norm that follows (``delta_scale``).
    Reference: src/mlx_one/models/language/lfm2/reference_math.py:160-179."""

    def __init__(self, spec, tensors, runtime, **roles):
        super().__init__(spec, tensors, runtime, **roles)
        self.scale = float(spec.get("residual_scale", 1.0))
        self.pending_scale = self.scale
        for part in (self.mixer, self.feed_forward):
            if part is not None:
                part.residual_scale = self.scale

    @staticmethod
    def _norm(norm, residual, delta, consumer, scale=1.0):
        extra = {} if scale == 1.0 else {"delta_scale": scale}
        if consumer.accepts_normed_input and norm.supports_lazy:
            return norm.forward(residual, delta, lazy=True, **extra)
        return norm.forward(residual, delta, **extra)

    def _fuses(self, part):
        return part.fuses_residual and (self.scale == 1.0 or part.scales_residual)

    def forward(self, residual, delta, ctx, cache, write, delta_scale=1.0):
        normed = self._norm(self.mixer_norm, residual, delta, self.mixer, delta_scale)
        if self._fuses(self.mixer):
            mixed = self.mixer.forward(normed, ctx, cache, write, residual=residual)
        else:
            mixed = self.mixer.forward(normed, ctx, cache, write)
        if self.feed_forward is None:
            return mixed
        normed = self._norm(self.feed_forward_norm, residual, mixed, self.feed_forward, self.scale)
        if self._fuses(self.feed_forward):
            return self.feed_forward.forward(normed, ctx, residual=residual)
        return self.feed_forward.forward(normed, ctx)
