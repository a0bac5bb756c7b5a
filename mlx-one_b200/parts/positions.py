"""Position encodings."""

from __future__ import annotations

import math

import torch

from .base import PositionEncoding
from .registry import POSITIONS


@POSITIONS.register("rope")
class RotaryEncoding(PositionEncoding):
    """Non-interleaved rotary encoding: dimension j of the first half pairs with j of the
    second half; inv_freq_j = theta^(-j / (rotary_dim / 2)), angle = position * inv_freq,
    all in 32-bit. Parameters: ``theta``, ``rotary_dim`` (even, at most the head size).
    Reference: src/mlx_one/models/shared/transformer.py:50-51, 67-72, 88-90."""

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.rotary_dim = int(spec["rotary_dim"])
        if self.rotary_dim <= 0 or self.rotary_dim % 2:
            raise ValueError("rotary_dim must be positive and even")
        half = self.rotary_dim // 2
        inv_freq = torch.pow(torch.tensor(float(spec["theta"]), dtype=torch.float32),
                             -torch.arange(half, dtype=torch.float32) / half)
        self.inv_freq = inv_freq.to(runtime.device)

    def rotary_table(self):
        return self.inv_freq, self.rotary_dim


@POSITIONS.register("yarn")
class ScaledRotaryEncoding(PositionEncoding):
    """Rotary encoding of the first ``rotary_dim`` dimensions of a head (pairs j and j +
    rotary_dim / 2) whose frequencies are stretched for a context ``factor`` times the
    ``original`` one: f_j = theta^(-2j / rotary_dim); with d(t) = rotary_dim * ln(original /
    (2 pi t)) / (2 ln theta), lo = max(floor(d(fast)), 0), hi = min(ceil(d(slow)), rotary_dim - 1)
    and r_j = clamp((j - lo) / max(hi - lo, 0.001), 0, 1) the frequency of pair j is
    (f_j / factor) r_j + f_j (1 - r_j): pairs that turn often within the original context keep
    their frequency, slow ones are interpolated. Cosine and sine are both multiplied by
    0.1 ln(factor) + 1. Parameters: ``theta``, ``rotary_dim``, and ``factor``, ``original``,
    ``fast``, ``slow`` (``factor`` None: plain frequencies, amplitude 1). The table is worked out
    in 64-bit on the host and rounded once."""

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.rotary_dim = dims = int(spec["rotary_dim"])
        if dims <= 0 or dims % 2:
            raise ValueError("rotary_dim must be positive and even")
        theta = float(spec["theta"])
        index = torch.arange(dims // 2, dtype=torch.float64)
        freq = theta ** (-2.0 * index / dims)
        self.scale = 1.0
        factor = spec.get("factor")
        if factor is not None:
            factor, original = float(factor), float(spec["original"])
            turns = lambda t: dims * math.log(original / (2 * math.pi * t)) / (2 * math.log(theta))
            lo = max(math.floor(turns(float(spec["fast"]))), 0)
            hi = min(math.ceil(turns(float(spec["slow"]))), dims - 1)
            ramp = torch.clamp((index - lo) / max(hi - lo, 0.001), 0.0, 1.0)
            freq = freq / factor * ramp + freq * (1.0 - ramp)
            self.scale = 0.1 * math.log(factor) + 1.0
        self.inv_freq = freq.to(torch.float32).to(runtime.device)

    def rotary_table(self):
        return self.inv_freq, self.rotary_dim

    def amplitude(self):
        return self.scale


@POSITIONS.register("rope_long")
class LongContextRotaryEncoding(PositionEncoding):
    """Rotary encoding of the first ``rotary_dim`` dimensions of a head with f_i =
    theta^(-2i / rotary_dim) and the long-context rule of Llama 3.1 for slow pairs: with the
    wavelength l = 2 pi / f, pairs with l < original / high keep f, pairs with l > original / low
    get f / factor, and between the two, with s = (original / l - low) / (high - low), the
    frequency is (1 - s) f / factor + s f. Parameters: ``theta``, ``rotary_dim``, ``factor``,
    ``original``, ``low``, ``high`` (``factor`` None: plain frequencies), and ``layout``:
    ``halves`` (pair i is dimensions i and i + rotary_dim / 2) or ``neighbours`` (pair i is
    dimensions 2i and 2i + 1). The kernels rotate halves; a mixer whose encoding pairs neighbours
    reorders the rows of its query and key projections with ``row_order`` when it is built, which
    leaves every score as it is. The table is worked out in 64-bit on the host and rounded once."""

    LAYOUTS = ("halves", "neighbours")

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.rotary_dim = dims = int(spec["rotary_dim"])
        if dims <= 0 or dims % 2:
            raise ValueError("rotary_dim must be positive and even")
        self.layout = spec.get("layout") or "halves"
        if self.layout not in self.LAYOUTS:
            raise ValueError(f"unknown layout {self.layout!r}")
        theta = float(spec["theta"])
        freq = theta ** (-2.0 * torch.arange(dims // 2, dtype=torch.float64) / dims)
        factor = spec.get("factor")
        if factor is not None:
            factor, original = float(factor), float(spec["original"])
            low, high = float(spec["low"]), float(spec["high"])
            wave = 2 * math.pi / freq
            blend = (original / wave - low) / (high - low)
            mixed = (1 - blend) * freq / factor + blend * freq
            freq = torch.where(wave < original / high, freq,
                               torch.where(wave > original / low, freq / factor, mixed))
        self.inv_freq = freq.to(torch.float32).to(runtime.device)

    def rotary_table(self):
        return self.inv_freq, self.rotary_dim

    def row_order(self, head_dim: int) -> torch.Tensor | None:
        """For a head of ``head_dim`` rows whose pairs are neighbours: the order of rows that
        puts pair i at i and i + rotary_dim / 2 (None: nothing to reorder)."""
        if self.layout == "halves":
            return None
        dims = self.rotary_dim
        return torch.cat([torch.arange(0, dims, 2), torch.arange(1, dims, 2),
                          torch.arange(dims, head_dim)])


@POSITIONS.register("none")
class NoPositionEncoding(PositionEncoding):
    """No rotation: order is known to the model only through causality."""

    def rotary_table(self):
        return None
