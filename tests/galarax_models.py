"""Tiny Galarax configurations for the tests, with weights drawn large enough that every
mechanism moves the logits.

The configurations differ in every size: width, vocabulary, head counts and groupings (2 per key
head, 1 per key head, all on one), key and value sizes (value shorter, longer, equal), the
rotated part of a head (a part, the whole head, none) with and without stretched frequencies,
score scales, convolution taps (2, 3, 4), key sizes of the delta rule that are and are not
powers of two, layers without a feed-forward, sizes that differ from layer to layer, and the
loop (over the first two layers, over a single layer, none, over all layers).
"""

from __future__ import annotations

import json
import tempfile
from pathlib import Path

import torch


def _layer(left, right, ff):
    return {"type": "parallel", "mixer": {"left": left, "right": right},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def _left(heads, kv_heads, dim, vdim, scale, rot):
    out = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if rot is not None:
        out["rot"] = rot
    return out


def _right(heads, kv_heads, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


_STRETCH_A = {"base": 10000.0, "dims": 16,
              "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}}
_STRETCH_B = {"base": 500.0, "dims": 32,
              "scaling": {"factor": 16.0, "original": 32, "fast": 4.0, "slow": 0.5}}

# value rows shorter than key rows; loop over the first two layers; a layer without feed-forward;
# the last layer has other sizes than the first two and rotates nothing
G1 = {"architecture": "Galarax", "vocab": 300, "width": 64, "norm": {"eps": 1e-5},
      "layers": [
          _layer(_left(4, 2, 32, 16, 0.2, _STRETCH_A), _right(4, 2, 16, 24, 4), 96),
          _layer(_left(4, 2, 32, 16, 0.2, _STRETCH_A), _right(4, 2, 16, 24, 4), None),
          _layer(_left(2, 1, 16, 16, 0.3, None), _right(2, 2, 32, 8, 2), 80)],
      "loop": {"start": 0, "stop": 2, "times": 2}}

# value rows longer than key rows; every query head its own key head; the whole head rotated,
# frequencies as they are; a delta key size that is no power of two; no loop
G2 = {"architecture": "Galarax", "vocab": 257, "width": 96, "norm": {"eps": 1e-6},
      "layers": [
          _layer(_left(3, 3, 16, 48, 0.25, {"base": 1000.0, "dims": 16}), _right(2, 1, 40, 8, 2), 200),
          _layer(_left(3, 3, 16, 48, 0.25, {"base": 1000.0, "dims": 16}), _right(2, 1, 40, 8, 2), 200)]}

# head size 64 on one key head (the tensor-core attention kernels), a loop over a single layer,
# a delta key size of 128 with as many query/key heads as value heads
G3 = {"architecture": "Galarax", "vocab": 512, "width": 128, "norm": {"eps": 2e-6},
      "layers": [
          _layer(_left(8, 1, 64, 64, 0.11, _STRETCH_B), _right(6, 6, 128, 32, 3), 256),
          _layer(_left(8, 1, 64, 64, 0.11, _STRETCH_B), _right(6, 6, 128, 32, 3), 256),
          _layer(_left(8, 1, 64, 64, 0.11, _STRETCH_B), _right(6, 6, 128, 32, 3), None),
          _layer(_left(8, 1, 64, 64, 0.11, _STRETCH_B), _right(6, 6, 128, 32, 3), 256)],
      "loop": {"start": 1, "stop": 2, "times": 3}}

# one pass of a loop over all layers (times = 1: only its vector is added), one head everywhere,
# convolutions of a single tap (no inputs to keep)
G4 = {"architecture": "Galarax", "vocab": 64, "width": 32, "norm": {"eps": 1e-5},
      "layers": [_layer(_left(1, 1, 8, 8, 0.5, {"base": 100.0, "dims": 2}), _right(1, 1, 8, 4, 1), 48)],
      "loop": {"start": 0, "stop": 1, "times": 1}}

# sizes that are multiples of nothing much: width 72, vocabulary 100, three query heads on one key
# head, keys of 24 and values of 40, six rotated dimensions, five taps, a loop over the last two
# of three layers, the looped layers of different sizes, one of them without a feed-forward
G5 = {"architecture": "Galarax", "vocab": 100, "width": 72, "norm": {"eps": 3e-6},
      "layers": [
          _layer(_left(3, 1, 24, 40, 0.21, {"base": 5000.0, "dims": 6, "scaling": {
              "factor": 2.0, "original": 16, "fast": 3.0, "slow": 0.25}}), _right(3, 3, 24, 20, 5), 100),
          _layer(_left(2, 2, 40, 24, 0.15, {"base": 5000.0, "dims": 40}), _right(4, 1, 12, 36, 3), None),
          _layer(_left(3, 1, 24, 40, 0.21, None), _right(3, 3, 24, 20, 5), 52)],
      "loop": {"start": 1, "stop": 3, "times": 2}}

CONFIGS = {"G1": (G1, 11, 4), "G2": (G2, 12, 8), "G3": (G3, 13, 16), "G4": (G4, 14, 2),
           "G5": (G5, 15, 8)}   # config, seed, page


def draw_tensors(config: dict, seed: int, decay_bias: float = 0.0) -> dict[str, torch.Tensor]:
    """Weights for ``config``, by the names and shapes of the engine's weight contract: matrices
    ~ N(0, 1/in), biases and vectors ~ N(0, 0.3), norm weights around their neutral value,
    convolution kernels ~ N(0, 0.5). ``decay_bias`` is added to A_log (very negative: the delta
    rule forgets slowly)."""
    from mlx_one_b200.config import GalaraxConfig
    from mlx_one_b200.architectures.galarax import describe
    from mlx_one_b200.parts import expected_tensors

    generator = torch.Generator().manual_seed(seed)
    out = {}
    for name, want in expected_tensors(describe(GalaraxConfig.from_dict(config))).items():
        values = torch.randn(want.shape, generator=generator)
        if want.init == "norm":
            values = 1.0 + 0.2 * values
        elif want.init == "norm0":
            values = 0.2 * values
        elif name.endswith(".conv"):
            values = 0.5 * values
        elif name.endswith("A_log"):
            values = 0.5 * values + decay_bias
        elif len(want.shape) == 2 and name != "loop.step":
            values = values / want.shape[1] ** 0.5
            if name == "embed":
                values = torch.randn(want.shape, generator=generator)
        else:
            values = 0.3 * values
        out[name] = values.to(torch.bfloat16)
    return out


def make_model_dir(name: str, root: Path | None = None, decay_bias: float = 0.0) -> Path:
    """Writes the tiny model ``name`` into a fresh temporary folder (never into the repo)."""
    from mlx_one_b200.weights.safetensors_io import write_safetensors

    config, seed, _ = CONFIGS[name]
    folder = Path(tempfile.mkdtemp(prefix=f"tiny_{name}_", dir=root))
    write_safetensors(folder / "model.safetensors", draw_tensors(config, seed, decay_bias),
                      {"format": "pt"})
    (folder / "config.json").write_text(json.dumps(config, indent=1))
    return folder


# bfloat16: a row's error is the root mean square over the vocabulary of (engine - plain), its
# mean taken off, relative to the spread of the plain logits. Rounding alone gives 1 to 3 % on
# these models (measured); a wrong key, a lost state or a token fed twice gives 15 % and more.
BF16_ROW_ERROR = 0.06
# A few positions of these random models are badly determined: the plain equations in 32-bit
# arithmetic land 1e-4 from the 64-bit ones there, a hundred times farther than elsewhere (1e-6),
# and every rounding of the engine is amplified alike. ``want.noise`` (see PlainModel.logits)
# measures that per position; a position's bounds grow with it.
USUAL_NOISE = 5e-6


def assert_rows_close(got: torch.Tensor, want: torch.Tensor, dtype, what: str = "") -> None:
    """float32: every logit within 1e-4 + 1e-4 |plain| + 4 x the position's noise. bfloat16: every
    row's error (see above) within ``BF16_ROW_ERROR`` x max(1, noise / USUAL_NOISE)."""
    noise = getattr(want, "noise", None)
    got, want = got.float().cpu(), want.float().cpu()
    assert got.shape == want.shape, f"{what}: {tuple(got.shape)} against {tuple(want.shape)}"
    noise = torch.zeros(want.shape[0]) if noise is None else noise.float().cpu()
    if dtype == torch.float32:
        excess = (got - want).abs() - (1e-4 + 1e-4 * want.abs() + 4 * noise[:, None])
        assert excess.max() <= 0, (f"{what}: logits differ by {(got - want).abs().max():.3e}; rows "
                                   f"{torch.nonzero((excess > 0).any(-1)).flatten().tolist()[:8]}")
        return
    difference = got - want
    difference = difference - difference.mean(-1, keepdim=True)
    spread = (want - want.mean(-1, keepdim=True)).pow(2).mean().sqrt()
    rows = difference.pow(2).mean(-1).sqrt() / spread
    allowed = BF16_ROW_ERROR * torch.clamp(noise / USUAL_NOISE, min=1.0)
    assert (rows <= allowed).all(), (f"{what}: row error {rows.max():.3f} of the spread; rows "
                                     f"{torch.nonzero(rows > allowed).flatten().tolist()[:8]}")
    # and most rows are determined well: the looser bound is for the exception
    assert (noise <= 4 * USUAL_NOISE).float().mean() >= 0.5 or want.shape[0] < 8, \
        f"{what}: most positions of this request are badly determined; choose other weights"
