"""Tiny Farorax configurations for the tests, with weights drawn large enough that every
mechanism moves the logits.

The configurations differ in every size: width, vocabulary, head counts and groupings, key and
value sizes (equal, value shorter, value longer; multiples of 32, of 16, of neither), the
rotated part of a head (all of it, a part, two dimensions, nothing) with and without the
long-context rule, windows (shorter than a page, a few pages, longer than every prompt, none,
one token), lightning heads with keys of 4 to 136 values and decays from fast to none at all,
feed-forwards (gated, routed with and without groups and a shared expert, one expert per token,
none), the order of the layers, the factor on the parts' outputs (also 1), the soft cap (also
none), and the loop (over the first layers, a single layer three times, all layers once, the
last layers, none).
"""

from __future__ import annotations

import json
import tempfile
from pathlib import Path

import torch


def attention(heads, kv_heads, dim, vdim, scale, window, rot, mlp):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window is not None:
        mixer["mask"] = {"size": window}
    if rot is not None:
        mixer["rot"] = rot
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def lightning(heads, dim, vdim, decay, mlp):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim,
                                           "decay": list(decay)}, "mlp": mlp}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def routed(ff, experts, top, groups=None, shared=None):
    out = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if groups is not None:
        out["router"]["groups"] = {"count": groups[0], "keep": groups[1]}
    if shared is not None:
        out["shared"] = {"ff": shared}
    return out


_LONG_A = {"base": 10000.0, "dims": 32,
           "scaling": {"factor": 8.0, "low": 1.0, "high": 3.0, "original": 64}}
_LONG_B = {"base": 300.0, "dims": 64,
           "scaling": {"factor": 2.0, "low": 0.5, "high": 6.0, "original": 40}}

# heads of 32 (the kernel that prepares and attends in one for single tokens), a window of a few
# pages, routed experts in three groups of which two are kept, a layer without a feed-forward,
# a loop over the first two layers
F1 = {"architecture": "Farorax", "vocab": 300, "width": 64, "norm": {"eps": 1e-5},
      "residual_mult": 0.5, "logit_softcap": 20.0,
      "layers": [
          attention(4, 2, 32, 32, 0.2, 24, _LONG_A, dense(96)),
          lightning(2, 16, 24, (0.9, 0.5), routed(32, 6, 2, (3, 2), 40)),
          lightning(4, 8, 16, (1.0, 0.97, 0.6, 0.2), None)],
      "loop": {"start": 0, "stop": 2, "times": 2}}

# every query head its own key head; values longer than keys; a part of the head rotated,
# frequencies as they are; a window shorter than a page; one expert per token and no shared one;
# the parts' outputs enter with factor 1; no loop
F2 = {"architecture": "Farorax", "vocab": 257, "width": 96, "norm": {"eps": 1e-6},
      "residual_mult": 1.0, "logit_softcap": 50.0,
      "layers": [
          attention(3, 3, 16, 48, 0.25, 7, {"base": 1000.0, "dims": 8}, routed(48, 4, 1)),
          lightning(3, 40, 8, (0.8, 0.999, 0.3), dense(200)),
          attention(3, 3, 16, 48, 0.25, 7, {"base": 1000.0, "dims": 8}, dense(64))]}

# heads of 64 on one key head, all of the head rotated, a window of 100; lightning keys of 128;
# eight experts in four groups; a single layer looped three times
F3 = {"architecture": "Farorax", "vocab": 512, "width": 128, "norm": {"eps": 2e-6},
      "residual_mult": 0.7, "logit_softcap": 15.0,
      "layers": [
          lightning(4, 128, 32, (0.95, 0.9, 0.99, 0.7), dense(256)),
          attention(8, 1, 64, 64, 0.11, 100, _LONG_B, routed(48, 8, 3, (4, 2), 64)),
          lightning(4, 128, 32, (0.95, 0.9, 0.99, 0.7), routed(48, 8, 3, (4, 2), 64)),
          attention(8, 1, 64, 64, 0.11, 100, _LONG_B, dense(256))],
      "loop": {"start": 1, "stop": 2, "times": 3}}

# one head everywhere, two rotated dimensions, a window of one token (a query sees itself and the
# sink), one pass of a loop over all layers, logits as they are
F4 = {"architecture": "Farorax", "vocab": 64, "width": 32, "norm": {"eps": 1e-5},
      "residual_mult": 1.5,
      "layers": [attention(1, 1, 8, 8, 0.5, 1, {"base": 100.0, "dims": 2}, dense(48)),
                 lightning(1, 4, 12, (0.5,), None)],
      "loop": {"start": 0, "stop": 2, "times": 1}}

# sizes that are multiples of nothing much: width 72, vocabulary 100, three query heads on one
# key head, keys of 24 and values of 40, six rotated dimensions, no window at all; lightning keys
# of 136; a second attention with values shorter than keys, nothing rotated and a window beyond
# every prompt; all of five experts in one group, two chosen; a loop over the last two layers
F5 = {"architecture": "Farorax", "vocab": 100, "width": 72, "norm": {"eps": 3e-6},
      "residual_mult": 0.25, "logit_softcap": 8.0,
      "layers": [
          attention(3, 1, 24, 40, 0.21, None, {"base": 5000.0, "dims": 6, "scaling": {
              "factor": 4.0, "low": 2.0, "high": 5.0, "original": 16}}, routed(20, 5, 2, None, 24)),
          lightning(2, 136, 20, (0.999, 0.9), dense(100)),
          attention(2, 2, 40, 24, 0.15, 200, None, None)],
      "loop": {"start": 1, "stop": 3, "times": 2}}

# no routed experts (in bfloat16 nothing is decided by a hair, so every row is held to the
# bound): heads of 64 in pairs on a key head with a window of 40, lightning keys of 64, a loop over
# the last two layers
F6 = {"architecture": "Farorax", "vocab": 384, "width": 128, "norm": {"eps": 1e-5},
      "residual_mult": 0.4, "logit_softcap": 12.0,
      "layers": [
          lightning(2, 64, 64, (0.98, 0.8), dense(192)),
          attention(4, 2, 64, 64, 0.125, 40, {"base": 8000.0, "dims": 64}, dense(192)),
          lightning(4, 32, 32, (0.99, 0.9, 0.7, 0.5), None)],
      "loop": {"start": 1, "stop": 3, "times": 2}}

CONFIGS = {"F6": (F6, 26, 16), "F1": (F1, 21, 4), "F2": (F2, 22, 8), "F3": (F3, 23, 16), "F4": (F4, 24, 2),
           "F5": (F5, 25, 8)}   # config, seed, page


def draw_tensors(config: dict, seed: int) -> dict[str, torch.Tensor]:
    """Weights for ``config``, by the names and shapes of the engine's weight contract: matrices
    ~ N(0, 1/in) (the embedding N(0, 1), routers three times as wide so that scores differ),
    norm weights around 1, sinks ~ N(0, 1.5), the loop's vectors ~ N(0, 0.3)."""
    from mlx_one_b200.architectures.farorax import describe
    from mlx_one_b200.config import FaroraxConfig
    from mlx_one_b200.parts import expected_tensors

    generator = torch.Generator().manual_seed(seed)
    out = {}
    for name, want in expected_tensors(describe(FaroraxConfig.from_dict(config))).items():
        values = torch.randn(want.shape, generator=generator)
        if want.init == "norm":
            values = 1.0 + 0.2 * values
        elif name.endswith(".sink"):
            values = 1.5 * values
        elif name.endswith(".router"):
            values = 3.0 * values / want.shape[1] ** 0.5
        elif name == "embed":
            pass
        elif name == "loop.step":
            values = 0.3 * values
        elif len(want.shape) == 2:
            values = values / want.shape[1] ** 0.5
        else:
            values = 0.3 * values
        out[name] = values.to(torch.bfloat16)
    return out


def make_model_dir(name: str, root: Path | None = None, config: dict | None = None) -> Path:
    """Writes the tiny model ``name`` into a fresh temporary folder (never into the repo)."""
    from mlx_one_b200.weights.safetensors_io import write_safetensors

    base, seed, _ = CONFIGS[name]
    config = base if config is None else config
    folder = Path(tempfile.mkdtemp(prefix=f"tiny_{name}_", dir=root))
    write_safetensors(folder / "model.safetensors", draw_tensors(config, seed), {"format": "pt"})
    (folder / "config.json").write_text(json.dumps(config, indent=1))
    return folder


# bfloat16: a row's error is the root mean square over the vocabulary of (engine - plain), its
# mean taken off, relative to the spread of the plain logits. Rounding alone gives a few percent
# on these models; a wrong key, a lost state or a token fed twice gives 15 % and more.
BF16_ROW_ERROR = 0.12
USUAL_NOISE = 5e-6
# The bfloat16 engine routes what its own 16-bit arithmetic has made of the stream (about a
# percent from the plain model's), so a position whose routing margin is below this may go to
# other experts than in the plain model; its own logits are then others, and so, a little, are
# those of every later position of the request (the layers after it carry it on: a lightning
# state forgets slowly). Rows from the first such position on are not compared in bfloat16; the
# 32-bit engine is compared everywhere, and so is bfloat16 on models without routed experts.
ROUTING_MARGIN = 0.05


def assert_rows_close(got: torch.Tensor, want: torch.Tensor, dtype, what: str = "") -> None:
    """float32: every logit within 1e-4 + 1e-4 |plain| + 4 x the position's noise (positions with
    a routing margin below 1e-5 left out). bfloat16: every row's error (see above) within
    ``BF16_ROW_ERROR`` up to the request's first position that is routed by a hair."""
    noise, margin = getattr(want, "noise", None), getattr(want, "margin", None)
    got, want = got.float().cpu(), want.float().cpu()
    assert got.shape == want.shape, f"{what}: {tuple(got.shape)} against {tuple(want.shape)}"
    noise = torch.zeros(want.shape[0]) if noise is None else noise.float().cpu()
    margin = torch.full((want.shape[0],), float("inf")) if margin is None else margin.float().cpu()
    if dtype == torch.float32:
        excess = (got - want).abs() - (1e-4 + 1e-4 * want.abs() + 4 * noise[:, None])
        excess[margin < 1e-5] = 0
        assert excess.max() <= 0, (f"{what}: logits differ by {(got - want).abs().max():.3e}; rows "
                                   f"{torch.nonzero((excess > 0).any(-1)).flatten().tolist()[:8]}")
        return
    difference = got - want
    difference = difference - difference.mean(-1, keepdim=True)
    spread = (want - want.mean(-1, keepdim=True)).pow(2).mean().sqrt()
    rows = difference.pow(2).mean(-1).sqrt() / spread
    allowed = BF16_ROW_ERROR * torch.clamp(noise / USUAL_NOISE, min=1.0)
    settled = torch.cumsum((margin < ROUTING_MARGIN).float(), 0) == 0
    bad = (rows > allowed) & settled
    assert not bad.any(), (f"{what}: row error {rows[settled].max():.3f} of the spread; rows "
                           f"{torch.nonzero(bad).flatten().tolist()[:8]}")


def sliced(want: torch.Tensor, count: int) -> torch.Tensor:
    """The first ``count`` rows of a plain model's logits, with their noise and margins."""
    out = want[:count]
    out.noise, out.margin = want.noise[:count], want.margin[:count]
    return out
