"""Typed configuration of Galarax, read from its config.json keys.

A Galarax config.json has ``architecture`` ("Galarax"), ``vocab``, ``width``, ``norm.eps``, a
list ``layers`` and an optional ``loop``. Every layer entry gives its ``type`` (the mixer it
has), the mixer's sizes under ``mixer`` and its feed-forward under ``mlp`` (null: none). The
one mixer type of the design, ``parallel``, runs two mixers side by side on the same input:
``left`` (grouped-query softmax attention with rotary positions) and ``right`` (a gated delta
rule with short convolutions). ``loop`` names a run of layers (``start`` .. ``stop`` - 1) that is
executed ``times`` times in a row with the same weights.

Nothing here has a default that stands for a size: a key that the design requires and that is
absent is an error with the key's path.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping

from .base import ConfigError, divisible, positive, positive_int

NAME = "Galarax"


def _need(data: Mapping[str, Any], key: str, where: str) -> Any:
    if not isinstance(data, Mapping) or key not in data:
        raise ConfigError(f"{where}{key} is missing")
    return data[key]


@dataclass(frozen=True)
class RotaryScaling:
    """Frequency interpolation between an original context and ``factor`` times it."""

    factor: float
    original: float
    fast: float
    slow: float

    @classmethod
    def from_dict(cls, data, where):
        out = cls(*(float(_need(data, key, where)) for key in ("factor", "original", "fast", "slow")))
        for key in ("factor", "original", "fast", "slow"):
            positive(where + key, getattr(out, key))
        return out

    def to_dict(self):
        original = int(self.original) if float(self.original).is_integer() else self.original
        return {"factor": self.factor, "fast": self.fast, "original": original, "slow": self.slow}


@dataclass(frozen=True)
class Rotary:
    base: float
    dims: int
    scaling: RotaryScaling | None = None

    @classmethod
    def from_dict(cls, data, where):
        dims = _need(data, "dims", where)
        positive_int(where + "dims", dims)
        if dims % 2:
            raise ConfigError(f"{where}dims ({dims}) must be even")
        base = float(_need(data, "base", where))
        positive(where + "base", base)
        scaling = data.get("scaling")
        return cls(base, dims, None if scaling is None
                   else RotaryScaling.from_dict(scaling, where + "scaling."))

    def to_dict(self):
        out = {"base": self.base, "dims": self.dims}
        if self.scaling is not None:
            out["scaling"] = self.scaling.to_dict()
        return out


@dataclass(frozen=True)
class SoftmaxBranch:
    """``left``: query heads, key/value heads, key size, value size, score scale, rotation."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: Rotary | None

    @classmethod
    def from_dict(cls, data, where):
        heads, kv_heads = _need(data, "heads", where), _need(data, "kv_heads", where)
        divisible(where + "heads", heads, where + "kv_heads", kv_heads)
        dim, vdim = _need(data, "dim", where), _need(data, "vdim", where)
        positive_int(where + "dim", dim)
        positive_int(where + "vdim", vdim)
        scale = float(_need(data, "scale", where))
        positive(where + "scale", scale)
        rot = data.get("rot")
        rot = None if rot is None else Rotary.from_dict(rot, where + "rot.")
        if rot is not None and rot.dims > dim:
            raise ConfigError(f"{where}rot.dims ({rot.dims}) exceeds {where}dim ({dim})")
        return cls(heads, kv_heads, dim, vdim, scale, rot)

    def to_dict(self):
        out = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads,
               "scale": self.scale, "vdim": self.vdim}
        if self.rot is not None:
            out["rot"] = self.rot.to_dict()
        return out


@dataclass(frozen=True)
class DeltaBranch:
    """``right``: value heads, query/key heads, key size, value size, convolution taps."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int

    @classmethod
    def from_dict(cls, data, where):
        heads, kv_heads = _need(data, "heads", where), _need(data, "kv_heads", where)
        divisible(where + "heads", heads, where + "kv_heads", kv_heads)
        for key in ("dim", "vdim", "conv"):
            positive_int(where + key, _need(data, key, where))
        return cls(heads, kv_heads, data["dim"], data["vdim"], data["conv"])

    def to_dict(self):
        return {"conv": self.conv, "dim": self.dim, "heads": self.heads,
                "kv_heads": self.kv_heads, "vdim": self.vdim}


@dataclass(frozen=True)
class GalaraxLayer:
    type: str
    left: SoftmaxBranch
    right: DeltaBranch
    ff: int | None                  # feed-forward width; None: the layer has no feed-forward

    @classmethod
    def from_dict(cls, data, where):
        kind = _need(data, "type", where)
        if kind != "parallel":
            raise ConfigError(f"{where}type {kind!r} is not a mixer of this design (parallel)")
        mixer = _need(data, "mixer", where)
        left = SoftmaxBranch.from_dict(_need(mixer, "left", where + "mixer."), where + "mixer.left.")
        right = DeltaBranch.from_dict(_need(mixer, "right", where + "mixer."), where + "mixer.right.")
        mlp = data.get("mlp")
        ff = None
        if mlp is not None:
            if _need(mlp, "kind", where + "mlp.") != "dense":
                raise ConfigError(f"{where}mlp.kind {mlp['kind']!r} is not known (dense)")
            ff = _need(mlp, "ff", where + "mlp.")
            positive_int(where + "mlp.ff", ff)
        return cls(kind, left, right, ff)

    def to_dict(self):
        return {"mixer": {"left": self.left.to_dict(), "right": self.right.to_dict()},
                "mlp": None if self.ff is None else {"ff": self.ff, "kind": "dense"},
                "type": self.type}


@dataclass(frozen=True)
class Loop:
    start: int
    stop: int
    times: int


@dataclass(frozen=True)
class GalaraxConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: tuple[GalaraxLayer, ...]
    loop: Loop | None = None
    extra: Mapping[str, Any] = field(default_factory=dict, repr=False)

    def __post_init__(self) -> None:
        positive_int("vocab", self.vocab)
        positive_int("width", self.width)
        positive("norm.eps", self.norm_eps)
        if not self.layers:
            raise ConfigError("layers is empty")
        if self.loop is not None:
            loop = self.loop
            for key in ("start", "stop", "times"):
                value = getattr(loop, key)
                if isinstance(value, bool) or not isinstance(value, int) or value < 0:
                    raise ConfigError(f"loop.{key} must be a non-negative integer, got {value!r}")
            if not loop.start < loop.stop <= len(self.layers):
                raise ConfigError(f"loop.start .. loop.stop ({loop.start} .. {loop.stop}) is not "
                                  f"a run of the {len(self.layers)} layers")
            positive_int("loop.times", loop.times)

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "GalaraxConfig":
        name = data.get("architecture", data.get("model_type"))
        if str(name).lower() != NAME.lower():
            raise ConfigError(f"architecture {name!r} is not a {NAME} configuration")
        layers = _need(data, "layers", "")
        if not isinstance(layers, (list, tuple)):
            raise ConfigError("layers must be a list")
        loop = data.get("loop")
        if loop is not None:
            loop = Loop(*(_need(loop, key, "loop.") for key in ("start", "stop", "times")))
        known = {"architecture", "model_type", "layers", "loop", "norm", "vocab", "width"}
        return cls(vocab=_need(data, "vocab", ""), width=_need(data, "width", ""),
                   norm_eps=float(_need(_need(data, "norm", ""), "eps", "norm.")),
                   layers=tuple(GalaraxLayer.from_dict(entry, f"layers[{i}].")
                                for i, entry in enumerate(layers)),
                   loop=loop, extra={k: v for k, v in data.items() if k not in known})

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = dict(self.extra)
        out.update(architecture=NAME, layers=[layer.to_dict() for layer in self.layers],
                   norm={"eps": self.norm_eps}, vocab=self.vocab, width=self.width)
        if self.loop is not None:
            out["loop"] = {"start": self.loop.start, "stop": self.loop.stop,
                           "times": self.loop.times}
        return out
