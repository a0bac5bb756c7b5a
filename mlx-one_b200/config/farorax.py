"""Typed configuration of Farorax, read from its config.json keys.

A Farorax config.json has ``architecture`` ("Farorax"), ``vocab``, ``width``, ``norm.eps``,
``residual_mult`` (the factor on every part's output before it enters the stream),
``logit_softcap`` (logits become cap * tanh(logits / cap)), a list ``layers`` and an optional
``loop``. Every layer entry gives its ``type`` (the mixer it has: ``attention``, grouped-query
softmax attention over a sliding window with a learned sink per head and rotary positions on
neighbouring pairs; or ``lightning``, linear attention with a constant decay per head and a
32-bit matrix state), the mixer's sizes under ``mixer`` and its feed-forward under ``mlp``
(null: none; ``kind`` ``dense``: a gated feed-forward; ``moe``: routed experts with an optional
shared expert). ``loop`` names a run of layers (``start`` .. ``stop`` - 1) that is executed
``times`` times in a row with the same weights.

Nothing here has a default that stands for a size: a key that the design requires and that is
absent is an error with the key's path.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping

from .base import ConfigError, divisible, positive, positive_int

NAME = "Farorax"


def _need(data: Mapping[str, Any], key: str, where: str) -> Any:
    if not isinstance(data, Mapping) or key not in data:
        raise ConfigError(f"{where}{key} is missing")
    return data[key]


@dataclass(frozen=True)
class FrequencyScaling:
    """Long-context rule for rotary frequencies: wavelengths below ``original / high`` keep
    their frequency, above ``original / low`` it is divided by ``factor``, between them the two
    are blended."""

    factor: float
    low: float
    high: float
    original: float

    KEYS = ("factor", "low", "high", "original")

    @classmethod
    def from_dict(cls, data, where):
        out = cls(*(float(_need(data, key, where)) for key in cls.KEYS))
        for key in cls.KEYS:
            positive(where + key, getattr(out, key))
        if out.high == out.low:
            raise ConfigError(f"{where}high and {where}low must differ")
        return out

    def to_dict(self):
        original = int(self.original) if float(self.original).is_integer() else self.original
        return {"factor": self.factor, "high": self.high, "low": self.low, "original": original}


@dataclass(frozen=True)
class Rotary:
    base: float
    dims: int
    scaling: FrequencyScaling | None = None

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
                   else FrequencyScaling.from_dict(scaling, where + "scaling."))

    def to_dict(self):
        out = {"base": self.base, "dims": self.dims}
        if self.scaling is not None:
            out["scaling"] = self.scaling.to_dict()
        return out


@dataclass(frozen=True)
class AttentionMixer:
    """Query heads, key/value heads, key size, value size, score scale, window, rotation."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int | None
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
        window = None
        if data.get("mask") is not None:
            window = _need(data["mask"], "size", where + "mask.")
            positive_int(where + "mask.size", window)
        rot = data.get("rot")
        rot = None if rot is None else Rotary.from_dict(rot, where + "rot.")
        if rot is not None and rot.dims > dim:
            raise ConfigError(f"{where}rot.dims ({rot.dims}) exceeds {where}dim ({dim})")
        return cls(heads, kv_heads, dim, vdim, scale, window, rot)

    def to_dict(self):
        out = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads,
               "scale": self.scale, "vdim": self.vdim}
        if self.window is not None:
            out["mask"] = {"size": self.window}
        if self.rot is not None:
            out["rot"] = self.rot.to_dict()
        return out


@dataclass(frozen=True)
class LightningMixer:
    """Heads, key size, value size and the decay of each head's state per token."""

    heads: int
    dim: int
    vdim: int
    decay: tuple[float, ...]

    @classmethod
    def from_dict(cls, data, where):
        for key in ("heads", "dim", "vdim"):
            positive_int(where + key, _need(data, key, where))
        decay = _need(data, "decay", where)
        if isinstance(decay, (int, float)) and not isinstance(decay, bool):
            decay = [decay] * data["heads"]
        if not isinstance(decay, (list, tuple)) or len(decay) != data["heads"]:
            raise ConfigError(f"{where}decay must give one number per head")
        for index, value in enumerate(decay):
            if isinstance(value, bool) or not isinstance(value, (int, float)) or not 0 <= value <= 1:
                raise ConfigError(f"{where}decay[{index}] must lie in 0..1, got {value!r}")
        return cls(data["heads"], data["dim"], data["vdim"], tuple(float(v) for v in decay))

    def to_dict(self):
        return {"decay": list(self.decay), "dim": self.dim, "heads": self.heads, "vdim": self.vdim}


@dataclass(frozen=True)
class DenseFeedForward:
    ff: int

    def to_dict(self):
        return {"ff": self.ff, "kind": "dense"}


@dataclass(frozen=True)
class RoutedFeedForward:
    """``experts`` feed-forwards of width ``ff`` of which a token uses ``top``; experts form
    ``groups`` equal runs of neighbours of which the best ``keep`` may be chosen from; a shared
    expert of width ``shared_ff`` (None: none) serves every token."""

    ff: int
    experts: int
    top: int
    groups: int
    keep: int
    shared_ff: int | None

    @classmethod
    def from_dict(cls, data, where):
        ff = _need(_need(data, "expert", where), "ff", where + "expert.")
        positive_int(where + "expert.ff", ff)
        router = _need(data, "router", where)
        experts, top = _need(router, "experts", where + "router."), _need(router, "top", where + "router.")
        positive_int(where + "router.experts", experts)
        positive_int(where + "router.top", top)
        groups, keep = 1, 1
        if router.get("groups") is not None:
            groups = _need(router["groups"], "count", where + "router.groups.")
            keep = _need(router["groups"], "keep", where + "router.groups.")
            divisible(where + "router.experts", experts, where + "router.groups.count", groups)
            positive_int(where + "router.groups.keep", keep)
            if keep > groups:
                raise ConfigError(f"{where}router.groups.keep ({keep}) exceeds "
                                  f"{where}router.groups.count ({groups})")
        if top > keep * (experts // groups):
            raise ConfigError(f"{where}router.top ({top}) exceeds the experts of the kept groups")
        shared_ff = None
        if data.get("shared") is not None:
            shared_ff = _need(data["shared"], "ff", where + "shared.")
            positive_int(where + "shared.ff", shared_ff)
        return cls(ff, experts, top, groups, keep, shared_ff)

    def to_dict(self):
        out = {"expert": {"ff": self.ff}, "kind": "moe",
               "router": {"experts": self.experts, "groups": {"count": self.groups, "keep": self.keep},
                          "top": self.top}}
        if self.shared_ff is not None:
            out["shared"] = {"ff": self.shared_ff}
        return out


MIXERS = {"attention": AttentionMixer, "lightning": LightningMixer}


@dataclass(frozen=True)
class FaroraxLayer:
    type: str
    mixer: Any                      # AttentionMixer or LightningMixer
    mlp: Any                        # DenseFeedForward, RoutedFeedForward or None

    @classmethod
    def from_dict(cls, data, where):
        kind = _need(data, "type", where)
        if kind not in MIXERS:
            raise ConfigError(f"{where}type {kind!r} is not a mixer of this design "
                              f"({', '.join(sorted(MIXERS))})")
        mixer = MIXERS[kind].from_dict(_need(data, "mixer", where), where + "mixer.")
        mlp = data.get("mlp")
        if mlp is not None:
            form = _need(mlp, "kind", where + "mlp.")
            if form == "dense":
                positive_int(where + "mlp.ff", _need(mlp, "ff", where + "mlp."))
                mlp = DenseFeedForward(mlp["ff"])
            elif form == "moe":
                mlp = RoutedFeedForward.from_dict(mlp, where + "mlp.")
            else:
                raise ConfigError(f"{where}mlp.kind {form!r} is not known (dense, moe)")
        return cls(kind, mixer, mlp)

    def to_dict(self):
        return {"mixer": self.mixer.to_dict(), "mlp": None if self.mlp is None else self.mlp.to_dict(),
                "type": self.type}


@dataclass(frozen=True)
class Loop:
    start: int
    stop: int
    times: int


@dataclass(frozen=True)
class FaroraxConfig:
    vocab: int
    width: int
    norm_eps: float
    residual_mult: float
    logit_softcap: float | None
    layers: tuple[FaroraxLayer, ...]
    loop: Loop | None = None
    extra: Mapping[str, Any] = field(default_factory=dict, repr=False)

    def __post_init__(self) -> None:
        positive_int("vocab", self.vocab)
        positive_int("width", self.width)
        positive("norm.eps", self.norm_eps)
        positive("residual_mult", self.residual_mult)
        if self.logit_softcap is not None:
            positive("logit_softcap", self.logit_softcap)
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
    def from_dict(cls, data: Mapping[str, Any]) -> "FaroraxConfig":
        name = data.get("architecture", data.get("model_type"))
        if str(name).lower() != NAME.lower():
            raise ConfigError(f"architecture {name!r} is not a {NAME} configuration")
        layers = _need(data, "layers", "")
        if not isinstance(layers, (list, tuple)):
            raise ConfigError("layers must be a list")
        loop = data.get("loop")
        if loop is not None:
            loop = Loop(*(_need(loop, key, "loop.") for key in ("start", "stop", "times")))
        known = {"architecture", "model_type", "layers", "loop", "norm", "vocab", "width",
                 "residual_mult", "logit_softcap"}
        softcap = data.get("logit_softcap")
        return cls(vocab=_need(data, "vocab", ""), width=_need(data, "width", ""),
                   norm_eps=float(_need(_need(data, "norm", ""), "eps", "norm.")),
                   residual_mult=float(data.get("residual_mult", 1.0)),
                   logit_softcap=None if softcap is None else float(softcap),
                   layers=tuple(FaroraxLayer.from_dict(entry, f"layers[{i}].")
                                for i, entry in enumerate(layers)),
                   loop=loop, extra={k: v for k, v in data.items() if k not in known})

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = dict(self.extra)
        out.update(architecture=NAME, layers=[layer.to_dict() for layer in self.layers],
                   norm={"eps": self.norm_eps}, residual_mult=self.residual_mult,
                   vocab=self.vocab, width=self.width)
        if self.logit_softcap is not None:
            out["logit_softcap"] = self.logit_softcap
        if self.loop is not None:
            out["loop"] = {"start": self.loop.start, "stop": self.loop.stop,
                           "times": self.loop.times}
        return out
