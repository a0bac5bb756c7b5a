"""Plain, slow Farorax written from the design's equations: whole sequences, no cache, one
function per mechanism. It shares no code with the engine: it reads config.json and the
safetensors file by itself and computes everything in one floating type (float64 by default).

Notation: x [T, W] the stream, h the normed input of a part, T tokens at positions 0..T-1.
"""

from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import torch

_KINDS = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16, "I32": torch.int32}


def read_tensors(path):
    """A safetensors file: 8 bytes little-endian header length, the JSON header, the data."""
    raw = Path(path).read_bytes()
    (length,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + length])
    data = raw[8 + length:]
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        out[name] = torch.frombuffer(bytearray(data[lo:hi]), dtype=_KINDS[info["dtype"]]) \
            .reshape(info["shape"]).clone()
    return out


# --------------------------------------------------------------------------- small pieces


def rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def silu(z):
    return z / (1 + torch.exp(-z))


def gelu_tanh(z):
    return 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))


def pair_frequencies(rot, kind):
    """f_i = base^(-2i/dims), then per frequency the long-context rule: wavelengths shorter than
    original/high keep f, longer than original/low get f/factor, between them a blend."""
    dims = rot["dims"]
    out = []
    for i in range(dims // 2):
        f = rot["base"] ** (-2.0 * i / dims)
        s = rot.get("scaling")
        if s:
            wave = 2 * math.pi / f
            if wave > s["original"] / s["low"]:
                f = f / s["factor"]
            elif wave >= s["original"] / s["high"]:
                t = (s["original"] / wave - s["low"]) / (s["high"] - s["low"])
                f = (1 - t) * f / s["factor"] + t * f
        out.append(f)
    return torch.tensor(out, dtype=kind)


def rotate_neighbours(x, positions, rot):
    """x [T, heads, D]: within the first dims dimensions, neighbours (2i, 2i+1) are turned by
    position * f_i; the other dimensions pass."""
    if not rot:
        return x
    f = pair_frequencies(rot, x.dtype)
    dims = rot["dims"]
    angle = positions.to(x.dtype)[:, None] * f[None, :]
    cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    turned = torch.stack([u * cos - v * sin, v * cos + u * sin], -1).flatten(-2)
    return torch.cat([turned, x[..., dims:]], -1)


def windowed_attention_with_sink(q, k, v, scale, window, sink):
    """q [T, H, D], k [T, G, D], v [T, G, V], sink [H] -> [T, H, V]. Query i sees keys j with
    0 <= i - j < window; the softmax's denominator also holds exp(sink_h), which has no value."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[-1], dtype=q.dtype)
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    visible = (i - j >= 0) & (i - j < window)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        s = s.masked_fill(~visible, -math.inf)
        top = torch.maximum(s.amax(-1, keepdim=True), sink[h])
        e = torch.exp(s - top)
        out[:, h] = (e @ v[:, g]) / (e.sum(-1, keepdim=True) + torch.exp(sink[h] - top))
    return out


def decayed_outer_product_state(q, k, v, decay):
    """q, k [T, H, D], v [T, H, V], decay [H] -> o [T, H, V], from a zero state.
    Per token and head: S = decay S + k v^T; o = S^T q."""
    T, H, V = v.shape
    o = torch.zeros(T, H, V, dtype=v.dtype)
    for h in range(H):
        S = torch.zeros(q.shape[2], V, dtype=v.dtype)
        for t in range(T):
            S = decay[h] * S + torch.outer(k[t, h], v[t, h])
            o[t, h] = S.T @ q[t, h]
    return o


def routing(h, router, experts, top, groups, keep, margins=None):
    """Weights [T, experts]: sigmoid scores; experts in ``groups`` equal runs of neighbours, a
    group's score the sum of its two largest, only the best ``keep`` groups stay; of those the
    ``top`` largest are chosen, their scores divided by their sum. ``margins`` collects, per
    token, how far the choice is from another one: the gap between the worst kept and the best
    dropped group, and between the worst chosen and the best allowed expert that was not."""
    s = torch.sigmoid(h @ router.T)
    T = s.shape[0]
    per = experts // groups
    grouped = s.view(T, groups, per)
    group_score = grouped.topk(min(2, per), dim=-1).values.sum(-1)
    kept = torch.zeros(T, groups, dtype=torch.bool)
    kept.scatter_(1, group_score.topk(keep, dim=-1).indices, True)
    allowed = kept[:, :, None].expand(T, groups, per).reshape(T, experts)
    chosen = s.masked_fill(~allowed, -1.0).topk(top, dim=-1).indices
    weights = torch.zeros_like(s)
    weights.scatter_(1, chosen, s.gather(1, chosen))
    if margins is not None:
        gap = torch.full((T,), math.inf, dtype=s.dtype)
        if keep < groups:
            ranked = group_score.sort(dim=-1, descending=True).values
            gap = torch.minimum(gap, ranked[:, keep - 1] - ranked[:, keep])
        ranked = s.masked_fill(~allowed, -1.0).sort(dim=-1, descending=True).values
        if top < keep * per:
            gap = torch.minimum(gap, ranked[:, top - 1] - ranked[:, top])
        margins.append(gap)
    return weights / (weights.sum(-1, keepdim=True) + 1e-20)


# --------------------------------------------------------------------------- parts


def attention_mixer(h, w, p, c):
    T = h.shape[0]
    H, G, D, V = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    positions = torch.arange(T)
    q = rotate_neighbours((h @ w[p + "q"].T).view(T, H, D), positions, c.get("rot"))
    k = rotate_neighbours((h @ w[p + "k"].T).view(T, G, D), positions, c.get("rot"))
    v = (h @ w[p + "v"].T).view(T, G, V)
    window = (c.get("mask") or {}).get("size") or T
    mixed = windowed_attention_with_sink(q, k, v, c["scale"], window, w[p + "sink"])
    return mixed.reshape(T, H * V) @ w[p + "o"].T


def lightning_mixer(h, w, p, c, eps):
    T = h.shape[0]
    H, D, V = c["heads"], c["dim"], c["vdim"]
    q = silu(h @ w[p + "q"].T).view(T, H, D)
    k = silu(h @ w[p + "k"].T).view(T, H, D)
    v = silu(h @ w[p + "v"].T).view(T, H, V)
    o = decayed_outer_product_state(q, k, v, torch.tensor(c["decay"], dtype=h.dtype))
    o = rms_norm(o.reshape(T, H * V), w[p + "norm"], eps) * torch.sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


def gated_feed_forward(h, w, p, act):
    return (act(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def routed_feed_forward(h, w, p, c, margins=None):
    r = c["router"]
    groups = r.get("groups") or {"count": 1, "keep": 1}
    weights = routing(h, w[p + "router"], r["experts"], r["top"], groups["count"], groups["keep"],
                      margins)
    out = torch.zeros_like(h)
    for e in range(r["experts"]):
        out = out + weights[:, e:e + 1] * gated_feed_forward(h, w, f"{p}e{e}.", silu)
    if c.get("shared"):
        out = out + gated_feed_forward(h, w, p + "shared.", silu)
    return out


# --------------------------------------------------------------------------- the model


def layer_runs(cfg):
    """(layer, pass number or None): the layers in the order they run; the pass number stands
    at the first layer of each pass of the loop."""
    count, loop = len(cfg["layers"]), cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(count)]
    runs = [(i, None) for i in range(loop["start"])]
    for turn in range(loop["times"]):
        runs += [(i, turn if i == loop["start"] else None)
                 for i in range(loop["start"], loop["stop"])]
    return runs + [(i, None) for i in range(loop["stop"], count)]


def forward(cfg, w, tokens, states=None, margins=None):
    """Logits [T, vocab] of a whole sequence; ``states`` collects the stream after each run,
    ``margins`` the routing margins of every routed feed-forward that runs."""
    eps, m = cfg["norm"]["eps"], cfg.get("residual_mult", 1.0)
    x = w["embed"][torch.as_tensor(tokens)]
    embedded = x.clone()
    for index, turn in layer_runs(cfg):
        if turn is not None:
            x = torch.cat([x, embedded], -1) @ w["loop.in"].T + w["loop.step"][turn]
        layer, p = cfg["layers"][index], f"l{index}."
        h = rms_norm(x, w[p + "norm1"], eps)
        if layer["type"] == "attention":
            x = x + m * attention_mixer(h, w, p + "mix.", layer["mixer"])
        elif layer["type"] == "lightning":
            x = x + m * lightning_mixer(h, w, p + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        mlp = layer.get("mlp")
        if mlp:
            h = rms_norm(x, w[p + "norm2"], eps)
            if mlp["kind"] == "dense":
                x = x + m * gated_feed_forward(h, w, p + "mlp.", gelu_tanh)
            elif mlp["kind"] == "moe":
                x = x + m * routed_feed_forward(h, w, p + "mlp.", mlp, margins)
            else:
                raise ValueError(mlp["kind"])
        if states is not None:
            states.append(x.clone())
    z = rms_norm(x, w["final.norm"], eps) @ w["head"].T
    cap = cfg.get("logit_softcap")
    return cap * torch.tanh(z / cap) if cap else z


class PlainModel:
    def __init__(self, model_dir, kind=torch.float64):
        self.cfg = json.loads((Path(model_dir) / "config.json").read_text())
        self.w = {name: t.to(kind) for name, t in
                  read_tensors(Path(model_dir) / "model.safetensors").items()}

        self.w32 = {name: t.to(torch.float32) for name, t in self.w.items()} \
            if kind == torch.float64 else None

    def logits(self, tokens, states=None):
        """Logits [T, vocab]. The result carries ``noise`` [T], how far the same equations in
        32-bit arithmetic land from the 64-bit ones at each position (largest difference of a
        logit), and ``margin`` [T], the smallest routing margin of the position (infinite
        without routed layers): a position whose margin is tiny is decided by rounding."""
        margins = []
        out = forward(self.cfg, self.w, tokens, states, margins).float()
        out.margin = torch.stack(margins).amin(0).float() if margins \
            else torch.full((len(tokens),), math.inf)
        if self.w32 is not None:
            out.noise = (forward(self.cfg, self.w32, tokens) - out).abs().amax(dim=-1)
        return out

    def greedy(self, prompt, count):
        tokens = list(prompt)
        for _ in range(count):
            tokens.append(int(torch.argmax(self.logits(tokens)[-1])))
        return tokens[len(prompt):]
