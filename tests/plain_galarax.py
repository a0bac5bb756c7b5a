"""Plain, slow Galarax written from the design's equations: whole sequences, no cache, one
function per mechanism. It shares no code with the engine: it reads config.json and the
safetensors file by itself and computes everything in one floating type (float64 by default).

Notation: x [T, W] the stream, h the normed input of a mixer, T tokens at positions 0..T-1.
"""

from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import torch

# --------------------------------------------------------------------------- loading

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


def rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_around_zero(x, w, eps):
    return rms(x, eps) * (1 + w)


def silu(z):
    return z / (1 + torch.exp(-z))


def rotary_frequencies(rot, kind):
    """Frequencies of the pairs and the factor on cosine and sine."""
    dims, base = rot["dims"], rot["base"]
    i = torch.arange(dims // 2, dtype=kind)
    f = base ** (-2 * i / dims)
    scaling = rot.get("scaling")
    if not scaling:
        return f, 1.0
    factor = scaling["factor"]
    d = lambda t: dims * math.log(scaling["original"] / (2 * math.pi * t)) / (2 * math.log(base))
    lo = max(math.floor(d(scaling["fast"])), 0)
    hi = min(math.ceil(d(scaling["slow"])), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0, 1)
    return f / factor * ramp + f * (1 - ramp), 0.1 * math.log(factor) + 1


def rotate(x, positions, rot):
    """x [T, heads, D]: the pair (i, i + dims/2) of the first dims dimensions is turned by
    position * frequency_i, cosine and sine scaled; the other dimensions pass."""
    if not rot:
        return x
    f, amplitude = rotary_frequencies(rot, x.dtype)
    dims, half = rot["dims"], rot["dims"] // 2
    angle = positions.to(x.dtype)[:, None] * f[None, :]
    cos, sin = (torch.cos(angle) * amplitude)[:, None, :], (torch.sin(angle) * amplitude)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., dims:]], -1)


def causal_softmax_attention(q, k, v, scale):
    """q [T, H, D], k [T, G, D], v [T, G, V] -> [T, H, V]; head h reads key head h // (H/G)."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[-1], dtype=q.dtype)
    visible = torch.tril(torch.ones(T, T, dtype=torch.bool))
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        s = s.masked_fill(~visible, -math.inf)
        out[:, h] = torch.softmax(s, -1) @ v[:, g]
    return out


def causal_conv(x, w):
    """x [T, C], w [C, taps] (last column the current token's), zeros before the start."""
    T, taps = x.shape[0], w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, x.shape[1], dtype=x.dtype), x], 0)
    return sum(padded[j:j + T] * w[:, j] for j in range(taps))


def delta_recurrence(q, k, v, beta, g):
    """q, k [T, G, D], v [T, H, V], beta, g [T, H] -> o [T, H, V], from a zero state.
    Per token: S = g S; u = beta (v - S^T k); S = S + k u^T; o = S^T q."""
    T, H, V = v.shape
    G, D = q.shape[1], q.shape[2]
    o = torch.zeros(T, H, V, dtype=v.dtype)
    for h in range(H):
        j = h // (H // G)
        S = torch.zeros(D, V, dtype=v.dtype)
        for t in range(T):
            S = g[t, h] * S
            u = beta[t, h] * (v[t, h] - S.T @ k[t, j])
            S = S + torch.outer(k[t, j], u)
            o[t, h] = S.T @ q[t, j]
    return o


# --------------------------------------------------------------------------- mixers


def left_mixer(h, w, p, c, eps):
    T = h.shape[0]
    H, G, D, V = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    q = (h @ w[p + "q"].T + w[p + "q.b"]).view(T, H, D)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).view(T, G, D)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).view(T, G, V)
    positions = torch.arange(T)
    q, k = rms(rotate(q, positions, c.get("rot")), eps), rms(rotate(k, positions, c.get("rot")), eps)
    mixed = causal_softmax_attention(q, k, v, c["scale"])
    return mixed.reshape(T, H * V) @ w[p + "o"].T


def right_mixer(h, w, p, c, eps):
    T = h.shape[0]
    H, G, D, V = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    unit = lambda x: x / torch.sqrt((x * x).sum(-1, keepdim=True) + 1e-6)
    q = unit(silu(causal_conv(h @ w[p + "q"].T, w[p + "q.conv"])).view(T, G, D)) * D ** -0.5
    k = unit(silu(causal_conv(h @ w[p + "k"].T, w[p + "k.conv"])).view(T, G, D))
    v = silu(causal_conv(h @ w[p + "v"].T, w[p + "v.conv"])).view(T, H, V)
    beta = torch.sigmoid(h @ w[p + "b"].T)
    g = torch.exp(-torch.exp(w[p + "A_log"]) *
                  torch.nn.functional.softplus(h @ w[p + "a"].T + w[p + "dt_bias"]))
    o = delta_recurrence(q, k, v, beta, g)
    o = rms(o, eps) * w[p + "norm"] * silu(h @ w[p + "g"].T).view(T, H, V)
    return o.reshape(T, H * V) @ w[p + "o"].T


def parallel_mixer(h, w, p, c, eps):
    a = left_mixer(h, w, p + "left.", c["left"], eps)
    b = right_mixer(h, w, p + "right.", c["right"], eps)
    return 0.5 * (rms(a, eps) * w[p + "left.out"] + rms(b, eps) * w[p + "right.out"])


def dense_feed_forward(h, w, p):
    return torch.relu(h @ w[p + "up"].T) ** 2 @ w[p + "down"].T


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


def forward(cfg, w, tokens, states=None):
    """Logits [T, vocab] of a whole sequence; ``states`` collects the stream after each run."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.as_tensor(tokens)]
    embedded = x.clone()
    for index, turn in layer_runs(cfg):
        if turn is not None:
            if turn > 0:
                x = x + embedded
            x = x + w["loop.step"][turn]
        layer, p = cfg["layers"][index], f"l{index}."
        x = x + parallel_mixer(norm_around_zero(x, w[p + "norm1"], eps), w, p + "mix.",
                               layer["mixer"], eps)
        if layer.get("mlp"):
            x = x + dense_feed_forward(norm_around_zero(x, w[p + "norm2"], eps), w, p + "mlp.")
        if states is not None:
            states.append(x.clone())
    return norm_around_zero(x, w["final.norm"], eps) @ w["head"].T


class PlainModel:
    def __init__(self, model_dir, kind=torch.float64):
        self.cfg = json.loads((Path(model_dir) / "config.json").read_text())
        self.w = {name: t.to(kind) for name, t in
                  read_tensors(Path(model_dir) / "model.safetensors").items()}
        self.w32 = {name: t.to(torch.float32) for name, t in self.w.items()} \
            if kind == torch.float64 else None

    def logits(self, tokens, states=None):
        """Logits [T, vocab]. The result carries ``noise`` [T]: how far the same equations in
        32-bit arithmetic land from the 64-bit ones at each position (largest difference of a
        logit), a measure of how well the position's logits are determined at all."""
        out = forward(self.cfg, self.w, tokens, states).float()
        if self.w32 is not None:
            out.noise = (forward(self.cfg, self.w32, tokens) - out).abs().amax(dim=-1)
        return out

    def greedy(self, prompt, count):
        tokens = list(prompt)
        for _ in range(count):
            tokens.append(int(torch.argmax(self.logits(tokens)[-1])))
        return tokens[len(prompt):]
