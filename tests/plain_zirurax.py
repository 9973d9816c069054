"""Plain, slow implementation of the Zirurax decoder, for tests only.

Whole sequences, no cache, one function per mechanism, float32 on the CPU unless
``precision(torch.float64)`` is in force.  It reads the raw ``config.json`` dictionary and the
checkpoint's own tensor names and shares no code with ``lily_b200``.

The design in this file's notation.  A layer is ``x <- x + mixer(h) + ff(h)`` with ``h = rms(x) * w``.
The mixer runs a windowed, soft-capped, gated softmax attention ("left") and a Mamba-2 state-space layer
("right") on the same ``h`` and returns ``(rms(left) * w_l + rms(right) * w_r) / 2``.  The feed-forward is
``down(gelu_tanh(gate h) * up h)``.  The logits are the final norm times the embedding table.
"""

from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import torch

Tensor = torch.Tensor

_COMPUTE = [torch.float32]


class precision:
    def __init__(self, dtype):
        self.dtype = dtype

    def __enter__(self):
        _COMPUTE.append(self.dtype)

    def __exit__(self, *exc):
        _COMPUTE.pop()


def _c(t: Tensor) -> Tensor:
    return t.to(_COMPUTE[-1])


def rms(x: Tensor, eps: float) -> Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def gelu_tanh(z: Tensor) -> Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def softplus(z: Tensor) -> Tensor:
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


# --------------------------------------------------------------------------- rotation

def rotary_frequencies(rot: dict) -> Tensor:
    """f_i = base^(-2i/dims), then the three-band rescaling by wavelength when ``scaling`` is given."""
    dims = rot["dims"]
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = float(rot["base"]) ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if sc:
        factor, low, high, orig = float(sc["factor"]), float(sc["low"]), float(sc["high"]), float(sc["original"])
        wave = 2.0 * math.pi / f
        out = f.clone()
        long_ = wave > orig / low
        out[long_] = f[long_] / factor
        mid = ~(wave < orig / high) & ~long_
        if high != low:
            s = (orig / wave - low) / (high - low)
            out[mid] = ((1.0 - s) * f / factor + s * f)[mid]
        f = out
    return f.to(torch.float32)


def rotate_interleaved(x: Tensor, positions: Tensor, freqs: Tensor) -> Tensor:
    """x [tokens, heads, dim]: features (2i, 2i+1) of the first 2 * len(freqs) are rotated by position * f_i."""
    n = freqs.numel()
    ang = positions.to(torch.float32)[:, None] * freqs[None, :]          # float32 angles
    cos, sin = _c(ang.cos())[:, None, :], _c(ang.sin())[:, None, :]
    u, v = x[..., 0:2 * n:2], x[..., 1:2 * n:2]
    out = x.clone()
    out[..., 0:2 * n:2] = u * cos - v * sin
    out[..., 1:2 * n:2] = v * cos + u * sin
    return out


# --------------------------------------------------------------------------- left: attention

def windowed_softcap_attention(q: Tensor, k: Tensor, v: Tensor, scale: float, softcap: Optional[float],
                               window: Optional[int]) -> Tensor:
    """q [t, H, d], k [t, G, d], v [t, G, dv] -> [t, H, dv].  Query i sees key j when 0 <= i - j < window."""
    t, heads, _ = q.shape
    per = heads // k.shape[1]
    i = torch.arange(t)[:, None]
    j = torch.arange(t)[None, :]
    seen = (j <= i) if window is None else ((j <= i) & (i - j < window))
    out = []
    for h in range(heads):
        s = (q[:, h] @ k[:, h // per].t()) * scale
        if softcap:
            s = softcap * torch.tanh(s / softcap)
        s = s.masked_fill(~seen, float("-inf"))
        out.append(torch.softmax(s, -1) @ v[:, h // per])
    return torch.stack(out, 1)


def left_mixer(h: Tensor, w: Dict[str, Tensor], p: str, c: dict, positions: Tensor) -> Tensor:
    t = h.shape[0]
    heads, kvh, d, dv = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    q = (h @ _c(w[f"{p}.q"]).t()).view(t, heads, d)
    k = (h @ _c(w[f"{p}.k"]).t()).view(t, kvh, d)
    v = (h @ _c(w[f"{p}.v"]).t()).view(t, kvh, dv)
    rot = c.get("rot")
    if rot:
        f = rotary_frequencies(rot)
        q, k = rotate_interleaved(q, positions, f), rotate_interleaved(k, positions, f)
    window = (c.get("mask") or {}).get("size")
    o = windowed_softcap_attention(q, k, v, float(c["scale"]), c.get("softcap"), window).reshape(t, heads * dv)
    o = o * torch.sigmoid(h @ _c(w[f"{p}.g"]).t())
    return o @ _c(w[f"{p}.o"]).t()


# --------------------------------------------------------------------------- right: state-space layer

def causal_conv(x: Tensor, taps: Tensor, bias: Tensor) -> Tensor:
    """x [t, channels], taps [channels, k] (last column multiplies the current token), zeros before the start."""
    t, ch = x.shape
    k = taps.shape[1]
    padded = torch.cat([x.new_zeros(k - 1, ch), x])
    out = bias[None, :].expand(t, ch).clone()
    for j in range(k):
        out = out + padded[j:j + t] * taps[:, j][None, :]
    return out


def ssd_scan(x: Tensor, dt: Tensor, a: Tensor, b: Tensor, cc: Tensor, d_skip: Tensor) -> Tensor:
    """x [t, heads, p], dt [t, heads], a [heads] (negative rates), b and cc [t, groups, n]:
    S_t = exp(a dt_t) S_(t-1) + dt_t b_t x_t^T,  y_t = S_t^T c_t + D x_t."""
    t, heads, p = x.shape
    groups, n = b.shape[1], b.shape[2]
    per = heads // groups
    state = x.new_zeros(heads, n, p)
    ys = []
    for s in range(t):
        bs = b[s].repeat_interleave(per, 0)               # [heads, n]
        cs = cc[s].repeat_interleave(per, 0)
        decay = torch.exp(a * dt[s])                      # [heads]
        state = decay[:, None, None] * state + dt[s][:, None, None] * bs[:, :, None] * x[s][:, None, :]
        ys.append(torch.einsum("hnp,hn->hp", state, cs) + d_skip[:, None] * x[s])
    return torch.stack(ys)


def grouped_rms(y: Tensor, parts: int, eps: float) -> Tensor:
    t, width = y.shape
    return rms(y.view(t, parts, width // parts), eps).view(t, width)


def right_mixer(h: Tensor, w: Dict[str, Tensor], p: str, c: dict, eps: float) -> Tensor:
    t = h.shape[0]
    heads, pd, n, groups = c["heads"], c["vdim"], c["state"], c["groups"]
    inner = heads * pd
    proj = h @ _c(w[f"{p}.in"]).t()
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * groups * n], proj[:, 2 * inner + 2 * groups * n:]
    xbc = causal_conv(xbc, _c(w[f"{p}.conv"]), _c(w[f"{p}.conv.b"]))
    xbc = xbc * torch.sigmoid(xbc)
    x = xbc[:, :inner].view(t, heads, pd)
    b = xbc[:, inner:inner + groups * n].view(t, groups, n)
    cc = xbc[:, inner + groups * n:].view(t, groups, n)
    dt = softplus(dt + _c(w[f"{p}.dt_bias"]))
    a = -torch.exp(_c(w[f"{p}.A_log"]))
    y = ssd_scan(x, dt, a, b, cc, _c(w[f"{p}.D"])).reshape(t, inner)
    y = y * (z * torch.sigmoid(z))
    y = grouped_rms(y, c["norm_groups"], eps) * _c(w[f"{p}.norm"])
    return y @ _c(w[f"{p}.o"]).t()


# --------------------------------------------------------------------------- layer, model

def parallel_mixer(h: Tensor, w: Dict[str, Tensor], p: str, c: dict, eps: float, positions: Tensor) -> Tensor:
    left = left_mixer(h, w, f"{p}.left", c["left"], positions)
    right = right_mixer(h, w, f"{p}.right", c["right"], eps)
    return 0.5 * (rms(left, eps) * _c(w[f"{p}.left.out"]) + rms(right, eps) * _c(w[f"{p}.right.out"]))


def feed_forward(h: Tensor, w: Dict[str, Tensor], p: str) -> Tensor:
    return (gelu_tanh(h @ _c(w[f"{p}.gate"]).t()) * (h @ _c(w[f"{p}.up"]).t())) @ _c(w[f"{p}.down"]).t()


def forward(cfg: dict, w: Dict[str, Tensor], ids: Sequence[int], layers_out: Optional[List[Tensor]] = None) -> Tensor:
    """Logits [tokens, vocab] of one whole sequence; ``layers_out`` collects the stream after each layer."""
    eps = float(cfg["norm"]["eps"])
    positions = torch.arange(len(ids))
    x = _c(w["embed"])[torch.tensor(list(ids))] * float(cfg["embedding"]["scale"])
    for i, layer in enumerate(cfg["layers"]):
        if layer["type"] != "parallel":
            raise ValueError(f"layer type {layer['type']!r}")
        h = rms(x, eps) * _c(w[f"l{i}.norm1"])
        delta = parallel_mixer(h, w, f"l{i}.mix", layer["mixer"], eps, positions)
        if layer.get("mlp"):
            if layer["mlp"]["kind"] != "dense":
                raise ValueError(f"feed-forward kind {layer['mlp']['kind']!r}")
            delta = delta + feed_forward(h, w, f"l{i}.mlp")
        x = x + delta
        if layers_out is not None:
            layers_out.append(x.clone())
    return (rms(x, eps) * _c(w["final.norm"])) @ _c(w["embed"]).t()
