"""Plain, slow implementation of the Godotar decoder, for tests only.

Whole sequences, no cache, one function per mechanism, float32 on the CPU unless
``precision(torch.float64)`` is in force.  It reads the raw ``config.json`` dictionary and the
checkpoint's own tensor names and shares no code with ``lily_b200``.

The design in this file's notation.  ``nrm(x, w) = x / sqrt(mean(x^2) + eps) * (1 + w)``.  The stream starts as
``x = nrm(E[token], w_embed)``.  A layer is ``x <- x + mixer(nrm(x, w1)) + ff(nrm(x, w2))``; the mixer is a
linear-attention recurrence with data-dependent decay ("wkv") or a softmax attention over a low-rank latent of
keys and values ("latent_attention"); the feed-forward is dense or a routed mixture with identity experts.  A
stretch of layers runs several times over with the same weights, each pass with a state of its own and a learned
vector added to ``x`` ahead of it.  The logits are ``logit_scale * E nrm(x, w_final)``.
"""

from __future__ import annotations

from typing import Dict, List, Optional, Tuple

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


def unit_rms(x: Tensor, eps: float) -> Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def offset_norm(x: Tensor, w: Tensor, eps: float) -> Tensor:
    """The model's norm: its gain is stored as a difference from one."""
    return unit_rms(x, eps) * (1.0 + _c(w))


def silu(z: Tensor) -> Tensor:
    return z * torch.sigmoid(z)


# --------------------------------------------------------------------------- wkv

def token_shift(h: Tensor, mu: Tensor, first: Optional[Tensor] = None) -> Tensor:
    """h_t + (h_(t-1) - h_t) * mu, with zeros (or ``first``) ahead of the first token."""
    prev = torch.cat([torch.zeros_like(h[:1]) if first is None else first[None], h[:-1]], 0)
    return h + (prev - h) * _c(mu)


def wkv_decay(mix_w: Tensor, w: Dict[str, Tensor], p: str) -> Tensor:
    """exp(-exp(W2 tanh(W1 m) + w0)): a number in (0, 1) for every head and key channel."""
    z = torch.tanh(mix_w @ _c(w[f"{p}.w1"]).t()) @ _c(w[f"{p}.w2"]).t() + _c(w[f"{p}.w0"])
    return torch.exp(-torch.exp(z))


def wkv_recurrence(r: Tensor, k: Tensor, v: Tensor, decay: Tensor, u: Tensor,
                   state: Optional[Tensor] = None) -> Tuple[Tensor, Tensor]:
    """r, k, v, decay [t, H, d]; u [H, d]; state [H, d(key), d(value)].  Token by token:
    o_t[j] = sum_i r_t[i] (S[i, j] + u[i] k_t[i] v_t[j]);  S[i, j] <- decay_t[i] S[i, j] + k_t[i] v_t[j]."""
    t, heads, d = r.shape
    S = torch.zeros(heads, d, d, dtype=r.dtype) if state is None else state.clone()
    out = torch.zeros(t, heads, d, dtype=r.dtype)
    for n in range(t):
        kv = k[n][:, :, None] * v[n][:, None, :]
        out[n] = torch.einsum("hi,hij->hj", r[n], S + u[:, :, None] * kv)
        S = decay[n][:, :, None] * S + kv
    return out, S


def wkv_mixer(h: Tensor, w: Dict[str, Tensor], p: str, c: dict, eps: float) -> Tensor:
    t = h.shape[0]
    heads, d = c["heads"], c["dim"]
    proj = lambda name, m: (m @ _c(w[f"{p}.{name}"]).t())
    r = proj("r", token_shift(h, w[f"{p}.mu.r"])).view(t, heads, d)
    k = proj("k", token_shift(h, w[f"{p}.mu.k"])).view(t, heads, d)
    v = proj("v", token_shift(h, w[f"{p}.mu.v"])).view(t, heads, d)
    gate = silu(proj("g", token_shift(h, w[f"{p}.mu.g"])))
    decay = wkv_decay(token_shift(h, w[f"{p}.mu.w"]), w, p).view(t, heads, d)
    o, _ = wkv_recurrence(r, k, v, decay, _c(w[f"{p}.u"]))
    o = unit_rms(o, eps).reshape(t, heads * d) * _c(w[f"{p}.norm"]) * gate
    return o @ _c(w[f"{p}.o"]).t()


# --------------------------------------------------------------------------- latent attention

def rotate_halves(x: Tensor, positions: Tensor, dims: int, base: float) -> Tensor:
    """x [t, ..., n]: feature i of the first ``dims`` is paired with feature i + dims / 2 and the pair is turned by
    the angle position * base^(-2 i / dims); the rest passes."""
    half = dims // 2
    f = (float(base) ** (-2.0 * torch.arange(half, dtype=torch.float64) / dims)).to(torch.float32)
    ang = positions.to(torch.float32)[:, None] * f[None, :]                # float32 angles
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    cos, sin = _c(ang.cos()).view(shape), _c(ang.sin()).view(shape)
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., dims:]], -1)


def windowed_softmax(scores: Tensor, window: Optional[int]) -> Tensor:
    """scores [t, t] (query, key): query i sees key j when 0 <= i - j < window."""
    t = scores.shape[0]
    i = torch.arange(t)[:, None]
    j = torch.arange(t)[None, :]
    seen = (j <= i) if window is None else ((j <= i) & (i - j < window))
    return torch.softmax(scores.masked_fill(~seen, float("-inf")), -1)


def latent_attention_mixer(h: Tensor, w: Dict[str, Tensor], p: str, c: dict, eps: float, positions: Tensor) -> Tensor:
    t = h.shape[0]
    heads, d, dr, dv, rank = c["heads"], c["dim"], c["rot_dim"], c["vdim"], c["kv_rank"]
    rot = c["rot"]
    cq = unit_rms(h @ _c(w[f"{p}.dq"]).t(), eps) * _c(w[f"{p}.dq.norm"])
    q = (cq @ _c(w[f"{p}.uq"]).t()).view(t, heads, d + dr)
    q_plain, q_rot = q[..., :d], rotate_halves(q[..., d:], positions, rot["dims"], rot["base"])
    down = h @ _c(w[f"{p}.dkv"]).t()
    latent = unit_rms(down[:, :rank], eps) * _c(w[f"{p}.dkv.norm"])
    k_rot = rotate_halves(down[:, rank:], positions, rot["dims"], rot["base"])      # one for all heads
    k_plain = (latent @ _c(w[f"{p}.uk"]).t()).view(t, heads, d)
    v = (latent @ _c(w[f"{p}.uv"]).t()).view(t, heads, dv)
    gate = torch.sigmoid(h @ _c(w[f"{p}.g"]).t())                           # [t, heads]
    window = (c.get("mask") or {}).get("size")
    out = []
    for n in range(heads):
        s = (q_plain[:, n] @ k_plain[:, n].t() + q_rot[:, n] @ k_rot.t()) * float(c["scale"])
        out.append((windowed_softmax(s, window) @ v[:, n]) * gate[:, n:n + 1])
    return torch.cat(out, -1) @ _c(w[f"{p}.o"]).t()


# --------------------------------------------------------------------------- feed-forward

def dense_ff(h: Tensor, w: Dict[str, Tensor], p: str) -> Tensor:
    return (silu(h @ _c(w[f"{p}.gate"]).t()) * (h @ _c(w[f"{p}.up"]).t())) @ _c(w[f"{p}.down"]).t()


def clamped_expert(h: Tensor, w: Dict[str, Tensor], p: str, limit: float) -> Tensor:
    g = torch.clamp(h @ _c(w[f"{p}.gate"]).t(), max=limit)
    u = torch.clamp(h @ _c(w[f"{p}.up"]).t(), min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ _c(w[f"{p}.down"]).t()


def route(h: Tensor, w: Dict[str, Tensor], p: str, top: int) -> Tuple[Tensor, Tensor]:
    """(chosen experts [t, top], their weights [t, top]).  The choice is by softmax score plus a correction; the
    weights are the scores themselves, renormalised over the chosen."""
    s = torch.softmax(h.float() @ w[f"{p}.router"].float().t(), -1)
    chosen = torch.topk(s + w[f"{p}.correction"].float(), top, dim=-1).indices
    picked = torch.gather(s, 1, chosen)
    return chosen, picked / (picked.sum(-1, keepdim=True) + 1e-20)


def moe_ff(h: Tensor, w: Dict[str, Tensor], p: str, c: dict) -> Tensor:
    experts, top = c["router"]["experts"], c["router"]["top"]
    chosen, weights = route(h, w, p, top)
    out = torch.zeros_like(h)
    for n in range(h.shape[0]):
        for e, a in zip(chosen[n].tolist(), weights[n].tolist()):
            x = h[n:n + 1]
            y = clamped_expert(x, w, f"{p}.e{e}", float(c["expert"]["limit"])) if e < experts else x      # identity experts
            out[n] += a * y[0]
    return out


# --------------------------------------------------------------------------- the model

def layer_runs(cfg: dict) -> List[Tuple[int, Optional[int]]]:
    """(layer, number of the pass that starts ahead of it or None) in running order."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    start, stop, times = loop["start"], loop["stop"], loop["times"]
    runs: List[Tuple[int, Optional[int]]] = [(i, None) for i in range(start)]
    for t in range(times):
        runs += [(i, t if i == start else None) for i in range(start, stop)]
    return runs + [(i, None) for i in range(stop, n)]


def forward(cfg: dict, w: Dict[str, Tensor], tokens, return_layers: bool = False):
    """Logits [t, vocab] of one sequence (and, on request, the stream after every layer run)."""
    eps = float(cfg["norm"]["eps"])
    ids = torch.as_tensor(tokens, dtype=torch.long)
    positions = torch.arange(len(ids))
    E = _c(w["embed"])
    x = offset_norm(E[ids], w["embed.norm"], eps)
    seen = []
    for i, starts_pass in layer_runs(cfg):
        ly, p = cfg["layers"][i], f"l{i}"
        if starts_pass is not None:
            x = x + _c(w["loop.step"])[starts_pass]
        h1 = offset_norm(x, w[f"{p}.norm1"], eps)
        if ly["type"] == "wkv":
            y = wkv_mixer(h1, w, f"{p}.mix", ly["mixer"], eps)
        elif ly["type"] == "latent_attention":
            y = latent_attention_mixer(h1, w, f"{p}.mix", ly["mixer"], eps, positions)
        else:
            raise ValueError(ly["type"])
        mlp = ly.get("mlp")
        if mlp is not None:
            h2 = offset_norm(x, w[f"{p}.norm2"], eps)
            y = y + (dense_ff(h2, w, f"{p}.mlp") if mlp["kind"] == "dense" else moe_ff(h2, w, f"{p}.mlp", mlp))
        x = x + y
        seen.append(x)
    logits = (offset_norm(x, w["final.norm"], eps) @ E.t()) * float(cfg.get("logit_scale", 1.0))
    return (logits, torch.stack(seen)) if return_layers else logits
