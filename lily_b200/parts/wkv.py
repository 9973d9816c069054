"""A linear-attention mixer with a data-dependent decay (the time mixing of the RWKV family), with its state in the
request's slot.

With ``h'`` the mixer's input at the token before (zeros ahead of a request's first token), each of the five streams
r, k, v, g, w reads its own mix ``h + (h' - h) * mu_s``.  r, k, v are projections of their mixes
(``heads * head_dim`` columns), ``gate = silu(W_g mix_g)``, and the decay of a head's key channel is
``w = exp(-exp(W_2 tanh(W_1 mix_w) + w_0))`` through a low-rank pair.  Per head, with S a ``head_dim x head_dim``
matrix that is zero when the request starts,

    o_t = (S_(t-1) + diag(u) k_t v_t^T)^T r_t          (the bonus u counts for the current token only)
    S_t = diag(w_t) S_(t-1) + k_t v_t^T

then each head's o is divided by its root mean square, the heads are concatenated and multiplied by a gain and by the
gate, and projected out.

What a request carries from step to step is one float32 row of its slot (``StateNeed``): the heads' matrices
``[heads, head_dim, head_dim]`` followed by the mixer's input at the request's last token ``[hidden]``.  The kernels
reach it through ``batch.slots`` on the device, so a step in which every request brings one token can be captured in a
CUDA graph (``graph_safe``); a portion of a prompt continues from the same row, whatever its length.  The decay and its
logarithm (from the low-rank product on: tanh, the second product, the exponentials), the state, the sums over it and
the unit norm are float32 in both precisions.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch

from lily_b200.parts.base import BuildContext, Mixer, StateNeed, TensorSpec, register_part

STREAMS = ("r", "k", "v", "g", "w")


@dataclass(frozen=True)
class WkvSpec:
    hidden_size: int
    heads: int
    head_dim: int
    decay_rank: int
    norm_eps: float
    kind: str = "wkv"
    # names of the tensors under the part's prefix
    names: Optional[Tuple[Tuple[str, str], ...]] = None

    _DEFAULTS = tuple((f"mu_{s}", f"mu.{s}") for s in STREAMS) + (
        ("r", "r"), ("k", "k"), ("v", "v"), ("g", "g"), ("w1", "w1"), ("w2", "w2"), ("w0", "w0"), ("u", "u"),
        ("norm", "norm"), ("o", "o"))

    def name(self, role: str) -> str:
        return dict(self.names or ()).get(role, dict(self._DEFAULTS)[role])

    @property
    def inner(self) -> int:
        return self.heads * self.head_dim


@register_part("mixer", "wkv")
class Wkv(Mixer):
    graph_safe = True

    def __init__(self, spec: WkvSpec, prefix: str, ctx: BuildContext):
        if min(spec.heads, spec.head_dim, spec.decay_rank) < 1:
            raise ValueError("heads, head size and the decay's rank are positive")
        self.spec, self.prefix, self.ctx = spec, prefix, ctx
        self.mu = self.w_r = self.w_k = self.w_v = self.w_g = self.w_1 = self.w_2t = self.w_0 = self.u = self.gain = self.w_o = None

    # ---- what it needs ----------------------------------------------------------

    @property
    def matrix_floats(self) -> int:
        return self.spec.heads * self.spec.head_dim * self.spec.head_dim

    def state_need(self) -> StateNeed:
        return StateNeed((self.matrix_floats + self.spec.hidden_size,), torch.float32)

    def tensors(self) -> Dict[str, TensorSpec]:
        s, p = self.spec, self.prefix
        out = {f"{p}.{s.name('mu_' + x)}": TensorSpec((s.hidden_size,), role="vector", init="normal") for x in STREAMS}
        out.update({f"{p}.{s.name(x)}": TensorSpec((s.inner, s.hidden_size)) for x in ("r", "k", "v", "g")})
        out.update({f"{p}.{s.name('w1')}": TensorSpec((s.decay_rank, s.hidden_size)),
                    f"{p}.{s.name('w2')}": TensorSpec((s.inner, s.decay_rank)),
                    f"{p}.{s.name('w0')}": TensorSpec((s.inner,), role="vector", init="normal"),
                    f"{p}.{s.name('u')}": TensorSpec((s.heads, s.head_dim), role="vector", init="normal"),
                    f"{p}.{s.name('norm')}": TensorSpec((s.inner,), role="vector", init="gain"),
                    f"{p}.{s.name('o')}": TensorSpec((s.hidden_size, s.inner))})
        return out

    def load(self, get) -> None:
        s, p = self.spec, self.prefix
        g = lambda role: get(f"{p}.{s.name(role)}")
        self.mu = torch.stack([g("mu_" + x).float() for x in STREAMS]).contiguous()        # [5, hidden]
        self.w_r, self.w_k, self.w_v, self.w_g = (g(x).contiguous() for x in ("r", "k", "v", "g"))
        self.w_1 = g("w1").contiguous()
        # from tanh on the decay's path is float32: the second matrix of the pair (transposed for the kernel), w_0, u
        self.w_2t = g("w2").float().t().contiguous()
        self.w_0 = g("w0").float().contiguous()
        self.u = g("u").float().contiguous()
        self.gain = g("norm").float().contiguous()
        self.w_o = g("o").contiguous()

    # ---- one step ----------------------------------------------------------------

    def forward(self, x, batch, cache, state, write_cache: bool = True):
        s, ops = self.spec, self.ctx.ops
        mixes = ops.token_shift_mix(x, self.mu, state, self.matrix_floats, batch.cu_seqlens, batch.token_req, batch.slots)
        r = ops.linear(mixes[0], self.w_r)
        k = ops.linear(mixes[1], self.w_k)
        v = ops.linear(mixes[2], self.w_v)
        gate = ops.linear(mixes[3], self.w_g)
        low = ops.linear(mixes[4], self.w_1, out_dtype=torch.float32)            # [tokens, rank], float32 from here on
        log_decay = ops.wkv_decay(low, self.w_2t, self.w_0)
        # long portions run as chunks side by side; the cut is planned once a step for all layers
        plan = batch.plan(("wkv_plan",), lambda b: ops.wkv_plan(b.h_new_lens, b.token_ids.device))
        need = ops.wkv_workspace_floats(plan, s.heads, s.head_dim)
        room = batch.workspace.floats("wkv_chunks", need) if need and batch.workspace is not None else None
        if need and room is None:
            plan = None                                    # no scratch to be had: every portion runs whole
        y = ops.wkv_scan(r, k, v, log_decay, self.u, state, batch.cu_seqlens, batch.slots, batch.num_requests, s.heads,
                         s.head_dim, plan=plan, workspace=room)
        normed = ops.group_rmsnorm_gate(y, gate, self.gain, s.heads, s.norm_eps)
        return ops.linear_auto(normed, self.w_o)
