"""A state-space mixer of the Mamba-2 kind (state-space duality), with its state in the request's slot.

One projection of the input gives ``[z | x | B | C | dt]`` (``inner = heads * head_dim`` columns for z and x,
``groups * state`` for B and C each, ``heads`` for dt).  x, B and C pass a short causal convolution per channel
(with bias) and SiLU; per head h of group g, with ``dt = softplus(dt + dt_bias)`` and ``a = -exp(A_log)``,

    S_t = exp(a_h dt_t) S_(t-1) + dt_t B_t x_t^T        (S is state x head_dim, zero when the request starts)
    y_t = S_t^T C_t + D_h x_t

then ``y * silu(z)`` is RMS-normed in ``norm_groups`` equal parts, multiplied by a gain and projected out.

What a request carries from step to step is one float32 row of its slot (``StateNeed``): the scan state
``[heads, head_dim, state]`` followed by the convolution's last ``taps - 1`` inputs ``[(taps - 1), channels]``.
The kernels reach it through ``batch.slots`` on the device, so a step in which every request brings one token can be
captured in a CUDA graph (``graph_safe``); a portion of a prompt continues from the same row, whatever its length.
The step size, the decay, the state and the sums over it are float32 in both precisions.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch

from lily_b200.parts.base import BuildContext, Mixer, StateNeed, TensorSpec, register_part


@dataclass(frozen=True)
class SSDSpec:
    hidden_size: int
    heads: int
    head_dim: int
    state: int
    groups: int
    conv_taps: int
    norm_groups: int
    norm_eps: float
    kind: str = "ssd"
    # names of the tensors under the part's prefix
    names: Optional[Tuple[Tuple[str, str], ...]] = None

    _DEFAULTS = (("in", "in_proj.weight"), ("conv", "conv1d.weight"), ("conv_bias", "conv1d.bias"), ("dt_bias", "dt_bias"),
                 ("A_log", "A_log"), ("D", "D"), ("norm", "norm.weight"), ("out", "out_proj.weight"))

    def name(self, role: str) -> str:
        return dict(self.names or ()).get(role, dict(self._DEFAULTS)[role])

    @property
    def inner(self) -> int:
        return self.heads * self.head_dim

    @property
    def channels(self) -> int:
        """Columns that pass the convolution: x, B and C."""
        return self.inner + 2 * self.groups * self.state

    @property
    def projected(self) -> int:
        return 2 * self.inner + 2 * self.groups * self.state + self.heads


@register_part("mixer", "ssd")
class SSD(Mixer):
    graph_safe = True

    def __init__(self, spec: SSDSpec, prefix: str, ctx: BuildContext):
        if spec.heads % spec.groups:
            raise ValueError(f"{spec.heads} heads do not group over {spec.groups} groups")
        if spec.inner % spec.norm_groups:
            raise ValueError(f"{spec.inner} columns do not split into {spec.norm_groups} norm groups")
        if spec.conv_taps < 1:
            raise ValueError("the convolution has at least one tap")
        self.spec, self.prefix, self.ctx = spec, prefix, ctx
        self.w_in = self.w_out = self.conv_w = self.conv_b = self.dt_bias = self.a_log = self.d_skip = self.gain = None

    # ---- what it needs ----------------------------------------------------------

    @property
    def scan_floats(self) -> int:
        return self.spec.inner * self.spec.state

    def state_need(self) -> StateNeed:
        s = self.spec
        return StateNeed((self.scan_floats + (s.conv_taps - 1) * s.channels,), torch.float32)

    def tensors(self) -> Dict[str, TensorSpec]:
        s, p = self.spec, self.prefix
        return {f"{p}.{s.name('in')}": TensorSpec((s.projected, s.hidden_size)),
                f"{p}.{s.name('conv')}": TensorSpec((s.channels, s.conv_taps), role="vector", init="normal"),
                f"{p}.{s.name('conv_bias')}": TensorSpec((s.channels,), role="vector", init="zeros"),
                f"{p}.{s.name('dt_bias')}": TensorSpec((s.heads,), role="vector", init="normal"),
                f"{p}.{s.name('A_log')}": TensorSpec((s.heads,), role="vector", init="normal"),
                f"{p}.{s.name('D')}": TensorSpec((s.heads,), role="vector", init="gain"),
                f"{p}.{s.name('norm')}": TensorSpec((s.inner,), role="vector", init="gain"),
                f"{p}.{s.name('out')}": TensorSpec((s.hidden_size, s.inner))}

    def load(self, get) -> None:
        s, p = self.spec, self.prefix
        self.w_in = get(f"{p}.{s.name('in')}").contiguous()
        self.w_out = get(f"{p}.{s.name('out')}").contiguous()
        # the small vectors enter the recurrence (or its short convolution) and are held in float32
        self.conv_w = get(f"{p}.{s.name('conv')}").float().contiguous()
        self.conv_b = get(f"{p}.{s.name('conv_bias')}").float().contiguous()
        self.dt_bias = get(f"{p}.{s.name('dt_bias')}").float().contiguous()
        self.a_log = get(f"{p}.{s.name('A_log')}").float().contiguous()
        self.d_skip = get(f"{p}.{s.name('D')}").float().contiguous()
        self.gain = get(f"{p}.{s.name('norm')}").float().contiguous()

    # ---- one step ----------------------------------------------------------------

    def forward(self, x, batch, cache, state, write_cache: bool = True):
        s, ops = self.spec, self.ctx.ops
        chunk = ops.SSM_CHUNK
        chunk_req, chunk_start = batch.plan(("token_chunks", chunk),
                                            lambda b: ops.token_chunks(b.h_new_lens, chunk, b.token_ids.device))
        proj = ops.linear(x, self.w_in)                                       # [tokens, z | x | B | C | dt]
        xbc = ops.causal_conv_silu(proj, s.inner, s.channels, self.conv_w, self.conv_b, state, self.scan_floats,
                                   chunk_req, chunk_start, batch.cu_seqlens, batch.slots, chunk)
        # long portions run as chunks side by side; what that takes is planned once a step for layers of one size
        plan = batch.plan(("scan_plan", self.scan_floats),
                          lambda b: ops.scan_plan(b.h_new_lens, b.token_ids.device, self.scan_floats))
        need = ops.scan_workspace_floats(plan, s.heads, s.head_dim, s.state)
        room = batch.workspace.floats("ssd_chunks", need) if need and batch.workspace is not None else None
        y = ops.ssd_scan(xbc, proj, s.inner + s.channels, self.dt_bias, self.a_log, self.d_skip, state,
                         batch.cu_seqlens, batch.slots, batch.num_requests, s.heads, s.head_dim, s.state, s.groups,
                         plan=plan, workspace=room)
        gated = ops.gated_group_rmsnorm(y, proj, self.gain, s.norm_groups, s.norm_eps)
        return ops.linear_auto(gated, self.w_out)
