"""A routed mixture of small gated feed-forward layers, some of whose router outputs stand for the identity.

The router scores ``s = softmax(W_router h)`` over all its outputs (logits and softmax in float32).  The ``top`` outputs
with the largest ``s + correction`` are chosen; their weights are their scores ``s`` (without the correction) divided
by the sum of the chosen scores.  The first ``experts`` outputs name experts with weights of their own,

    y = W_down (g * sigmoid(alpha g) * (u + 1)),   g = min(W_gate h, limit),   u = clamp(W_up h, -limit, limit),

the last ``identity`` outputs name experts without tensors whose output is ``h`` itself.  The result is the weighted
sum of the chosen outputs, returned in float32 as one plane of partial sums for the next residual add.

Routing, grouping by expert and the grouped products all stay on the device (``ops.moe_route``, ``ops.moe_experts``):
nothing is read back by the host, so a step replays from a CUDA graph, and each (token, choice) pair is a row of a
grouped product whose sum runs over k in a fixed order, so a token's result does not depend on its neighbours in the
batch.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch

from lily_b200.parts.base import BuildContext, FeedForward, TensorSpec, register_part


@dataclass(frozen=True)
class RoutedExpertsSpec:
    hidden_size: int
    intermediate_size: int        # of one expert
    experts: int                  # router outputs with weights of their own
    identity: int                 # router outputs after those that stand for the identity
    top: int
    limit: float                  # the clamp on the gate (from above) and on the up product (both sides)
    alpha: float = 1.702          # the slope inside the gate's sigmoid
    kind: str = "routed_experts"
    # names under the part's prefix: the router, its correction, and the pattern of an expert's prefix
    names: Optional[Tuple[Tuple[str, str], ...]] = None

    _DEFAULTS = (("router", "router"), ("correction", "correction"), ("expert", "e{}"), ("gate", "gate"), ("up", "up"),
                 ("down", "down"))

    def name(self, role: str) -> str:
        return dict(self.names or ()).get(role, dict(self._DEFAULTS)[role])

    @property
    def outputs(self) -> int:
        return self.experts + self.identity


@register_part("feed_forward", "routed_experts")
class RoutedExperts(FeedForward):
    def __init__(self, spec: RoutedExpertsSpec, prefix: str, ctx: BuildContext):
        if spec.experts < 0 or spec.identity < 0 or not 1 <= spec.top <= spec.outputs:
            raise ValueError(f"top {spec.top} of {spec.experts} experts and {spec.identity} identity outputs")
        self.spec, self.prefix, self.ctx = spec, prefix, ctx
        self.router = self.correction = self.w_gate_up = self.w_down = None

    def _expert(self, e: int, role: str) -> str:
        return f"{self.prefix}.{self.spec.name('expert').format(e)}.{self.spec.name(role)}"

    def tensors(self) -> Dict[str, TensorSpec]:
        s, p = self.spec, self.prefix
        out = {f"{p}.{s.name('router')}": TensorSpec((s.outputs, s.hidden_size)),
               f"{p}.{s.name('correction')}": TensorSpec((s.outputs,), role="vector", init="zeros")}
        for e in range(s.experts):
            out[self._expert(e, "gate")] = TensorSpec((s.intermediate_size, s.hidden_size))
            out[self._expert(e, "up")] = TensorSpec((s.intermediate_size, s.hidden_size))
            out[self._expert(e, "down")] = TensorSpec((s.hidden_size, s.intermediate_size))
        return out

    def load(self, get) -> None:
        s, p = self.spec, self.prefix
        self.router = get(f"{p}.{s.name('router')}").float().contiguous()           # the router works in float32
        self.correction = get(f"{p}.{s.name('correction')}").float().contiguous()
        ff, h = s.intermediate_size, s.hidden_size
        if s.experts:
            first = get(self._expert(0, "gate"))
            self.w_gate_up = torch.empty((s.experts, 2 * ff, h), dtype=first.dtype, device=first.device)
            self.w_down = torch.empty((s.experts, h, ff), dtype=first.dtype, device=first.device)
            for e in range(s.experts):
                self.w_gate_up[e, :ff].copy_(get(self._expert(e, "gate")))
                self.w_gate_up[e, ff:].copy_(get(self._expert(e, "up")))
                self.w_down[e].copy_(get(self._expert(e, "down")))
        else:
            self.w_gate_up = self.w_down = torch.empty((0,), dtype=self.ctx.dtype, device=self.router.device)

    def forward(self, x, batch):
        s, ops = self.spec, self.ctx.ops
        routing = ops.moe_route(x, self.router, self.correction, s.top, s.experts)
        out = ops.moe_experts(x, routing, self.w_gate_up, self.w_down, s.limit, s.alpha)
        return out.unsqueeze(0)                   # float32 [1, tokens, hidden]: one plane of partial sums
