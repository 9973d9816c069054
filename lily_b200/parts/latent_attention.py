"""Softmax attention over a low-rank latent of keys and values, with the latent alone in the paged cache.

Queries go through a latent of their own: ``c_q = rms(W_dq h) * g_q``, ``q = W_uq c_q``, head by head
``[head_dim unrotated | rot_dim rotated]``.  ``W_dkv h`` gives ``kv_rank + rot_dim`` numbers: the first ``kv_rank``,
RMS-normed with a gain, are the latent ``c``; the rest, rotated by position, are one key part shared by all heads.
Per head the unrotated key is ``W_uk c`` and the value ``W_uv c``; the score is
``(q_unrotated . k_unrotated + q_rotated . k_rotated) * scale`` over the visible positions (all, or the last
``window``); each head's output is multiplied by ``sigmoid(W_g h)`` of that head, and ``W_o`` closes the part.

Only ``[c | rotated key part]`` is cached: one row of ``kv_rank + rot_dim`` numbers per position for all heads
(``CacheNeed`` with one kv head and ``values_in_keys``).  Since ``q_u . (W_uk c) = (W_uk^T q_u) . c``, the unrotated
query part of each head is carried into the latent's space once per token (a product per head), the attention kernel
then runs over the cached rows as they are, all heads sharing them, with the first ``kv_rank`` columns of a row as its
values, and ``W_uv`` is applied to each head's weighted sum of latents afterwards (``W_uv sum_j p_j c_j``).  A prompt's
portion and a decoded token take the same path, so what a position's logits are does not depend on how it arrived.

The three projections that read the mixer's input (query latent, key/value latent, gate) are one product with a
float32 result; the two RMS norms, the rotation angles, the scores and the softmax are float32 in both precisions.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

import torch

from lily_b200.parts.attention import AttentionPlan, LayerCache
from lily_b200.parts.base import BuildContext, CacheNeed, Mixer, TensorSpec, build_part, register_part


@dataclass(frozen=True)
class LatentAttentionSpec:
    hidden_size: int
    num_heads: int
    head_dim: int                 # unrotated query/key columns a head
    rot_dim: int                  # rotated query/key columns a head (the key's are shared by all heads)
    v_head_dim: int
    q_rank: int
    kv_rank: int
    scale: float
    norm_eps: float
    window: Optional[int] = None  # None: all keys; n: the last n keys
    position: Any = None          # a position spec over the rot_dim columns (e.g. RopeSpec) or None
    out_gate: bool = True         # each head's output times sigmoid(W_g h) of the head
    kind: str = "latent_attention"
    # names of the tensors under the part's prefix
    names: Optional[Tuple[Tuple[str, str], ...]] = None

    _DEFAULTS = (("dq", "dq"), ("dq_norm", "dq.norm"), ("uq", "uq"), ("dkv", "dkv"), ("dkv_norm", "dkv.norm"),
                 ("uk", "uk"), ("uv", "uv"), ("g", "g"), ("o", "o"))

    def name(self, role: str) -> str:
        return dict(self.names or ()).get(role, dict(self._DEFAULTS)[role])

    @property
    def row(self) -> int:
        """Numbers cached for one position."""
        return self.kv_rank + self.rot_dim


@register_part("mixer", "latent_attention")
class LatentAttention(Mixer):
    graph_safe = True

    def __init__(self, spec: LatentAttentionSpec, prefix: str, ctx: BuildContext):
        if min(spec.num_heads, spec.head_dim, spec.v_head_dim, spec.q_rank, spec.kv_rank) < 1 or spec.rot_dim < 0:
            raise ValueError("sizes of the latent attention are positive")
        self.spec, self.prefix, self.ctx = spec, prefix, ctx
        self.position = build_part("position", spec.position, prefix, ctx) if spec.position is not None else None
        if self.position is not None and self.position.rotary_dim > spec.rot_dim:
            raise ValueError(f"{self.position.rotary_dim} rotated columns do not fit the {spec.rot_dim} set aside for them")
        self.w_down = self.w_uq = self.w_uk = self.w_uv = self.w_o = self.q_gain = self.kv_gain = None

    # ---- what it needs ----------------------------------------------------------

    def cache_need(self) -> CacheNeed:
        s = self.spec
        return CacheNeed(1, s.row, s.window, s.kv_rank, values_in_keys=True)

    def tensors(self) -> Dict[str, TensorSpec]:
        s, p = self.spec, self.prefix
        h = s.num_heads
        out = {f"{p}.{s.name('dq')}": TensorSpec((s.q_rank, s.hidden_size)),
               f"{p}.{s.name('dq_norm')}": TensorSpec((s.q_rank,), role="vector", init="gain"),
               f"{p}.{s.name('uq')}": TensorSpec((h * (s.head_dim + s.rot_dim), s.q_rank)),
               f"{p}.{s.name('dkv')}": TensorSpec((s.row, s.hidden_size)),
               f"{p}.{s.name('dkv_norm')}": TensorSpec((s.kv_rank,), role="vector", init="gain"),
               f"{p}.{s.name('uk')}": TensorSpec((h * s.head_dim, s.kv_rank)),
               f"{p}.{s.name('uv')}": TensorSpec((h * s.v_head_dim, s.kv_rank)),
               f"{p}.{s.name('o')}": TensorSpec((s.hidden_size, h * s.v_head_dim))}
        if s.out_gate:
            out[f"{p}.{s.name('g')}"] = TensorSpec((h, s.hidden_size))
        return out

    def load(self, get) -> None:
        s, p = self.spec, self.prefix
        g = lambda role: get(f"{p}.{s.name(role)}")
        parts = [g("dq"), g("dkv")] + ([g("g")] if s.out_gate else [])
        self.w_down = torch.cat(parts, 0).contiguous()                 # [q_rank | kv_rank + rot | heads] rows
        self.q_gain = g("dq_norm").float().contiguous()
        self.kv_gain = g("dkv_norm").float().contiguous()
        self.w_uq = g("uq").contiguous()
        h = s.num_heads
        # per head [out, in]: q' = W_uk^T q_u takes W_uk^T [kv_rank, head_dim]; the value takes W_uv [v, kv_rank] as stored
        self.w_uk = g("uk").view(h, s.head_dim, s.kv_rank).transpose(1, 2).contiguous()
        self.w_uv = g("uv").view(h, s.v_head_dim, s.kv_rank).contiguous()
        self.w_o = g("o").contiguous()

    # ---- one step ----------------------------------------------------------------

    def _plan(self, batch, group: int, dtype, page: int):
        """How this step's attention runs for these sizes in cache group ``group`` (made once a step, shared by the
        layers of one size): the heads are the query heads of one kv head."""
        s, ops = self.spec, self.ctx.ops
        key = ("latent_attention", group, s.num_heads, s.row, s.kv_rank, dtype, page)

        def make(b):
            nd = b.num_decode
            decode = ops.plan_decode_attention(dtype, nd, s.num_heads, 1, s.row, b.max_decode_len, even=b.decode_even,
                                               dv=s.kv_rank, values_in_keys=True)
            rows = tiles = None
            if b.num_requests > nd:
                rows = ops.prefill_tile_rows(dtype, s.row, page, b.num_tokens - nd, dv=s.kv_rank, values_in_keys=True,
                                             heads=s.num_heads)
                tiles = ops.prefill_tiles(b.h_prefix_lens, b.h_new_lens, nd, rows, b.token_ids.device)
            return AttentionPlan(decode, rows, tiles)
        return batch.plan(key, make)

    def forward(self, x, batch, cache: LayerCache, state=None, write_cache: bool = True):
        s, ops = self.spec, self.ctx.ops
        page, h = self.ctx.page_size, s.num_heads
        table = batch.block_tables[cache.group]
        plan = self._plan(batch, cache.group, cache.data.dtype, page)
        cos, sin = self.position.tables() if self.position is not None else (None, None)
        rotary_dim = self.position.rotary_dim if self.position is not None else 0
        down = ops.linear(x, self.w_down, out_dtype=torch.float32)      # [tokens, q latent | kv latent | rotated | gates]
        cq = ops.latent_prepare(down, 0, s.q_rank, s.q_rank, s.kv_rank, s.rot_dim, rotary_dim, self.q_gain, self.kv_gain,
                                s.norm_eps, cos, sin, batch.positions, batch.token_req, table, cache.data, page,
                                write_kv=write_cache)
        q = ops.linear(cq, self.w_uq)                                    # [tokens, heads * (head_dim + rot)]
        tokens = q.shape[0]
        q_heads = q.view(tokens, h, s.head_dim + s.rot_dim)
        carried = ops.head_linear(q_heads[:, :, :s.head_dim], self.w_uk, out_dtype=torch.float32)      # [heads, tokens, kv_rank]
        queries = ops.latent_query(carried, q, h, s.head_dim, s.kv_rank, s.rot_dim, rotary_dim, cos, sin, batch.positions)
        mixed = torch.empty((tokens, h * s.kv_rank), dtype=q.dtype, device=q.device)
        nd, dec = batch.num_decode, plan.decode
        if nd:
            scratch = batch.workspace.floats("attention_decode", dec.scratch_floats) if dec.scratch_floats else None
            ops.attention_decode(queries[:nd], cache.data, table, batch.seq_lens, mixed[:nd], scratch, dec.splits, h, 1,
                                 s.row, page, s.scale, s.window, dv=s.kv_rank, values_in_keys=True)
        if batch.num_requests > nd:
            tile_req, tile_start = plan.tiles
            ops.attention_prefill(queries, cache.data, table, batch.cu_seqlens, batch.prefix_lens, tile_req, tile_start,
                                  mixed, h, 1, s.row, page, s.scale, s.window, tile_rows=plan.tile_rows, dv=s.kv_rank,
                                  values_in_keys=True)
        values = ops.head_linear(mixed.view(tokens, h, s.kv_rank), self.w_uv, out_dtype=torch.float32)  # [heads, tokens, v]
        if s.out_gate:
            out = ops.head_gate(values, down, s.q_rank + s.row, q.dtype)
        else:
            out = ops.cast(values.transpose(0, 1).reshape(tokens, h * s.v_head_dim).contiguous(), q.dtype)
        return ops.linear_auto(out, self.w_o)
