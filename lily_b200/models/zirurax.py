"""The Zirurax decoder as a ``ModelSpec``.

Every layer is a parallel block: one RMSNorm, then side by side a windowed grouped-query attention (rotation of
interleaved pairs with Llama-3 frequency scaling, soft-capped scores, an output gate) and a Mamba-2 state-space
mixer, each output RMS-normed with a gain of its own and the two averaged, plus a dense GELU-gated feed-forward
that reads the same norm.  The embedding is scaled; the head is the embedding table without the scale.  Sizes may
differ from layer to layer; tensor names are the checkpoint's own (``l<i>.norm1``, ``l<i>.mix.left.q``, ...).
"""

from __future__ import annotations

from lily_b200.config.registry import register_architecture
from lily_b200.config.zirurax_config import ZiruraxConfig
from lily_b200.parts.attention import AttentionSpec
from lily_b200.parts.base import ModelSpec, ScheduleEntry
from lily_b200.parts.block import ParallelBlockSpec
from lily_b200.parts.mlp import SwiGLUSpec
from lily_b200.parts.norm import RMSNormSpec
from lily_b200.parts.rope import RopeSpec
from lily_b200.parts.ssm import SSDSpec

_LEFT_NAMES = (("q", "q"), ("k", "k"), ("v", "v"), ("o", "o"), ("g", "g"))
_RIGHT_NAMES = (("in", "in"), ("conv", "conv"), ("conv_bias", "conv.b"), ("dt_bias", "dt_bias"), ("A_log", "A_log"),
                ("D", "D"), ("norm", "norm"), ("out", "o"))
_FF_NAMES = (("gate", "gate"), ("up", "up"), ("down", "down"))


def build_spec(cfg: ZiruraxConfig) -> ModelSpec:
    norm = RMSNormSpec(cfg.width, cfg.eps, suffix="")
    blocks = []
    for i, layer in enumerate(cfg.layers):
        a, m = layer.left, layer.right
        rope = None
        if a.rotary_dims:
            rope = RopeSpec(a.dim, a.rotary_dims, a.rotary_base, a.rotary_scaling, interleaved=True, exact_frequencies=True)
        left = AttentionSpec(cfg.width, a.heads, a.kv_heads, a.dim, window=a.window, scale=a.scale, position=rope,
                             v_head_dim=a.vdim, softcap=a.softcap, out_gate=True, names=_LEFT_NAMES)
        right = SSDSpec(cfg.width, m.heads, m.vdim, m.state, m.groups, m.conv, m.norm_groups, cfg.eps, names=_RIGHT_NAMES)
        ff = None if layer.ff is None else SwiGLUSpec(cfg.width, layer.ff, activation="gelu_tanh", names=_FF_NAMES)
        blocks.append(ParallelBlockSpec(prefix=f"l{i}", hidden_size=cfg.width,
                                        mixers=(("mix.left", left, "mix.left.out"), ("mix.right", right, "mix.right.out")),
                                        feed_forward=ff, norm=norm, eps=cfg.eps))
    return ModelSpec(architecture=cfg.architecture, vocab_size=cfg.vocab, hidden_size=cfg.width, blocks=blocks,
                     schedule=[ScheduleEntry(i) for i in range(len(blocks))], final_norm=norm, embed_name="embed",
                     final_norm_prefix="final.norm", head_name=None, max_position=cfg.max_positions,
                     ignored_tensors=(), embed_scale=cfg.embedding_scale)


register_architecture("Zirurax", ZiruraxConfig.from_dict, build_spec)
