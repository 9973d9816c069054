"""The Godotar decoder as a ``ModelSpec``.

The stream starts as the embedding rows under the model's norm (RMS norm whose gain is stored as a difference from
one).  Every layer is a parallel block with two norms: ``x += mixer(norm1(x)) + ff(norm2(x))``.  The mixer is a
linear-attention recurrence with a data-dependent decay (``wkv``) or a softmax attention over a cached low-rank latent
(``latent_attention``, windowed, rotated in halves, with an output gate per head); the feed-forward is a dense SwiGLU or
a routed mixture of clamped experts, some router outputs standing for the identity; a layer may have none.  A stretch of
layers runs several times over with the same weights: each pass is a run of the schedule with caches and states of its
own, and a row of ``loop.step`` is added to the stream ahead of it.  The head is the embedding table; the logits are
scaled.  Tensor names are the checkpoint's own (``l<i>.norm1``, ``l<i>.mix.dkv``, ``l<i>.mlp.e3.gate``, ...).
"""

from __future__ import annotations

from lily_b200.config.godotar_config import DenseFFConfig, GodotarConfig, RoutedFFConfig
from lily_b200.config.model_config import ConfigError
from lily_b200.config.registry import register_architecture
from lily_b200.parts.base import ModelSpec, ScheduleEntry
from lily_b200.parts.block import ParallelBlockSpec
from lily_b200.parts.experts import RoutedExpertsSpec
from lily_b200.parts.latent_attention import LatentAttentionSpec
from lily_b200.parts.mlp import SwiGLUSpec
from lily_b200.parts.norm import RMSNormSpec
from lily_b200.parts.rope import RopeSpec
from lily_b200.parts.wkv import WkvSpec

_FF_NAMES = (("gate", "gate"), ("up", "up"), ("down", "down"))
STEP_TENSOR = "loop.step"


def build_spec(cfg: GodotarConfig) -> ModelSpec:
    norm = RMSNormSpec(cfg.width, cfg.eps, suffix="", offset=1.0)
    blocks = []
    ignored = []
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        if layer.type == "wkv":
            if m.decay_rank is None:
                raise ConfigError(f"layers[{i}]: the decay's rank is unknown (give mixer.decay_rank, or load a checkpoint)")
            mixer = WkvSpec(cfg.width, m.heads, m.dim, m.decay_rank, cfg.eps)
        else:
            rope = RopeSpec(m.rot_dim, m.rotary_dims, m.rotary_base, exact_frequencies=True) if m.rotary_dims else None
            mixer = LatentAttentionSpec(cfg.width, m.heads, m.dim, m.rot_dim, m.vdim, m.q_rank, m.kv_rank, m.scale, cfg.eps,
                                        window=m.window, position=rope)
        if layer.mlp is None:
            ff = None
            ignored.append(f"l{i}.norm2")                   # a layer without feed-forward has no use for its norm
        elif isinstance(layer.mlp, DenseFFConfig):
            ff = SwiGLUSpec(cfg.width, layer.mlp.ff, names=_FF_NAMES)
        else:
            r: RoutedFFConfig = layer.mlp
            ff = RoutedExpertsSpec(cfg.width, r.ff, r.experts, r.identity, r.top, r.limit)
        blocks.append(ParallelBlockSpec(prefix=f"l{i}", hidden_size=cfg.width, mixers=(("mix", mixer, None),),
                                        feed_forward=ff, norm=norm, eps=cfg.eps, ff_norm=norm if ff is not None else None))
    schedule = [ScheduleEntry(i, step=None if t is None else (STEP_TENSOR, t)) for i, t in cfg.runs()]
    if cfg.loop is not None and all(entry.step is None for entry in schedule):
        ignored.append(STEP_TENSOR)                         # a loop over no layer has no pass to add its vectors ahead of
    return ModelSpec(architecture=cfg.architecture, vocab_size=cfg.vocab, hidden_size=cfg.width, blocks=blocks,
                     schedule=schedule, final_norm=norm, embed_name="embed", final_norm_prefix="final.norm", head_name=None,
                     max_position=cfg.max_positions, ignored_tensors=tuple(ignored), logit_scale=cfg.logit_scale,
                     embed_norm=norm, embed_norm_prefix="embed.norm")


register_architecture("Godotar", GodotarConfig.from_dict, build_spec)
