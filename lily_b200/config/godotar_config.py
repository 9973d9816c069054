"""Typed configuration of the Godotar decoder, read from its ``config.json``.

The file lists the layers one by one; every layer names its type (which mixer it has) and carries the sizes and
constants of its mixer and of its feed-forward (or ``null`` for none), so layers of one model may differ.  A stretch of
layers may run several times over (``loop``).  Keys read here:

    architecture, vocab, width, norm.eps, logit_scale (optional), max_positions (optional),
    loop.{start, stop, times} (optional)
    layers[i].type                       "wkv" | "latent_attention"
    layers[i].mixer  (wkv)               heads, dim, decay_rank (optional: else read off the checkpoint's tensor)
    layers[i].mixer  (latent_attention)  heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, mask.size (optional),
                                         rot.{dims, base}
    layers[i].mlp                        null, {kind: "dense", ff}, or
                                         {kind: "moe", expert.{ff, limit}, router.{experts, identity, top}}

A size that neither the file nor the design fixes (the rank of the decay's low-rank pair) is taken from the shape of
the checkpoint tensor that has it (``sizes_from_tensors``).
"""

from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Any, Dict, List, Optional, Tuple, Union

from lily_b200.config.model_config import ConfigError
from lily_b200.config.zirurax_config import _need


@dataclass(frozen=True)
class WkvConfig:
    heads: int
    dim: int
    decay_rank: Optional[int]         # None until the checkpoint's tensors have been seen

    @classmethod
    def from_dict(cls, d: Dict[str, Any], where: str) -> "WkvConfig":
        rank = d.get("decay_rank")
        out = cls(_need(d, "heads", where), _need(d, "dim", where), int(rank) if rank else None)
        if min(out.heads, out.dim) < 1 or (out.decay_rank is not None and out.decay_rank < 1):
            raise ConfigError(f"{where}: sizes must be positive")
        return out


@dataclass(frozen=True)
class LatentAttentionConfig:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    window: Optional[int]
    rotary_dims: int                  # 0: no rotation
    rotary_base: float

    @classmethod
    def from_dict(cls, d: Dict[str, Any], where: str) -> "LatentAttentionConfig":
        rot = d.get("rot") or {}
        mask = d.get("mask") or {}
        out = cls(heads=_need(d, "heads", where), dim=_need(d, "dim", where), rot_dim=_need(d, "rot_dim", where),
                  vdim=_need(d, "vdim", where), q_rank=_need(d, "q_rank", where), kv_rank=_need(d, "kv_rank", where),
                  scale=_need(d, "scale", where, float), window=int(mask["size"]) if mask.get("size") else None,
                  rotary_dims=int(rot.get("dims") or 0), rotary_base=float(rot.get("base") or 10000.0))
        if min(out.heads, out.dim, out.vdim, out.q_rank, out.kv_rank) < 1 or out.rot_dim < 0:
            raise ConfigError(f"{where}: sizes must be positive")
        if out.rotary_dims < 0 or out.rotary_dims % 2 or out.rotary_dims > out.rot_dim:
            raise ConfigError(f"{where}.rot.dims {out.rotary_dims} must be even and within rot_dim {out.rot_dim}")
        if out.window is not None and out.window < 1:
            raise ConfigError(f"{where}.mask.size must be positive")
        return out


@dataclass(frozen=True)
class DenseFFConfig:
    ff: int


@dataclass(frozen=True)
class RoutedFFConfig:
    ff: int
    limit: float
    experts: int
    identity: int
    top: int

    @classmethod
    def from_dict(cls, d: Dict[str, Any], where: str) -> "RoutedFFConfig":
        expert, router = d.get("expert") or {}, d.get("router") or {}
        out = cls(ff=_need(expert, "ff", f"{where}.expert"), limit=_need(expert, "limit", f"{where}.expert", float),
                  experts=_need(router, "experts", f"{where}.router"), identity=int(router.get("identity") or 0),
                  top=_need(router, "top", f"{where}.router"))
        if out.ff < 1 or out.experts < 0 or out.identity < 0 or not 1 <= out.top <= out.experts + out.identity:
            raise ConfigError(f"{where}: top {out.top} of {out.experts} experts and {out.identity} identity outputs, ff {out.ff}")
        return out


@dataclass(frozen=True)
class GodotarLayerConfig:
    type: str                                                   # "wkv" | "latent_attention"
    mixer: Union[WkvConfig, LatentAttentionConfig]
    mlp: Union[None, DenseFFConfig, RoutedFFConfig]


@dataclass(frozen=True)
class LoopConfig:
    start: int
    stop: int
    times: int


_MIXERS = {"wkv": WkvConfig, "latent_attention": LatentAttentionConfig}


@dataclass
class GodotarConfig:
    architecture: str
    vocab: int
    width: int
    eps: float
    logit_scale: float
    layers: List[GodotarLayerConfig]
    loop: Optional[LoopConfig]
    max_positions: int = 1 << 17
    torch_dtype: str = "bfloat16"

    @classmethod
    def from_dict(cls, cfg: Dict[str, Any], generation: Optional[Dict[str, Any]] = None,
                  architecture: Optional[str] = None) -> "GodotarConfig":
        listed = cfg.get("layers")
        if not isinstance(listed, list) or not listed:
            raise ConfigError("config.json lacks the list 'layers'")
        layers = []
        for i, layer in enumerate(listed):
            where = f"layers[{i}]"
            kind = layer.get("type")
            if kind not in _MIXERS:
                raise ConfigError(f"{where}.type {kind!r} is not a layer type of this architecture (have: {', '.join(sorted(_MIXERS))})")
            mixer = _MIXERS[kind].from_dict(layer.get("mixer") or {}, f"{where}.mixer")
            mlp = layer.get("mlp")
            if mlp is None:
                ff = None
            elif mlp.get("kind") == "dense":
                ff = DenseFFConfig(_need(mlp, "ff", f"{where}.mlp"))
                if ff.ff < 1:
                    raise ConfigError(f"{where}.mlp.ff must be positive")
            elif mlp.get("kind") == "moe":
                ff = RoutedFFConfig.from_dict(mlp, f"{where}.mlp")
            else:
                raise ConfigError(f"{where}.mlp.kind {mlp.get('kind')!r} is not a feed-forward of this architecture (have: dense, moe)")
            layers.append(GodotarLayerConfig(kind, mixer, ff))
        loop = None
        if cfg.get("loop"):
            lp = cfg["loop"]
            loop = LoopConfig(_need(lp, "start", "loop"), _need(lp, "stop", "loop"), _need(lp, "times", "loop"))
            if not (0 <= loop.start <= loop.stop <= len(layers)) or loop.times < 1:
                raise ConfigError(f"loop {loop.start}..{loop.stop} x {loop.times} does not fit {len(layers)} layers")
        out = cls(architecture=architecture or str(cfg.get("architecture", "Godotar")),
                  vocab=_need(cfg, "vocab", "config"), width=_need(cfg, "width", "config"),
                  eps=_need(cfg.get("norm") or {}, "eps", "norm", float),
                  logit_scale=float(cfg["logit_scale"]) if cfg.get("logit_scale") is not None else 1.0, layers=layers,
                  loop=loop, max_positions=int(cfg.get("max_positions") or (1 << 17)),
                  torch_dtype=str(cfg.get("torch_dtype") or "bfloat16"))
        if out.vocab < 1 or out.width < 1 or not out.eps > 0:
            raise ConfigError("vocab and width must be positive, norm.eps above zero")
        return out

    def sizes_from_tensors(self, shapes: Dict[str, Tuple[int, ...]]) -> "GodotarConfig":
        """Fills in what config.json leaves to the checkpoint: the rank of each wkv layer's decay pair is the number of
        rows of its first matrix ``l<i>.mix.w1``."""
        layers = []
        for i, layer in enumerate(self.layers):
            if layer.type == "wkv" and layer.mixer.decay_rank is None:
                shape = shapes.get(f"l{i}.mix.w1")
                if shape is None or len(shape) != 2:
                    raise ConfigError(f"layers[{i}]: the decay's rank is neither in config.json nor readable from l{i}.mix.w1")
                layer = replace(layer, mixer=replace(layer.mixer, decay_rank=int(shape[0])))
            layers.append(layer)
        return replace(self, layers=layers)

    def runs(self) -> List[Tuple[int, Optional[int]]]:
        """(layer, number of the pass that starts ahead of it or None) in running order."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, None) for i in range(n)]
        lp = self.loop
        out: List[Tuple[int, Optional[int]]] = [(i, None) for i in range(lp.start)]
        for t in range(lp.times):
            out += [(i, t if i == lp.start else None) for i in range(lp.start, lp.stop)]
        return out + [(i, None) for i in range(lp.stop, n)]

    def summary(self) -> str:
        return (f"{self.architecture} layers={len(self.layers)} width={self.width} vocab={self.vocab} eps={self.eps} "
                f"loop={self.loop}")
