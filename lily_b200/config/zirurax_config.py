"""Typed configuration of the Zirurax decoder, read from its ``config.json``.

The file lists the layers one by one; every layer names its type and carries the sizes and constants of its
mixer and of its feed-forward (or ``null`` for none), so layers of one model may differ.  Keys read here:

    architecture, vocab, width, embedding.scale, norm.eps, max_positions (optional),
    layers[i].type                                  "parallel"
    layers[i].mixer.left    heads, kv_heads, dim, vdim, scale, softcap (optional), mask.size (optional),
                            rot.{dims, base, scaling.{factor, low, high, original}} (rot and scaling optional)
    layers[i].mixer.right   heads, vdim, state, groups, conv, norm_groups
    layers[i].mlp           null, or {kind: "dense", ff}
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional

from lily_b200.config.model_config import ConfigError, RopeScaling


def _need(d: Dict[str, Any], key: str, where: str, kind=int):
    if not isinstance(d, dict) or key not in d or d[key] is None:
        raise ConfigError(f"config.json lacks {where}.{key}")
    try:
        return kind(d[key])
    except (TypeError, ValueError):
        raise ConfigError(f"config.json {where}.{key} = {d[key]!r} is not {kind.__name__}") from None


@dataclass(frozen=True)
class WindowedAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: Optional[float]
    window: Optional[int]
    rotary_dims: int                  # 0: no rotation
    rotary_base: float
    rotary_scaling: RopeScaling

    @classmethod
    def from_dict(cls, d: Dict[str, Any], where: str) -> "WindowedAttentionConfig":
        rot = d.get("rot") or {}
        sc = rot.get("scaling")
        scaling = RopeScaling()
        if sc:
            scaling = RopeScaling("llama3", _need(sc, "factor", f"{where}.rot.scaling", float),
                                  _need(sc, "low", f"{where}.rot.scaling", float),
                                  _need(sc, "high", f"{where}.rot.scaling", float),
                                  _need(sc, "original", f"{where}.rot.scaling", int))
        mask = d.get("mask") or {}
        softcap = d.get("softcap")
        out = cls(heads=_need(d, "heads", where), kv_heads=_need(d, "kv_heads", where), dim=_need(d, "dim", where),
                  vdim=_need(d, "vdim", where), scale=_need(d, "scale", where, float),
                  softcap=float(softcap) if softcap else None,
                  window=int(mask["size"]) if mask.get("size") else None,
                  rotary_dims=int(rot.get("dims") or 0), rotary_base=float(rot.get("base") or 10000.0),
                  rotary_scaling=scaling)
        if min(out.heads, out.kv_heads, out.dim, out.vdim) < 1 or out.heads % out.kv_heads:
            raise ConfigError(f"{where}: {out.heads} heads over {out.kv_heads} kv heads of sizes {out.dim} / {out.vdim}")
        if out.rotary_dims < 0 or out.rotary_dims % 2 or out.rotary_dims > out.dim:
            raise ConfigError(f"{where}.rot.dims {out.rotary_dims} must be even and within dim {out.dim}")
        if out.window is not None and out.window < 1:
            raise ConfigError(f"{where}.mask.size must be positive")
        return out


@dataclass(frozen=True)
class StateSpaceConfig:
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int

    @classmethod
    def from_dict(cls, d: Dict[str, Any], where: str) -> "StateSpaceConfig":
        out = cls(*(_need(d, k, where) for k in ("heads", "vdim", "state", "groups", "conv", "norm_groups")))
        if min(out.heads, out.vdim, out.state, out.groups, out.conv, out.norm_groups) < 1:
            raise ConfigError(f"{where}: sizes must be positive")
        if out.heads % out.groups or (out.heads * out.vdim) % out.norm_groups:
            raise ConfigError(f"{where}: {out.heads} heads over {out.groups} groups, {out.heads * out.vdim} columns in "
                              f"{out.norm_groups} norm groups")
        return out


@dataclass(frozen=True)
class ZiruraxLayerConfig:
    left: WindowedAttentionConfig
    right: StateSpaceConfig
    ff: Optional[int]                 # None: the layer has no feed-forward


@dataclass
class ZiruraxConfig:
    architecture: str
    vocab: int
    width: int
    embedding_scale: float
    eps: float
    layers: List[ZiruraxLayerConfig]
    max_positions: int = 1 << 17
    torch_dtype: str = "bfloat16"

    @classmethod
    def from_dict(cls, cfg: Dict[str, Any], generation: Optional[Dict[str, Any]] = None,
                  architecture: Optional[str] = None) -> "ZiruraxConfig":
        layers = []
        listed = cfg.get("layers")
        if not isinstance(listed, list) or not listed:
            raise ConfigError("config.json lacks the list 'layers'")
        for i, layer in enumerate(listed):
            where = f"layers[{i}]"
            if layer.get("type") != "parallel":
                raise ConfigError(f"{where}.type {layer.get('type')!r} is not a layer type of this architecture (have: parallel)")
            mixer = layer.get("mixer") or {}
            if "left" not in mixer or "right" not in mixer:
                raise ConfigError(f"{where}.mixer needs 'left' and 'right'")
            mlp = layer.get("mlp")
            if mlp is not None and mlp.get("kind") != "dense":
                raise ConfigError(f"{where}.mlp.kind {mlp.get('kind')!r} is not a feed-forward of this architecture (have: dense)")
            layers.append(ZiruraxLayerConfig(WindowedAttentionConfig.from_dict(mixer["left"], f"{where}.mixer.left"),
                                             StateSpaceConfig.from_dict(mixer["right"], f"{where}.mixer.right"),
                                             None if mlp is None else _need(mlp, "ff", f"{where}.mlp")))
        out = cls(architecture=architecture or str(cfg.get("architecture", "Zirurax")),
                  vocab=_need(cfg, "vocab", "config"), width=_need(cfg, "width", "config"),
                  embedding_scale=float((cfg.get("embedding") or {}).get("scale", 1.0)),
                  eps=_need(cfg.get("norm") or {}, "eps", "norm", float), layers=layers,
                  max_positions=int(cfg.get("max_positions") or (1 << 17)),
                  torch_dtype=str(cfg.get("torch_dtype") or "bfloat16"))
        if out.vocab < 1 or out.width < 1 or not out.eps > 0:
            raise ConfigError("vocab and width must be positive, norm.eps above zero")
        return out

    def summary(self) -> str:
        return (f"{self.architecture} layers={len(self.layers)} width={self.width} vocab={self.vocab} "
                f"eps={self.eps} embedding_scale={self.embedding_scale}")
