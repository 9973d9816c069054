"""Small Zirurax configurations and random weights for the tests, made here from the design alone (no code of
``lily_b200`` decides a name or a shape)."""

from __future__ import annotations

import json
import math
import os
from typing import Dict, Optional

import torch


def layer(heads=4, kv_heads=2, dim=16, vdim=24, window=13, rot_dims=8, base=10000.0, scaling=None, scale=0.4,
          softcap=5.0, s_heads=4, s_vdim=8, state=12, groups=2, conv=3, norm_groups=4, ff: Optional[int] = 40) -> dict:
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window:
        left["mask"] = {"size": window}
    if softcap:
        left["softcap"] = softcap
    if rot_dims:
        left["rot"] = {"dims": rot_dims, "base": base}
        if scaling:
            left["rot"]["scaling"] = scaling
    right = {"heads": s_heads, "vdim": s_vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}
    return {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


SCALING = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}      # all three bands occur below 64 positions

# Sizes that differ in every respect from layer to layer: head sizes for keys and values, partial and full rotation,
# no rotation, with and without window, cap, feed-forward; 1, 2 and 4 groups; 2 to 4 taps.
VARIED = {"architecture": "Zirurax", "vocab": 131, "width": 48, "embedding": {"scale": 3.0}, "norm": {"eps": 1e-5},
          "layers": [layer(),
                     layer(heads=6, kv_heads=3, dim=8, vdim=8, window=7, rot_dims=8, scaling=SCALING, softcap=None,
                           s_heads=2, s_vdim=16, state=20, groups=1, conv=4, norm_groups=1, ff=None),
                     layer(heads=2, kv_heads=2, dim=24, vdim=16, window=None, rot_dims=0, scale=0.3, softcap=2.0,
                           s_heads=8, s_vdim=4, state=5, groups=4, conv=2, norm_groups=2, ff=56)]}

# Sharp attention: a large scale under a high cap puts nearly all weight on the best visible key, so a key that is
# wrongly seen or wrongly dropped at a window's edge changes the output outright.
SHARP = {"architecture": "Zirurax", "vocab": 97, "width": 32, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6},
         "layers": [layer(heads=2, kv_heads=1, dim=16, vdim=16, window=9, rot_dims=16, scale=3.0, softcap=40.0,
                          s_heads=2, s_vdim=8, state=8, groups=1, conv=4, norm_groups=2, ff=32),
                    layer(heads=2, kv_heads=1, dim=16, vdim=16, window=17, rot_dims=16, scale=3.0, softcap=40.0,
                          s_heads=2, s_vdim=8, state=8, groups=1, conv=4, norm_groups=2, ff=32)]}

# Head sizes the tensor-core attention kernels take, wider layers.
WIDE = {"architecture": "Zirurax", "vocab": 257, "width": 128, "embedding": {"scale": 2.0}, "norm": {"eps": 1e-6},
        "layers": [layer(heads=4, kv_heads=2, dim=64, vdim=64, window=40, rot_dims=32, scale=0.2, softcap=10.0,
                         s_heads=4, s_vdim=32, state=64, groups=2, conv=4, norm_groups=2, ff=192),
                   layer(heads=2, kv_heads=1, dim=128, vdim=128, window=None, rot_dims=128, scaling=SCALING, scale=0.15,
                         softcap=8.0, s_heads=8, s_vdim=16, state=16, groups=1, conv=4, norm_groups=1, ff=128)]}


def shapes(cfg: dict) -> Dict[str, tuple]:
    w = cfg["width"]
    out = {"embed": (cfg["vocab"], w), "final.norm": (w,)}
    for i, ly in enumerate(cfg["layers"]):
        a, m = ly["mixer"]["left"], ly["mixer"]["right"]
        p = f"l{i}"
        inner = m["heads"] * m["vdim"]
        channels = inner + 2 * m["groups"] * m["state"]
        out.update({f"{p}.norm1": (w,),
                    f"{p}.mix.left.q": (a["heads"] * a["dim"], w), f"{p}.mix.left.k": (a["kv_heads"] * a["dim"], w),
                    f"{p}.mix.left.v": (a["kv_heads"] * a["vdim"], w), f"{p}.mix.left.g": (a["heads"] * a["vdim"], w),
                    f"{p}.mix.left.o": (w, a["heads"] * a["vdim"]),
                    f"{p}.mix.right.in": (inner + channels + m["heads"], w), f"{p}.mix.right.conv": (channels, m["conv"]),
                    f"{p}.mix.right.conv.b": (channels,), f"{p}.mix.right.dt_bias": (m["heads"],),
                    f"{p}.mix.right.A_log": (m["heads"],), f"{p}.mix.right.D": (m["heads"],),
                    f"{p}.mix.right.norm": (inner,), f"{p}.mix.right.o": (w, inner),
                    f"{p}.mix.left.out": (w,), f"{p}.mix.right.out": (w,)})
        if ly["mlp"]:
            out.update({f"{p}.mlp.gate": (ly["mlp"]["ff"], w), f"{p}.mlp.up": (ly["mlp"]["ff"], w),
                        f"{p}.mlp.down": (w, ly["mlp"]["ff"])})
    return out


def make_weights(cfg: dict, seed: int, dtype=torch.float32) -> Dict[str, torch.Tensor]:
    """Random weights at scales that keep every mechanism alive: projections of unit gain, slow and fast decays,
    step sizes around one, gains around one."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in shapes(cfg).items():
        n = lambda: torch.randn(shape, generator=g)
        if name == "embed":
            t = n()
        elif name.endswith(("norm1", "final.norm", ".out", "right.norm", ".D")):
            t = 1.0 + 0.2 * n()
        elif name.endswith("A_log"):
            t = torch.rand(shape, generator=g) * 4.0 - 4.0          # decays exp(-dt e^A): memory of 1 to 50 tokens
        elif name.endswith("dt_bias"):
            t = n() - 0.5
        elif name.endswith("conv"):
            t = 0.6 * n()
        elif name.endswith("conv.b"):
            t = 0.2 * n()
        else:
            t = n() / math.sqrt(shape[-1])
        out[name] = t.to(dtype)
    return out


def write_model_dir(path: str, cfg: dict, weights: Dict[str, torch.Tensor]) -> str:
    from lily_b200.weights.safetensors_io import write_safetensors

    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(path, "model.safetensors"),
                      [(n, t.dtype, tuple(t.shape)) for n, t in weights.items()], {"format": "pt"},
                      produce=lambda n: weights[n])
    return path


def tokens(n: int, vocab: int, seed: int):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()
