"""Small Godotar configurations and random weights for the tests, made here from the design alone (no code of
``lily_b200`` decides a name or a shape)."""

from __future__ import annotations

import json
import math
import os
from typing import Dict, Optional

import torch


def wkv(heads=3, dim=8, kind="dense", **mlp) -> dict:
    return {"type": "wkv", "mixer": {"heads": heads, "dim": dim}, "mlp": feed_forward(kind, **mlp)}


def latent(heads=3, dim=8, rot_dim=4, vdim=12, q_rank=20, kv_rank=24, window: Optional[int] = 11, scale=0.35, base=10000.0,
           kind="moe", **mlp) -> dict:
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale,
         "rot": {"dims": rot_dim, "base": base}}
    if window:
        m["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": m, "mlp": feed_forward(kind, **mlp)}


def feed_forward(kind, ff=40, experts=5, identity=2, top=2, limit=1.5):
    if kind is None:
        return None
    if kind == "dense":
        return {"kind": "dense", "ff": ff}
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "identity": identity, "top": top}}


# Sizes that differ from layer to layer; the looped stretch starts after the first layer and holds both mixers; a layer
# without feed-forward; experts without identity outputs and with one choice; head sizes that are no power of two.
VARIED = {"architecture": "Godotar", "vocab": 131, "width": 48, "norm": {"eps": 1e-5}, "logit_scale": 0.7,
          "loop": {"start": 1, "stop": 3, "times": 3},
          "layers": [latent(),
                     wkv(heads=2, dim=12, kind="moe", ff=24, experts=4, identity=0, top=1, limit=0.8),
                     latent(heads=2, dim=6, rot_dim=8, vdim=6, q_rank=10, kv_rank=18, window=7, scale=0.5, base=100.0, kind=None),
                     wkv(heads=5, dim=4, kind="dense", ff=56)]}

# Sharp attention and long memory: a large scale puts nearly all weight on the best visible key, so a key that is
# wrongly seen or wrongly dropped at a window's edge changes the output outright; no loop at all.
SHARP = {"architecture": "Godotar", "vocab": 97, "width": 32, "norm": {"eps": 1e-6},
         "layers": [latent(heads=2, dim=8, rot_dim=8, vdim=8, q_rank=16, kv_rank=16, window=9, scale=3.0, kind="dense", ff=32),
                    wkv(heads=2, dim=16, kind="moe", ff=16, experts=3, identity=3, top=3, limit=1.0),
                    latent(heads=1, dim=16, rot_dim=2, vdim=16, q_rank=8, kv_rank=32, window=17, scale=3.0, kind="dense", ff=32)]}

# Wider layers; the whole model is one loop that runs once; all keys visible in one layer; a wkv head of 64 and of 40.
WIDE = {"architecture": "Godotar", "vocab": 257, "width": 128, "norm": {"eps": 1e-6}, "logit_scale": 0.25,
        "loop": {"start": 0, "stop": 3, "times": 1},
        "layers": [wkv(heads=2, dim=64, kind="moe", ff=64, experts=8, identity=1, top=4, limit=1.0),
                   latent(heads=4, dim=32, rot_dim=16, vdim=32, q_rank=48, kv_rank=64, window=None, scale=0.2, kind="dense", ff=192),
                   wkv(heads=3, dim=40, kind="dense", ff=128)]}

DECAY_RANK = 6           # rows of every layer's first decay matrix in these checkpoints (config.json does not say)


def random_config(seed: int) -> dict:
    """A configuration drawn at random: 2 to 5 layers of either mixer in any order, any feed-forward or none, widths
    in steps of 8 (and two that are not), head sizes and ranks in steps of 2 or 8, with and without loop, windows from 3 to 70 or none."""
    import random
    rng = random.Random(seed)
    width = rng.choice([24, 40, 64, 72, 96, 136, 44, 50])
    layers = []
    for _ in range(rng.randint(2, 5)):
        kind = rng.choice(["dense", "moe", "moe", None])
        mlp = {}
        if kind == "dense":
            mlp = {"ff": rng.choice([16, 40, 72])}
        elif kind == "moe":
            experts, identity = rng.randint(1, 9), rng.randint(0, 3)
            mlp = {"ff": rng.choice([8, 24, 40]), "experts": experts, "identity": identity,
                   "top": rng.randint(1, min(4, experts + identity)), "limit": rng.choice([0.5, 1.0, 7.0])}
        if rng.random() < 0.5:
            layers.append(wkv(heads=rng.randint(1, 4), dim=rng.choice([4, 8, 12, 16, 24, 32, 64]), kind=kind, **mlp))
        else:
            rot = rng.choice([2, 4, 8, 16])
            rank = rng.choice([8, 24, 40, 64, 120]) if rng.random() < 0.7 else rng.choice([10, 18, 34])
            layers.append(latent(heads=rng.randint(1, 6), dim=rng.choice([4, 8, 16, 32]), rot_dim=rot, vdim=rng.choice([4, 8, 20, 32]),
                                 q_rank=rng.choice([8, 12, 32]), kv_rank=rank, window=rng.choice([None, 3, 17, 40, 70]),
                                 scale=rng.choice([0.2, 0.5]), base=rng.choice([100.0, 10000.0]), kind=kind, **mlp))
    cfg = {"architecture": "Godotar", "vocab": rng.choice([61, 128, 300]), "width": width, "norm": {"eps": rng.choice([1e-5, 1e-6])},
           "logit_scale": rng.choice([0.3, 1.0]), "layers": layers}
    if rng.random() < 0.7:
        start = rng.randint(0, len(layers) - 1)
        cfg["loop"] = {"start": start, "stop": rng.randint(start + 1, len(layers)), "times": rng.randint(1, 3)}
    return cfg


def shapes(cfg: dict) -> Dict[str, tuple]:
    w = cfg["width"]
    out = {"embed": (cfg["vocab"], w), "embed.norm": (w,), "final.norm": (w,)}
    if cfg.get("loop"):
        out["loop.step"] = (cfg["loop"]["times"], w)
    for i, ly in enumerate(cfg["layers"]):
        m, p = ly["mixer"], f"l{i}"
        out[f"{p}.norm1"] = (w,)
        if ly["type"] == "wkv":
            hd = m["heads"] * m["dim"]
            rank = m.get("decay_rank", DECAY_RANK)
            out.update({f"{p}.mix.mu.{s}": (w,) for s in "rkvgw"})
            out.update({f"{p}.mix.{s}": (hd, w) for s in "rkvg"})
            out.update({f"{p}.mix.w1": (rank, w), f"{p}.mix.w2": (hd, rank), f"{p}.mix.w0": (hd,),
                        f"{p}.mix.u": (m["heads"], m["dim"]), f"{p}.mix.norm": (hd,), f"{p}.mix.o": (w, hd)})
        else:
            h = m["heads"]
            out.update({f"{p}.mix.dq": (m["q_rank"], w), f"{p}.mix.dq.norm": (m["q_rank"],),
                        f"{p}.mix.uq": (h * (m["dim"] + m["rot_dim"]), m["q_rank"]),
                        f"{p}.mix.dkv": (m["kv_rank"] + m["rot_dim"], w), f"{p}.mix.dkv.norm": (m["kv_rank"],),
                        f"{p}.mix.uk": (h * m["dim"], m["kv_rank"]), f"{p}.mix.uv": (h * m["vdim"], m["kv_rank"]),
                        f"{p}.mix.g": (h, w), f"{p}.mix.o": (w, h * m["vdim"])})
        mlp = ly["mlp"]
        if mlp is None:
            continue
        out[f"{p}.norm2"] = (w,)
        if mlp["kind"] == "dense":
            out.update({f"{p}.mlp.gate": (mlp["ff"], w), f"{p}.mlp.up": (mlp["ff"], w), f"{p}.mlp.down": (w, mlp["ff"])})
        else:
            r, ff = mlp["router"], mlp["expert"]["ff"]
            n = r["experts"] + r["identity"]
            out.update({f"{p}.mlp.router": (n, w), f"{p}.mlp.correction": (n,)})
            for e in range(r["experts"]):
                out.update({f"{p}.mlp.e{e}.gate": (ff, w), f"{p}.mlp.e{e}.up": (ff, w), f"{p}.mlp.e{e}.down": (w, ff)})
    return out


def make_weights(cfg: dict, seed: int, dtype=torch.float32) -> Dict[str, torch.Tensor]:
    """Random weights at scales that keep every mechanism alive: projections of unit gain, decays that forget in two
    to a few hundred tokens, a bonus of order one, router logits that spread, corrections that change the choice,
    expert products that reach their clamps, gains stored around zero."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in shapes(cfg).items():
        n = lambda: torch.randn(shape, generator=g)
        last = name.rsplit(".", 1)[-1]
        if name in ("embed",):
            t = n()
        elif last in ("norm1", "norm2") or name in ("embed.norm", "final.norm"):
            t = 0.2 * n()                                            # stored as a difference from one
        elif name.endswith(("mix.norm", "dq.norm", "dkv.norm")):
            t = 1.0 + 0.2 * n()
        elif name == "loop.step":
            t = 0.5 * n()
        elif ".mix.mu." in name:
            t = torch.rand(shape, generator=g)
        elif last == "w0":
            t = torch.rand(shape, generator=g) * 5.0 - 5.5          # decays exp(-e^w0): memory of 2 to 250 tokens
        elif last == "w2":
            t = n() / math.sqrt(shape[-1])
        elif last == "u":
            t = 0.5 * n()
        elif last == "router":
            t = 3.0 * n() / math.sqrt(shape[-1])
        elif last == "correction":
            t = 0.1 * n()
        elif ".mlp.e" in name and last in ("gate", "up"):
            t = 1.5 * n() / math.sqrt(shape[-1])
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
