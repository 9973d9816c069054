"""The Godotar decoder beside the framework's two other decoders at equal sizes: prefill and decode throughput of all
three through the same step function, and each kernel of the new design alone against its roofline, beside the like
kernel of the closest existing model (the Zirurax decoder: a recurrent mixer with its state in the request's slot and
a windowed attention; the dense decoder for the feed-forward).

    python -m lily_b200.bench.godotar_bench [--sizes small mid] [--layers 4] [--no-kernels] [--no-models] [--table]
    python bench.py --design godotar ...          (the same, as one JSON line)

Random weights in bfloat16.  A size gives the models the same width and layers.  The Godotar layers alternate as
[wkv + dense, latent attention + experts, wkv + experts, wkv + experts]; the wkv mixer has width / 64 heads of 64, the
latent attention the size's heads with 128 unrotated and 64 rotated query/key columns, values of 128, a key/value
latent of 512 and a query latent of 3 width / 8; the experts are 16 (+ 2 identity outputs) of a quarter of the dense
feed-forward width each, of which a token takes 4, so a token's feed-forward work equals the dense layer's.
Timing as in ``design_bench``: device time by CUDA events after warm-up, weights and caches larger than L2, kernels
over rotated inputs replayed from a graph.
"""

from __future__ import annotations

import argparse
import json
import sys
from typing import List

import torch

from lily_b200.bench.design_bench import SIZES, dense_config, model_throughput, zirurax_config
from lily_b200.bench.kbench import peaks, time_ms


def godotar_config(z: dict, layers: int) -> dict:
    width = z["width"]
    wkv = {"heads": width // 64, "dim": 64, "decay_rank": 64}
    lat = {"heads": z["heads"], "dim": 128, "rot_dim": 64, "vdim": 128, "q_rank": 3 * width // 8, "kv_rank": 512,
           "scale": 192 ** -0.5, "mask": {"size": z["window"]}, "rot": {"dims": 64, "base": 1000000.0}}
    moe = {"kind": "moe", "expert": {"ff": z["ff"] // 4, "limit": 7.0}, "router": {"experts": 16, "identity": 2, "top": 4}}
    dense = {"kind": "dense", "ff": z["ff"]}
    kinds = [("wkv", wkv, dense), ("latent_attention", lat, moe), ("wkv", wkv, moe), ("wkv", wkv, moe)]
    return {"architecture": "Godotar", "vocab": z["vocab"], "width": width, "norm": {"eps": 1e-6}, "logit_scale": 1.0,
            "layers": [{"type": t, "mixer": m, "mlp": f} for t, m, f in (kinds[i % 4] for i in range(layers))]}


def kernel_table(z: dict, tokens: int, batch: int, context: int, reps: int = 30, copies: int = 3) -> List[dict]:
    """Each kernel of the design alone, prefill shape (``tokens`` of one request) and decode shape (``batch`` requests of
    one token), with the like kernel of the closest existing model beside it."""
    from lily_b200.csrc import ops

    dev, dt = "cuda", torch.bfloat16
    pk = peaks()
    props = torch.cuda.get_device_properties(0)
    fp32_tflops = props.multi_processor_count * 128 * 2 * 1965000 / 1e9
    g = torch.Generator(device=dev).manual_seed(0)
    rnd = lambda *shape: torch.randn(*shape, device=dev, generator=g)
    cfg = godotar_config(z, 2)
    wk, la = cfg["layers"][0]["mixer"], cfg["layers"][1]["mixer"]
    moe = cfg["layers"][1]["mlp"]
    width = z["width"]
    heads, d = wk["heads"], wk["dim"]
    hd = heads * d
    rows: List[dict] = []

    def add(name, like, fns, bytes_moved, flops=0.0, flop_peak=None, shape=""):
        ms = time_ms(fns, reps, graph=True)
        row = {"kernel": name, "like": like, "shape": shape, "us": round(ms * 1e3, 2),
               "hbm_frac": round(bytes_moved / ms / 1e6 / pk["hbm_gbs"], 3)}
        if flops:
            row["flop_frac"] = round(flops / ms / 1e9 / (flop_peak or pk["bf16_tflops"]), 3)
            row["flop_peak"] = "fp32 fma" if flop_peak else "bf16 tensor"
        row["roofline_frac"] = max(row["hbm_frac"], row.get("flop_frac", 0.0))
        row["bound"] = row.get("flop_peak", "hbm") if row.get("flop_frac", 0.0) > row["hbm_frac"] else "hbm"
        rows.append(row)

    for label, n, reqs in (("prefill", tokens, 1), ("decode", batch, batch)):
        per = n // reqs
        cu = torch.arange(0, n + 1, per, device=dev, dtype=torch.int32)
        slots = torch.arange(1, reqs + 1, device=dev, dtype=torch.int32)
        token_req = torch.arange(reqs, device=dev, dtype=torch.int32).repeat_interleave(per)
        state_floats = hd * d + width
        states = [torch.zeros(reqs + 1, state_floats, device=dev) for _ in range(copies)]
        # ---- the wkv mixer's kernels
        hs = [rnd(n, width).to(dt) for _ in range(copies)]
        mu = torch.rand(5, width, device=dev, generator=g)
        add("token_shift_mix", "causal_conv_silu", [lambda h=h, s=s: ops.token_shift_mix(h, mu, s, hd * d, cu, token_req, slots)
                                                    for h, s in zip(hs, states)], n * width * 2 * 6, shape=label)
        lows = [rnd(n, wk["decay_rank"]) for _ in range(copies)]
        w2t, w0 = rnd(wk["decay_rank"], hd) / 8, torch.rand(hd, device=dev, generator=g) * 5 - 5.5
        add("wkv_decay", "-", [lambda a=a: ops.wkv_decay(a, w2t, w0) for a in lows], n * (hd + wk["decay_rank"]) * 4,
            2.0 * n * hd * wk["decay_rank"], fp32_tflops, shape=label)
        rkv = [(rnd(n, hd).to(dt), (rnd(n, hd) / 8).to(dt), rnd(n, hd).to(dt), ops.wkv_decay(a, w2t, w0)) for a in lows]
        u = rnd(heads, d)
        plan = ops.wkv_plan([per] * reqs, dev)                                  # long portions run as chunks, as in the model
        room = torch.empty(max(1, ops.wkv_workspace_floats(plan, heads, d)), device=dev)
        add("wkv_scan", "ssd_scan", [lambda x=x, s=s: ops.wkv_scan(x[0], x[1], x[2], x[3], u, s, cu, slots, reqs, heads, d,
                                                                    plan=plan, workspace=room)
                                     for x, s in zip(rkv, states)],
            n * hd * (3 * 2 + 4 + 4) + 2 * reqs * hd * d * 4, 4.0 * n * hd * d, fp32_tflops, shape=label)
        ys = [rnd(n, hd) for _ in range(copies)]
        gain = rnd(hd)
        add("group_rmsnorm_gate", "gated_group_rmsnorm", [lambda y=y, x=x: ops.group_rmsnorm_gate(y, x[0], gain, heads, 1e-6)
                                                          for y, x in zip(ys, rkv)], n * hd * (4 + 2 + 2), shape=label)
        # ---- the block's two norms in one pass, beside the dense decoder's fused add + norm
        resid = [rnd(n, width) for _ in range(copies)]
        deltas = [(rnd(n, width).to(dt), rnd(1, n, width)) for _ in range(copies)]
        g1, g2 = rnd(width), rnd(width)
        add("add_rmsnorm_multi (2 deltas, 2 norms)", "add_rmsnorm", [lambda r=r, x=x: ops.add_rmsnorm_multi(r, list(x), [g1, g2], 1e-6, dt)
                                                                      for r, x in zip(resid, deltas)],
            n * width * (8 + 2 + 4 + 2 * 2), shape=label)
        wn = torch.ones(width, device=dev, dtype=dt)
        add("add_rmsnorm (dense)", "-", [lambda r=r, x=x: ops.add_rmsnorm(r, x[0], wn, 1e-6, dt) for r, x in zip(resid, deltas)],
            n * width * (8 + 2 * 2), shape=label)
        # ---- the experts
        r_ = moe["router"]
        outputs, experts, top, ff = r_["experts"] + r_["identity"], r_["experts"], r_["top"], moe["expert"]["ff"]
        router, corr = rnd(outputs, width) * 3 / width ** 0.5, rnd(outputs) / (2 * outputs)
        add("moe_route + align", "-", [lambda h=h: ops.moe_route(h, router, corr, top, experts) for h in hs],
            n * width * 2 + outputs * width * 4, shape=label)
        gu = (rnd(experts, 2 * ff, width) / width ** 0.5).to(dt)
        dn = (rnd(experts, width, ff) / ff ** 0.5).to(dt)
        routings = [ops.moe_route(h, router, corr, top, experts) for h in hs]
        pairs = n * top
        touched = min(experts, pairs)
        add("moe_experts", "gate/up + down products", [lambda h=h, r=r: ops.moe_experts(h, r, gu, dn, 7.0, 1.702) for h, r in zip(hs, routings)],
            touched * 3 * ff * width * 2 + pairs * (width * 2 + ff * 4 + width * 4), 6.0 * pairs * ff * width, shape=label)
        dense_gu = (rnd(2 * z["ff"], width) / width ** 0.5).to(dt)
        dense_dn = (rnd(width, z["ff"]) / z["ff"] ** 0.5).to(dt)
        add("gate/up + down products (dense)", "-", [lambda h=h: ops.linear(ops.silu_mul(ops.linear(h, dense_gu)), dense_dn) for h in hs],
            3 * z["ff"] * width * 2, 6.0 * n * z["ff"] * width, shape=label)

    # ---- attention over the cached latent beside the dense decoder's attention
    h_, rank, rot, page = la["heads"], la["kv_rank"], la["rot_dim"], 64
    row = rank + rot
    window = la["mask"]["size"]
    nq, nkv, dd = z["heads"], z["kv_heads"], z["head"]
    pages = -(-tokens // page)
    cu1 = torch.tensor([0, tokens], device=dev, dtype=torch.int32)
    pre = torch.zeros(1, device=dev, dtype=torch.int32)
    span = min(window, tokens)
    pairs_w = tokens * span - span * (span - 1) / 2
    fns = []
    for _ in range(copies):
        cache = rnd(pages + 1, page * row).to(dt)
        table = (torch.randperm(pages, device=dev, generator=g) + 1).view(1, pages).to(torch.int32)
        q = (rnd(tokens, h_ * row) / 8).to(dt)
        out = torch.empty((tokens, h_ * rank), device=dev, dtype=dt)
        tile = ops.prefill_tile_rows(dt, row, page, tokens, dv=rank, values_in_keys=True, heads=h_)
        tr, ts = ops.prefill_tiles([0], [tokens], 0, tile, dev)
        fns.append(lambda q=q, cache=cache, table=table, out=out, tr=tr, ts=ts, tile=tile: ops.attention_prefill(
            q, cache, table, cu1, pre, tr, ts, out, h_, 1, row, page, la["scale"], window, tile_rows=tile, dv=rank, values_in_keys=True))
    add("latent attention, prefill (window)", "attention_prefill", fns, tokens * (row + h_ * (row + rank)) * 2,
        2.0 * h_ * (row + rank) * pairs_w, shape=f"{tokens} tokens")
    fns = []
    for _ in range(copies):
        cache = rnd(pages + 1, 2, nkv, page, dd).to(dt)
        table = (torch.randperm(pages, device=dev, generator=g) + 1).view(1, pages).to(torch.int32)
        q = rnd(tokens, nq * dd).to(dt)
        out = torch.empty_like(q)
        tile = ops.prefill_tile_rows(dt, dd, page, tokens)
        tr, ts = ops.prefill_tiles([0], [tokens], 0, tile, dev)
        fns.append(lambda q=q, cache=cache, table=table, out=out, tr=tr, ts=ts, tile=tile: ops.attention_prefill(
            q, cache, table, cu1, pre, tr, ts, out, nq, nkv, dd, page, dd ** -0.5, window, tile_rows=tile))
    add("attention_prefill (dense heads, same window)", "-", fns, tokens * (2 * nkv + 2 * nq) * dd * 2, 4.0 * nq * dd * pairs_w,
        shape=f"{tokens} tokens")
    pages = -(-context // page)
    seen = min(window, context)
    fns = []
    for _ in range(copies):
        cache = rnd(batch * pages + 1, page * row).to(dt)
        table = (torch.randperm(batch * pages, device=dev, generator=g) + 1).view(batch, pages).to(torch.int32)
        q = (rnd(batch, h_ * row) / 8).to(dt)
        out = torch.empty((batch, h_ * rank), device=dev, dtype=dt)
        seq = torch.full((batch,), context, device=dev, dtype=torch.int32)
        plan = ops.plan_decode_attention(dt, batch, h_, 1, row, seen, dv=rank, values_in_keys=True)
        scratch = torch.empty(max(1, plan.scratch_floats), device=dev)
        fns.append(lambda q=q, cache=cache, table=table, out=out, seq=seq, scratch=scratch, plan=plan: ops.attention_decode(
            q, cache, table, seq, out, scratch, plan.splits, h_, 1, row, page, la["scale"], window, dv=rank, values_in_keys=True))
    add("latent attention, decode (window)", "attention_decode", fns, batch * seen * row * 2 + batch * h_ * (row + rank) * 2,
        2.0 * batch * h_ * (row + rank) * seen, shape=f"{batch} x {context}")
    fns = []
    for _ in range(copies):
        cache = rnd(batch * pages + 1, 2, nkv, page, dd).to(dt)
        table = (torch.randperm(batch * pages, device=dev, generator=g) + 1).view(batch, pages).to(torch.int32)
        q = rnd(batch, nq * dd).to(dt)
        out = torch.empty_like(q)
        seq = torch.full((batch,), context, device=dev, dtype=torch.int32)
        plan = ops.plan_decode_attention(dt, batch, nq, nkv, dd, seen)
        scratch = torch.empty(max(1, plan.scratch_floats), device=dev)
        fns.append(lambda q=q, cache=cache, table=table, out=out, seq=seq, scratch=scratch, plan=plan: ops.attention_decode(
            q, cache, table, seq, out, scratch, plan.splits, nq, nkv, dd, page, dd ** -0.5, window, stages=plan.stages))
    add("attention_decode (dense heads, same window)", "-", fns, batch * seen * 2 * nkv * dd * 2 + 2 * batch * nq * dd * 2,
        4.0 * batch * nq * dd * seen, shape=f"{batch} x {context}")
    return rows


def run(sizes, layers, tokens, batch, context, steps, kernels=True, models=True) -> dict:
    out = {"design": "Godotar", "beside": "the Zirurax and the dense (Qwen3 layer) decoders at equal width and layers",
           "dtype": "bf16", "data": "synthetic: seeded random weights", "peaks": peaks(), "layers": layers,
           "prefill_tokens": tokens, "decode_batch": batch, "context": context, "sizes": {}}
    for name in sizes:
        z = SIZES[name]
        entry = {"shape": z}
        if models:
            entry["godotar"] = model_throughput(godotar_config(z, layers), tokens, batch, context, steps)
            entry["zirurax"] = model_throughput(zirurax_config(z, layers), tokens, batch, context, steps)
            entry["dense"] = model_throughput(dense_config(z, layers, context), tokens, batch, context, steps)
        if kernels:
            entry["kernels"] = kernel_table(z, tokens, batch, context)
        out["sizes"][name] = entry
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--sizes", nargs="+", default=["small", "mid"], choices=sorted(SIZES))
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--no-kernels", action="store_true")
    ap.add_argument("--no-models", action="store_true")
    ap.add_argument("--table", action="store_true", help="print the kernels as a table on stderr as well")
    a = ap.parse_args(argv)
    out = run(a.sizes, a.layers, a.tokens, a.batch, a.context, a.steps, kernels=not a.no_kernels, models=not a.no_models)
    if a.table:
        for name, entry in out["sizes"].items():
            for k in ("godotar", "zirurax", "dense"):
                if k in entry:
                    print(name, k, entry[k], file=sys.stderr)
            for row in entry.get("kernels", []):
                print(f"{name:6s} {row['kernel']:46s} {row['shape']:14s} {row['us']:10.2f} us  hbm {row['hbm_frac']:.3f}"
                      + (f"  {row['flop_peak']} {row['flop_frac']:.3f}" if "flop_frac" in row else "") + f"  ({row['bound']})",
                      file=sys.stderr)
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
