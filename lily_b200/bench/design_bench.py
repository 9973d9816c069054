"""The Zirurax decoder beside the dense (Qwen3-like) decoder at equal sizes: prefill and decode throughput of both
through the same step function, and each kernel of the new design alone against its roofline, beside the like kernel
of the dense decoder.

    python -m lily_b200.bench.design_bench [--sizes small mid] [--layers 4] [--kernels] [--models]
    python bench.py --design zirurax ...          (the same, as one JSON line)

Random weights in bfloat16.  A size gives both models the same width, feed-forward width, attention heads and
layers; the Zirurax layer adds the state-space mixer (inner = 2 x width, heads of 64, state 128), the window, the cap
and the output gate.  Throughput: tokens a second of a prefill of ``--tokens`` tokens, and of decode steps of
``--batch`` requests at ``--context`` positions through CUDA graphs (device time by CUDA events, after warm-up; the
weights and caches of every size are larger than L2).  Kernels: CUDA-event time over rotated inputs
(``kbench.time_ms``), achieved bytes and FLOP against the measured copy bandwidth and, for the float32 recurrences that
may not use tensor cores, against the FP32 FMA rate of the device (SMs x 128 lanes x 2 x clock).
"""

from __future__ import annotations

import argparse
import json
import statistics
import sys
from typing import Dict, List

import torch

from lily_b200.bench.kbench import peaks, time_ms

SIZES = {
    "small": dict(width=2048, ff=8192, heads=16, kv_heads=4, head=128, window=1024, s_heads=64, s_head=64, state=128,
                  groups=8, vocab=32000),
    "mid": dict(width=4096, ff=12288, heads=32, kv_heads=8, head=128, window=2048, s_heads=128, s_head=64, state=128,
                groups=8, vocab=32000),
}


def zirurax_config(z: dict, layers: int) -> dict:
    layer = {"type": "parallel",
             "mixer": {"left": {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["head"], "vdim": z["head"],
                                "scale": z["head"] ** -0.5, "softcap": 30.0, "mask": {"size": z["window"]},
                                "rot": {"dims": z["head"], "base": 1000000.0}},
                       "right": {"heads": z["s_heads"], "vdim": z["s_head"], "state": z["state"], "groups": z["groups"],
                                 "conv": 4, "norm_groups": z["groups"]}},
             "mlp": {"kind": "dense", "ff": z["ff"]}}
    return {"architecture": "Zirurax", "vocab": z["vocab"], "width": z["width"], "embedding": {"scale": 1.0},
            "norm": {"eps": 1e-6}, "layers": [layer] * layers}


def dense_config(z: dict, layers: int, context: int) -> dict:
    return {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": layers,
            "hidden_size": z["width"], "num_attention_heads": z["heads"], "num_key_value_heads": z["kv_heads"],
            "head_dim": z["head"], "intermediate_size": z["ff"], "vocab_size": z["vocab"], "rope_theta": 1000000.0,
            "rms_norm_eps": 1e-6, "tie_word_embeddings": True, "max_position_embeddings": context, "hidden_act": "silu",
            "torch_dtype": "bfloat16"}


def device_ms(fn, reps: int) -> float:
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(reps):
        fn()
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) / reps


def model_throughput(cfg: dict, tokens: int, batch: int, context: int, steps: int) -> Dict[str, float]:
    from lily_b200.config.server_args import ServerArgs
    from lily_b200.csrc import ops
    from lily_b200.engine.batch import FUTURE, StepEntry
    from lily_b200.engine.runner import ModelRunner

    args = ServerArgs(dtype="bfloat16", device="cuda:0", context_length=context, page_size=64,
                      max_total_tokens=(batch + 1) * (context + 64), max_running_requests=batch + 1, random_seed=0)
    runner = ModelRunner.from_random(cfg, seed=0, args=args)
    vocab = runner.spec.vocab_size
    g = torch.Generator().manual_seed(1)
    ids = lambda n: torch.randint(0, vocab, (n,), generator=g).tolist()
    prompt = ids(tokens)

    def prefill_once():
        slot = runner.open_request()
        runner.step([StepEntry(slot, prompt, [tokens - 1])])
        runner.close_request(slot)
    for _ in range(3):
        prefill_once()
    prefill_ms = device_ms(prefill_once, 5)

    total = 3 + 3 * steps
    slots = [runner.open_request() for _ in range(batch)]
    for s in slots:
        runner.step([StepEntry(s, ids(context - total - 2), [])])
    runner.store_future(ops.argmax(runner.step([StepEntry(s, [ids(1)[0]], [0]) for s in slots])))
    entries = [StepEntry(s, [FUTURE], [0]) for s in slots]
    one = lambda: runner.store_future(ops.argmax(runner.step(entries)))
    for _ in range(3):
        one()
    l0 = ops.launches["count"]
    decode_ms = statistics.median(device_ms(one, steps) for _ in range(3))
    launches = (ops.launches["count"] - l0) // (3 * steps)
    graphs = runner.graph_steps
    torch.cuda.synchronize()
    for s in slots:
        runner.close_request(s)
    out = {"prefill_tokens_s": round(tokens / prefill_ms * 1e3, 1), "prefill_ms": round(prefill_ms, 3),
           "decode_tokens_s": round(batch / decode_ms * 1e3, 1), "decode_ms": round(decode_ms, 4),
           "launches_per_decode_step": int(launches), "graph_steps": int(graphs), "weight_gb": round(runner.weight_bytes / 1e9, 2)}
    del runner
    torch.cuda.empty_cache()
    return out


def kernel_table(z: dict, tokens: int, batch: int, context: int, reps: int = 30, copies: int = 3) -> List[dict]:
    """Each kernel of the new design alone, prefill shape (``tokens`` of one request) and decode shape (``batch``
    requests of one token), beside the like kernel of the dense decoder."""
    from lily_b200.csrc import ops

    dev, dt = "cuda", torch.bfloat16
    pk = peaks()
    props = torch.cuda.get_device_properties(0)
    fp32_tflops = props.multi_processor_count * 128 * 2 * (props.clock_rate if hasattr(props, "clock_rate") else 1965000) / 1e9
    g = torch.Generator(device=dev).manual_seed(0)
    rnd = lambda *shape: torch.randn(*shape, device=dev, generator=g)
    width, inner = z["width"], z["s_heads"] * z["s_head"]
    channels = inner + 2 * z["groups"] * z["state"]
    projected = 2 * inner + 2 * z["groups"] * z["state"] + z["s_heads"]
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
        state_floats = inner * z["state"] + 3 * channels
        # ---- the state-space mixer's kernels
        conv_w, conv_b = rnd(channels, 4), rnd(channels)
        cr, cs = ops.token_chunks([per] * reqs, ops.SSM_CHUNK, dev)
        projs = [rnd(n, projected).to(dt) for _ in range(copies)]
        states = [torch.zeros(reqs + 1, state_floats, device=dev) for _ in range(copies)]
        add("causal_conv_silu", "qk_norm_rope_write", [lambda p=p, s=s: ops.causal_conv_silu(p, inner, channels, conv_w, conv_b, s, inner * z["state"], cr, cs, cu, slots)
                                                        for p, s in zip(projs, states)],
            n * channels * 4 + (reqs * 3 * channels * 8 if label == "decode" else 0), shape=label)
        xbcs = [rnd(n, channels).to(dt) for _ in range(copies)]
        vecs = [rnd(z["s_heads"]) - 2 for _ in range(3)]
        scan_flops = 6.0 * n * inner * z["state"]
        scan_bytes = n * (channels * 2 + inner * 4) + 2 * reqs * inner * z["state"] * 4
        plan = ops.scan_plan([per] * reqs, dev, inner * z["state"])            # long portions run as chunks, as in the model
        room = torch.empty(max(1, ops.scan_workspace_floats(plan, z["s_heads"], z["s_head"], z["state"])), device=dev)
        add("ssd_scan", "attention", [lambda x=x, p=p, s=s: ops.ssd_scan(x, p, inner + channels, vecs[0], vecs[1], vecs[2], s, cu, slots, reqs,
                                                                          z["s_heads"], z["s_head"], z["state"], z["groups"],
                                                                          plan=plan, workspace=room)
                                      for x, p, s in zip(xbcs, projs, states)],
            scan_bytes, scan_flops, fp32_tflops, shape=label)
        ys = [rnd(n, inner) for _ in range(copies)]
        gain = rnd(inner)
        add("gated_group_rmsnorm", "add_rmsnorm", [lambda y=y, p=p: ops.gated_group_rmsnorm(y, p, gain, z["groups"], 1e-6) for y, p in zip(ys, projs)],
            n * inner * (4 + 2 + 2), shape=label)
        # ---- joining the sublayers
        outs = [(rnd(n, width).to(dt), rnd(n, width).to(dt), rnd(n, width).to(dt)) for _ in range(copies)]
        gains = [rnd(width), rnd(width)]
        add("normed_mean", "add_rmsnorm", [lambda o=o: ops.normed_mean([o[0], o[1]], gains, 1e-6, add=o[2]) for o in outs],
            n * width * (3 * 2 + 4), shape=label)
        resid = [rnd(n, width) for _ in range(copies)]
        w = torch.ones(width, device=dev, dtype=dt)
        add("add_rmsnorm (dense)", "-", [lambda r=r, o=o: ops.add_rmsnorm(r, o[0], w, 1e-6, dt) for r, o in zip(resid, outs)],
            n * width * (8 + 2 * 2), shape=label)
        heads_out = z["heads"] * z["head"]
        att = [(rnd(n, heads_out).to(dt), rnd(n, heads_out).to(dt)) for _ in range(copies)]
        add("sigmoid_gate", "silu_mul", [lambda a=a: ops.sigmoid_gate(a[0], a[1]) for a in att], n * heads_out * 6, shape=label)
        gus = [rnd(n, 2 * z["ff"]).to(dt) for _ in range(copies)]
        add("gelu_tanh * up", "silu_mul", [lambda x=x: ops.silu_mul(x, block=128, activation="gelu_tanh") for x in gus], n * z["ff"] * 6, shape=label)
        add("silu * up (dense)", "-", [lambda x=x: ops.silu_mul(x, block=128) for x in gus], n * z["ff"] * 6, shape=label)

    # ---- attention: window and cap beside the dense decoder's plain scores
    nq, nkv, d, page = z["heads"], z["kv_heads"], z["head"], 64
    for label, window, cap in (("attention_prefill window+cap", z["window"], 30.0), ("attention_prefill (dense)", None, None)):
        pages = -(-tokens // page)
        fns = []
        for _ in range(copies):
            cache = rnd(pages + 1, 2, nkv, page, d).to(dt)
            table = (torch.randperm(pages, device=dev, generator=g) + 1).view(1, pages).to(torch.int32)
            q = rnd(tokens, nq * d).to(dt)
            out = torch.empty_like(q)
            tile = ops.prefill_tile_rows(dt, d, page, tokens, softcap=cap)
            tr, ts = ops.prefill_tiles([0], [tokens], 0, tile, dev)
            cu1 = torch.tensor([0, tokens], device=dev, dtype=torch.int32)
            pre = torch.zeros(1, device=dev, dtype=torch.int32)
            fns.append(lambda q=q, cache=cache, table=table, out=out, tr=tr, ts=ts: ops.attention_prefill(
                q, cache, table, cu1, pre, tr, ts, out, nq, nkv, d, page, d ** -0.5, window, tile_rows=tile, softcap=cap))
        span = min(window or tokens, tokens)
        pairs = tokens * span - span * (span - 1) / 2 if window else tokens * (tokens + 1) / 2
        add(label, "attention_prefill" if window else "-", fns, tokens * (2 * nkv + 2 * nq) * d * 2, 4.0 * nq * d * pairs, shape=f"{tokens} tokens")
    for label, window, cap in (("attention_decode window+cap", z["window"], 30.0), ("attention_decode (dense)", None, None)):
        pages = -(-context // page)
        seen = min(window or context, context)
        fns = []
        for _ in range(copies):
            cache = rnd(batch * pages + 1, 2, nkv, page, d).to(dt)
            table = (torch.randperm(batch * pages, device=dev, generator=g) + 1).view(batch, pages).to(torch.int32)
            q = rnd(batch, nq * d).to(dt)
            out = torch.empty_like(q)
            seq = torch.full((batch,), context, device=dev, dtype=torch.int32)
            plan = ops.plan_decode_attention(dt, batch, nq, nkv, d, seen)
            scratch = torch.empty(max(1, plan.scratch_floats), device=dev)
            fns.append(lambda q=q, cache=cache, table=table, out=out, seq=seq, scratch=scratch, plan=plan: ops.attention_decode(
                q, cache, table, seq, out, scratch, plan.splits, nq, nkv, d, page, d ** -0.5, window, stages=plan.stages, softcap=cap))
        add(label, "attention_decode" if window else "-", fns, batch * seen * 2 * nkv * d * 2 + 2 * batch * nq * d * 2,
            4.0 * batch * nq * d * seen, shape=f"{batch} x {context}")
    return rows


def run(sizes, layers, tokens, batch, context, steps, kernels=True, models=True) -> dict:
    out = {"design": "Zirurax", "beside": "dense decoder (Qwen3 layer) at equal width, heads, feed-forward and layers",
           "dtype": "bf16", "data": "synthetic: seeded random weights", "peaks": peaks(), "layers": layers,
           "prefill_tokens": tokens, "decode_batch": batch, "context": context, "sizes": {}}
    for name in sizes:
        z = SIZES[name]
        entry = {"shape": z}
        if models:
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
            for k in ("zirurax", "dense"):
                if k in entry:
                    print(name, k, entry[k], file=sys.stderr)
            for row in entry.get("kernels", []):
                print(f"{name:6s} {row['kernel']:32s} {row['shape']:14s} {row['us']:10.2f} us  hbm {row['hbm_frac']:.3f}"
                      + (f"  {row['flop_peak']} {row['flop_frac']:.3f}" if "flop_frac" in row else "") + f"  ({row['bound']})",
                      file=sys.stderr)
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
