"""The Godotar decoder through the engine against its plain implementation (``plain_godotar``), in every cutting:
whole prompts, token-by-token decoding, portions down to two tokens, mixed batches of unequal requests, pages and
slots that are freed and used again, long decoding past every window, greedy generation through the entry point and
the scheduler.  The CPU variants run the engine's host side over the kernels' plain statements; the ``gpu`` variants
run the CUDA kernels in float32 and bfloat16."""

import copy
import tempfile

import pytest
import torch

import godotar_models as gm
import plain_godotar
from harness import make_runner, run_mixed, run_portions, run_whole
from lily_b200.config.model_config import ConfigError
from lily_b200.engine.batch import StepEntry

DEVICES = ["cpu", pytest.param("cuda", marks=pytest.mark.gpu)]
CONFIGS = {"varied": gm.VARIED, "sharp": gm.SHARP, "wide": gm.WIDE}


def plain_logits(cfg, weights, ids, dtype="float32"):
    if dtype == "bfloat16":
        weights = {k: v.bfloat16().float() for k, v in weights.items()}
    with plain_godotar.precision(torch.float64):
        return plain_godotar.forward(cfg, weights, ids).float()


def close(got, want, dtype, what=""):
    err = (got - want).abs()
    if dtype == "float32":
        assert float(err.max()) < 2e-4 * max(1.0, float(want.abs().max())), f"{what}: max error {float(err.max()):.3e}"
    else:
        # A score rounded to bfloat16 hands a token to another expert where two choice scores are next to equal; that
        # token's row then differs outright, and through the recurrent state so may a few after it.  So bfloat16 is
        # judged by rows: nine in ten within the bound that correct kernels keep, the median row well within it.
        # (float32 above is the sharp comparison.)
        scale = float(want.abs().max())
        rows = err.max(-1).values.sort().values
        assert float(rows[int(0.9 * (len(rows) - 1))]) < 0.06 * scale and float(rows[len(rows) // 2]) < 0.03 * scale, \
            f"{what}: row errors median {float(rows[len(rows) // 2]):.3e}, max {float(rows[-1]):.3e} (logits up to {scale:.2f})"


@pytest.fixture(scope="module", params=sorted(CONFIGS))
def setup(request):
    cfg = CONFIGS[request.param]
    with tempfile.TemporaryDirectory() as tmp:
        weights = gm.make_weights(cfg, 11)
        yield cfg, weights, gm.write_model_dir(tmp + "/m", cfg, weights)


def runner_for(path, device, dtype="float32", max_tokens=512, page_size=16, max_requests=4):
    return make_runner(path, dtype=dtype, device=device, max_tokens=max_tokens, page_size=page_size,
                       max_requests=max_requests, context_length=1024)


def dtypes(device, cfg=None):
    """bfloat16 on the GPU too, except for the configuration whose near one-hot attention and routing turn a rounding
    into another key or expert (it is there for the exact comparison in float32)."""
    return ["float32"] if device == "cpu" or cfg is gm.SHARP else ["float32", "bfloat16"]


@pytest.mark.parametrize("device", DEVICES)
def test_whole_decoded_and_in_portions(setup, device):
    """A prompt whole; its last 40 tokens one by one (past every window of the small configurations, over several
    page borders); portions of changing sizes down to two tokens and single tokens between them."""
    cfg, weights, path = setup
    ids = gm.tokens(150, cfg["vocab"], 5)
    for dtype in dtypes(device, cfg):
        want = plain_logits(cfg, weights, ids, dtype)
        runner = runner_for(path, device, dtype)
        close(run_whole(runner, ids), want, dtype, "whole")
        close(run_portions(runner, ids, [110] + [1] * 40), want, dtype, "decoded")
        close(run_portions(runner, ids, [3, 2, 31, 2, 1, 1, 17, 2, 5, 1, 64, 2]), want, dtype, "portions")
        close(run_portions(runner, ids, [1] * 24 + [2] * 10), want, dtype, "from the first token on")
        assert runner.cache.held_pages() == [0] * len(runner.cache.groups) and runner.cache.slots.available == 4


@pytest.mark.parametrize("device", DEVICES)
def test_mixed_batches_with_pages_and_slots_used_again(setup, device):
    """Up to four live requests of unequal lengths, portions of some beside single tokens of others, in a pool that
    holds fewer tokens than all requests together and with four slots for six requests."""
    cfg, weights, path = setup
    lens = {"a": 90, "b": 41, "c": 70, "d": 33, "e": 58, "f": 20}
    reqs = {k: gm.tokens(n, cfg["vocab"], 40 + i) for i, (k, n) in enumerate(lens.items())}
    plan = [{"a": 30, "b": 2, "c": 17}, {"a": 1, "b": 20, "c": 2, "d": 33}, {"a": 1, "b": 1, "c": 1},
            {"a": 28, "b": 18, "c": 50}, {"a": 1, "e": 16}, {"a": 1, "e": 1, "f": 3}, {"a": 28, "e": 41, "f": 17}]
    ends = {1: ["d"], 3: ["b", "c"]}
    for dtype in dtypes(device, cfg):
        runner = runner_for(path, device, dtype, max_tokens=16 * 16)
        got = run_mixed(runner, reqs, plan, ends)
        for k, ids in reqs.items():
            close(got[k], plain_logits(cfg, weights, ids, dtype), dtype, f"request {k}")
        assert runner.cache.held_pages() == [0] * len(runner.cache.groups) and runner.cache.slots.available == 4


@pytest.mark.parametrize("device", DEVICES)
def test_a_batch_changes_no_request(setup, device):
    """The logits of a request do not depend on what else is in the batch or on the slot and pages it got."""
    cfg, weights, path = setup
    reqs = {k: gm.tokens(n, cfg["vocab"], 70 + i) for i, (k, n) in enumerate({"a": 37, "b": 64, "c": 9}.items())}
    runner = runner_for(path, device)
    alone = {k: run_portions(runner, ids, [len(ids) - 4, 1, 1, 1, 1]) for k, ids in reqs.items()}
    filler = runner.open_request()                       # the batch's requests get other slots and pages than alone
    runner.step([StepEntry(filler, gm.tokens(21, cfg["vocab"], 1), [])])
    plan = [{k: len(ids) - 4 for k, ids in reqs.items()}] + [{k: 1 for k in reqs}] * 4
    together = run_mixed(runner, reqs, plan)
    runner.close_request(filler)
    for k in reqs:
        assert float((together[k] - alone[k]).abs().max()) < 1e-5 * max(1.0, float(alone[k].abs().max())), k


@pytest.mark.parametrize("device", DEVICES)
def test_long_decoding_through_graphs(setup, device):
    """Three requests decode 70 tokens side by side (captured steps on the GPU), far past their windows, while the
    windowed cache groups give pages back and every pass of the looped layers carries its own state."""
    cfg, weights, path = setup
    reqs = {k: gm.tokens(n, cfg["vocab"], 90 + i) for i, (k, n) in enumerate({"a": 100, "b": 81, "c": 75}.items())}
    plan = [{"a": 30, "b": 11, "c": 5}] + [{"a": 1, "b": 1, "c": 1}] * 70
    for dtype in dtypes(device, cfg):
        runner = runner_for(path, device, dtype)
        before = runner.graph_steps
        got = run_mixed(runner, reqs, plan)
        for k, ids in reqs.items():
            close(got[k], plain_logits(cfg, weights, ids, dtype), dtype, f"request {k}")
        if device == "cuda":
            assert runner.model.graph_safe and runner.graph_steps - before == 70


@pytest.mark.gpu
@pytest.mark.parametrize("seed", range(24))
def test_configurations_drawn_at_random(seed):
    """Two dozen configurations drawn at random (layer order, sizes, loop, windows, feed-forwards): whole, decoded, in portions
    and two requests side by side, in both precisions, on whichever kernels their sizes get."""
    cfg = gm.random_config(seed)
    with tempfile.TemporaryDirectory() as tmp:
        weights = gm.make_weights(cfg, 100 + seed)
        path = gm.write_model_dir(tmp + "/m", cfg, weights)
        ids, other = gm.tokens(140, cfg["vocab"], seed), gm.tokens(45, cfg["vocab"], seed + 50)
        for dtype in ("float32", "bfloat16"):
            want, want_other = plain_logits(cfg, weights, ids, dtype), plain_logits(cfg, weights, other, dtype)
            runner = runner_for(path, "cuda", dtype, page_size=16 if seed % 2 else 64)
            close(run_whole(runner, ids), want, dtype, f"whole {cfg}")
            close(run_portions(runner, ids, [100] + [1] * 40), want, dtype, "decoded")
            close(run_portions(runner, ids, [2, 33, 1, 2, 70, 1, 1, 30]), want, dtype, "portions")
            got = run_mixed(runner, {"a": ids, "b": other}, [{"a": 90, "b": 3}, {"a": 1, "b": 40}, {"a": 49, "b": 1}, {"b": 1}])
            close(got["a"], want, dtype, "beside another")
            close(got["b"], want_other, dtype, "the other")


@pytest.mark.parametrize("device", DEVICES)
def test_a_slot_used_again_starts_from_nothing(device):
    """A request that takes the slot and pages of one that ended sees nothing of it: neither the heads' matrices, nor
    the carried input of the token shift, nor a cached latent."""
    cfg = gm.VARIED
    with tempfile.TemporaryDirectory() as tmp:
        weights = gm.make_weights(cfg, 13)
        path = gm.write_model_dir(tmp + "/m", cfg, weights)
        runner = runner_for(path, device, max_tokens=64, max_requests=1)
        first, second = gm.tokens(50, cfg["vocab"], 1), gm.tokens(23, cfg["vocab"], 2)
        run_portions(runner, first, [20, 30])
        close(run_portions(runner, second, [10, 1, 12]), plain_logits(cfg, weights, second), "float32", "second request")


@pytest.mark.parametrize("device", DEVICES)
def test_greedy_generation_through_the_entry_point(device):
    """``Engine.generate`` (scheduler, sampler, cache manager) against greedy decoding with the plain implementation."""
    from lily_b200.engine.engine import Engine, EngineConfig
    from lily_b200.sampling.params import SamplingParams

    cfg = gm.VARIED
    with tempfile.TemporaryDirectory() as tmp:
        weights = gm.make_weights(cfg, 12)
        path = gm.write_model_dir(tmp + "/m", cfg, weights)
        runner = runner_for(path, device, max_tokens=640, max_requests=3)
        engine = Engine(EngineConfig(model_path=path, dtype="float32", device=device,
                                     server_args={"chunked_prefill_size": 32, "max_prefill_tokens": 48}), runner=runner)
        prompts = [gm.tokens(n, cfg["vocab"], 200 + n) for n in (45, 7, 70, 1, 33)]
        out = engine.generate(prompts, SamplingParams(max_new_tokens=12, ignore_eos=True))
        for ids, res in zip(prompts, out):
            seq = list(ids)
            for tok in res["output_ids"]:
                logits = plain_logits(cfg, weights, seq)[-1]
                best = int(torch.argmax(logits))
                # a near-tie may fall either way: the chosen token must be (almost) the best one
                assert tok == best or float(logits[best] - logits[tok]) < 1e-3
                seq.append(tok)
            assert len(res["output_ids"]) == 12


@pytest.mark.gpu
def test_command_line_writes_random_weights_and_generates():
    """``python -m lily_b200 init-random`` from a config.json that gives the decay's rank, then ``generate`` from the
    folder it wrote: the tokens are the plain implementation's greedy choice over the written weights."""
    import json
    import os
    import subprocess
    import sys

    from lily_b200.weights.safetensors_io import SafetensorsFile

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = copy.deepcopy(gm.VARIED)
    for layer in cfg["layers"]:
        if layer["type"] == "wkv":
            layer["mixer"]["decay_rank"] = 5
    with tempfile.TemporaryDirectory() as tmp:
        with open(tmp + "/config.json", "w") as f:
            json.dump(cfg, f)
        run = lambda *args: subprocess.run([sys.executable, "-m", "lily_b200", *args], cwd=root, capture_output=True, text=True, timeout=900)
        out = run("init-random", "--config", tmp + "/config.json", "--out", tmp + "/m", "--seed", "3")
        assert out.returncode == 0, out.stderr[-2000:]
        prompt = gm.tokens(19, cfg["vocab"], 8)
        out = run("generate", "--model-path", tmp + "/m", "--dtype", "float32", "--max-total-tokens", "256", "--page-size", "16",
                  "--prompt-ids", ",".join(map(str, prompt)), "--max-new-tokens", "5", "--ignore-eos")
        assert out.returncode == 0, out.stderr[-2000:]
        got = json.loads(out.stdout.strip().splitlines()[-1])["output_ids"]
        held = SafetensorsFile(tmp + "/m/model.safetensors")
        weights = {n: held.tensor(n).float() for n in held.entries}
        seq = list(prompt)
        for tok in got:
            logits = plain_logits(cfg, weights, seq)[-1]
            best = int(torch.argmax(logits))
            assert tok == best or float(logits[best] - logits[tok]) < 1e-3
            seq.append(tok)
        assert len(got) == 5


def test_config_refuses_what_the_design_does_not_have():
    from lily_b200.config.godotar_config import GodotarConfig

    GodotarConfig.from_dict(gm.VARIED)
    for path, value in ((("layers", 0, "type"), "serial"), (("layers", 0, "mlp", "kind"), "sparse"),
                        (("layers", 0, "mixer", "rot", "dims"), 3), (("layers", 0, "mlp", "router", "top"), 9),
                        (("loop", "stop"), 7), (("loop", "times"), 0)):
        cfg = copy.deepcopy(gm.VARIED)
        node = cfg
        for key in path[:-1]:
            node = node[key]
        node[path[-1]] = value
        with pytest.raises(ConfigError):
            GodotarConfig.from_dict(cfg)


def test_schedule_cache_groups_and_states():
    """The looped stretch becomes runs of the schedule with caches and states of their own; a size that config.json
    leaves out is read off the checkpoint."""
    with tempfile.TemporaryDirectory() as tmp:
        path = gm.write_model_dir(tmp + "/m", gm.VARIED, gm.make_weights(gm.VARIED, 3))
        runner = make_runner(path, max_tokens=64, page_size=8, max_requests=2, context_length=64)
        spec = runner.spec
        assert [(e.block, e.step) for e in spec.schedule] == [
            (0, None), (1, ("loop.step", 0)), (2, None), (1, ("loop.step", 1)), (2, None), (1, ("loop.step", 2)), (2, None),
            (3, None)]
        needs = [(n.kv_heads, n.head_dim, n.v_head_dim, n.window, n.values_in_keys, layers) for n, layers in runner.model.cache_groups]
        assert needs == [(1, 28, 24, 11, True, 1), (1, 26, 18, 7, True, 3)]
        # heads * head size squared for the matrices, then the carried input of the token shift
        assert [tuple(s.shape[1:]) for s in runner.cache.states] == [(2 * 12 * 12 + 48,)] * 3 + [(5 * 4 * 4 + 48,)]
        assert spec.blocks[1].mixers[0][1].decay_rank == gm.DECAY_RANK


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_tool_in_every_cutting(dtype):
    """``bin/trace_run`` as a subprocess: whole, last tokens one by one, portions, then four live requests with pages
    and state slots used again (six requests over four slots and a pool of five pages of 64)."""
    from test_trace_run_gpu import Trace, replay

    cfg = gm.WIDE
    with tempfile.TemporaryDirectory() as tmp:
        weights = gm.make_weights(cfg, 21)
        path = gm.write_model_dir(tmp + "/m", cfg, weights)
        reqs = {k: gm.tokens(n, cfg["vocab"], 300 + i) for i, (k, n) in enumerate(
            {"w": 150, "t": 140, "p": 131, "a": 100, "b": 70, "c": 64, "d": 90, "e": 40}.items())}
        t = Trace(reqs)
        t.step({"w": 150}, end=["w"])
        t.step({"t": 90})
        for i in range(50):
            t.step({"t": 1}, end=["t"] if i == 49 else [])
        for i, n in enumerate([8, 2, 30, 17, 2, 3, 40, 2, 5, 22]):
            t.step({"p": n}, end=["p"] if i == 9 else [])
        t.step({"a": 60})
        t.step({"a": 1, "b": 33})
        t.step({"a": 1, "b": 2, "c": 64}, want={"c": [63, 0]})
        t.step({"b": 35, "a": 1, "d": 5}, end=["c"])
        t.step({"a": 37, "d": 2}, end=["b"])
        t.step({"d": 83, "e": 3}, end=["a"])
        t.step({"e": 1}, end=["d"])
        t.step({"e": 36}, end=["e"])
        rows = replay(path, dtype, t.steps, 320, tmp, cfg["vocab"])
        plain = {k: plain_logits(cfg, weights, ids, dtype) for k, ids in reqs.items()}
        for i, expect in enumerate(t.expect):
            want = torch.stack([plain[k][pos] for k, pos in expect])
            close(rows[i], want, dtype, f"step {i}")


@pytest.mark.parametrize("device", DEVICES)
def test_a_long_prompt_whole_and_cut(device):
    """600 tokens, whole and cut at odd places, beside a short request in the same step: the recurrence carried over
    hundreds of tokens, the window of all keys over several pages."""
    cfg = gm.WIDE
    with tempfile.TemporaryDirectory() as tmp:
        weights = gm.make_weights(cfg, 14)
        path = gm.write_model_dir(tmp + "/m", cfg, weights)
        ids, other = gm.tokens(600, cfg["vocab"], 6), gm.tokens(30, cfg["vocab"], 7)
        for dtype in dtypes(device, cfg):
            want, want_other = plain_logits(cfg, weights, ids, dtype), plain_logits(cfg, weights, other, dtype)
            runner = runner_for(path, device, dtype, max_tokens=1024, page_size=64)
            close(run_whole(runner, ids), want, dtype, "whole")
            close(run_portions(runner, ids, [333, 2, 1, 264]), want, dtype, "portions")
            got = run_mixed(runner, {"a": ids, "b": other}, [{"a": 450, "b": 29}, {"a": 150, "b": 1}])
            close(got["a"], want, dtype, "beside a short request")
            close(got["b"], want_other, dtype, "the short request")
