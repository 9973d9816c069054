"""Each mechanism of the Godotar decoder alone: the kernels' faces (CUDA on the GPU, their plain statements on the
CPU) against the functions of ``plain_godotar``, with inputs made so that a fault shows: one cached position scaled to
stand out far back, at a page border, just inside and just outside the window; states carried over portions of every
length; a slow decay that keeps the first token alive for hundreds of steps; router scores at a correction's mercy;
sizes that are not powers of two."""

import math

import pytest
import torch

import kernel_refs
import plain_godotar as pg

DEVICES = ["cpu", pytest.param("cuda", marks=pytest.mark.gpu)]


def ops_for(device):
    if device == "cpu":
        return kernel_refs
    from lily_b200.csrc import ops
    return ops


def i32(values, device):
    return torch.tensor(values, dtype=torch.int32, device=device)


def dtypes_of(device):
    return [torch.float32] if device == "cpu" else [torch.float32, torch.bfloat16]


def rounded(x, dtype):
    return x.to(dtype).float()


# ------------------------------------------------------------------ token shift

@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("width", [48, 301])
def test_token_shift_carries_the_last_input(device, width):
    """Two requests side by side, cut differently; the slot hands the last input of a portion to the next one, and a
    request's first token sees zeros."""
    ops = ops_for(device)
    g = torch.Generator().manual_seed(width)
    mu = torch.rand(5, width, generator=g)
    seqs = [torch.randn(37, width, generator=g), torch.randn(20, width, generator=g)]
    cuts = [[5, 1, 1, 30], [2, 9, 8, 1]]
    for dtype in dtypes_of(device):
        state = torch.zeros(4, 11 + width, device=device)
        state[0] = 7.0                                        # slot 0 belongs to no one; nothing may read it
        got = [[], []]
        done = [0, 0]
        for step in range(4):
            n = [cuts[0][step], cuts[1][step]]
            h = torch.cat([seqs[r][done[r]:done[r] + n[r]] for r in range(2)]).to(device=device, dtype=dtype)
            out = ops.token_shift_mix(h, mu.to(device), state, 11, i32([0, n[0], n[0] + n[1]], device),
                                      i32([0] * n[0] + [1] * n[1], device), i32([2, 1], device))
            got[0].append(out[:, :n[0]].float().cpu())
            got[1].append(out[:, n[0]:].float().cpu())
            done = [done[r] + n[r] for r in range(2)]
        for r in range(2):
            x = rounded(seqs[r], dtype)
            want = torch.stack([pg.token_shift(x, mu[s]) for s in range(5)])
            tol = 1e-6 if dtype == torch.float32 else 2e-2
            assert float((torch.cat(got[r], 1) - want).abs().max()) < tol * float(want.abs().max())
        assert float(state[:, :11].abs().max().cpu()) in (0.0, 7.0)          # columns ahead of the carried input are not its


# ------------------------------------------------------------------ decay and recurrence

@pytest.mark.parametrize("device", DEVICES)
def test_decay_logarithm(device):
    ops = ops_for(device)
    g = torch.Generator().manual_seed(3)
    t, width, rank, cols = 33, 40, 7, 90
    mix = torch.randn(t, width, generator=g)
    w = {"p.w1": torch.randn(rank, width, generator=g) / 6, "p.w2": torch.randn(cols, rank, generator=g),
         "p.w0": torch.rand(cols, generator=g) * 5 - 5}
    want = pg.wkv_decay(mix, w, "p")
    a = (mix @ w["p.w1"].t()).to(device)
    got = ops.wkv_decay(a, w["p.w2"].t().contiguous().to(device), w["p.w0"].to(device))
    assert float((torch.exp(got.cpu()) - want).abs().max()) < 1e-6
    assert float(want.min()) < 0.7 and float(want.max()) > 0.99             # fast and slow decays both occur


def scan_in_portions(ops, device, dtype, r, k, v, lw, u, cuts, slot=2, slots=4):
    t, heads, d = r.shape
    state = torch.zeros(slots, heads * d * d + 5, device=device)
    flat = lambda x: x.reshape(t, heads * d).to(device=device, dtype=dtype)
    rf, kf, vf = flat(r), flat(k), flat(v)
    lwf = lw.reshape(t, heads * d).to(device)
    out, done = [], 0
    for n in cuts:
        sl = slice(done, done + n)
        out.append(ops.wkv_scan(rf[sl].contiguous(), kf[sl].contiguous(), vf[sl].contiguous(), lwf[sl].contiguous(),
                                u.to(device), state, i32([0, n], device), i32([slot], device), 1, heads, d).cpu())
        done += n
    assert done == t
    return torch.cat(out).view(t, heads, d), state[slot, :heads * d * d].view(heads, d, d).cpu()


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("heads,d", [(2, 16), (3, 12), (1, 64), (2, 40), (1, 100), (1, 136)])
def test_recurrence_against_the_plain_loop(device, heads, d):
    """Whole, decoded one by one, and in portions of every kind; head sizes that are no multiple of the kernel's tiles."""
    ops = ops_for(device)
    g = torch.Generator().manual_seed(d)
    t = 90 if d > 64 else 150
    r, k, v = (torch.randn(t, heads, d, generator=g) for _ in range(3))
    k = k / math.sqrt(d)
    lw = -torch.exp(torch.rand(t, heads, d, generator=g) * 6 - 6)            # decays from 0.37 to 0.9975
    u = torch.randn(heads, d, generator=g)
    for dtype in dtypes_of(device):
        rr, kk, vv = (rounded(x, dtype) for x in (r, k, v))
        want, want_state = pg.wkv_recurrence(rr.double(), kk.double(), vv.double(), torch.exp(lw.double()), u.double())
        for cuts in ([t], [t - 40] + [1] * 40, [3, 2, 17, 1, 1, 2, 33, t - 59], [1] * 20 + [t - 20]):
            got, state = scan_in_portions(ops, device, dtype, r, k, v, lw, u, cuts)
            scale = float(want.abs().max())
            assert float((got - want.float()).abs().max()) < 2e-5 * scale, (dtype, cuts[:3])
            assert float((state - want_state.float()).abs().max()) < 2e-5 * max(1.0, float(want_state.abs().max()))


@pytest.mark.gpu
@pytest.mark.parametrize("heads,d", [(2, 64), (3, 24)])
def test_recurrence_in_chunks_side_by_side(heads, d):
    """Long portions run as chunks side by side (each first from zero, then from the matrices it starts from), beside
    short portions of the same step that run whole; two steps, so the second continues from the slots."""
    from lily_b200.csrc import ops
    device = "cuda"
    g = torch.Generator().manual_seed(d)
    lens = [[700, 40, 300], [257, 1, 520]]                       # per step: new tokens of three requests
    total = [sum(step[q] for step in lens) for q in range(3)]
    seqs = []
    for n in total:
        r, k, v = (torch.randn(n, heads, d, generator=g) for _ in range(3))
        seqs.append((r, k / math.sqrt(d), v, -torch.exp(torch.rand(n, heads, d, generator=g) * 6 - 6)))
    u = torch.randn(heads, d, generator=g)
    state = torch.zeros(5, heads * d * d + 3, device=device)
    slots = i32([3, 1, 4], device)
    got = [[], [], []]
    done = [0, 0, 0]
    for step in lens:
        cat = lambda j: torch.cat([seqs[q][j][done[q]:done[q] + step[q]] for q in range(3)]).reshape(sum(step), heads * d).to(device)
        cu = i32([0, step[0], step[0] + step[1], sum(step)], device)
        plan = ops.wkv_plan(step, device)
        assert plan is not None and plan.longs == 2 and plan.shorts == 1
        room = torch.empty(ops.wkv_workspace_floats(plan, heads, d), device=device)
        y = ops.wkv_scan(cat(0), cat(1), cat(2), cat(3), u.to(device), state, cu, slots, 3, heads, d, plan=plan, workspace=room).cpu()
        at = 0
        for q in range(3):
            got[q].append(y[at:at + step[q]])
            at += step[q]
            done[q] += step[q]
    for q in range(3):
        r, k, v, lw = seqs[q]
        want, want_state = pg.wkv_recurrence(r.double(), k.double(), v.double(), torch.exp(lw.double()), u.double())
        out = torch.cat(got[q]).view(-1, heads, d)
        assert float((out - want.float()).abs().max()) < 3e-5 * float(want.abs().max()), q
        kept = state[int(slots[q]), :heads * d * d].view(heads, d, d).cpu()
        assert float((kept - want_state.float()).abs().max()) < 3e-5 * max(1.0, float(want_state.abs().max()))


@pytest.mark.parametrize("device", DEVICES)
def test_recurrence_remembers_the_first_token(device):
    """With decays next to one, a value written by the first token is read 400 tokens later, through 399 decoded
    steps; with the bonus the current token counts once more, and only for itself."""
    ops = ops_for(device)
    heads, d, t = 1, 8, 401
    r = torch.zeros(t, heads, d)
    k = torch.zeros(t, heads, d)
    v = torch.zeros(t, heads, d)
    k[0, 0, 3] = 1.0
    v[0, 0, 5] = 2.0
    r[-1, 0, 3] = 1.0
    k[200, 0, 1] = 1.0
    v[200, 0, 2] = 3.0
    r[200, 0, 1] = 1.0
    lw = torch.full((t, heads, d), -1e-3)
    u = torch.full((heads, d), 0.5)
    got, _ = scan_in_portions(ops, device, torch.float32, r, k, v, lw, u, [1] * t)
    assert abs(float(got[-1, 0, 5]) - 2.0 * math.exp(-1e-3 * 399)) < 1e-4
    assert abs(float(got[200, 0, 2]) - 0.5 * 3.0) < 1e-6                    # the bonus alone: the state had nothing in row 1
    assert float(got[201:-1].abs().max()) == 0.0


@pytest.mark.parametrize("device", DEVICES)
def test_unit_norm_by_head_with_gain_and_gate(device):
    ops = ops_for(device)
    g = torch.Generator().manual_seed(5)
    t, heads, d = 19, 3, 20
    y = torch.randn(t, heads * d, generator=g) * 4
    gate, gain = torch.randn(t, heads * d, generator=g), 1 + 0.3 * torch.randn(heads * d, generator=g)
    for dtype in dtypes_of(device):
        z = rounded(gate, dtype)
        want = pg.unit_rms(y.view(t, heads, d), 1e-5).reshape(t, -1) * gain * pg.silu(z)
        got = ops.group_rmsnorm_gate(y.to(device), gate.to(device=device, dtype=dtype), gain.to(device), heads, 1e-5).float().cpu()
        assert float((got - want).abs().max()) < (1e-5 if dtype == torch.float32 else 2e-2) * float(want.abs().max())


# ------------------------------------------------------------------ attention over the cached latent

def latent_weights(g, width, heads, d, rot, dv, q_rank, rank):
    n = lambda *shape: torch.randn(*shape, generator=g)
    return {"p.dq": n(q_rank, width) / math.sqrt(width), "p.dq.norm": 1 + 0.2 * n(q_rank),
            "p.uq": n(heads * (d + rot), q_rank) / math.sqrt(q_rank), "p.dkv": n(rank + rot, width) / math.sqrt(width),
            "p.dkv.norm": 1 + 0.2 * n(rank), "p.uk": n(heads * d, rank) / math.sqrt(rank),
            "p.uv": n(heads * dv, rank) / math.sqrt(rank), "p.g": n(heads, width) / math.sqrt(width),
            "p.o": n(width, heads * dv) / math.sqrt(heads * dv)}


def run_latent(ops, device, dtype, h, w, c, eps, page, cuts):
    """The mixer's own sequence of kernel faces over a sequence cut into ``cuts`` (a portion of one token takes the
    decode kernel); pages are handed out in a scrambled order."""
    t, width = h.shape
    heads, d, rot, dv, q_rank, rank = c["heads"], c["dim"], c["rot_dim"], c["vdim"], c["q_rank"], c["kv_rank"]
    row = rank + rot
    pages = -(-t // page)
    order = torch.randperm(pages, generator=torch.Generator().manual_seed(1)) + 1
    table = i32(order.tolist(), device).view(1, pages)
    cache = torch.zeros((pages + 1, page * row), dtype=dtype, device=device)
    dev = lambda x, dt=dtype: x.to(device=device, dtype=dt).contiguous()
    w_down = dev(torch.cat([w["p.dq"], w["p.dkv"], w["p.g"]], 0))
    w_uq, w_o = dev(w["p.uq"]), dev(w["p.o"])
    w_uk = dev(w["p.uk"].view(heads, d, rank).transpose(1, 2))
    w_uv = dev(w["p.uv"].view(heads, dv, rank))
    dims, base = c["rot"]["dims"], c["rot"]["base"]
    f = (float(base) ** (-2.0 * torch.arange(dims // 2, dtype=torch.float64) / dims)).float()
    ang = torch.arange(t, dtype=torch.float32)[:, None] * f[None, :]
    cos, sin = ang.cos().to(device), ang.sin().to(device)
    window = (c.get("mask") or {}).get("size")
    outs, done = [], 0
    for n in cuts:
        x = dev(h[done:done + n])
        pos = i32(list(range(done, done + n)), device)
        down = ops.linear(x, w_down, out_dtype=torch.float32)
        cq = ops.latent_prepare(down, 0, q_rank, q_rank, rank, rot, dims, dev(w["p.dq.norm"], torch.float32),
                                dev(w["p.dkv.norm"], torch.float32), eps, cos, sin, pos, i32([0] * n, device), table, cache, page)
        q = ops.linear(cq, w_uq)
        carried = ops.head_linear(q.view(n, heads, d + rot)[:, :, :d], w_uk, out_dtype=torch.float32)
        queries = ops.latent_query(carried, q, heads, d, rank, rot, dims, cos, sin, pos)
        mixed = torch.empty((n, heads * rank), dtype=dtype, device=device)
        if n == 1:
            plan = ops.plan_decode_attention(dtype, 1, heads, 1, row, done + 1, dv=rank, values_in_keys=True)
            scratch = torch.empty(max(1, plan.scratch_floats), dtype=torch.float32, device=device)
            ops.attention_decode(queries, cache, table, i32([done + 1], device), mixed, scratch, plan.splits, heads, 1, row,
                                 page, float(c["scale"]), window, dv=rank, values_in_keys=True)
        else:
            tile = ops.prefill_tile_rows(dtype, row, page, n, dv=rank, values_in_keys=True, heads=heads)
            tr, ts = ops.prefill_tiles([done], [n], 0, tile, device)
            ops.attention_prefill(queries, cache, table, i32([0, n], device), i32([done], device), tr, ts, mixed, heads, 1,
                                  row, page, float(c["scale"]), window, tile_rows=tile, dv=rank, values_in_keys=True)
        values = ops.head_linear(mixed.view(n, heads, rank), w_uv, out_dtype=torch.float32)
        gated = ops.head_gate(values, down, q_rank + row, dtype)
        outs.append(ops.linear(gated, w_o).float().cpu())
        done += n
    assert done == t
    return torch.cat(outs)


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("heads,d,rot,dv,q_rank,rank", [(3, 8, 4, 12, 20, 24), (2, 32, 16, 32, 48, 128), (1, 16, 2, 5, 9, 33),
                                                        (5, 12, 32, 8, 16, 72), (40, 16, 64, 16, 32, 512), (16, 8, 8, 8, 24, 264),
                                                        (4, 32, 16, 24, 32, 64)])
@pytest.mark.parametrize("window", [37, None, 64])
def test_one_position_that_stands_out(device, heads, d, rot, dv, q_rank, rank, window):
    """The inputs at three positions (at a page border and far back) are made so that their cached latent scores high
    against every later query: queries up to ``window - 1`` positions behind such a position see it, the next one does
    not.  Whole, decoded, and in portions, over pages in a scrambled order."""
    ops = ops_for(device)
    g = torch.Generator().manual_seed(rank + d)
    t, page, width, eps = 230, 16, 40, 1e-5
    c = {"heads": heads, "dim": d, "rot_dim": rot, "vdim": dv, "q_rank": q_rank, "kv_rank": rank, "scale": 4.0 / math.sqrt(d + rot),
         "rot": {"dims": rot, "base": 50.0}}
    if window:
        c["mask"] = {"size": window}
    w = latent_weights(g, width, heads, d, rot, dv, q_rank, rank)
    h = torch.randn(t, width, generator=g)
    marks = [15, 16, 101]
    # a direction of the input that the key/value latent keeps and every query's carried part answers to
    probe = torch.randn(width, generator=g)
    for m in marks:
        h[m] = 3.0 * probe
    for dtype in dtypes_of(device):
        wr = {k: rounded(v, dtype) for k, v in w.items()}
        with pg.precision(torch.float64):
            want = pg.latent_attention_mixer(rounded(h, dtype).double(), wr, "p", c, eps, torch.arange(t)).float()
        for cuts in ([t], [120] + [1] * 40 + [70], [7, 2, 41, 2, 1, 1, 64, 3, 109]):
            got = run_latent(ops, device, dtype, h, w, c, eps, page, cuts)
            tol = 5e-5 if dtype == torch.float32 else 6e-2
            assert float((got - want).abs().max()) < tol * max(1.0, float(want.abs().max())), (dtype, cuts[:3])
    if device == "cuda":
        assert ops.latent_attention_status() == 0                 # no bounded wait of the tensor-core kernel ran out


@pytest.mark.gpu
@pytest.mark.parametrize("heads,row,rank", [(4, 144, 128), (16, 576, 512), (33, 72, 40), (3, 28, 24), (4, 80, 64), (2, 136, 128),
                                            (5, 264, 256), (8, 392, 384), (2, 520, 512), (1, 16, 8), (6, 24, 16), (3, 200, 130)])
@pytest.mark.parametrize("window", [None, 100])
def test_latent_decode_in_key_ranges(heads, row, rank, window):
    """One new token a request over cached rows of unequal lengths, the keys cut into 1 to 7 ranges that are merged
    afterwards (tensor cores where the sizes allow, CUDA cores else): against a plain softmax over the same rows."""
    from lily_b200.csrc import ops
    device, page, scale = "cuda", 16, 0.2
    g = torch.Generator().manual_seed(row)
    lens = [1, 37, 300, 64, 129]
    pages = [-(-n // page) for n in lens]
    width = max(pages)
    order = (torch.randperm(sum(pages), generator=g) + 1).tolist()
    table = torch.zeros(len(lens), width, dtype=torch.int32)
    at = 0
    for r, n in enumerate(pages):
        table[r, :n] = torch.tensor(order[at:at + n], dtype=torch.int32)
        at += n
    for dtype in (torch.float32, torch.bfloat16):
        cache = (torch.randn(sum(pages) + 1, page * row, generator=g) * 0.7).to(device=device, dtype=dtype)
        q = torch.randn(len(lens), heads * row, generator=g).to(device=device, dtype=dtype)
        rows = cache.view(-1, page, row).float()
        want = torch.empty(len(lens), heads, rank)
        for r, n in enumerate(lens):
            keys = torch.stack([rows[int(table[r, j // page]), j % page] for j in range(n)]).cpu()
            sc = (q[r].float().cpu().view(heads, row) @ keys.t()) * scale
            if window:
                sc[:, :max(0, n - window)] = float("-inf")
            want[r] = torch.softmax(sc, -1) @ keys[:, :rank]
        for splits in (1, 2, 7):
            out = torch.empty(len(lens), heads * rank, device=device, dtype=dtype)
            scratch = torch.empty(max(1, ops.decode_scratch_floats(len(lens), heads, rank, splits)), device=device)
            ops.attention_decode(q, cache, table.to(device), i32(lens, device), out, scratch, splits, heads, 1, row, page, scale,
                                 window, dv=rank, values_in_keys=True)
            tol = 1e-5 if dtype == torch.float32 else 2e-2
            assert float((out.float().cpu().view(len(lens), heads, rank) - want).abs().max()) < tol * float(want.abs().max()), (dtype, splits)
    assert ops.latent_attention_status() == 0                     # no bounded wait of the tensor-core kernel ran out


@pytest.mark.parametrize("device", DEVICES)
def test_window_edge_of_the_latent_attention(device):
    """The plain functions say what the construction is for: with a sharp softmax the query at the window's edge and the
    next one differ outright, so a window that is one off cannot pass the test above."""
    g = torch.Generator().manual_seed(1)
    t = 60
    s = torch.zeros(t, t)
    s[:, 10] = 50.0
    inside, outside = pg.windowed_softmax(s, 20)[29], pg.windowed_softmax(s, 20)[30]
    assert float(inside[10]) > 0.99 and float(outside[10]) == 0.0 and abs(float(outside.sum()) - 1.0) < 1e-6


# ------------------------------------------------------------------ routed experts

def expert_weights(g, width, ff, experts, outputs):
    n = lambda *shape: torch.randn(*shape, generator=g)
    w = {"p.router": 3 * n(outputs, width) / math.sqrt(width), "p.correction": n(outputs) / (2 * outputs)}       # of the size of a score
    for e in range(experts):
        w.update({f"p.e{e}.gate": 2 * n(ff, width) / math.sqrt(width), f"p.e{e}.up": 2 * n(ff, width) / math.sqrt(width),
                  f"p.e{e}.down": n(width, ff) / math.sqrt(ff)})
    return w


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("experts,identity,top,ff,width", [(5, 2, 2, 24, 40), (12, 4, 3, 64, 72), (4, 0, 1, 10, 33), (1, 3, 4, 7, 20),
                                                           (0, 3, 2, 8, 16), (40, 1, 8, 16, 48)])
def test_routed_experts(device, experts, identity, top, ff, width):
    """Choice by score plus correction, weights by score alone; clamps that are reached; identity outputs; one token
    and many, alone and in a batch."""
    ops = ops_for(device)
    g = torch.Generator().manual_seed(experts * 10 + top)
    outputs = experts + identity
    w = expert_weights(g, width, ff, experts, outputs)
    c = {"router": {"experts": experts, "identity": identity, "top": top}, "expert": {"ff": ff, "limit": 0.9}}
    h = torch.randn(77, width, generator=g)
    for dtype in dtypes_of(device):
        wr = {k: (v if k in ("p.router", "p.correction") else rounded(v, dtype)) for k, v in w.items()}
        x = rounded(h, dtype)
        chosen_want, weights_want = pg.route(x, w, "p", top)
        want = pg.moe_ff(x, wr, "p", c)
        router, corr = w["p.router"].to(device), w["p.correction"].to(device)
        if experts:
            gu = torch.stack([torch.cat([w[f"p.e{e}.gate"], w[f"p.e{e}.up"]]) for e in range(experts)]).to(device=device, dtype=dtype)
            dn = torch.stack([w[f"p.e{e}.down"] for e in range(experts)]).to(device=device, dtype=dtype)
        else:
            gu = dn = torch.empty(0, device=device, dtype=dtype)
        for rows in (slice(0, 77), slice(5, 6), slice(40, 49)):
            xs = h[rows].to(device=device, dtype=dtype).contiguous()
            routing = ops.moe_route(xs, router, corr, top, experts)
            assert torch.equal(routing.chosen.cpu().long().sort(-1).values, chosen_want[rows].sort(-1).values)
            order = routing.chosen.cpu().long().argsort(-1)
            assert float((routing.weights.cpu().gather(1, order) - weights_want[rows].gather(1, chosen_want[rows].argsort(-1))).abs().max()) < 1e-5
            got = ops.moe_experts(xs, routing, gu, dn, 0.9, 1.702).cpu()
            tol = 1e-5 if dtype == torch.float32 else 2e-2
            assert float((got - want[rows]).abs().max()) < tol * max(1.0, float(want.abs().max())), (dtype, rows)
    # many tokens (several share a block on the GPU): the same choices and weights as the plain router
    big = torch.randn(1100, width, generator=g)
    routing = ops.moe_route(big.to(device), w["p.router"].to(device), w["p.correction"].to(device), top, experts)
    chosen_big, weights_big = pg.route(big, w, "p", top)
    assert torch.equal(routing.chosen.cpu().long().sort(-1).values, chosen_big.sort(-1).values)
    order = routing.chosen.cpu().long().argsort(-1)
    assert float((routing.weights.cpu().gather(1, order) - weights_big.gather(1, chosen_big.argsort(-1))).abs().max()) < 1e-5
    # the construction does what it says: corrections change choices, clamps bite, identity outputs are chosen
    s = torch.softmax(h @ w["p.router"].t(), -1)
    if outputs > top:
        assert not torch.equal(torch.topk(s, top).indices.sort(-1).values, chosen_want.sort(-1).values)
    if experts:
        assert float((h @ w["p.e0.gate"].t()).max()) > 0.9
    if identity > 1 and experts:
        assert bool((chosen_want >= experts).any()) and bool((chosen_want < experts).any())


# ------------------------------------------------------------------ residual add with two deltas, a vector and two gains

@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("hidden", [48, 321, 1024])
def test_residual_add_with_two_norms(device, hidden):
    ops = ops_for(device)
    g = torch.Generator().manual_seed(hidden)
    t = 21
    resid = torch.randn(t, hidden, generator=g) * 3
    a, b = torch.randn(t, hidden, generator=g), torch.randn(3, t, hidden, generator=g)
    bias, g1, g2 = torch.randn(hidden, generator=g), torch.randn(hidden, generator=g) * 0.2, torch.randn(hidden, generator=g) * 0.2
    for dtype in dtypes_of(device):
        stream = resid.clone().to(device)
        ar = rounded(a, dtype)
        total = resid + ar + b.sum(0) + bias
        o1, o2 = ops.add_rmsnorm_multi(stream, [a.to(device=device, dtype=dtype), b.to(device)], [(1 + g1).to(device), (1 + g2).to(device)],
                                       1e-5, dtype, bias=bias.to(device))
        tol = 1e-5 if dtype == torch.float32 else 2e-2
        assert float((stream.cpu() - total).abs().max()) < 1e-5 * float(total.abs().max())
        assert float((o1.float().cpu() - pg.offset_norm(total, g1, 1e-5)).abs().max()) < tol * 5
        assert float((o2.float().cpu() - pg.offset_norm(total, g2, 1e-5)).abs().max()) < tol * 5


@pytest.mark.parametrize("device", DEVICES)
def test_products_by_head(device):
    ops = ops_for(device)
    g = torch.Generator().manual_seed(2)
    t, heads, k, n, extra = 70, 3, 20, 37, 6
    rows = torch.randn(t, heads * (k + extra), generator=g)
    w = torch.randn(heads, n, k, generator=g)
    want = torch.einsum("thk,hnk->htn", rows.view(t, heads, k + extra)[:, :, :k], w)
    for dtype in dtypes_of(device):
        x = rows.to(device=device, dtype=dtype)
        got = ops.head_linear(x.view(t, heads, k + extra)[:, :, :k], w.to(device=device, dtype=dtype), out_dtype=torch.float32)
        ref = torch.einsum("thk,hnk->htn", rounded(rows, dtype).view(t, heads, k + extra)[:, :, :k], rounded(w, dtype)) if dtype != torch.float32 else want
        assert float((got.float().cpu() - ref).abs().max()) < 1e-4 * float(ref.abs().max())
