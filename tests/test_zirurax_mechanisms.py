"""Each mechanism of the Zirurax decoder alone: the kernels' faces (CUDA on the GPU, their plain statements on the
CPU) against the functions of ``plain_zirurax``, with inputs made so that a fault shows: one key scaled to stand out
far back, at a page border, just inside and just outside the window; states carried over portions of every length;
sizes that are not powers of two."""

import math

import pytest
import torch

import kernel_refs
import plain_zirurax as pz

DEVICES = ["cpu", pytest.param("cuda", marks=pytest.mark.gpu)]


def ops_for(device):
    if device == "cpu":
        return kernel_refs
    from lily_b200.csrc import ops
    return ops


def i32(values, device):
    return torch.tensor(values, dtype=torch.int32, device=device)


# ------------------------------------------------------------------ attention: window, cap, value size, pages

def run_attention(ops, device, dtype, q, k, v, scale, softcap, window, page, cuts):
    """q [t, H, d], k [t, G, d], v [t, G, dv] through the cache write and the attention kernels, the sequence cut into
    the portions ``cuts`` (a portion of one token takes the decode kernel); pages are handed out in a scrambled order."""
    t, heads, d = q.shape
    kvh, dv = k.shape[1], v.shape[2]
    pages = -(-t // page)
    order = torch.randperm(pages, generator=torch.Generator().manual_seed(1)) + 1
    table = i32(order.tolist(), device).view(1, pages)
    shape = (pages + 1, 2, kvh, page, d) if dv == d else (pages + 1, kvh * page * (d + dv))
    cache = torch.zeros(shape, dtype=dtype, device=device)
    out = torch.empty((t, heads * dv), dtype=dtype, device=device)
    qkv = torch.cat([q.reshape(t, -1), k.reshape(t, -1), v.reshape(t, -1)], 1).to(device=device, dtype=dtype)
    done = 0
    for n in cuts:
        rows = qkv[done:done + n].contiguous()
        pos = i32(list(range(done, done + n)), device)
        qq = ops.qk_norm_rope_write(rows, None, None, 1e-6, None, None, pos, i32([0] * n, device), table, cache, heads, kvh,
                                    d, 0, page, dv=dv)
        o = torch.empty((n, heads * dv), dtype=dtype, device=device)
        if n == 1:
            plan = ops.plan_decode_attention(dtype, 1, heads, kvh, d, done + 1, dv=dv)
            scratch = torch.empty(max(1, plan.scratch_floats), dtype=torch.float32, device=device)
            ops.attention_decode(qq, cache, table, i32([done + 1], device), o, scratch, plan.splits, heads, kvh, d, page, scale,
                                 window, softcap=softcap, dv=dv)
        else:
            tile = ops.prefill_tile_rows(dtype, d, page, n, softcap=softcap, dv=dv)
            tr, ts = ops.prefill_tiles([done], [n], 0, tile, device)
            ops.attention_prefill(qq, cache, table, i32([0, n], device), i32([done], device), tr, ts, o, heads, kvh, d, page,
                                  scale, window, tile_rows=tile, softcap=softcap, dv=dv)
        out[done:done + n] = o
        done += n
    assert done == t
    return out.float().cpu().view(t, heads, dv)


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("heads,kvh,d,dv", [(4, 2, 16, 24), (3, 1, 40, 8), (4, 2, 64, 64), (2, 1, 128, 128)])
@pytest.mark.parametrize("window,softcap", [(37, 6.0), (None, None), (64, 50.0)])
def test_one_key_that_stands_out(device, heads, kvh, d, dv, window, softcap):
    """A key many times larger than the rest draws nearly all weight of every query that sees it: queries up to
    ``window - 1`` positions behind it do, the next one does not.  The marked keys sit at a page border and far back."""
    ops = ops_for(device)
    g = torch.Generator().manual_seed(d + dv)
    t, page = 230, 16
    q = torch.randn(t, heads, d, generator=g)
    k = torch.randn(t, kvh, d, generator=g) * 0.3
    v = torch.randn(t, kvh, dv, generator=g)
    marks = [15, 16, 101]
    for m in marks:                               # every later query scores high against these keys
        k[m] = 0.0
        k[m, :, 0] = 6.0 * math.sqrt(d)
    q[:, :, 0] = q[:, :, 0].abs() + 1.0
    scale = 1.0 / math.sqrt(d)
    want = pz.windowed_softcap_attention(q.double(), k.double(), v.double(), scale, softcap, window).float()
    cuts_list = [[t], [120] + [1] * 40 + [70], [7, 2, 41, 2, 1, 1, 64, 3, 109]]
    pages = [page] if d != dv or device == "cpu" else [page, 64]      # pages of 64: long portions take the tcgen05 kernel
    dtypes = [torch.float32] if device == "cpu" else [torch.float32, torch.bfloat16]
    for dtype in dtypes:
        if dtype == torch.bfloat16:
            r = lambda x: x.bfloat16().float()
            ref = pz.windowed_softcap_attention(r(q).double(), r(k).double(), r(v).double(), scale, softcap, window).float()
        else:
            ref = want
        for cuts in cuts_list:
            for pg in pages:
                got = run_attention(ops, device, dtype, q, k, v, scale, softcap, window, pg, cuts)
                tol = 2e-5 if dtype == torch.float32 else 3e-2
                assert float((got - ref).abs().max()) < tol * max(1.0, float(ref.abs().max())), (dtype, cuts[:3], pg)
    if window:
        # the construction does what it says: the query at the window's edge and the next one differ a lot
        edge = marks[2] + window - 1
        assert float((want[edge] - want[edge + 1]).abs().max()) > 0.2


# ------------------------------------------------------------------ the state-space mixer's kernels

@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("width,col0", [(91, 13), (92, 12)])        # odd rows and offsets, and even ones
@pytest.mark.parametrize("taps", [1, 2, 4, 7])
def test_convolution_carries_its_inputs(device, taps, width, col0):
    ops = ops_for(device)
    g = torch.Generator().manual_seed(taps)
    t, channels = 200, 70
    proj = torch.randn(t, width, generator=g)
    w = torch.randn(channels, taps, generator=g) * 0.5
    b = torch.randn(channels, generator=g) * 0.2
    conv = pz.causal_conv(proj[:, col0:col0 + channels], w, b)
    want = conv * torch.sigmoid(conv)
    for cuts in ([t], [1] * 9 + [2, 2, 3, 1, 64, 1, 65, 53], [130, 70]):
        state = torch.zeros(3, 17 + (taps - 1) * channels, device=device)
        got = []
        done = 0
        for n in cuts:
            # two requests in the step: the one under test in slot 2 and a bystander in slot 1
            rows = torch.cat([proj[done:done + n], proj[:5]]).to(device)
            cr, cs = ops.token_chunks([n, 5], ops.SSM_CHUNK, device)
            out = ops.causal_conv_silu(rows, col0, channels, w.to(device), b.to(device), state, 17, cr, cs,
                                       i32([0, n, n + 5], device), i32([2, 1], device))
            got.append(out[:n].float().cpu())
            done += n
        assert float((torch.cat(got) - want).abs().max()) < 1e-5, cuts[:3]
        assert float(state[0].abs().max()) == 0.0 and float(state[:, :17].abs().max()) == 0.0


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("heads,pd,n_state,groups", [(4, 8, 12, 2), (2, 64, 128, 1), (6, 5, 33, 3), (2, 16, 200, 2), (8, 4, 5, 4)])
def test_scan_carries_its_state(device, heads, pd, n_state, groups):
    ops = ops_for(device)
    g = torch.Generator().manual_seed(n_state)
    t = 470                     # portions past ``ops.SCAN_DIRECT`` tokens run as chunks side by side on the GPU
    inner = heads * pd
    xbc = torch.randn(t, inner + 2 * groups * n_state, generator=g)
    proj = torch.randn(t, 3 + heads, generator=g)
    dt_bias = torch.randn(heads, generator=g) - 0.5
    a_log = torch.rand(heads, generator=g) * 4.0 - 4.0
    d_skip = 1.0 + 0.3 * torch.randn(heads, generator=g)
    dt = pz.softplus(proj[:, 3:].double() + dt_bias.double())
    want = pz.ssd_scan(xbc[:, :inner].double().view(t, heads, pd), dt, -torch.exp(a_log.double()),
                       xbc[:, inner:inner + groups * n_state].double().view(t, groups, n_state),
                       xbc[:, inner + groups * n_state:].double().view(t, groups, n_state), d_skip.double()).float().view(t, inner)
    for cuts in ([t], [420] + [1] * 50, [1, 2, 17, 2, 1, 1, 40, 3, 193, 210]):
        state = torch.zeros(4, inner * n_state + 9, device=device)
        got, done = [], 0
        for n in cuts:
            rows_x = torch.cat([xbc[:3], xbc[done:done + n]]).to(device)          # a bystander's three tokens first
            rows_p = torch.cat([proj[:3], proj[done:done + n]]).to(device)
            y = ops.ssd_scan(rows_x, rows_p, 3, dt_bias.to(device), a_log.to(device), d_skip.to(device), state,
                             i32([0, 3, 3 + n], device), i32([1, 3], device), 2, heads, pd, n_state, groups,
                             plan=ops.scan_plan([3, n], device, inner * n_state))
            got.append(y[3:].float().cpu())
            done += n
        scale = max(1.0, float(want.abs().max()))
        assert float((torch.cat(got) - want).abs().max()) < 2e-5 * scale, cuts[:3]
        assert float(state[0].abs().max()) == 0.0 and float(state[2].abs().max()) == 0.0


@pytest.mark.parametrize("device", DEVICES)
def test_gate_then_grouped_norm(device):
    ops = ops_for(device)
    g = torch.Generator().manual_seed(3)
    for inner, groups, extra in ((48, 4, 11), (90, 1, 11), (256, 2, 11), (256, 2, 12), (2048, 2, 128), (40, 5, 4)):
        y = torch.randn(21, inner, generator=g) * 3
        proj = torch.randn(21, inner + extra, generator=g)       # rows of odd and of even length (16-byte accesses)
        gain = 1 + 0.2 * torch.randn(inner, generator=g)
        z = proj[:, :inner]
        want = pz.grouped_rms(y * (z * torch.sigmoid(z)), groups, 1e-5) * gain
        got = ops.gated_group_rmsnorm(y.to(device), proj.to(device), gain.to(device), groups, 1e-5).float().cpu()
        assert float((got - want).abs().max()) < 1e-5, (inner, groups, extra)
        if device != "cpu":
            zb = proj.bfloat16().float()[:, :inner]
            ref = pz.grouped_rms(y * (zb * torch.sigmoid(zb)), groups, 1e-5) * gain
            got = ops.gated_group_rmsnorm(y.to(device), proj.bfloat16().to(device), gain.to(device), groups, 1e-5).float().cpu()
            assert float((got - ref).abs().max()) < 0.02 * float(ref.abs().max()), (inner, groups, extra)


@pytest.mark.parametrize("device", DEVICES)
def test_normed_mean_gate_and_gelu(device):
    ops = ops_for(device)
    g = torch.Generator().manual_seed(4)
    # odd widths, and wide rows of a few tokens (which a cluster of blocks shares on the GPU) and of many
    for n, width in ((19, 72), (5, 1024), (70, 1024), (3, 4096)):
        a, b, f = (torch.randn(n, width, generator=g) * s for s in (5.0, 0.1, 1.0))
        ga, gb = 1 + 0.2 * torch.randn(width, generator=g), 1 + 0.2 * torch.randn(width, generator=g)
        want = 0.5 * (pz.rms(a, 1e-6) * ga + pz.rms(b, 1e-6) * gb) + f
        parts = torch.stack([0.25 * a, 0.75 * a]).contiguous()                 # one input arrives as two partial sums
        got = ops.normed_mean([parts.to(device), b.to(device)], [ga.to(device), gb.to(device)], 1e-6, add=f.to(device))
        assert got.shape == (1, n, width) and float((got[0].cpu() - want).abs().max()) < 2e-5, (n, width)
        alone = ops.normed_mean([b.to(device)], [gb.to(device)], 1e-6)
        assert float((alone[0].cpu() - pz.rms(b, 1e-6) * gb).abs().max()) < 2e-5, (n, width)
        half = ops.normed_mean([a.bfloat16().to(device), b.bfloat16().to(device)], [ga.to(device), gb.to(device)], 1e-6)
        ref = 0.5 * (pz.rms(a.bfloat16().float(), 1e-6) * ga + pz.rms(b.bfloat16().float(), 1e-6) * gb)
        assert float((half[0].cpu() - ref).abs().max()) < 2e-5, (n, width)
    n, width = 19, 72
    a, b = torch.randn(n, width, generator=g) * 5.0, torch.randn(n, width, generator=g) * 0.1

    out = a.clone().to(device)
    ops.sigmoid_gate(out, b.to(device))
    assert float((out.cpu() - a * torch.sigmoid(b)).abs().max()) < 1e-5

    gu = torch.randn(n, 2 * 40, generator=g) * 2
    want = pz.gelu_tanh(gu[:, :40]) * gu[:, 40:]
    got = ops.silu_mul(gu.to(device), activation="gelu_tanh").cpu()
    assert float((got - want).abs().max()) < 1e-5


def test_interleaved_pairs_by_reordered_rows():
    """Rotating pairs (2i, 2i + 1) of q and k equals rotating halves after both were reordered alike: same scores."""
    from lily_b200.parts.rope import RopeSpec, inverse_frequencies, pairing_order
    from lily_b200.config.model_config import RopeScaling

    g = torch.Generator().manual_seed(5)
    t, d, rd = 40, 24, 16
    q, k = torch.randn(t, 2, d, generator=g), torch.randn(t, 2, d, generator=g)
    rot = {"dims": rd, "base": 5000.0, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}}
    f = pz.rotary_frequencies(rot)
    assert torch.equal(f, inverse_frequencies(RopeSpec(d, rd, 5000.0, RopeScaling("llama3", 8.0, 1.0, 4.0, 64), exact_frequencies=True)))
    assert len({float(x) for x in (f * (5000.0 ** (torch.arange(rd // 2) * 2.0 / rd)))}) > 2      # all three bands occur
    pos = torch.arange(t)
    want = torch.einsum("thd,shd->hts", pz.rotate_interleaved(q, pos, f), pz.rotate_interleaved(k, pos, f))
    order = pairing_order(d, rd)
    ang = pos[:, None].float() * f[None, :]

    def halves(x):
        x = x[..., order]
        x1, x2 = x[..., :rd // 2], x[..., rd // 2:rd]
        c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
        return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s, x[..., rd:]], -1)
    got = torch.einsum("thd,shd->hts", halves(q), halves(k))
    assert float((got - want).abs().max()) < 1e-4
