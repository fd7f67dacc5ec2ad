"""Gugalorn on the GPU: every new kernel and part alone against the plain implementation, then whole models replayed in
every way of cutting, in both dtypes, through the engine's step function, scheduler and command line."""
import math

import pytest
import torch

import plain_gugalorn as plain
import replay
import tiny
import tiny_gugalorn as tg
from test_kernels_gpu import _Batch, paged_setup

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 2e-5, "bfloat16": 2e-2}


def ops():
    from rust_mlx_b200.kernels import ops as o
    return o


def rnd(shape, seed, scale=1.0):
    return torch.randn(shape, generator=torch.Generator().manual_seed(seed)) * scale


class Steps:
    """Sequences of given lengths cut into steps: ``cuts[s]`` lists the portion sizes of sequence s; step i takes the i-th
    portion of every sequence that still has one.  Yields (batch, rows): a batch as kernels read it and, per sequence of
    the batch, (sequence, first position, count)."""

    def __init__(self, cuts):
        self.cuts = cuts

    def __iter__(self):
        at = [0] * len(self.cuts)
        for i in range(max(len(c) for c in self.cuts)):
            rows = [(s, at[s], c[i]) for s, c in enumerate(self.cuts) if i < len(c)]
            status = torch.zeros(1, dtype=torch.int32, device=DEV)
            batch = _Batch([a + n for _, a, n in rows], [n for _, _, n in rows], status)
            yield batch, rows
            for s, a, n in rows:
                at[s] = a + n


def close(got, want, dtype, what=""):
    got, want = got.double().cpu(), want.double()
    err = (got - want).abs() / (1.0 + want.abs())
    assert err.max().item() < TOL[dtype], (what, err.max().item())


# ------------------------------------------------------------------------------------------------ kernels alone

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("taps, channels, act, residual, bias", [(4, 40, "silu", False, True), (3, 17, None, True, False),
                                                                 (2, 64, None, False, False), (1, 24, None, True, False), (6, 9, "silu", True, True)])
def test_short_convolution_in_portions_through_its_ring(dtype, taps, channels, act, residual, bias):
    """Portions of every size from one token up, sequences that start in different steps and share the batch, slots that
    are not the sequences' numbers; the ring holds NaN where nothing was written yet."""
    cuts = [[1, 1, 2, 1, 7, 1, 1, 30, 3], [9, 1, 1, 1, 2], [2, 2, 1, 5, 1, 1, 1, 1, 40, 1]]
    lengths = [sum(c) for c in cuts]
    dt = DT[dtype]
    x = [rnd((n, channels), 10 + s).to(dt) for s, n in enumerate(lengths)]
    w = rnd((channels, taps), 3, 0.5)
    b = rnd((channels,), 4, 0.3) if bias else None
    want = []
    for xs in x:
        y = plain.causal_conv(xs.double(), w.double(), b.double() if bias else None)
        y = plain.silu(y) if act else y
        want.append(y + xs.double() if residual else y)
    ring = torch.full((5, max(taps - 1, 1), channels), float("nan"), dtype=dt, device=DEV)
    slots = torch.tensor([3, 0, 4], dtype=torch.int32, device=DEV)
    ring[[3, 0, 4]] = 0         # a request's state is zero when it starts
    got = [torch.zeros(n, channels, dtype=dt) for n in lengths]
    for batch, rows in Steps(cuts):
        xin = torch.cat([x[s][a:a + n] for s, a, n in rows]).to(DEV)
        # columns of wider rows: at a place that the kernel of eight channels a thread takes (bfloat16), or not
        lead, extra = (8, 16) if channels % 8 == 0 and taps != 2 else (2, 5)
        wide = torch.full((xin.shape[0], channels + extra), float("nan"), dtype=dt, device=DEV)
        wide[:, lead:lead + channels] = xin
        out = torch.empty_like(xin)
        ops().short_conv(wide[:, lead:lead + channels], w.t().contiguous().to(DEV), b.to(DEV) if bias else None, out, ring, batch,
                         slots[[s for s, _, _ in rows]].contiguous(), act, residual)
        at = 0
        for s, a, n in rows:
            got[s][a:a + n] = out[at:at + n].cpu()
            at += n
    for s in range(len(cuts)):
        close(got[s], want[s], dtype, s)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads, groups, k, v", [(4, 2, 16, 8), (6, 1, 40, 6), (3, 3, 7, 10), (8, 2, 128, 64), (2, 1, 200, 24)])
def test_state_space_recurrence_in_portions(dtype, heads, groups, k, v):
    cuts = [[5, 1, 1, 40, 2, 1], [1, 1, 1, 3], [33, 1, 17]]
    lengths = [sum(c) for c in cuts]
    dt = DT[dtype]
    cc = heads * v + 2 * groups * k
    conv = [rnd((n, cc), 20 + s).to(dt) for s, n in enumerate(lengths)]
    raw = [rnd((n, heads), 30 + s, 2.0).to(dt) for s, n in enumerate(lengths)]
    dt_bias, a_log, skip = rnd((heads,), 1), rnd((heads,), 2, 0.5), rnd((heads,), 3)
    want = []
    for c, r in zip(conv, raw):
        n = c.shape[0]
        c, step = c.double(), plain.softplus(r.double() + dt_bias.double())
        decay = torch.exp(-torch.exp(a_log.double()) * step)
        xs = c[:, :heads * v].view(n, heads, v)
        B = c[:, heads * v:heads * v + groups * k].view(n, groups, k).repeat_interleave(heads // groups, dim=1)
        C = c[:, heads * v + groups * k:].view(n, groups, k).repeat_interleave(heads // groups, dim=1)
        S = torch.zeros(heads, k, v, dtype=torch.float64)
        y = torch.zeros(n, heads, v, dtype=torch.float64)
        for i in range(n):
            S = decay[i][:, None, None] * S + step[i][:, None, None] * B[i][:, :, None] * xs[i][:, None, :]
            y[i] = torch.einsum("hkv,hk->hv", S, C[i]) + skip.double()[:, None] * xs[i]
        want.append(y.reshape(n, heads * v))
    state = torch.full((6, heads, v, k), float("nan"), dtype=torch.float32, device=DEV)
    slots = torch.tensor([5, 1, 2], dtype=torch.int32, device=DEV)
    state[[5, 1, 2]] = 0
    got = [torch.zeros(n, heads * v) for n in lengths]
    for batch, rows in Steps(cuts):
        cin = torch.cat([conv[s][a:a + n] for s, a, n in rows]).to(DEV)
        rin = torch.cat([raw[s][a:a + n] for s, a, n in rows]).to(DEV)
        out = torch.empty(cin.shape[0], heads * v, dtype=torch.float32, device=DEV)
        ops().recurrence_ssd(cin, rin, dt_bias.to(DEV), a_log.to(DEV), skip.to(DEV), state, out, batch,
                             slots[[s for s, _, _ in rows]].contiguous(), heads, groups, k, v)
        at = 0
        for s, a, n in rows:
            got[s][a:a + n] = out[at:at + n].cpu()
            at += n
    for s in range(len(cuts)):
        close(got[s], want[s], "float32", s)        # (the kernel's own arithmetic is float in both runs)
    assert torch.isnan(state[[0, 3, 4]]).all()      # other requests' slots were not touched


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads, k, v", [(2, 8, 12), (3, 20, 8), (1, 7, 10), (6, 48, 64), (5, 5, 6), (2, 130, 16)])
def test_gated_linear_recurrence_in_portions(dtype, heads, k, v):
    cuts = [[3, 1, 1, 1, 50, 2], [1, 1, 2, 1], [20, 1, 9]]
    lengths = [sum(c) for c in cuts]
    dt = DT[dtype]
    q = [rnd((n, heads * k), 40 + s).to(dt) for s, n in enumerate(lengths)]
    f = [rnd((n, heads * k), 50 + s, 2.0).to(dt) for s, n in enumerate(lengths)]
    val = [rnd((n, heads * v), 60 + s).to(dt) for s, n in enumerate(lengths)]
    bias, lower = rnd((heads * k,), 5), torch.rand(heads * k, generator=torch.Generator().manual_seed(6))
    want = []
    for qs, fs, vs in zip(q, f, val):
        n = qs.shape[0]
        gate = (lower.double() + (1 - lower.double()) * torch.sigmoid(fs.double() + bias.double())).view(n, heads, k)
        qq, vv = plain.silu(qs.double()).view(n, heads, k), vs.double().view(n, heads, v)
        S = torch.zeros(heads, k, v, dtype=torch.float64)
        o = torch.zeros(n, heads, v, dtype=torch.float64)
        for i in range(n):
            S = gate[i][:, :, None] * S + (1 - gate[i])[:, :, None] * vv[i][:, None, :]
            o[i] = torch.einsum("hkv,hk->hv", S, qq[i])
        want.append(o.reshape(n, heads * v))
    state = torch.zeros((4, heads, v, k), dtype=torch.float32, device=DEV)
    slots = torch.tensor([2, 0, 3], dtype=torch.int32, device=DEV)
    got = [torch.zeros(n, heads * v) for n in lengths]
    for batch, rows in Steps(cuts):
        wide = torch.cat([torch.cat([q[s][a:a + n], f[s][a:a + n], val[s][a:a + n]], dim=1) for s, a, n in rows]).to(DEV)
        hk = heads * k
        out = torch.empty(wide.shape[0], heads * v, dtype=torch.float32, device=DEV)
        ops().recurrence_gate(wide[:, :hk], wide[:, hk:2 * hk], wide[:, 2 * hk:], bias.to(DEV), lower.to(DEV), state, out, batch,
                              slots[[s for s, _, _ in rows]].contiguous(), heads, k, v)
        at = 0
        for s, a, n in rows:
            got[s][a:a + n] = out[at:at + n].cpu()
            at += n
    for s in range(len(cuts)):
        close(got[s], want[s], "float32", s)
    assert (state[1] == 0).all()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_group_norm_with_its_gate_and_the_elementwise_gate(dtype):
    dt = DT[dtype]
    n, groups, size = 13, 3, 20
    y, z, w = rnd((n, groups * size), 1, 3.0), rnd((n, groups * size), 2).to(dt), 1 + rnd((groups * size,), 3, 0.2)
    out = torch.empty(n, groups * size, dtype=dt, device=DEV)
    wide = torch.zeros(n, groups * size + 7, dtype=dt, device=DEV)
    wide[:, 7:] = z.to(DEV)
    ops().group_rmsnorm(y.to(DEV), w.to(DEV), 1e-5, out, groups, gate=wide[:, 7:])
    u = y.double() * plain.silu(z.double())
    close(out, plain.rms(u.view(n, groups, size), 1e-5).reshape(n, -1) * w.double(), dtype)
    # a weight of one group's size shared by the groups, no gate
    ops().group_rmsnorm(y.to(DEV), w[:size].contiguous().to(DEV), 1e-5, out, groups)
    close(out, (plain.rms(y.double().view(n, groups, size), 1e-5) * w[:size].double()).reshape(n, -1), dtype)
    # heads padded to a wider size keep their first numbers
    heads, vdim, pad = 3, 6, 10
    o, g = rnd((n, heads * pad), 4).to(dt), rnd((n, heads * vdim), 5).to(dt)
    dense = torch.empty(n, heads * vdim, dtype=dt, device=DEV)
    ops().sigmoid_gate(o.to(DEV), pad, g.to(DEV), dense, heads, vdim)
    close(dense, (o.double().view(n, heads, pad)[:, :, :vdim] * torch.sigmoid(g.double()).view(n, heads, vdim)).reshape(n, -1), dtype)
    same = o[:, :heads * vdim].contiguous().to(DEV)
    want = same.double().cpu() * torch.sigmoid(g.double())
    ops().sigmoid_gate(same, vdim, g.to(DEV), same, heads, vdim)
    close(same, want, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nq, nkv, dq, dv, rot, page", [(4, 2, 16, 16, 8, 16), (6, 3, 12, 20, 4, 8), (3, 1, 24, 8, 24, 4), (2, 2, 8, 8, 0, 16)])
def test_whole_projection_norm_rotation_and_cache_write(dtype, nq, nkv, dq, dv, rot, page):
    dt = DT[dtype]
    hd = max(dq, dv)
    lengths, new = [37, 5, 1], [9, 5, 1]
    n = sum(new)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    batch = _Batch(lengths, new, status)
    rows = rnd((n, (nq + nkv) * dq + nkv * dv + 3), 7).to(dt)
    wq, wk = 1 + rnd((nq * dq,), 8, 0.3), 1 + rnd((nkv * dq,), 9, 0.3)
    inv_freq = torch.tensor([50.0 ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=torch.float32) if rot else None
    n_pages = sum(-(-x // page) for x in lengths)
    k_pool = torch.full((n_pages, nkv, page, hd), float("nan"), dtype=dt, device=DEV)
    v_pool = torch.full_like(k_pool, float("nan"))
    table, at = torch.full((3, max(-(-x // page) for x in lengths)), -1, dtype=torch.int32), 0
    for s, x in enumerate(lengths):
        for i in range(-(-x // page)):
            table[s, i] = n_pages - 1 - at
            at += 1
    q_out = torch.full((n, nq * hd), float("nan"), dtype=dt, device=DEV)
    ops().qk_whole_norm_rope_cache(rows.to(DEV), wq.to(DEV), wk.to(DEV), 1e-5, inv_freq.to(DEV) if rot else None, rot, batch.positions,
                                   batch.seq_index, table.to(DEV), page, k_pool, v_pool, q_out, nq, nkv, dq, dv, hd, True, status)
    assert status.item() == 0
    r = rows.double()
    pos = batch.positions.cpu()
    q = plain.rotate((plain.rms(r[:, :nq * dq], 1e-5) * wq.double()).view(n, nq, dq), pos, rot, 50.0)
    k = plain.rotate((plain.rms(r[:, nq * dq:(nq + nkv) * dq], 1e-5) * wk.double()).view(n, nkv, dq), pos, rot, 50.0)
    v = r[:, (nq + nkv) * dq:(nq + nkv) * dq + nkv * dv].view(n, nkv, dv)
    got_q = q_out.double().cpu().view(n, nq, hd)
    close(got_q[:, :, :dq], q, dtype)
    assert (got_q[:, :, dq:] == 0).all()
    for t in range(n):
        s, p = int(batch.seq_index[t]), int(pos[t])
        page_id, slot = int(table[s, p // page]), p % page
        close(k_pool[page_id, :, slot, :dq], k[t], dtype)
        close(v_pool[page_id, :, slot, :dv], v[t], dtype)
        assert (k_pool[page_id, :, slot, dq:] == 0).all() and (v_pool[page_id, :, slot, dv:] == 0).all()
    assert torch.isnan(k_pool.float()).sum().item() == (n_pages * page - n) * nkv * hd      # nothing else was written


def sink_attention_over_pages(q, k, v, qpos, window, scale):
    """q [T, nq, hd] at positions qpos over keys 0..S-1: the plain softmax with one more term, exp(0), in the denominator."""
    T, nq, hd = q.shape
    group = nq // k.shape[1]
    kpos = torch.arange(k.shape[0])
    allowed = kpos[None, :] <= qpos[:, None]
    if window:
        allowed &= kpos[None, :] > qpos[:, None] - window
    out = torch.empty(T, nq, hd, dtype=torch.float64)
    for h in range(nq):
        s = (q[:, h].double() @ k[:, h // group].double().t()) * scale
        e = torch.exp(s).masked_fill(~allowed, 0.0)
        out[:, h] = (e / (1.0 + e.sum(-1, keepdim=True))) @ v[:, h // group].double()
    return out


@pytest.mark.parametrize("dtype, nq, nkv, hd, page, kernel", [
    ("float32", 6, 3, 24, 16, "plain"), ("bfloat16", 4, 1, 48, 8, "plain"), ("bfloat16", 6, 2, 64, 16, "flash"),
    ("bfloat16", 4, 4, 32, 16, "flash"), ("bfloat16", 8, 2, 128, 64, "flash"), ("bfloat16", 8, 2, 64, 64, "tcgen05"),
    ("bfloat16", 4, 4, 128, 64, "tcgen05")])
@pytest.mark.parametrize("window", [0, 70])
def test_attention_with_a_sink_in_every_kernel(dtype, nq, nkv, hd, page, kernel, window):
    """Small scores, so that the sink's share of a row's weight is large: left out, counted twice (once a split, once a
    warp) or scaled wrongly it shows at once.  Portions beside decoded tokens, long sequences in several splits."""
    from rust_mlx_b200.engine.workspace import Workspace
    dt = DT[dtype]
    lengths, new = [700, 1, 33, 130, 300, 64, 1500], [200, 1, 33, 1, 1, 64, 1]
    k_pool, v_pool, table, ks, vs = paged_setup(lengths, nkv, hd, page, dt, seed=hd + nq)
    qs = [(rnd((c, nq, hd), 70 + i) * 0.3).to(dt) for i, c in enumerate(new)]
    q = torch.cat(qs).to(DEV).reshape(-1, nq * hd)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    batch = _Batch(lengths, new, status)
    out = torch.full_like(q, float("nan"))
    scale = 0.7 * hd ** -0.5
    sinks = torch.zeros(nq, dtype=torch.float32, device=DEV)
    ws = Workspace(DEV)
    if kernel == "plain":
        ops().attention_plain(q, k_pool, v_pool, batch.positions, batch.seq_index, table, page, out, nq, nkv, hd, window, scale, status, sinks)
    elif kernel == "flash":
        for splits in (None, 1, 3):
            out.fill_(float("nan"))
            ops().attention_flash(q, k_pool, v_pool, batch, table, page, out, nq, nkv, hd, window, scale, ws, n_splits=splits, sinks=sinks)
            check_sink_rows(out, qs, ks, vs, lengths, new, nq, hd, window, scale, dtype)
        ops().default.attention(q, k_pool, v_pool, batch, table, page, out, nq, nkv, hd, window, scale, ws, sinks=sinks)   # the engine's choice
    else:
        for per_block, runs in ((2, 1), (1, 3), (None, None)):
            out.fill_(float("nan"))
            ops().attention_tcgen05(q, k_pool, v_pool, batch, table, page, out, nq, nkv, hd, window, scale, per_block=per_block,
                                    n_splits=runs, workspace=ws, sinks=sinks)
            check_sink_rows(out, qs, ks, vs, lengths, new, nq, hd, window, scale, dtype)
    assert status.item() == 0
    check_sink_rows(out, qs, ks, vs, lengths, new, nq, hd, window, scale, dtype)


def check_sink_rows(out, qs, ks, vs, lengths, new, nq, hd, window, scale, dtype):
    at = 0
    for s, (n, c) in enumerate(zip(lengths, new)):
        want = sink_attention_over_pages(qs[s], ks[s], vs[s], torch.arange(n - c, n), window, scale)
        got = out[at:at + c].double().cpu().reshape(c, nq, hd)
        assert not torch.isnan(got).any(), (s, n, c)
        tol = 1e-2 if dtype == "bfloat16" else 1e-5
        assert ((got - want).abs() <= tol * (1 + want.abs())).all(), (s, n, c, (got - want).abs().max().item())
        at += c


def test_a_sink_changes_rows_by_what_the_formula_says():
    """The kernels' result with a sink equals their result without, times sum / (1 + sum): checked where the sum is small."""
    nq, nkv, hd, page = 2, 1, 16, 8
    lengths, new = [3], [3]
    k_pool, v_pool, table, ks, vs = paged_setup(lengths, nkv, hd, page, torch.float32, seed=1)
    q = (rnd((3, nq, hd), 1) * 0.1).to(DEV).reshape(3, nq * hd)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    batch = _Batch(lengths, new, status)
    with_sink, without = torch.empty_like(q), torch.empty_like(q)
    ops().attention_plain(q, k_pool, v_pool, batch.positions, batch.seq_index, table, page, without, nq, nkv, hd, 0, 1.0, status)
    ops().attention_plain(q, k_pool, v_pool, batch.positions, batch.seq_index, table, page, with_sink, nq, nkv, hd, 0, 1.0, status,
                          torch.zeros(nq, dtype=torch.float32, device=DEV))
    s = torch.einsum("thd,sd->ths", q.cpu().view(3, nq, hd).double(), ks[0][:, 0].double())
    total = torch.stack([torch.exp(s[t, :, :t + 1]).sum(-1) for t in range(3)])          # [3, nq]
    ratio = (total / (1 + total))[:, :, None]
    close(with_sink.view(3, nq, hd), without.double().cpu().view(3, nq, hd) * ratio, "float32")
    assert (ratio < 0.8).all()


# ------------------------------------------------------------------------------------------------ whole models

@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("gugalorn")
    return {name: tg.make_folder(tmp, raw, seed=i + 1) for i, (name, (raw, _)) in enumerate(tg.CONFIGS.items())}


_plain_memo = {}


def plain_logits(folder, raw, tokens):
    key = (folder, tuple(tokens))
    if key not in _plain_memo:
        _plain_memo[key] = plain.forward(raw, tg.weights(folder), tokens)
    return _plain_memo[key]


def requests_for(raw, lengths, seed):
    return {f"q{i}": p for i, p in enumerate(tiny.prompts(raw["vocab"], lengths, seed=seed))}


WAYS = {"whole": replay.whole, "tail": lambda r: replay.tail_one_by_one(r, 40), "portions": replay.portions, "mixed": replay.mixed}
LENGTHS = {"G1": [150, 1, 2, 61, 34, 97], "G2": [260, 70, 1, 129, 3], "G3": [120, 3, 66, 2]}


@pytest.mark.parametrize("name", ["G1", "G2", "G3"])
def test_float32_replay_every_way_against_the_plain_implementation(folders, name):
    from rust_mlx_b200.engine import Engine
    raw, page = tg.CONFIGS[name]
    reqs = requests_for(raw, LENGTHS[name], seed=11)
    want = {rid: plain_logits(folders[name], raw, toks) for rid, toks in reqs.items()}
    first = None
    for way, cut in WAYS.items():
        steps = cut(reqs)
        # a cache just large enough and four state slots: pages and slots are used again as requests end
        eng = Engine(folders[name], dtype="float32", max_tokens=replay.tokens_needed(steps, page), page_size=page, max_requests=4)
        got = replay.run_engine(eng, steps)
        eng.pools.table.check()
        assert eng.pools.table.live() == 0
        for rid in reqs:
            err = tg.row_error(got[rid], want[rid])
            assert err.max().item() < 2e-4, (name, way, rid, int(err.argmax()), err.max().item())
        if first is None:
            first = got
        else:       # every sum of the 32-bit path is formed in an order that the position alone decides
            for rid in reqs:
                assert torch.equal(got[rid], first[rid]), (name, way, rid)


@pytest.mark.parametrize("name", ["G1", "G2", "G3"])
def test_bfloat16_replay_every_way(folders, name):
    from rust_mlx_b200.engine import Engine
    raw, page = tg.CONFIGS[name]
    reqs = requests_for(raw, LENGTHS[name], seed=12)
    want = {rid: plain_logits(folders[name], raw, toks) for rid, toks in reqs.items()}
    for way, cut in WAYS.items():
        steps = cut(reqs)
        eng = Engine(folders[name], dtype="bfloat16", max_tokens=replay.tokens_needed(steps, page), page_size=page, max_requests=4)
        got = replay.run_engine(eng, steps)
        eng.pools.table.check()
        errs = torch.cat([tg.row_error(got[rid], want[rid]) for rid in reqs])
        assert errs.max().item() < 0.12 and errs.median().item() < 0.03, (name, way, errs.max().item(), errs.median().item())


def test_every_layer_against_the_plain_implementation(folders):
    """The residual stream after every layer, and the recurrences' raw outputs, in 32-bit: a difference is found at the
    first layer that shows it."""
    from rust_mlx_b200.engine import Engine
    for name in ("G1", "G3"):
        raw, page = tg.CONFIGS[name]
        toks = tiny.prompts(raw["vocab"], [45], seed=5)[0]
        layers = []
        plain.forward(raw, tg.weights(folders[name]), toks, layers)
        eng = Engine(folders[name], dtype="float32", max_tokens=128, page_size=page, max_requests=2)
        _, taken = eng.step_with_intermediates([("a", toks, [])], ["a"])
        for i in range(1, len(raw["layers"])):
            got = taken[f"run{i}.residual"].double().cpu()       # the stream as layer i finds it = after layer i - 1
            assert (got - layers[i - 1]).abs().max().item() < 1e-4 * (1 + layers[i - 1].abs().max().item()), (name, i)


def needle_model(tmp_path, dims=16):
    """One parallel layer whose softmax side decides: a query finds one key far back by a large score."""
    raw = tg.model(90, 48, 2, [tg.par((2, 1, dims, dims, 8, 1e4, 1.0), (1, 4, 4), 1.0, 0.05)])
    return raw, tg.make_folder(tmp_path, raw, seed=5, sharp=40.0, out_boost=30.0)


def test_far_keys_decide_and_are_found_in_prompts_and_in_decoding(tmp_path):
    from rust_mlx_b200.engine import Engine
    raw, folder = needle_model(tmp_path)
    toks = tiny.prompts(90, [520], seed=3)[0]
    want = plain.forward(raw, tg.weights(folder), toks)
    for cut in (replay.whole, lambda r: replay.tail_one_by_one(r, 60), replay.portions):
        steps = cut({"a": toks})
        eng = Engine(folder, dtype="float32", max_tokens=replay.tokens_needed(steps, 16), page_size=16, max_requests=2)
        got = replay.run_engine(eng, steps)["a"]
        assert tg.row_error(got, want).max().item() < 2e-4
    # the scores are spread so widely that the plain implementation itself, told to forget everything older than 300
    # positions, gives other logits: keys far away carry weight
    s = plain.sink_attention
    try:
        plain.sink_attention = lambda q, k, v, scale, window=0: s(q, k, v, scale, 300)
        near = plain.forward(raw, tg.weights(folder), toks)
    finally:
        plain.sink_attention = s
    assert tg.row_error(near[400:], want[400:]).max().item() > 0.05
    eng = Engine(folder, dtype="bfloat16", max_tokens=1024, page_size=16, max_requests=2)
    got = replay.run_engine(eng, replay.tail_one_by_one({"a": toks}, 60))["a"]
    err = tg.row_error(got, want)
    assert err.max().item() < 0.4 and err.median().item() < 0.08


def test_states_and_rings_start_from_zero_when_slots_and_pages_are_used_again(folders):
    """Two slots and pages for one long request: every request takes over what the one before it left; the same request
    run again in a used slot gives the same bits as in a fresh engine."""
    from rust_mlx_b200.engine import Engine
    raw, page = tg.CONFIGS["G1"]
    prompts = tiny.prompts(raw["vocab"], [70, 40, 70, 9], seed=9)
    fresh = []
    for p in prompts:
        eng = Engine(folders["G1"], dtype="float32", max_tokens=128, page_size=page, max_requests=2)
        fresh.append(eng.step([("x", p, list(range(len(p))))], ["x"]).cpu())
    eng = Engine(folders["G1"], dtype="float32", max_tokens=128, page_size=page, max_requests=2)
    for turn in range(2):
        for i, p in enumerate(prompts):
            half = len(p) // 2
            eng.step([((turn, i), p[:half], [])])
            got = eng.step([((turn, i), p[half:], list(range(len(p) - half)))], [(turn, i)]).cpu()
            assert torch.equal(got, fresh[i][half:]), (turn, i)
    eng.pools.table.check()


def test_long_decoding(folders):
    from rust_mlx_b200.engine import Engine
    raw, page = tg.CONFIGS["G3"]
    toks = tiny.prompts(raw["vocab"], [330], seed=21)[0]
    want = plain_logits(folders["G3"], raw, toks)
    eng = Engine(folders["G3"], dtype="float32", max_tokens=512, page_size=page, max_requests=2)
    got = replay.run_engine(eng, replay.tail_one_by_one({"a": toks}, 325))["a"]
    assert tg.row_error(got, want).max().item() < 2e-4


def greedy(raw, w, prompt, n):
    ids = list(prompt)
    for _ in range(n):
        ids.append(int(plain.forward(raw, w, ids)[-1].argmax()))
    return ids[len(prompt):]


def test_greedy_generation_through_the_scheduler(folders):
    from rust_mlx_b200.engine import Engine
    for name in ("G1", "G3"):
        raw, page = tg.CONFIGS[name]
        w = tg.weights(folders[name])
        prompts = tiny.prompts(raw["vocab"], [30, 3, 55, 9, 41], seed=31)
        want = [greedy(raw, w, p, 8) for p in prompts]
        # a cache too small for all five at once and three state slots: requests wait, step back and are computed again
        eng = Engine(folders[name], dtype="float32", max_tokens=4 * page * 2 + 2 * page, page_size=page, max_requests=3)
        got = eng.generate(prompts, max_tokens=8, prefill_chunk=13, ignore_eos=True)
        assert got == want, name
        eng.pools.table.check()


def test_bfloat16_generation_in_graphs_equals_plain_launches(folders):
    """Decode steps captured in CUDA graphs (padded to the next batch size, whose spare places must not step a request's
    state; captured after an eager run whose state is put back) choose the tokens that plain launches choose."""
    from rust_mlx_b200.engine import Engine
    for name in ("G2", "G1"):
        raw, page = tg.CONFIGS[name]
        w = tg.weights(folders[name])
        prompts = tiny.prompts(raw["vocab"], [70, 9, 140, 33, 5], seed=41)
        # (five requests decode in a graph of six places: in 32-bit the tokens are the same bit for bit)
        exact = [Engine(folders[name], dtype="float32", max_tokens=4096, page_size=page, max_requests=8, cuda_graphs=g)
                 .generate(prompts, max_tokens=12, prefill_chunk=64, ignore_eos=True) for g in (True, False)]
        assert exact[0] == exact[1], name
        eng = Engine(folders[name], dtype="bfloat16", max_tokens=4096, page_size=page, max_requests=8)
        assert eng.graphs is not None
        got = eng.generate(prompts, max_tokens=12, prefill_chunk=64, ignore_eos=True)
        assert eng.graphs.replays > 0
        plain_steps = Engine(folders[name], dtype="bfloat16", max_tokens=4096, page_size=page, max_requests=8, cuda_graphs=False)
        assert plain_steps.generate(prompts, max_tokens=12, prefill_chunk=64, ignore_eos=True) == got
        for p, g in zip(prompts, got):
            ids = list(p)
            for t in g:
                logits = plain.forward(raw, w, ids)[-1]
                spread = (logits - logits.mean()).pow(2).mean().sqrt()
                assert logits[t] >= logits.max() - 0.15 * spread, (name, t, int(logits.argmax()))
                ids.append(t)


def test_trace_tool_runs_this_family(folders, tmp_path):
    raw, page = tg.CONFIGS["G1"]
    reqs = requests_for(raw, [40, 1, 77, 20, 5], seed=51)
    steps = replay.mixed(reqs)
    got = replay.run_trace_tool(folders["G1"], "float32", steps, str(tmp_path / "out"), replay.tokens_needed(steps, 64), raw["vocab"])
    for rid, toks in reqs.items():
        assert tg.row_error(got[rid], plain_logits(folders["G1"], raw, toks)).max().item() < 2e-4


def random_configuration(seed):
    """Sizes, constants and the order of layers drawn from a seed (every choice a model of this family may make)."""
    import random
    r = random.Random(seed)
    width = r.choice([48, 72, 96, 136])
    layers = []
    for _ in range(r.randint(2, 5)):
        ff = r.choice([0, 0, 32, 80])
        if r.random() < 0.5:
            heads = r.choice([2, 3, 4, 6])
            vdim = r.choice([4, 8, 12, 16])
            groups = r.choice([g for g in (1, 2, 3, 6) if heads % g == 0])
            norm_groups = r.choice([g for g in (1, 2, heads) if (heads * vdim) % g == 0])
            layers.append(tg.ssm(heads, vdim, r.choice([8, 16, 24, 32, 48]), groups, r.choice([1, 2, 3, 4]), norm_groups, ff))
        else:
            kv = r.choice([1, 2, 3])
            heads = kv * r.choice([1, 2, 3])
            dim, vdim = r.choice([8, 16, 32, 64]), r.choice([8, 16, 32, 64])
            dims = r.choice([0, dim // 2, dim]) // 2 * 2
            left = (heads, kv, dim, vdim, dims, r.choice([50.0, 1e4, 1e6]), r.uniform(0.1, 0.3))
            right = (r.choice([1, 2, 4, 6]), r.choice([4, 8, 12, 16, 48]), r.choice([8, 16, 64]))
            layers.append(tg.par(left, right, round(r.uniform(0.5, 1.5), 3), round(r.uniform(0.5, 1.5), 3), ff))
    return tg.model(r.randint(50, 300), width, r.choice([0, 2, 3, 4, 5]), layers, eps=r.choice([1e-5, 1e-6]), scale=r.choice([0.5, 1.0, 2.0]))


@pytest.mark.parametrize("seed", range(8))
def test_random_configurations_replayed_in_mixed_steps(tmp_path, seed):
    from rust_mlx_b200.engine import Engine
    raw = random_configuration(seed)
    folder = tg.make_folder(tmp_path, raw, seed=100 + seed)
    reqs = requests_for(raw, [70, 1, 33, 2, 90, 17], seed=seed)
    want = {rid: plain.forward(raw, tg.weights(folder), toks) for rid, toks in reqs.items()}
    page = [16, 32, 64][seed % 3]
    for dtype, bound in (("float32", 2e-4), ("bfloat16", 0.15)):
        for cut in (replay.mixed, replay.portions):
            steps = cut(reqs)
            eng = Engine(folder, dtype=dtype, max_tokens=replay.tokens_needed(steps, page), page_size=page, max_requests=4)
            got = replay.run_engine(eng, steps)
            eng.pools.table.check()
            for rid in reqs:
                err = tg.row_error(got[rid], want[rid])
                assert err.max().item() < bound, (seed, dtype, rid, int(err.argmax()), err.max().item(), raw)
