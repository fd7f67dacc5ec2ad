"""The Resolorn family on the GPU against its plain implementation (tests/plain_resolorn.py): each mechanism alone,
every way of cutting requests into steps, pages and slots used again, windows' edges, generation."""
import math
import os

import pytest
import torch

import plain_resolorn as plain
import replay
import tiny
import tiny_resolorn as tr

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
F = torch.float64


def context(dtype=torch.float32):
    from rust_mlx_b200.engine.workspace import Workspace
    from rust_mlx_b200.kernels import ops
    from rust_mlx_b200.parts import BuildContext
    return BuildContext(DEV, dtype, ops.default, Workspace(DEV))


def bind(part, seed=0, dtype=torch.float32, scale=None):
    """Random tensors for ``part`` (``scale``: name ending -> factor), bound; returns them in float64 on the host."""
    from rust_mlx_b200.weights.random_init import random_tensors
    tensors = random_tensors(part.all_param_specs(), seed, dtype, DEV)
    for ending, factor in (scale or {}).items():
        for k in tensors:
            if k.endswith(ending):
                tensors[k] = (tensors[k].float() * factor).to(tensors[k].dtype)
    host = {k: v.detach().cpu().to(F) for k, v in tensors.items()}
    part.bind_all(tensors, context(dtype))
    return host


# ---------------------------------------------------------------------------------------------- kernels alone

def test_embedding_adds_the_position_rows():
    from rust_mlx_b200.kernels import ops
    table = torch.randn(50, 36, device=DEV)
    pos = torch.randn(20, 36, device=DEV)
    ids = torch.tensor([3, 49, 0, 7], dtype=torch.int32, device=DEV)
    positions = torch.tensor([0, 19, 5, 5], dtype=torch.int32, device=DEV)
    h = torch.empty(4, 36, device=DEV)
    ops.embedding(ids, table, h, pos_table=pos, positions=positions)
    assert torch.equal(h, table[ids.long()] + pos[positions.long()])
    tb, pb = table.to(torch.bfloat16), pos.to(torch.bfloat16)
    ops.embedding(ids, tb, h, pos_table=pb, positions=positions)
    assert torch.equal(h, tb[ids.long()].float() + pb[positions.long()].float())


@pytest.mark.parametrize("width, rows", [(64, 5), (200, 300), (70, 3), (5000, 2)])
def test_norm_adds_a_scaled_sum_of_two(width, rows):
    from rust_mlx_b200.kernels import ops
    for dtype in (torch.float32, torch.bfloat16):
        h = torch.randn(rows, width, device=DEV)
        a = torch.randn(rows, width, device=DEV).to(dtype)
        b = torch.randn(rows, width, device=DEV).to(dtype)
        w = torch.rand(width, device=DEV) + 0.5
        x = torch.empty(rows, width, dtype=dtype, device=DEV)
        want_h = h.double() + 0.3 * (a.double() + b.double())
        want_x = plain.rms_norm(want_h, w.double(), 1e-5)
        h1 = h.clone()
        ops.add_rmsnorm(h1, a, w, 1e-5, x, delta2=b, mult=0.3)
        assert tiny.max_abs(h1, want_h) < 1e-5
        assert tiny.max_abs(x, want_x) < (1e-5 if dtype == torch.float32 else 4e-2)
        # one delta, factor 1: the bits of the kernel as other families use it
        h2, h3 = h.clone(), h.clone()
        x2 = torch.empty_like(x)
        ops.add_rmsnorm(h2, a, w, 1e-5, x)
        ops.add_rmsnorm(h3, a, w, 1e-5, x2, delta2=None, mult=1.0)
        assert torch.equal(h2, h + a.float()) and torch.equal(h2, h3) and torch.equal(x, x2)


@pytest.mark.parametrize("inner", [40, 64, 100])
def test_gated_activation_with_gelu(inner):
    from rust_mlx_b200.kernels import ops
    for dtype, tol in ((torch.float32, 2e-6), (torch.bfloat16, 2e-2)):
        gu = (torch.randn(7, 2 * inner, device=DEV) * 3).to(dtype)
        out = torch.empty(7, inner, dtype=dtype, device=DEV)
        ops.swiglu(gu, out, 0, "gelu_tanh")
        g, u = gu[:, :inner].double(), gu[:, inner:].double()
        want = plain.gelu_tanh(g) * u
        assert ((out.double() - want).abs() <= tol * (1 + want.abs())).all()
        ops.swiglu(gu, out, 0, "silu")
        want = plain.silu(g) * u
        assert ((out.double() - want).abs() <= tol * (1 + want.abs())).all()


@pytest.mark.parametrize("rows, width, experts, top", [(1, 64, 8, 2), (37, 96, 6, 6), (300, 50, 5, 1), (64, 128, 40, 7)])
def test_router_sort_products_and_weighted_sum(rows, width, experts, top):
    from rust_mlx_b200.kernels import ops
    torch.manual_seed(rows)
    for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 3e-2)):
        x = torch.randn(rows, width, device=DEV).to(dtype)
        wr = torch.randn(experts, width, device=DEV)
        ids = torch.empty(rows, top, dtype=torch.int32, device=DEV)
        wts = torch.empty(rows, top, dtype=torch.float32, device=DEV)
        ops.moe_route(x, wr, top, ids, wts)
        logits = x.double() @ wr.double().T
        want = torch.topk(logits, top, dim=-1)
        assert torch.equal(ids.long().sort(-1).values, want.indices.sort(-1).values)
        assert torch.equal(ids.long(), want.indices)             # in descending order of the logits
        assert tiny.max_abs(wts, torch.softmax(want.values, -1)) < 1e-5
        offsets = torch.empty(experts + 1, dtype=torch.int32, device=DEV)
        pairs = torch.empty(rows * top, dtype=torch.int32, device=DEV)
        where = torch.empty(rows * top, dtype=torch.int32, device=DEV)
        ops.moe_sort(ids, experts, offsets, pairs, where)
        flat = ids.flatten().long()
        counts = torch.bincount(flat, minlength=experts)
        assert offsets.tolist() == [0] + counts.cumsum(0).tolist()
        assert sorted(pairs.tolist()) == list(range(rows * top))
        assert torch.equal(where[pairs.long()], torch.arange(rows * top, dtype=torch.int32, device=DEV))
        for e in range(experts):
            run = pairs[offsets[e]:offsets[e + 1]].long()
            assert (flat[run] == e).all()
        n_out = 72
        w = (torch.randn(experts, n_out, width, device=DEV) * 0.1).to(dtype)
        y = torch.full((rows * top, n_out), float("nan"), dtype=dtype, device=DEV)
        ops.moe_gemm(x, w, y, offsets, sorted_pairs=pairs, top=top)
        src = pairs.long() // top
        want_y = torch.einsum("pk,pnk->pn", x[src].double(), w[flat[pairs.long()]].double())
        assert ((y.double() - want_y).abs() <= tol * (1 + want_y.abs())).all()
        w2 = (torch.randn(experts, width, n_out, device=DEV) * 0.1).to(dtype)
        z = torch.full((rows * top, width), float("nan"), dtype=dtype, device=DEV)
        ops.moe_gemm(y, w2, z, offsets)
        want_z = torch.einsum("pk,pnk->pn", y.double(), w2[flat[pairs.long()]].double())
        assert ((z.double() - want_z).abs() <= tol * (1 + want_z.abs())).all()
        shared = torch.randn(rows, width, device=DEV).to(dtype)
        out = torch.empty(rows, width, dtype=dtype, device=DEV)
        ops.moe_combine(z, where, wts, shared, out)
        want_out = (wts.double().unsqueeze(-1) * z.double()[where.long().view(rows, top)]).sum(1) + shared.double()
        assert ((out.double() - want_out).abs() <= tol * (1 + want_out.abs())).all()
        ops.moe_combine(z, where, wts, None, out)
        assert ((out.double() - (want_out - shared.double())).abs() <= tol * (1 + want_out.abs())).all()


@pytest.mark.parametrize("rows, top, experts, n_out, k", [(3, 2, 8, 72, 64), (64, 4, 6, 128, 200), (700, 2, 3, 320, 96),
                                                         (40, 1, 5, 200, 136), (2048, 2, 4, 256, 512)])
def test_experts_products_on_the_tensor_cores(rows, top, experts, n_out, k):
    """Few, some and many rows an expert (tiles of 16, 64 and 128 rows), experts without rows, weight rows that are
    no multiple of 128, K with a ragged last block of 64; plain and with the gated epilogue."""
    from rust_mlx_b200.kernels import ops
    torch.manual_seed(rows + k)
    x = torch.randn(rows, k, device=DEV).to(torch.bfloat16)
    ids = torch.stack([torch.randperm(experts, device=DEV)[:top] for _ in range(rows)]).to(torch.int32)
    if top == 1 and experts > 2:
        ids[ids == 1] = 0                                         # expert 1 gets no rows at all
    offsets = torch.empty(experts + 1, dtype=torch.int32, device=DEV)
    pairs = torch.empty(rows * top, dtype=torch.int32, device=DEV)
    where = torch.empty(rows * top, dtype=torch.int32, device=DEV)
    ops.moe_sort(ids, experts, offsets, pairs, where)
    xs = torch.empty(rows * top, k, dtype=torch.bfloat16, device=DEV)
    ops.moe_gather(x, pairs, top, xs)
    assert torch.equal(xs, x[pairs.long() // top])
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    which = ids.flatten().long()[pairs.long()]
    w = (torch.randn(experts, n_out, k, device=DEV) * 0.1).to(torch.bfloat16)
    y = torch.full((rows * top, n_out), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.moe_gemm_tcgen05(xs, w, y, offsets, status)
    assert status.item() == 0
    want = torch.stack([w[e].double() @ xs[i].double() for i, e in enumerate(which.tolist())]) if rows * top <= 256 else \
        torch.cat([xs[offsets[e]:offsets[e + 1]].double() @ w[e].double().T for e in range(experts)])
    assert ((y.double() - want).abs() <= 2e-2 * (1 + want.abs())).all()
    if n_out % 128 == 0:
        for activation, f in (("silu", plain.silu), ("gelu_tanh", plain.gelu_tanh)):
            act = torch.full((rows * top, n_out // 2), float("nan"), dtype=torch.bfloat16, device=DEV)
            ops.moe_gemm_tcgen05(xs, w, act, offsets, status, gated=True, activation=activation)
            blocks = want.view(rows * top, n_out // 128, 2, 64)
            want_act = (f(blocks[:, :, 0]) * blocks[:, :, 1]).reshape(rows * top, n_out // 2)
            assert status.item() == 0
            assert ((act.double() - want_act).abs() <= 2e-2 * (1 + want_act.abs())).all()


def test_experts_products_tile_arrangements_agree():
    """The arrangements kept for comparisons (two weight tiles a block; tiles of 256 rows) against the default."""
    import ctypes
    from rust_mlx_b200.kernels import ops
    from rust_mlx_b200.kernels.library import kernels_library
    lib = kernels_library()
    torch.manual_seed(5)
    experts, n_out, k, rows, top = 3, 384, 200, 900, 2
    x = torch.randn(rows * top, k, device=DEV).to(torch.bfloat16)
    ids = torch.randint(0, experts, (rows * top, 1), device=DEV, dtype=torch.int32)
    offsets = torch.empty(experts + 1, dtype=torch.int32, device=DEV)
    pairs = torch.empty(rows * top, dtype=torch.int32, device=DEV)
    where = torch.empty(rows * top, dtype=torch.int32, device=DEV)
    ops.moe_sort(ids, experts, offsets, pairs, where)
    w = (torch.randn(experts, n_out, k, device=DEV) * 0.1).to(torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    outs = {}
    try:
        for variant in (0, 1, 2):
            lib.rmx_moe_set_tile_variant(ctypes.c_int(variant))
            for gated in (False, True):
                y = torch.full((rows * top, n_out // 2 if gated else n_out), float("nan"), dtype=torch.bfloat16, device=DEV)
                ops.moe_gemm_tcgen05(x, w, y, offsets, status, gated=gated)
                outs[(variant, gated)] = y
    finally:
        lib.rmx_moe_set_tile_variant(ctypes.c_int(0))
    assert status.item() == 0
    for gated in (False, True):
        assert not torch.isnan(outs[(0, gated)].float()).any()
        for variant in (1, 2):
            a, b = outs[(0, gated)].double(), outs[(variant, gated)].double()
            assert ((a - b).abs() <= 1e-2 * (1 + a.abs())).all()


def test_routed_part_in_bfloat16_on_the_tensor_cores_against_the_fma_kernels():
    from rust_mlx_b200.kernels import ops
    from rust_mlx_b200.parts.feedforward import SwiGLUFeedForward
    from rust_mlx_b200.parts.routed import RoutedFeedForward

    class Batch:
        status = torch.zeros(1, dtype=torch.int32, device=DEV)

    for inner in (64, 40):            # with and without blocks of 64 (the gated epilogue)
        ff = RoutedFeedForward("m", 96, inner, 6, 2, shared=SwiGLUFeedForward("m.shared", 96, 32, names=("gate", "up", "down")))
        w = bind(ff, seed=inner, dtype=torch.bfloat16, scale={".router": 50.0, ".gate": 10.0, ".up": 10.0, ".down": 10.0})
        for rows in (5, 300):
            x = torch.randn(rows, 96, device=DEV).to(torch.bfloat16)
            got = ff.forward(x, Batch()).clone()
            ff.ctx.ops.use_tcgen05_experts = False
            try:
                other = ff.forward(x, Batch()).clone()
            finally:
                ff.ctx.ops.use_tcgen05_experts = True
            mlp = {"router": {"experts": 6, "top": 2}, "shared": {"ff": 32}}
            want = plain.routed_experts(x.double().cpu(), w, "m", mlp, bf16=True)
            for y in (got, other):
                err = tr.row_error(y.cpu(), want)
                assert (err > 0.05).sum().item() <= 0.02 * rows, err.max().item()
            assert Batch.status.item() == 0


def test_products_of_heads_with_their_own_matrices():
    from rust_mlx_b200.kernels import ops
    rows, heads, k, n = 13, 3, 24, 40
    for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 2e-2)):
        a = torch.randn(rows, heads * k, device=DEV).to(dtype)
        w = torch.randn(heads, n, k, device=DEV).to(dtype)
        wide = torch.full((rows, heads * n + 8), 7.0, dtype=dtype, device=DEV)
        out = wide[:, :heads * n]                                       # rows of a wider buffer
        ops.default.linear_heads(a.view(rows, heads, k), w, out.view(rows, heads, n) if out.is_contiguous() else
                                 out.unflatten(1, (heads, n)))
        want = torch.einsum("thk,hnk->thn", a.view(rows, heads, k).double(), w.double()).reshape(rows, heads * n)
        assert ((out.double() - want).abs() <= tol * (1 + want.abs())).all()
        assert (wide[:, heads * n:] == 7.0).all()


def test_latent_norms_write_the_latent_into_its_page_and_gates_scale_heads():
    from rust_mlx_b200.kernels import ops
    q_rank, kv_rank, heads, page = 20, 24, 3, 4
    n = 6
    for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 2e-2)):
        proj = torch.randn(n, q_rank + kv_rank + heads, device=DEV).to(dtype)
        wq, wkv = torch.rand(q_rank, device=DEV) + 0.5, torch.rand(kv_rank, device=DEV) + 0.5
        cq = torch.empty(n, q_rank, dtype=dtype, device=DEV)
        pool = torch.full((5, 1, page, kv_rank), float("nan"), dtype=dtype, device=DEV)
        positions = torch.tensor([4, 5, 6, 0, 1, 9], dtype=torch.int32, device=DEV)
        seq_index = torch.tensor([0, 0, 0, 1, 1, 2], dtype=torch.int32, device=DEV)
        table = torch.tensor([[-1, 3, -1], [0, -1, -1], [-1, -1, 4]], dtype=torch.int32, device=DEV)
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        ops.latent_norms(proj, q_rank, kv_rank, wq, wkv, 1e-6, cq, pool, positions, seq_index, table, page, status)
        assert status.item() == 0
        want_q = plain.rms_norm(proj[:, :q_rank].double(), wq.double(), 1e-6)
        want_c = plain.rms_norm(proj[:, q_rank:q_rank + kv_rank].double(), wkv.double(), 1e-6)
        assert ((cq.double() - want_q).abs() <= tol * (1 + want_q.abs())).all()
        places = [(3, 0), (3, 1), (3, 2), (0, 0), (0, 1), (4, 1)]
        for t, (pg, slot) in enumerate(places):
            assert ((pool[pg, 0, slot].double() - want_c[t]).abs() <= tol * (1 + want_c[t].abs())).all()
        written = torch.zeros(5, page, dtype=torch.bool)
        for pg, slot in places:
            written[pg, slot] = True
        assert torch.isnan(pool[:, 0][~written.to(DEV)]).all()          # nothing else was touched
        # a layer that reads another's latents writes none
        pool2 = torch.full_like(pool, float("nan"))
        ops.latent_norms(proj, q_rank, 0, wq, None, 1e-6, cq, None, positions, seq_index, table, page, status)
        assert torch.isnan(pool2).all()
        # a position without a page is reported, not written
        bad = torch.tensor([[-1, -1, -1]] * 3, dtype=torch.int32, device=DEV)
        ops.latent_norms(proj, q_rank, kv_rank, wq, wkv, 1e-6, cq, pool2, positions, seq_index, bad, page, status)
        assert status.item() == 1 and torch.isnan(pool2).all()
        o = torch.randn(n, heads * 5, device=DEV).to(dtype)
        want_o = o.double().view(n, heads, 5) * torch.sigmoid(proj[:, q_rank + kv_rank:].double()).unsqueeze(-1)
        ops.gate_heads(o, proj[:, q_rank + kv_rank:], heads, 5)
        assert ((o.double().view(n, heads, 5) - want_o).abs() <= tol * (1 + want_o.abs())).all()


# ---------------------------------------------------------------------------------------------- parts alone

def test_gated_feed_forward_part_with_gelu_and_other_names():
    from rust_mlx_b200.parts.feedforward import SwiGLUFeedForward
    for inner in (72, 128):
        ff = SwiGLUFeedForward("l0.mlp", 48, inner, activation="gelu_tanh", names=("gate", "up", "down"))
        w = bind(ff, seed=5, scale={".gate": 20.0})
        x = torch.randn(9, 48, device=DEV)
        want = plain.gated_unit(x.double().cpu(), w["l0.mlp.gate"], w["l0.mlp.up"], w["l0.mlp.down"], plain.gelu_tanh)
        assert tiny.max_abs(ff.forward(x).cpu(), want) < 1e-5


def test_gated_feed_forward_in_bfloat16_forms_gelu_in_the_product():
    """Few rows: gate/up with GELU(gate) * up in the tcgen05 product's epilogue, one launch, against the plain pieces."""
    from rust_mlx_b200.kernels import ops
    from rust_mlx_b200.parts.feedforward import SwiGLUFeedForward
    ff = SwiGLUFeedForward("m", 256, 640, activation="gelu_tanh", names=("gate", "up", "down"))
    w = bind(ff, seed=6, dtype=torch.bfloat16, scale={".gate": 30.0})
    assert ops.prefers_fused_swiglu(9, 1280, 256)
    for rows in (1, 9, 40):
        x = torch.randn(rows, 256, device=DEV).to(torch.bfloat16)
        before = ops.launch_count
        y = ff.forward(x)
        assert ops.launch_count - before <= 2
        want = plain.gated_unit(x.double().cpu(), w["m.gate"], w["m.up"], w["m.down"], plain.gelu_tanh, bf16=True)
        assert ((y.double().cpu() - want).abs() <= 2e-2 * (1 + want.abs())).all()


@pytest.mark.parametrize("experts, top, shared, rows", [(6, 2, 32, 50), (4, 4, 0, 9), (5, 1, 16, 1), (3, 2, 8, 700)])
def test_routed_feed_forward_part(experts, top, shared, rows):
    from rust_mlx_b200.parts.feedforward import SwiGLUFeedForward
    from rust_mlx_b200.parts.routed import RoutedFeedForward
    width, inner = 40, 24
    sh = SwiGLUFeedForward("m.shared", width, shared, names=("gate", "up", "down")) if shared else None
    ff = RoutedFeedForward("m", width, inner, experts, top, shared=sh)
    w = bind(ff, seed=experts, scale={".router": 50.0, ".gate": 10.0, ".up": 10.0, ".down": 10.0})
    x = torch.randn(rows, width, device=DEV)
    mlp = {"router": {"experts": experts, "top": top}}
    if shared:
        mlp["shared"] = {"ff": shared}
    want = plain.routed_experts(x.double().cpu(), w, "m", mlp)
    got = ff.forward(x).cpu()
    assert ((got.double() - want).abs() <= 1e-5 * (1 + want.abs())).all()
    # a row's result does not depend on the rows beside it
    alone = ff.forward(x[rows // 2:rows // 2 + 1].contiguous()).cpu()
    assert torch.equal(alone[0], got[rows // 2])


@pytest.mark.parametrize("window, own", [(0, True), (6, True), (1, True), (9, False)])
def test_latent_attention_part_over_steps(window, own):
    """The mixer alone with a cache of its own: a portion, then single tokens and small portions.  ``own`` False: it
    reads latents that another mixer (with a narrower window of its own) wrote."""
    from rust_mlx_b200.cache import CachePools
    from rust_mlx_b200.engine.batch import SequenceInput, build_batch
    from rust_mlx_b200.parts.latent_attention import LatentAttentionMixer
    width, heads, dim, vdim, q_rank, kv_rank, page = 40, 3, 8, 12, 20, 24, 4
    writer = LatentAttentionMixer("w", width, heads, dim, vdim, q_rank, kv_rank, 1e-5, window=4, cache_window=max(window, 4))
    mixer = writer if own else LatentAttentionMixer("r", width, 2, 16, 8, 12, kv_rank, 1e-5, scale=0.4, window=window,
                                                    cache_window=max(window, 4), own_latent=False)
    if own:
        writer.window, writer.cache_window = window, window
    sharp = {".uq": 12.0, ".uk": 12.0}
    ww = bind(writer, seed=8, scale=sharp)
    wm = ww if own else bind(mixer, seed=9, scale=sharp)
    pools = CachePools({0: writer.cache_spec()}, max_tokens=64, page_size=page, max_requests=2, dtype=torch.float32, device=DEV)
    pools.groups[0].k_pool.fill_(float("nan"))
    T = 27
    x = torch.randn(T, width, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    pools.open(3)
    outs, at = [], 0
    for c in (11, 1, 2, 1, 1, 7, 1, 1, 2):
        pools.table.reserve(3, at + c)
        batch = build_batch([SequenceInput(3, at, [0] * c, [])], pools, DEV, status, 10)
        xs = x[at:at + c].contiguous()
        if not own:
            writer.forward(xs, batch, pools.view(0, batch, False))
        outs.append(mixer.forward(xs, batch, pools.view(0, batch, not own)).clone())
        at += c
        pools.table.commit(3, at)
    assert status.item() == 0 and at == T
    xd = x.double().cpu()
    c_lat = plain.latent(xd, ww, "w", 1e-5)
    m = {"heads": mixer.heads, "dim": mixer.dim, "vdim": mixer.vdim, "scale": mixer.scale}
    if window:
        m["mask"] = {"size": window}
    want = plain.latent_attention(xd, c_lat, wm, mixer.prefix, m, 1e-5)
    assert tiny.max_abs(torch.cat(outs).cpu(), want) < 2e-5


def test_parallel_block_adds_both_outputs_scaled():
    from rust_mlx_b200.parts.base import ScaledSum
    from rust_mlx_b200.parts.block import ParallelBlock
    from rust_mlx_b200.parts.feedforward import SwiGLUFeedForward
    from rust_mlx_b200.parts.norm import RMSNorm

    class Twice:                        # a mixer that remembers nothing: y = 2 x
        graph_safe = True
        def children(self): return []
        def all_param_specs(self): return []
        def bind_all(self, tensors, ctx): self.ctx = ctx
        def cache_specs(self): return []
        def forward(self, x, batch, cache): return (2 * x).contiguous()

    width = 32
    block = ParallelBlock(RMSNorm("n", width, 1e-5), Twice(), SwiGLUFeedForward("f", width, 48, names=("gate", "up", "down")), 0.25)
    w = bind(block, seed=3, scale={".gate": 10.0, ".up": 10.0, ".down": 10.0})
    end = RMSNorm("e", width, 1e-5)
    bind(end, seed=4)
    h = torch.randn(5, width, device=DEV)
    h0 = h.double().cpu()
    h, pending = block.forward(h, None, None, None)
    assert isinstance(pending, ScaledSum) and pending.factor == 0.25
    end.forward(h, pending)
    x = plain.rms_norm(h0, w["n"], 1e-5)
    want = h0 + 0.25 * (2 * x + plain.gated_unit(x, w["f.gate"], w["f.up"], w["f.down"], plain.silu))
    assert tiny.max_abs(h.cpu(), want) < 1e-5
    # a layer of a mixer alone
    block = ParallelBlock(RMSNorm("n", width, 1e-5), Twice(), None, 0.5)
    w = bind(block, seed=3)
    h = h0.float().to(DEV)
    h, pending = block.forward(h, None, None, None)
    end.forward(h, pending)
    assert tiny.max_abs(h.cpu(), h0 + 0.5 * 2 * plain.rms_norm(h0, w["n"], 1e-5)) < 1e-5


# ---------------------------------------------------------------------------------------------- whole models

@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("resolorn")
    return {name: tr.make_folder(tmp, raw, seed=i + 1) for i, (name, (raw, _)) in enumerate(tr.CONFIGS.items())}


_plain_memo = {}


def plain_logits(folder, raw, tokens, bf16=False):
    key = (folder, tuple(tokens), bf16)
    if key not in _plain_memo:
        _plain_memo[key] = plain.forward(raw, tr.weights(folder), tokens, bf16=bf16)
    return _plain_memo[key]


def requests_for(raw, lengths, seed):
    return {f"q{i}": p for i, p in enumerate(tiny.prompts(raw["vocab"], lengths, seed=seed))}


WAYS = {"whole": replay.whole, "tail": lambda r: replay.tail_one_by_one(r, 40), "portions": replay.portions, "mixed": replay.mixed}
# lengths past every window and several pages; one and two tokens (the first tokens of a sequence)
LENGTHS = {"R1": [150, 1, 2, 61, 34, 97], "R2": [300, 2, 131, 75, 1], "R3": [260, 70, 1, 129], "R4": [90, 33, 2], "R5": [120, 3, 66]}


@pytest.mark.parametrize("name", ["R1", "R2", "R3", "R4", "R5"])
def test_float32_replay_every_way_against_the_plain_implementation(folders, name):
    from rust_mlx_b200.engine import Engine
    raw, page = tr.CONFIGS[name]
    reqs = requests_for(raw, LENGTHS[name], seed=11)
    want = {rid: plain_logits(folders[name], raw, toks) for rid, toks in reqs.items()}
    first = None
    for way, cut in WAYS.items():
        steps = cut(reqs)
        # a cache just large enough: pages and slots are used again as requests end
        eng = Engine(folders[name], dtype="float32", max_tokens=replay.tokens_needed(steps, page), page_size=page, max_requests=4)
        got = replay.run_engine(eng, steps)
        eng.pools.table.check()
        assert eng.pools.table.live() == 0
        for rid in reqs:
            err = tr.row_error(got[rid], want[rid])
            assert err.max().item() < 2e-4, (name, way, rid, int(err.argmax()), err.max().item())
        if first is None:
            first = got
        else:       # the 32-bit path adds in an order that the position alone decides: the same bits however it is cut
            for rid in reqs:
                assert torch.equal(got[rid], first[rid]), (name, way, rid)


@pytest.mark.parametrize("name", ["R1", "R2", "R3", "R4", "R5"])
def test_bfloat16_replay_every_way(folders, name):
    """Against the plain implementation with bfloat16 roundings.  A router's close call may fall the other way in
    two bfloat16 evaluations, which changes a row by far more than rounding: models with routed experts are
    allowed a few such rows, the others none."""
    from rust_mlx_b200.engine import Engine
    raw, page = tr.CONFIGS[name]
    reqs = requests_for(raw, LENGTHS[name], seed=12)
    want = {rid: plain_logits(folders[name], raw, toks, bf16=True) for rid, toks in reqs.items()}
    routed = any(layer["mlp"] and layer["mlp"]["kind"] == "moe" for layer in raw["layers"])
    for way, cut in WAYS.items():
        steps = cut(reqs)
        eng = Engine(folders[name], dtype="bfloat16", max_tokens=replay.tokens_needed(steps, page), page_size=page, max_requests=4)
        got = replay.run_engine(eng, steps)
        eng.pools.table.check()
        errs = torch.cat([tr.row_error(got[rid], want[rid]) for rid in reqs])
        over = (errs > 0.06).sum().item()
        assert over <= (0.04 * errs.numel() if routed else 0), (name, way, over, errs.numel(), errs.max().item())
        assert errs.median().item() < 0.03


def test_far_keys_decide_and_are_found_in_prompts_and_in_decoding(tmp_path):
    """One layer without a window and scores spread so widely that a position's output rests on one or two keys
    anywhere in the hundreds of tokens before it, across many pages: a key that is lost shows at once."""
    from safetensors.torch import load_file, save_file
    from rust_mlx_b200.engine import Engine
    raw = {"architecture": "Resolorn", "vocab": 90, "width": 48, "max_positions": 700, "norm": {"eps": 1e-6}, "residual_mult": 1.0,
           "layers": [tr._layer(tr._mixer(2, 16, 16, 16, 32), None)]}
    folder = tr.make_folder(tmp_path, raw, seed=5, sharp=30.0)
    toks = tiny.prompts(90, [520], seed=3)[0]
    want = plain.forward(raw, tr.weights(folder), toks)
    for cut in (replay.whole, lambda r: replay.tail_one_by_one(r, 60), replay.portions):
        steps = cut({"a": toks})
        eng = Engine(folder, dtype="float32", max_tokens=replay.tokens_needed(steps, 16), page_size=16, max_requests=2)
        got = replay.run_engine(eng, steps)["a"]
        assert tr.row_error(got, want).max().item() < 2e-4
    eng = Engine(folder, dtype="bfloat16", max_tokens=1024, page_size=16, max_requests=2)
    got = replay.run_engine(eng, replay.tail_one_by_one({"a": toks}, 60))["a"]
    err = tr.row_error(got, plain.forward(raw, tr.weights(folder), toks, bf16=True))
    assert err.max().item() < 0.3 and err.median().item() < 0.05     # (a lost key of such weight changes a row by about 1)


def test_just_inside_and_just_outside_a_window(tmp_path):
    """With a window of w, position i sees i - w + 1 and not i - w.  The plain implementation with the window one
    wider or one narrower must differ clearly from the engine, the right one must agree: in a prompt's portion and
    decoding, at page borders (window 16 = page, 17, 15)."""
    from rust_mlx_b200.engine import Engine
    for w in (15, 16, 17):
        raw = {"architecture": "Resolorn", "vocab": 80, "width": 32, "max_positions": 128, "norm": {"eps": 1e-6},
               "residual_mult": 1.0, "layers": [tr._layer(tr._mixer(2, 8, 8, 12, 16, window=w), None)]}
        folder = tr.make_folder(tmp_path, raw, seed=w, sharp=10.0, out_boost=40.0)
        toks = tiny.prompts(80, [70], seed=w)[0]
        weights = tr.weights(folder)
        want = plain.forward(raw, weights, toks)
        wrong = []
        for other in (w - 1, w + 1):
            alt = {**raw, "layers": [tr._layer(tr._mixer(2, 8, 8, 12, 16, window=other), None)]}
            wrong.append(plain.forward(alt, weights, toks))
        for cut in (replay.whole, lambda r: replay.tail_one_by_one(r, 45), replay.portions):
            eng = Engine(folder, dtype="float32", max_tokens=128, page_size=16, max_requests=2)
            got = replay.run_engine(eng, cut({"a": toks}))["a"]
            assert tr.row_error(got, want).max().item() < 2e-4
            for alt in wrong:
                assert tr.row_error(got[w + 1:], alt[w + 1:]).median().item() > 1e-2


def test_long_decoding_past_the_windows_with_pages_given_back(folders):
    from rust_mlx_b200.engine import Engine
    raw, page = tr.CONFIGS["R2"]
    toks = tiny.prompts(raw["vocab"], [400], seed=21)[0]
    want = plain_logits(folders["R2"], raw, toks)
    steps = replay.tail_one_by_one({"a": toks}, 395)
    eng = Engine(folders["R2"], dtype="float32", max_tokens=1024, page_size=page, max_requests=2)
    got = replay.run_engine(eng, steps[:-1])["a"]
    assert tr.row_error(got, want[:399]).max().item() < 2e-4
    # every cache has a window here: pages behind the widest were given back while the request went on
    rid = eng._req_ids["a"]
    for g, grp in enumerate(eng.pools.paged_groups):
        assert eng.pools.table.pages_held(rid, grp.table_index) <= -(-grp.spec.window // page) + 1
    eng.step([("a", toks[-1:], [])], ["a"])
    eng.pools.table.check()


def test_greedy_generation_through_the_scheduler(folders):
    from rust_mlx_b200.engine import Engine
    for name in ("R1", "R2"):
        raw, page = tr.CONFIGS[name]
        w = tr.weights(folders[name])
        prompts = tiny.prompts(raw["vocab"], [30, 3, 55, 9, 41], seed=31)
        want = []
        for p in prompts:
            ids = list(p)
            for _ in range(8):
                ids.append(int(plain.forward(raw, w, ids)[-1].argmax()))
            want.append(ids[len(p):])
        # a cache too small for all five at once, so that requests wait and take over pages and slots of others
        eng = Engine(folders[name], dtype="float32", max_tokens=4 * page * 2 + 2 * page, page_size=page, max_requests=3)
        got = eng.generate(prompts, max_tokens=8, prefill_chunk=13, ignore_eos=True)
        assert got == want, name
        eng.pools.table.check()


def test_bfloat16_generation_in_graphs_follows_the_plain_implementation(folders):
    from rust_mlx_b200.engine import Engine
    raw, page = tr.CONFIGS["R3"]
    w = tr.weights(folders["R3"])
    prompts = tiny.prompts(raw["vocab"], [70, 9, 140], seed=41)
    eng = Engine(folders["R3"], dtype="bfloat16", max_tokens=2048, page_size=page, max_requests=4)
    assert eng.graphs is not None
    got = eng.generate(prompts, max_tokens=10, prefill_chunk=64, ignore_eos=True)
    assert eng.graphs.replays > 0
    plain_steps = Engine(folders["R3"], dtype="bfloat16", max_tokens=2048, page_size=page, max_requests=4, cuda_graphs=False)
    assert plain_steps.generate(prompts, max_tokens=10, prefill_chunk=64, ignore_eos=True) == got
    for p, g in zip(prompts, got):
        ids = list(p)
        for t in g:
            logits = plain.forward(raw, w, ids, bf16=True)[-1]
            spread = (logits - logits.mean()).pow(2).mean().sqrt()
            assert logits[t] >= logits.max() - 0.1 * spread, (t, int(logits.argmax()))
            ids.append(t)


def test_trace_tool_runs_this_family(folders, tmp_path):
    raw, page = tr.CONFIGS["R1"]
    reqs = requests_for(raw, [40, 1, 77], seed=51)
    steps = replay.mixed(reqs)
    got = replay.run_trace_tool(folders["R1"], "float32", steps, str(tmp_path / "out"), replay.tokens_needed(steps, 64),
                                raw["vocab"])
    for rid, toks in reqs.items():
        assert tr.row_error(got[rid], plain_logits(folders["R1"], raw, toks)).max().item() < 2e-4


def test_a_request_beyond_the_position_table_is_refused(folders):
    from rust_mlx_b200.engine import Engine, EngineError
    raw, page = tr.CONFIGS["R1"]
    eng = Engine(folders["R1"], dtype="float32", max_tokens=1024, page_size=page, max_requests=2)
    with pytest.raises(EngineError, match="position"):
        eng.step([("a", [1] * (raw["max_positions"] + 1), [])])
    eng.pools.table.check()
    assert eng.pools.table.live() == 0
