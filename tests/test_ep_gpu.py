"""Expert-parallel pieces on the GPU: the row-level entry points on one device, and the
two-rank NCCL exchange (needs two GPUs; skipped otherwise) against the single-GPU block."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available()
    return torch.device("cuda:0")


def test_rows_entry_points_single_gpu(orc):
    from maxuna_b200.moe import MoeBlock

    dev = torch.device("cuda:0")
    blk = MoeBlock.random(256, 512, 8, 2, seed=41, device=dev, weight_std=0.25)
    host = blk.host_layer(orc)
    rng = np.random.default_rng(42)
    rows = 77
    x = rng.standard_normal((rows, 256)).astype(np.float32)
    ids = rng.integers(0, 8, rows).astype(np.int32)
    w = rng.uniform(0.1, 1.0, rows).astype(np.float32)
    got = blk.experts_forward_rows(torch.from_numpy(x).to(dev), torch.from_numpy(ids).to(dev), torch.from_numpy(w).to(dev))
    idn = ids.astype(np.uint32).reshape(-1, 1)
    g = orc.mul_id(orc.Q4_K, host.gate, 8, 512, 256, x[:, None, :], idn)
    u = orc.mul_id(orc.Q4_K, host.up, 8, 512, 256, x[:, None, :], idn)
    want = orc.mul_id(orc.Q6_K, host.down, 8, 256, 512, orc.silu_mul(g, u), idn)[:, 0, :] * w[:, None]
    assert orc.rel_l2(got.cpu().numpy(), want) < 2e-3
    z = np.zeros((rows, 1), np.uint32)
    gs = orc.mul_id(orc.Q4_K, host.sh_gate, 1, 512, 256, x[:, None, :], z)
    us = orc.mul_id(orc.Q4_K, host.sh_up, 1, 512, 256, x[:, None, :], z)
    want_s = orc.mul_id(orc.Q6_K, host.sh_down, 1, 256, 512, orc.silu_mul(gs, us), z)[:, 0, :]
    got_s = blk.shared_forward(torch.from_numpy(x).to(dev))
    assert orc.rel_l2(got_s.cpu().numpy(), want_s) < 2e-3
    torch.cuda.synchronize()


def test_rows_f16_equals_f32_rows(orc):
    """The half-precision wire format gives the same result as the same values passed as f32."""
    from maxuna_b200.moe import MoeBlock

    dev = torch.device("cuda:0")
    blk = MoeBlock.random(256, 512, 8, 2, seed=43, device=dev, weight_std=0.25)
    gen = torch.Generator(device=dev)
    gen.manual_seed(5)
    rows = 130
    x16 = torch.randn(rows, 256, generator=gen, device=dev).to(torch.float16)
    ids = torch.randint(0, 8, (rows,), generator=gen, device=dev, dtype=torch.int32)
    w = torch.rand(rows, generator=gen, device=dev)
    a = blk.experts_forward_rows(x16, ids, w)
    b = blk.experts_forward_rows(x16.to(torch.float32), ids, w)
    torch.cuda.synchronize()
    assert torch.equal(a, b)


@pytest.mark.parametrize("t,k", [(1, 1), (130, 3), (700, 4)])
def test_tokens_entry_matches_rows_entry(t, k):
    """The token-level entry (empty slots allowed) against the row-level one on the expanded slots."""
    from maxuna_b200.moe import MoeBlock

    dev = torch.device("cuda:0")
    ne = 8
    blk = MoeBlock.random(256, 512, ne, 2, seed=47, device=dev, weight_std=0.25)
    gen = torch.Generator(device=dev)
    gen.manual_seed(9 + t)
    x16 = torch.randn(t, 256, generator=gen, device=dev).to(torch.float16)
    # distinct experts per token; about a third of the slots empty (id == ne), slot 0 always used
    ids = torch.rand(t, ne, generator=gen, device=dev).argsort(dim=1)[:, :k].to(torch.int32)
    empty = torch.rand(t, k, generator=gen, device=dev) < 0.35
    empty[:, 0] = False
    ids = torch.where(empty, torch.full_like(ids, ne), ids)
    w = torch.rand(t, k, generator=gen, device=dev)
    got = blk.experts_forward_tokens(x16, ids, w)
    tok, slot = torch.nonzero(ids < ne, as_tuple=True)
    y = blk.experts_forward_rows(x16[tok].contiguous(), ids[tok, slot].contiguous(), w[tok, slot].contiguous())
    want = torch.zeros(t, 256, device=dev)
    for s_ in range(k):
        m = slot == s_
        want.index_add_(0, tok[m], y[m])
    torch.cuda.synchronize()
    assert float((got - want).norm() / want.norm()) < 1e-6
    blk.check_device_flag()


@pytest.mark.parametrize("world", [2, 4])
def test_ep_pack_and_combine_match_the_index_arithmetic(world):
    """lmoe_ep_pack / lmoe_ep_combine against the torch plan they replace (one device, any world size)."""
    from maxuna_b200._native import check, lib
    from maxuna_b200.gguf import stream_ptr

    dev = torch.device("cuda:0")
    gen = torch.Generator(device=dev)
    gen.manual_seed(11)
    t, h, k, ne = 37, 128, 3, 8
    x = torch.randn(t, h, generator=gen, device=dev)
    # distinct experts per token, arbitrary order
    ids = torch.stack([torch.randperm(ne, generator=gen, device=dev)[:k] for _ in range(t)]).to(torch.int32)
    w = torch.rand(t, k, generator=gen, device=dev)
    n = t * k
    rows = torch.empty(n, h, dtype=torch.float16, device=dev)
    lids = torch.empty(n, dtype=torch.int32, device=dev)
    rw = torch.empty(n, dtype=torch.float32, device=dev)
    pos = torch.empty(n, dtype=torch.int32, device=dev)
    counts = torch.empty(world, dtype=torch.int64, device=dev)
    ws = torch.empty(lib().lmoe_ep_pack_workspace_bytes(ne, t), dtype=torch.uint8, device=dev)
    check(lib().lmoe_ep_pack(x.data_ptr(), ids.data_ptr(), w.data_ptr(), t, h, k, ne, world, rows.data_ptr(), lids.data_ptr(),
                             rw.data_ptr(), pos.data_ptr(), counts.data_ptr(), ws.data_ptr(), ws.numel(), stream_ptr()))
    torch.cuda.synchronize()
    e_local = ne // world
    flat = ids.reshape(-1).to(torch.int64)
    assert counts.tolist() == torch.bincount(flat // e_local, minlength=world).tolist()
    p = pos.to(torch.int64)
    assert sorted(p.tolist()) == list(range(n))                      # a permutation
    dest_sorted = torch.empty(n, dtype=torch.int64, device=dev)
    dest_sorted[p] = flat // e_local
    assert bool(torch.all(dest_sorted[1:] >= dest_sorted[:-1]))      # grouped by destination rank
    assert torch.equal(rows[p], x.to(torch.float16).repeat_interleave(k, dim=0))
    assert torch.equal(lids.to(torch.int64)[p], flat % e_local)
    assert torch.equal(rw[p], w.reshape(-1))
    # return leg: rows come back in the order they were sent
    back = torch.randn(n, h, generator=gen, device=dev)
    shared = torch.randn(t, h, generator=gen, device=dev)
    out = torch.empty(t, h, device=dev)
    check(lib().lmoe_ep_combine(back.data_ptr(), pos.data_ptr(), shared.data_ptr(), t, k, h, out.data_ptr(), stream_ptr()))
    torch.cuda.synchronize()
    want = torch.zeros(t, h, device=dev)
    y3 = back[p].view(t, k, h)
    for s_ in range(k):
        want += y3[:, s_]
    want += shared
    assert torch.equal(out, want)


def _ep_worker(rank, world, port, q, token_level):
    import sys

    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import torch.distributed as dist

    from maxuna_b200.ep import make_gpu_ep_block
    from maxuna_b200.moe import MoeBlock

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    full = MoeBlock.random(256, 512, 8, 3, seed=51, device=dev, weight_std=0.25)  # same seed on every rank
    ep = make_gpu_ep_block(full.router, full.exp_probs_b, full.shard(rank, world), 8, 3, token_level=token_level)
    gen = torch.Generator(device=dev)
    gen.manual_seed(7)
    x_all = torch.randn(2 * 96, 256, generator=gen, device=dev)
    x = x_all[rank * 96:(rank + 1) * 96].contiguous()
    out = ep.forward(x)
    ref = full.forward(x_all)[rank * 96:(rank + 1) * 96]
    torch.cuda.synchronize()
    err = float((out - ref).norm() / ref.norm())
    ids, _ = ep.route_fn(x)
    pairs = int(torch.zeros(96, world, dtype=torch.bool, device=dev).scatter_(1, ids.to(torch.int64) // (8 // world), True).sum())
    q.put((rank, err, ep.last_stats, pairs))
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("token_level", [False, True])
def test_expert_parallel_two_gpus(token_level):
    import torch.multiprocessing as mp

    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_ep_worker, args=(r, 2, port, q, token_level)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, err, stats, pairs in res:
        assert err < 1e-5, (rank, err)  # same f16 operands; the token-level sum is grouped by rank (f32 rounding)
        assert stats["rows_sent"] == (pairs if token_level else 96 * 3)


# ---- expert-parallel batched decode (BASELINE config 5) ------------------------------------------------------
@pytest.mark.parametrize("world,t_loc", [(2, 8), (4, 4), (8, 8)])
def test_ep_decode_ranks_emulated_on_one_gpu(orc, dev, world, t_loc):
    """The per-rank pieces of the expert-parallel decode step, with the ranks run one after the other on one
    GPU (no collective: the gathered batch and the returned partial rows are plain slices): routing of all
    tokens, id localisation, `lmoe_experts_forward_ep` on every shard with the shared expert for the shard's
    own tokens, rank-order sum + residual.  Against the oracle on the whole batch; ids bit for bit."""
    from maxuna_b200 import ops
    from maxuna_b200._native import check, lib
    from maxuna_b200.gguf import stream_ptr
    from maxuna_b200.moe import MoeBlock

    hidden, ne, k = 512, 32, 4      # every shard keeps at least top_k experts, so its handle has the block's top_k
    full = MoeBlock.random(hidden, 512, ne, k, seed=71, device=dev, weight_std=0.2)
    host = full.host_layer(orc)
    t = world * t_loc
    rng = np.random.default_rng(72)
    ffn_inp = (rng.standard_normal((t, hidden)) * 2).astype(np.float32)
    g = rng.uniform(0.5, 1.5, hidden).astype(np.float32)
    inp = torch.from_numpy(ffn_inp).to(dev)
    gw = torch.from_numpy(g).to(dev)
    normed = torch.empty_like(inp)
    check(lib().lmoe_rms_norm(inp.data_ptr(), gw.data_ptr(), 1e-6, t, hidden, normed.data_ptr(), stream_ptr()))
    ids, w = ops.route(full.router, full.exp_probs_b, normed, k, 2.5, True)
    e_local = ne // world
    parts = []
    for r in range(world):
        shard = full.shard(r, world)
        lids = torch.empty_like(ids)
        check(lib().lmoe_ep_localize_ids(ids.data_ptr(), ids.numel(), r * e_local, e_local, lids.data_ptr(), stream_ptr()))
        want_l = torch.where((ids // e_local) == r, ids - r * e_local, e_local)
        assert torch.equal(lids, want_l.to(torch.int32))
        part = torch.empty(t, hidden, device=dev)
        n = lib().lmoe_experts_workspace_bytes(shard.handle, t)
        ws = torch.full((n,), 0xFF, dtype=torch.uint8, device=dev)
        check(lib().lmoe_experts_forward_ep(shard.handle, normed.data_ptr(), lids.data_ptr(), w.data_ptr(), t, r * t_loc, t_loc,
                                            part.data_ptr(), ws.data_ptr(), n, stream_ptr()))
        torch.cuda.synchronize()
        check(lib().lmoe_check_device_flag(ws.data_ptr(), stream_ptr()))
        parts.append(part)
    out = torch.empty(t, hidden, device=dev)
    pos = (torch.arange(world, dtype=torch.int32, device=dev)[None, :] * t_loc +
           torch.arange(t_loc, dtype=torch.int32, device=dev)[:, None]).contiguous()
    for s_ in range(world):       # what rank s receives: chunk s of every rank's partial rows
        recv = torch.cat([p[s_ * t_loc:(s_ + 1) * t_loc] for p in parts]).contiguous()
        res = inp[s_ * t_loc:(s_ + 1) * t_loc].contiguous()
        o = torch.empty(t_loc, hidden, device=dev)
        check(lib().lmoe_ep_combine(recv.data_ptr(), pos.data_ptr(), res.data_ptr(), t_loc, world, hidden, o.data_ptr(), stream_ptr()))
        out[s_ * t_loc:(s_ + 1) * t_loc] = o
    torch.cuda.synchronize()
    ffn_out, ids_o, _ = host.forward(orc.rms_norm(ffn_inp, g, 1e-6))
    assert np.array_equal(ids.cpu().numpy().astype(np.uint32), ids_o)
    assert orc.rel_l2(out.cpu().numpy(), ffn_inp + ffn_out) < 2e-3
    # and against the single-GPU layer entry: the same kernels, sums grouped by rank instead of by slot
    single = full.layer_forward(inp, gw, 1e-6)
    torch.cuda.synchronize()
    assert float((out - single).norm() / single.norm()) < 1e-5


def _ep_decode_worker(rank, world, port, q, peer=False):
    import sys

    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import torch.distributed as dist

    from maxuna_b200.ep import make_gpu_ep_decode
    from maxuna_b200.moe import MoeBlock

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    n_layers, t_loc, hidden = 3, 32, 512
    fulls = [MoeBlock.random(hidden, 512, 16, 4, seed=81 + i, device=dev, weight_std=0.2) for i in range(n_layers)]
    gen = torch.Generator(device=dev)
    gen.manual_seed(9)
    norms = [0.5 + torch.rand(hidden, generator=gen, device=dev) for _ in fulls]
    px = None
    if peer:
        from maxuna_b200.ep import PeerExchange
        px = PeerExchange(t_loc, hidden)
    steps = [make_gpu_ep_decode(f.router, f.exp_probs_b, nw, f.shard(rank, world), 16, 4, exchange=px) for f, nw in zip(fulls, norms)]
    x_all = torch.randn(world * t_loc, hidden, generator=gen, device=dev)
    x = x_all[rank * t_loc:(rank + 1) * t_loc].contiguous()
    ref = x.clone()
    err0 = None
    for step, f, nw in zip(steps, fulls, norms):
        x = step.forward(x)
        ref = f.layer_forward(ref, nw, 1e-6)
        if err0 is None:          # first layer: identical inputs on both paths
            torch.cuda.synchronize()
            err0 = float((x - ref).norm() / ref.norm())
            moved = float((x - x_all[rank * t_loc:(rank + 1) * t_loc]).norm() / x.norm())   # the block's share of the output
    torch.cuda.synchronize()
    if px is not None:
        assert px.timed_out() == 0
        px.close()
    q.put((rank, err0, float((x - ref).norm() / ref.norm()), moved))
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("peer", [False, True])
def test_expert_parallel_decode_two_gpus(peer):
    """A three-layer residual stack, 64 sequences over two ranks, against the single-GPU layer entry; with NCCL
    collectives, and with both exchanges as stores into the other rank's memory (`PeerExchange`)."""
    import torch.multiprocessing as mp

    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_ep_decode_worker, args=(r, 2, port, q, peer)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, err0, err, moved in res:
        assert moved > 1e-2, (rank, moved)  # the block's output is a visible part of what is compared
        assert err0 < 1e-5, (rank, err0)   # same kernels on the same inputs; the sum is grouped by rank: f32 rounding
        assert err < 2e-3, (rank, err)     # later layers see inputs that differ in the last bits (a near-tie may re-route)


def _ep_prefill_worker(rank, world, port, q, waves):
    import sys

    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import torch.distributed as dist

    from maxuna_b200.ep import make_gpu_ep_prefill
    from maxuna_b200.moe import MoeBlock

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    full = MoeBlock.random(256, 512, 8, 3, seed=51, device=dev, weight_std=0.25)  # same seed on every rank
    ep = make_gpu_ep_prefill(full.router, full.exp_probs_b, full.shard(rank, world), 8, 3, waves=waves)
    gen = torch.Generator(device=dev)
    gen.manual_seed(7)
    x_all = torch.randn(world * 130, 256, generator=gen, device=dev)
    x = x_all[rank * 130:(rank + 1) * 130].contiguous()
    out = ep.forward(x)
    ref = full.forward(x_all, path="prefill")[rank * 130:(rank + 1) * 130]
    torch.cuda.synchronize()
    q.put((rank, float((out - ref).norm() / ref.norm()), ep.last_stats))
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("waves", [1, 3])
def test_expert_parallel_prefill_two_gpus(waves):
    import torch.multiprocessing as mp

    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_ep_prefill_worker, args=(r, 2, port, q, waves)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, err, stats in res:
        assert err < 1e-5, (rank, err)  # same f16 operands; the sum is grouped by rank (f32 rounding)
        assert stats["waves"] == waves
