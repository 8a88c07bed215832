"""Expert-parallel host logic on two CPU ranks (gloo): dispatch plan, the two exchanges and the
slot-order combine, with the CPU oracle standing in for the CUDA expert kernels."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _layer(orc, seed=3, hidden=256, ff=256, ne=8, top_k=3):
    rng = np.random.default_rng(seed)
    q = lambda dt, shape: orc.quantize(dt, rng.uniform(-0.5, 0.5, shape).astype(np.float32))
    return orc.HostLayer(hidden, ff, ne, top_k, router=(rng.standard_normal((ne, hidden)) * 0.1).astype(np.float32),
                         bias=rng.uniform(-0.1, 0.1, ne).astype(np.float32), gate=q(orc.Q4_K, (ne, ff, hidden)),
                         up=q(orc.Q4_K, (ne, ff, hidden)), down=q(orc.Q6_K, (ne, hidden, ff)),
                         sh_gate=q(orc.Q4_K, (ff, hidden)), sh_up=q(orc.Q4_K, (ff, hidden)), sh_down=q(orc.Q6_K, (hidden, ff)))


def _worker(rank, world, port, q, token_level=False):
    import sys

    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    from maxuna_b200.ep import ExpertParallelMoe
    from oracle import oracle as orc

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    L = _layer(orc)
    ne_local = L.n_expert // world
    gexp, dexp = L.gate.size // L.n_expert, L.down.size // L.n_expert
    lo, hi = rank * ne_local, (rank + 1) * ne_local
    # this rank's shard: local experts only (no shared expert inside; it is applied by shared_fn)
    shard = orc.HostLayer(L.hidden, L.expert_ff, ne_local, 1, L.router[lo:hi], None, L.gate[lo * gexp:hi * gexp],
                          L.up[lo * gexp:hi * gexp], L.down[lo * dexp:hi * dexp])
    shared_only = orc.HostLayer(L.hidden, L.expert_ff, 1, 1, L.router[:1], None, L.sh_gate, L.sh_up, L.sh_down)

    def route_fn(x):
        ids, w = orc.route(L.router, L.bias, x.numpy(), L.top_k, L.scale, L.norm)
        return torch.from_numpy(ids.astype(np.int32)), torch.from_numpy(w)

    def rows_fn(x, ids, w):
        xn, idn = x.numpy(), ids.numpy().astype(np.uint32).reshape(-1, 1)
        down = orc.mul_id(orc.Q6_K, shard.down, ne_local, L.hidden, L.expert_ff,
                          orc.silu_mul(orc.mul_id(orc.Q4_K, shard.gate, ne_local, L.expert_ff, L.hidden, xn[:, None, :], idn),
                                       orc.mul_id(orc.Q4_K, shard.up, ne_local, L.expert_ff, L.hidden, xn[:, None, :], idn)),
                          idn)
        return torch.from_numpy(down[:, 0, :] * w.numpy()[:, None])

    def shared_fn(x):
        xn = x.numpy()
        z = np.zeros((xn.shape[0], 1), np.uint32)
        d = orc.mul_id(orc.Q6_K, shared_only.down, 1, L.hidden, L.expert_ff,
                       orc.silu_mul(orc.mul_id(orc.Q4_K, shared_only.gate, 1, L.expert_ff, L.hidden, xn[:, None, :], z),
                                    orc.mul_id(orc.Q4_K, shared_only.up, 1, L.expert_ff, L.hidden, xn[:, None, :], z)), z)
        return torch.from_numpy(d[:, 0, :])

    def tokens_fn(x, ids, w):
        # the token-level form out of the row-level one: expand the non-empty slots, sum them back in slot order
        tok, slot = torch.nonzero(ids < ne_local, as_tuple=True)
        y = rows_fn(x[tok], ids[tok, slot], w[tok, slot])
        out = torch.zeros(x.shape[0], L.hidden)
        for s_ in range(ids.shape[1]):
            m = slot == s_
            out.index_add_(0, tok[m], y[m])
        return out

    ep = ExpertParallelMoe(route_fn, rows_fn, shared_fn, L.n_expert, L.top_k, payload_dtype=torch.float32,
                           tokens_fn=tokens_fn if token_level else None)
    rng = np.random.default_rng(100 + rank)
    t = 5 + 3 * rank  # ragged token counts per rank
    x = rng.standard_normal((t, L.hidden)).astype(np.float32)
    out = ep.forward(torch.from_numpy(x)).numpy()
    want, _, _ = L.forward(x)
    err = orc.rel_l2(out, want)
    # plan sanity: every row goes to the rank that owns its expert
    ids, _ = route_fn(torch.from_numpy(x))
    order, counts = ep.plan(ids)
    dest = (ids.reshape(-1).to(torch.int64) // ne_local)[order]
    ok_sorted = bool(torch.all(dest[1:] >= dest[:-1])) and int(counts.sum()) == t * L.top_k
    # token-level plan: one (token, rank) pair per rank that owns at least one of the token's experts
    tok, dst, tcounts = ep.plan_tokens(ids)
    want_pairs = sorted({(int(e) // ne_local, i) for i in range(t) for e in ids[i].tolist()})
    ok_sorted = ok_sorted and list(zip(dst.tolist(), tok.tolist())) == want_pairs
    ok_sorted = ok_sorted and tcounts.tolist() == [sum(1 for g, _ in want_pairs if g == r) for r in range(world)]
    q.put((rank, err, ok_sorted, ep.last_stats, len(want_pairs)))
    dist.destroy_process_group()


@pytest.mark.parametrize("token_level,world", [(False, 2), (True, 2), (True, 4)])
def test_expert_parallel_cpu_ranks(orc, token_level, world):
    orc.build()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q, token_level)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, err, ok_sorted, stats, n_pairs in res:
        assert err < 1e-5, (rank, err)
        assert ok_sorted
        assert stats["rows_sent"] == (n_pairs if token_level else (5 + 3 * rank) * 3)


def _prefill_worker(rank, world, port, q, waves):
    import sys

    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    from maxuna_b200.ep import ExpertParallelPrefill
    from oracle import oracle as orc

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    L = _layer(orc)
    ne_local = L.n_expert // world
    gexp, dexp = L.gate.size // L.n_expert, L.down.size // L.n_expert
    lo, hi = rank * ne_local, (rank + 1) * ne_local
    shard = orc.HostLayer(L.hidden, L.expert_ff, ne_local, L.top_k, L.router[lo:hi], None, L.gate[lo * gexp:hi * gexp],
                          L.up[lo * gexp:hi * gexp], L.down[lo * dexp:hi * dexp])
    shared_only = orc.HostLayer(L.hidden, L.expert_ff, 1, 1, L.router[:1], None, L.sh_gate, L.sh_up, L.sh_down)

    def route_fn(x):
        ids, w = orc.route(L.router, L.bias, x.numpy(), L.top_k, L.scale, L.norm)
        return torch.from_numpy(ids.astype(np.int32)), torch.from_numpy(w)

    def localize_fn(ids, first, count):
        e = ids.to(torch.int64) - first
        return torch.where((e >= 0) & (e < count), e, torch.full_like(e, count)).to(torch.int32)

    def tokens_fn(x, ids_local, w):
        return torch.from_numpy(shard.experts_forward(x.numpy(), ids_local.numpy().astype(np.uint32), w.numpy()))

    def shared_fn(x):
        n = x.shape[0]
        return torch.from_numpy(shared_only.experts_forward(x.numpy(), np.zeros((n, 1), np.uint32), np.ones((n, 1), np.float32)))

    def sum_fn(parts, shared):
        n = parts.shape[0] // world
        out = torch.zeros(n, parts.shape[1])
        for s_ in range(world):
            out += parts[s_ * n:(s_ + 1) * n]
        return out if shared is None else out + shared

    ep = ExpertParallelPrefill(route_fn, localize_fn, tokens_fn, shared_fn, sum_fn, L.n_expert, L.top_k,
                               payload_dtype=torch.float32, waves=waves)
    t_loc = 11                                            # the same count on every rank; not a multiple of the waves
    x = np.random.default_rng(300 + rank).standard_normal((t_loc, L.hidden)).astype(np.float32)
    out = ep.forward(torch.from_numpy(x)).numpy()
    want, _, _ = L.forward(x)
    q.put((rank, orc.rel_l2(out, want), ep.last_stats))
    dist.destroy_process_group()


@pytest.mark.parametrize("world,waves", [(2, 1), (2, 3), (4, 2)])
def test_expert_parallel_prefill_fixed_size_exchange(orc, world, waves):
    """`ExpertParallelPrefill`: every rank receives every token (all-gather), keeps the slots of its own experts,
    returns one partial row per token (all-to-all); no counts travel and nothing is read back on the host."""
    orc.build()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_prefill_worker, args=(r, world, port, q, waves)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, err, stats in res:
        assert err < 1e-5, (rank, err)
        assert stats["waves"] == waves and stats["tokens_gathered"] == world * 11
