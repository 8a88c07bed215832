"""Host logic of the expert-parallel decode step (`ExpertParallelDecode`) on 2 and 4 CPU ranks (gloo), with
the CPU oracle standing in for the CUDA entry points: all-gather of the normed rows, replicated routing,
local experts for all tokens + shared expert for the rank's own, all-to-all of the partial rows, rank-order
sum + residual.  A short residual stack of layers is compared with the oracle's single-process stack."""
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


def _layer(orc, seed, hidden=256, ff=256, ne=8, top_k=3):
    rng = np.random.default_rng(seed)
    q = lambda dt, shape: orc.quantize(dt, rng.uniform(-0.5, 0.5, shape).astype(np.float32))
    return orc.HostLayer(hidden, ff, ne, top_k, router=(rng.standard_normal((ne, hidden)) * 0.1).astype(np.float32),
                         bias=rng.uniform(-0.1, 0.1, ne).astype(np.float32), gate=q(orc.Q4_K, (ne, ff, hidden)),
                         up=q(orc.Q4_K, (ne, ff, hidden)), down=q(orc.Q6_K, (ne, hidden, ff)),
                         sh_gate=q(orc.Q4_K, (ff, hidden)), sh_up=q(orc.Q4_K, (ff, hidden)), sh_down=q(orc.Q6_K, (hidden, ff)))


class _HostExchange:
    """What `PeerExchange` does, on the host: `gather` / `scatter` with the same shapes and slot order, over gloo."""

    def __init__(self, world):
        self.world = world

    def gather(self, x):
        out = torch.empty(self.world * x.shape[0], x.shape[1], dtype=x.dtype)
        dist.all_gather_into_tensor(out, x.contiguous())
        return out

    def scatter(self, parts):
        out = torch.empty_like(parts)
        dist.all_to_all_single(out, parts.contiguous())
        return out


def _worker(rank, world, port, q, exchange=False):
    import sys

    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    from maxuna_b200.ep import ExpertParallelDecode
    from oracle import oracle as orc

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    n_layers, t_loc, hidden = 3, 4, 256
    layers = [_layer(orc, 40 + i) for i in range(n_layers)]
    norms = [np.random.default_rng(60 + i).uniform(0.5, 1.5, hidden).astype(np.float32) for i in range(n_layers)]
    steps = []
    for L, g in zip(layers, norms):
        ne_local = L.n_expert // world
        gexp, dexp = L.gate.size // L.n_expert, L.down.size // L.n_expert
        lo, hi = rank * ne_local, (rank + 1) * ne_local
        shard = orc.HostLayer(L.hidden, L.expert_ff, ne_local, L.top_k, L.router[lo:hi], None, L.gate[lo * gexp:hi * gexp],
                              L.up[lo * gexp:hi * gexp], L.down[lo * dexp:hi * dexp])
        shared_only = orc.HostLayer(L.hidden, L.expert_ff, 1, 1, L.router[:1], None, L.sh_gate, L.sh_up, L.sh_down)

        def norm_fn(x, g=g):
            return torch.from_numpy(orc.rms_norm(x.numpy(), g, 1e-6))

        def route_fn(x, L=L):
            ids, w = orc.route(L.router, L.bias, x.numpy(), L.top_k, L.scale, L.norm)
            return torch.from_numpy(ids.astype(np.int32)), torch.from_numpy(w)

        def localize_fn(ids, first, count):
            e = ids.to(torch.int64) - first
            return torch.where((e >= 0) & (e < count), e, torch.full_like(e, count)).to(torch.int32)

        def experts_fn(x, ids_local, w, sh_first, sh_count, shard=shard, shared_only=shared_only):
            xn = x.numpy()
            out = shard.experts_forward(xn, ids_local.numpy().astype(np.uint32), w.numpy())
            own = slice(sh_first, sh_first + sh_count)
            out[own] += shared_only.experts_forward(xn[own], np.zeros((sh_count, 1), np.uint32), np.ones((sh_count, 1), np.float32))
            return torch.from_numpy(out)

        def sum_fn(parts, residual, world=world):
            t = residual.shape[0]
            out = torch.zeros_like(residual)
            for s_ in range(world):                       # rank order
                out += parts[s_ * t:(s_ + 1) * t]
            return out + residual

        steps.append(ExpertParallelDecode(norm_fn, route_fn, localize_fn, experts_fn, sum_fn, L.n_expert,
                                          exchange=_HostExchange(world) if exchange else None))
    # all ranks draw the same batch; each keeps its slice
    x_all = np.random.default_rng(7).standard_normal((world * t_loc, hidden)).astype(np.float32)
    x = torch.from_numpy(x_all[rank * t_loc:(rank + 1) * t_loc].copy())
    for step in steps:
        x = step.forward(x)
    # the single-process reference: x <- x + block(norm(x)) on this rank's tokens
    want = x_all[rank * t_loc:(rank + 1) * t_loc].copy()
    for L, g in zip(layers, norms):
        ffn, _, _ = L.forward(orc.rms_norm(want, g, 1e-6))
        want = want + ffn
    q.put((rank, orc.rel_l2(x.numpy(), want)))
    dist.destroy_process_group()


@pytest.mark.parametrize("world,exchange", [(2, False), (4, False), (2, True)])
def test_expert_parallel_decode_cpu_ranks(orc, world, exchange):
    """The host logic of the expert-parallel decode step on gloo ranks against the single-process oracle; once with
    the exchanges behind the `exchange` object (the seam `PeerExchange` plugs into)."""
    orc.build()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q, exchange)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, err in res:
        assert err < 1e-5, (rank, err)   # same arithmetic per expert; the sum is grouped by rank: f32 rounding only
