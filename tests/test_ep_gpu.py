"""Expert-parallel pieces on the GPU: the row-level entry points on one device, and the
two-rank NCCL exchange (needs two GPUs; skipped otherwise) against the single-GPU block."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


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


def _ep_worker(rank, world, port, q):
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
    ep = make_gpu_ep_block(full.router, full.exp_probs_b, full.shard(rank, world), 8, 3)
    gen = torch.Generator(device=dev)
    gen.manual_seed(7)
    x_all = torch.randn(2 * 96, 256, generator=gen, device=dev)
    x = x_all[rank * 96:(rank + 1) * 96].contiguous()
    out = ep.forward(x)
    ref = full.forward(x_all)[rank * 96:(rank + 1) * 96]
    torch.cuda.synchronize()
    err = float((out - ref).norm() / ref.norm())
    q.put((rank, err, ep.last_stats))
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_expert_parallel_two_gpus():
    import torch.multiprocessing as mp

    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_ep_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, err, stats in res:
        assert err < 1e-5, (rank, err)  # same f16 operands, same per-element accumulation order
        assert stats["rows_sent"] == 96 * 3
