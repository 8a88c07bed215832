"""The grouped tensor-core GEMM (`mul_mm_id`) and the prefill block against the CPU oracle.
Cases follow src/ops/mm_id.rs:94-166, 379-437 of the reference; bound rel-L2 < 1e-3 for the
f16-tile path (the reference measures ~2.6e-4 for its own f16 tiles)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DTYPES = [(12, "Q4K"), (14, "Q6K")]


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available()
    return torch.device("cuda:0")


def _case(orc, dev, dt, n_expert, n_out, k, t, top_k, xpr, ids, seed, shared_map=False):
    from maxuna_b200 import ops
    from maxuna_b200.gguf import ExpertStack

    raw = orc.quantize(dt, orc.pseudo_random(n_expert * n_out * k, seed, -1.0, 1.0))
    stack = ExpertStack.from_bytes(raw, dt, n_expert, n_out, k, device=dev)
    x = orc.pseudo_random(t * xpr * k, seed ^ 0xABCD, -1.0, 1.0).reshape(t, xpr, k)
    xd, idd = torch.from_numpy(x).to(dev), torch.from_numpy(ids.astype(np.int32)).to(dev)
    if shared_map:
        got = ops.mul_mm_id_shared(stack, xd, idd, ops.prepare_map0(n_expert, idd))
    else:
        got = ops.mul_mm_id(stack, xd, idd)
    torch.cuda.synchronize()
    assert tuple(got.shape) == (t, top_k, n_out)
    return got.cpu().numpy(), orc.mul_id(dt, raw, n_expert, n_out, k, x, ids)


@pytest.mark.parametrize("dt,name", DTYPES)
@pytest.mark.parametrize("t,top_k,ne,xpr,seed,iseed", [(16, 2, 4, 1, 0x1600, 0x41), (64, 2, 4, 1, 0x6400, 0x42),
                                                      (40, 4, 6, 4, 0x1601, 0x43)])
def test_mm_small(orc, dev, dt, name, t, top_k, ne, xpr, seed, iseed):
    ids = orc.distinct_ids(t, top_k, ne, iseed)
    got, want = _case(orc, dev, dt, ne, 8, 256, t, top_k, xpr, ids, seed)
    assert orc.rel_l2(got, want) < 1e-3


@pytest.mark.parametrize("dt,name", DTYPES)
def test_mm_production_scale(orc, dev, dt, name):
    # 256 experts, top-10, a 512-token chunk; both activation layouts (src/ops/mm_id.rs:121-166)
    ids = orc.distinct_ids(512, 10, 256, 0x52)
    for xpr, seed in ((1, 0x53), (10, 0x54)):
        got, want = _case(orc, dev, dt, 256, 64, 256, 512, 10, xpr, ids, seed)
        assert orc.rel_l2(got, want) < 1e-3


@pytest.mark.parametrize("dt,name", DTYPES)
def test_mm_ragged_rows_multi_block_k_and_big_expert(orc, dev, dt, name):
    # n_out = 200 (two weight tiles, ragged), k = 768, one expert taking > 256 rows (two row tiles)
    t, top_k, ne = 300, 2, 3
    ids = np.stack([np.zeros(t, np.uint32), 1 + (np.arange(t) % 2).astype(np.uint32)], axis=1)
    got, want = _case(orc, dev, dt, ne, 200, 768, t, top_k, 1, ids, 0x77)
    assert orc.rel_l2(got, want) < 1e-3


def test_mm_shared_map0_bitwise_equals_self_contained(orc, dev):
    ids = orc.distinct_ids(96, 4, 8, 0x61)
    a, _ = _case(orc, dev, 12, 8, 64, 512, 96, 4, 1, ids, 0x62, shared_map=False)
    b, _ = _case(orc, dev, 12, 8, 64, 512, 96, 4, 1, ids, 0x62, shared_map=True)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


def test_mm_errors_not_faults(orc, dev):
    from maxuna_b200 import LmoeError, ops
    from maxuna_b200.gguf import ExpertStack

    raw = orc.quantize(12, orc.pseudo_random(4 * 8 * 256, 1, -1.0, 1.0))
    stack = ExpertStack.from_bytes(raw, 12, 4, 8, 256, device=dev)
    ids = torch.zeros(2, 2, dtype=torch.int32, device=dev)
    with pytest.raises(LmoeError):
        ops.mul_mm_id(stack, torch.zeros(2, 1, 128, device=dev), ids)
    scratch = ops.prepare_map0(4, ids)
    with pytest.raises(LmoeError):  # scratch laid out for another geometry
        ops.mul_mm_id_shared(stack, torch.zeros(3, 1, 256, device=dev), torch.zeros(3, 2, dtype=torch.int32, device=dev), scratch)
    assert ops.supported(12, 10) and ops.supported(14, 10) and not ops.supported(8, 10)
    torch.cuda.synchronize()


def _check_block(orc, blk, host, x, tol):
    xd = torch.from_numpy(x).to(blk.router.device)
    out, ids, w = blk.forward(xd, return_routing=True, path="prefill")
    torch.cuda.synchronize()
    blk.check_device_flag()
    want, ids_o, w_o = host.forward(x)
    assert np.array_equal(ids.cpu().numpy().astype(np.uint32), ids_o)
    assert np.array_equal(w.cpu().numpy().view(np.uint32), w_o.view(np.uint32))
    err = orc.rel_l2(out.cpu().numpy(), want)
    assert err < tol, err
    return err


def test_prefill_block_tiny(orc, dev):
    from maxuna_b200.moe import MoeBlock

    blk = MoeBlock.random(256, 256, 8, 3, seed=21, device=dev, weight_std=0.25)
    host = blk.host_layer(orc)
    rng = np.random.default_rng(22)
    for t in (32, 33, 100, 300):
        _check_block(orc, blk, host, rng.standard_normal((t, 256)).astype(np.float32), 2e-3)
    # the op-by-op sequence of the reference (mm_id + rescale + combine) agrees too
    x = rng.standard_normal((64, 256)).astype(np.float32)
    want, _, _ = host.forward(x)
    got = blk.forward_unfused(torch.from_numpy(x).to(dev), use_mm=True).cpu().numpy()
    assert orc.rel_l2(got, want) < 2e-3


def test_prefill_block_wide_ff(orc, dev):
    # expert_ff = 512: two Q6_K super-blocks per down row (the 256-row down kernel), ragged row tiles
    from maxuna_b200.moe import MoeBlock

    blk = MoeBlock.random(256, 512, 6, 2, seed=31, device=dev, weight_std=0.25)
    host = blk.host_layer(orc)
    rng = np.random.default_rng(32)
    for t in (40, 700):
        _check_block(orc, blk, host, rng.standard_normal((t, 256)).astype(np.float32), 2e-3)


def test_prefill_block_production_shape(orc, dev):
    from maxuna_b200.moe import MoeBlock

    blk = MoeBlock.random(3072, 1024, 256, 10, seed=2, device=dev)
    host = blk.host_layer(orc)
    x = np.random.default_rng(23).standard_normal((48, 3072)).astype(np.float32)
    _check_block(orc, blk, host, x, 2e-3)
