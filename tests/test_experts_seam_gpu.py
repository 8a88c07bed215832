"""`lmoe_experts_forward` = the `ExpertFfn::forward` seam of the reference (src/moe.rs:19-21): the routed
experts on a routing decision made by the CALLER.  Checked against the oracle's restatement of
`ReferenceExperts::forward` (src/moe.rs:142-187) with ids the router would not have picked, with empty
slots, and - on the mat-vec path, like the reference's own mul_mv_id cases (src/ops/mv_id.rs:100-203) -
with the same expert more than once in a row.  Bound: 2e-3 relative L2."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available()
    return torch.device("cuda:0")


@pytest.fixture(scope="module")
def small(orc, dev):
    from maxuna_b200.moe import MoeBlock

    blk = MoeBlock.random(512, 512, 16, 4, seed=41, device=dev, weight_std=0.2)
    return blk, blk.host_layer(orc)


def _run(orc, blk, host, x, ids, w, add_shared=False):
    dev = blk.router.device
    idd = torch.from_numpy(np.ascontiguousarray(ids).view(np.int32)).to(dev)      # the u32 bits in int32 storage
    out = blk.experts_forward(torch.from_numpy(x).to(dev), idd, torch.from_numpy(w).to(dev), add_shared)
    torch.cuda.synchronize()
    blk.check_device_flag()
    want = host.experts_forward(x, ids, w)
    if add_shared:
        full, _, _ = host.forward(x)                     # routed (router's own choice) + shared
        routed_own = host.experts_forward(x, *orc.route(host.router, host.bias, x, host.top_k))
        want = want + (full - routed_own)                # the shared expert's rows (to f32 rounding)
    return out.cpu().numpy(), want


@pytest.mark.parametrize("t", [1, 2, 5, 40, 64])
def test_matvec_path_any_ids(orc, small, t):
    blk, host = small
    rng = np.random.default_rng(100 + t)
    x = rng.standard_normal((t, 512)).astype(np.float32)
    ids = orc.distinct_ids(t, 4, 16, 0x70 + t)
    w = rng.uniform(0.1, 1.0, (t, 4)).astype(np.float32)
    got, want = _run(orc, blk, host, x, ids, w)
    assert orc.rel_l2(got, want) < 2e-3


def test_matvec_path_repeats_and_empty_slots(orc, small):
    blk, host = small
    rng = np.random.default_rng(7)
    t = 9
    x = rng.standard_normal((t, 512)).astype(np.float32)
    ids = orc.random_ids(t, 4, 16, 0x33)                  # repeats inside a row are likely and allowed here
    ids[0] = [3, 3, 3, 3]
    ids[1] = [16, 5, 0xFFFFFFFF, 5]                       # two empty slots (id >= n_expert), one expert twice
    ids[2] = [16, 16, 16, 16]                             # a token with no expert at all -> a zero row
    w = rng.uniform(0.1, 1.0, (t, 4)).astype(np.float32)
    got, want = _run(orc, blk, host, x, ids, w)
    assert np.all(got[2] == 0.0)
    assert orc.rel_l2(got, want) < 2e-3


@pytest.mark.parametrize("t", [65, 300])
def test_grouped_path_distinct_ids_and_empty_slots(orc, small, t):
    blk, host = small
    rng = np.random.default_rng(200 + t)
    x = rng.standard_normal((t, 512)).astype(np.float32)
    ids = orc.distinct_ids(t, 4, 16, 0x90 + t)
    ids[::7, 1] = 16                                      # some empty slots
    ids[5] = 16                                           # and a token without experts
    w = rng.uniform(0.1, 1.0, (t, 4)).astype(np.float32)
    got, want = _run(orc, blk, host, x, ids, w)
    assert np.all(got[5] == 0.0)
    assert orc.rel_l2(got, want) < 2e-3


@pytest.mark.parametrize("t", [3, 100])
def test_with_shared_expert(orc, small, t):
    blk, host = small
    rng = np.random.default_rng(300 + t)
    x = rng.standard_normal((t, 512)).astype(np.float32)
    ids = orc.distinct_ids(t, 4, 16, 0xA0 + t)
    w = rng.uniform(0.1, 1.0, (t, 4)).astype(np.float32)
    got, want = _run(orc, blk, host, x, ids, w, add_shared=True)
    assert orc.rel_l2(got, want) < 2e-3


@pytest.mark.parametrize("t", [1, 7, 130])
def test_router_ids_through_the_seam_equal_the_block(orc, small, t):
    """route() + experts_forward(add_shared) is `MoeBlock::forward` (src/moe.rs:73-78): with the router's own
    decision the seam runs the same kernels on the same lists, so the result is bit-identical to the block's."""
    blk, _ = small
    dev = blk.router.device
    x = torch.randn(t, 512, device=dev)
    ids, w = blk.route(x)
    a = blk.experts_forward(x, ids, w, add_shared=True)
    b = blk.forward(x)
    torch.cuda.synchronize()
    assert torch.equal(a, b)


@pytest.mark.parametrize("t", [8, 96])
def test_production_shape(orc, dev, t):
    from maxuna_b200.moe import MoeBlock

    blk = MoeBlock.random(3072, 1024, 256, 10, seed=3, device=dev)
    host = blk.host_layer(orc)
    rng = np.random.default_rng(400 + t)
    x = rng.standard_normal((t, 3072)).astype(np.float32)
    ids = orc.distinct_ids(t, 10, 256, 0xB0 + t)
    w = rng.uniform(0.05, 0.5, (t, 10)).astype(np.float32)
    got, want = _run(orc, blk, host, x, ids, w)
    assert orc.rel_l2(got, want) < 2e-3


def test_argument_errors(small, dev):
    from maxuna_b200 import LmoeError

    blk, _ = small
    x = torch.zeros(3, 512, device=dev)
    with pytest.raises(LmoeError):
        blk.experts_forward(x, torch.zeros(3, 3, dtype=torch.int32, device=dev), torch.zeros(3, 3, device=dev))
    with pytest.raises(LmoeError):
        blk.experts_forward(torch.zeros(3, 256, device=dev), torch.zeros(3, 4, dtype=torch.int32, device=dev),
                            torch.zeros(3, 4, device=dev))
    torch.cuda.synchronize()
