"""The FFN half of a layer around the block (`lmoe_rms_norm`, `lmoe_moe_layer_forward`; src/model.rs:340-350)
against the oracle: the norm bit-exact (it feeds the router), the layer output within the block's bound."""
import numpy as np
import pytest
import torch


def test_oracle_rms_norm_matches_float64_formula(orc):
    orc.build()
    rng = np.random.default_rng(21)
    x = (rng.standard_normal((7, 3072)) * rng.uniform(0.1, 30, (7, 1))).astype(np.float32)
    w = rng.uniform(0.5, 1.5, 3072).astype(np.float32)
    got = orc.rms_norm(x, w, 1e-6)
    x64 = x.astype(np.float64)
    want = x64 / np.sqrt((x64 * x64).mean(axis=1, keepdims=True) + 1e-6) * w
    assert np.max(np.abs(got - want) / (np.abs(want) + 1e-12)) < 1e-6


@pytest.mark.gpu
@pytest.mark.parametrize("t,hidden", [(1, 256), (5, 260), (19, 3072), (300, 512)])
def test_rms_norm_bit_exact(orc, t, hidden):
    from maxuna_b200._native import check, lib
    from maxuna_b200.gguf import stream_ptr

    orc.build()
    rng = np.random.default_rng(22 + t)
    x = (rng.standard_normal((t, hidden)) * 3).astype(np.float32)
    w = rng.uniform(0.5, 1.5, hidden).astype(np.float32)
    xd, wd = torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda()
    out = torch.empty_like(xd)
    check(lib().lmoe_rms_norm(xd.data_ptr(), wd.data_ptr(), 1e-6, t, hidden, out.data_ptr(), stream_ptr()))
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy().view(np.uint32), orc.rms_norm(x, w, 1e-6).view(np.uint32))


@pytest.mark.gpu
@pytest.mark.parametrize("t", [1, 3, 17, 40, 64, 65, 200])   # 65 and 200 take the grouped-GEMM branch
def test_layer_forward_matches_oracle(orc, t):
    from maxuna_b200.moe import MoeBlock

    orc.build()
    dev = torch.device("cuda:0")
    blk = MoeBlock.random(256, 512, 8, 3, seed=61, device=dev, weight_std=0.25)
    host = blk.host_layer(orc)
    rng = np.random.default_rng(62 + t)
    ffn_inp = (rng.standard_normal((t, 256)) * 2).astype(np.float32)
    g = rng.uniform(0.5, 1.5, 256).astype(np.float32)
    out, ids, w = blk.layer_forward(torch.from_numpy(ffn_inp).to(dev), torch.from_numpy(g).to(dev), 1e-6,
                                    return_routing=True)
    torch.cuda.synchronize()
    blk.check_device_flag()
    normed = orc.rms_norm(ffn_inp, g, 1e-6)
    ffn_out, ids_o, w_o = host.forward(normed)
    assert np.array_equal(ids.cpu().numpy().astype(np.uint32), ids_o)
    assert np.array_equal(w.cpu().numpy().view(np.uint32), w_o.view(np.uint32))
    assert orc.rel_l2(out.cpu().numpy() - ffn_inp, ffn_out) < 2e-3
    assert orc.rel_l2(out.cpu().numpy(), ffn_inp + ffn_out) < 2e-3


@pytest.mark.gpu
def test_layer_forward_argument_errors():
    from maxuna_b200._native import LmoeError
    from maxuna_b200.moe import MoeBlock

    dev = torch.device("cuda:0")
    blk = MoeBlock.random(256, 256, 8, 3, seed=63, device=dev)
    with pytest.raises(LmoeError):
        blk.layer_forward(torch.zeros(2, 128, device=dev), torch.ones(128, device=dev))


@pytest.mark.gpu
@pytest.mark.parametrize("t", [4, 40, 130])
def test_stack_of_layers_matches_oracle(orc, t):
    """A short residual stack (the shape of BASELINE config 5 at toy size): x <- x + block_l(norm_l(x))."""
    from maxuna_b200.moe import MoeBlock

    orc.build()
    dev = torch.device("cuda:0")
    rng = np.random.default_rng(70 + t)
    layers = [MoeBlock.random(256, 256, 8, 3, seed=80 + i, device=dev, weight_std=0.25) for i in range(3)]
    norms = [rng.uniform(0.5, 1.5, 256).astype(np.float32) for _ in layers]
    x0 = rng.standard_normal((t, 256)).astype(np.float32)
    x = torch.from_numpy(x0).to(dev)
    want = x0.copy()
    for i, (blk, g) in enumerate(zip(layers, norms)):
        x, ids, _ = blk.layer_forward(x, torch.from_numpy(g).to(dev), 1e-6, return_routing=True)
        host = blk.host_layer(orc)
        ffn_out, ids_o, _ = host.forward(orc.rms_norm(want, g, 1e-6))
        if i == 0:      # later layers see inputs that differ in the last bits, so only the values are compared
            assert np.array_equal(ids.cpu().numpy().astype(np.uint32), ids_o)
        want = want + ffn_out
    torch.cuda.synchronize()
    assert orc.rel_l2(x.cpu().numpy(), want) < 2e-3
