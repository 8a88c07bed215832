"""Parity at the sizes the benchmark quotes (BASELINE configs 3 and 5, production shape: hidden 3072,
256 experts + shared, top-10, Q4_K gate/up, Q6_K down) and the edge cases around them.

The CPU oracle cannot run 4096 tokens in seconds, so the routing decision is compared for EVERY token
(ids and weights bit for bit) and the block output for a sample of tokens that includes rows of the most
loaded experts; a token's result does not depend on the other tokens of the call, so the oracle run on
the sample alone is the reference for those rows.  Bound: 2e-3 relative L2, like every block test."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

H, F, E, K = 3072, 1024, 256, 10


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available()
    return torch.device("cuda:0")


def _near_ties(orc, host, x, k, eps=1e-6):
    """Tokens whose k-th and (k+1)-th selection scores, evaluated in float64 from the oracle's logits,
    lie closer than `eps`: the ones where f32 noise in another implementation could change the top-k."""
    logits = orc.route_logits(host.router, x).astype(np.float64)
    sel = 1.0 / (1.0 + np.exp(-logits)) + (0.0 if host.bias is None else host.bias.astype(np.float64))
    part = -np.sort(-sel, axis=1)
    return int(np.count_nonzero(part[:, k - 1] - part[:, k] < eps))


def _sample_tokens(ids, n_expert, n_sample, rng):
    """Token sample that covers the three most loaded experts (their row tiles are the multi-tile case)."""
    tpe = np.bincount(ids.reshape(-1), minlength=n_expert)
    heavy = np.argsort(-tpe)[:3]
    pick = []
    for e in heavy:
        tok = np.nonzero((ids == e).any(axis=1))[0]
        pick += [tok[0], tok[len(tok) // 2], tok[-1]]          # first, middle and last row of the expert's list
    rest = rng.choice(ids.shape[0], n_sample, replace=False)
    return np.unique(np.concatenate([np.array(pick), rest]))[:n_sample + 9], tpe


@pytest.fixture(scope="module")
def zipf_block(dev):
    from bench import zipf_bias
    from maxuna_b200.moe import MoeBlock

    return MoeBlock.random(H, F, E, K, seed=4242, device=dev, bias=zipf_bias(E, 3, dev))


def test_prefill_config3_4096_tokens_zipf(orc, dev, zipf_block):
    """BASELINE config 3 at its own size: 4096 tokens, Zipf-skewed selection bias."""
    blk = zipf_block
    host = blk.host_layer(orc)
    gen = torch.Generator(device=dev)
    gen.manual_seed(99)
    xd = torch.randn(4096, H, generator=gen, device=dev)
    out, ids, w = blk.forward(xd, return_routing=True, path="prefill")
    torch.cuda.synchronize()
    blk.check_device_flag()
    x = xd.cpu().numpy()
    ids_o, w_o = orc.route(host.router, host.bias, x, K)
    ids_g = ids.cpu().numpy().astype(np.uint32)
    assert np.array_equal(ids_g, ids_o), "expert ids differ from the oracle"
    assert np.array_equal(w.cpu().numpy().view(np.uint32), w_o.view(np.uint32)), "routing weights differ"
    sample, tpe = _sample_tokens(ids_o, E, 64, np.random.default_rng(5))
    # the heavy experts take more than one row tile of the grouped GEMM (192 rows per tile)
    assert tpe.max() > 256, f"routing is not skewed enough to need several row tiles: max {tpe.max()}"
    want, ids_s, _ = host.forward(x[sample])
    assert np.array_equal(ids_s, ids_o[sample])
    got = out.cpu().numpy()[sample]
    err = orc.rel_l2(got, want)
    worst = max(orc.rel_l2(got[i], want[i]) for i in range(len(sample)))
    ties = _near_ties(orc, host, x, K)
    print(f"config3: tokens/expert max {tpe.max()} mean {tpe.mean():.0f}; sample of {len(sample)} tokens: rel-L2 {err:.2e}, "
          f"worst token {worst:.2e}; near-ties (<1e-6) {ties} of 4096 tokens")
    assert err < 2e-3 and worst < 4e-3


def test_layer_entry_2048_tokens(orc, dev, zipf_block):
    """The prefill half of BASELINE config 5, one layer: 2048 tokens through lmoe_moe_layer_forward."""
    blk = zipf_block
    host = blk.host_layer(orc)
    rng = np.random.default_rng(2048)
    ffn_inp = (rng.standard_normal((2048, H)) * 1.5).astype(np.float32)
    g = rng.uniform(0.5, 1.5, H).astype(np.float32)
    out, ids, w = blk.layer_forward(torch.from_numpy(ffn_inp).to(dev), torch.from_numpy(g).to(dev), 1e-6, return_routing=True)
    torch.cuda.synchronize()
    blk.check_device_flag()
    normed = orc.rms_norm(ffn_inp, g, 1e-6)
    ids_o, w_o = orc.route(host.router, host.bias, normed, K)
    assert np.array_equal(ids.cpu().numpy().astype(np.uint32), ids_o)
    assert np.array_equal(w.cpu().numpy().view(np.uint32), w_o.view(np.uint32))
    sample, _ = _sample_tokens(ids_o, E, 40, rng)
    want, _, _ = host.forward(normed[sample])
    assert orc.rel_l2(out.cpu().numpy()[sample] - ffn_inp[sample], want) < 2e-3


def test_decode_outlier_channels(orc, dev, zipf_block):
    """Hidden states with a few channels 100x the rest (and one token 100x the others): the decode kernel
    carries activations as 21-bit integers under a per-256 scale, so the small channels next to an outlier
    lose relative precision; the block output must stay inside the bound all the same."""
    blk = zipf_block
    host = blk.host_layer(orc)
    rng = np.random.default_rng(77)
    x = rng.standard_normal((8, H)).astype(np.float32)
    x[:, rng.choice(H, 6, replace=False)] *= 100.0
    x[3] *= 100.0
    out, ids, _ = blk.forward(torch.from_numpy(x).to(dev), return_routing=True, path="decode")
    torch.cuda.synchronize()
    blk.check_device_flag()
    want, ids_o, _ = host.forward(x)
    assert np.array_equal(ids.cpu().numpy().astype(np.uint32), ids_o)
    err = orc.rel_l2(out.cpu().numpy(), want)
    worst = max(orc.rel_l2(out.cpu().numpy()[i], want[i]) for i in range(8))
    print(f"decode with outlier channels: rel-L2 {err:.2e}, worst token {worst:.2e}")
    assert err < 2e-3 and worst < 2e-3


def test_prefill_l2_guard_large_magnitude(orc, dev):
    """Inputs large enough that silu(gate)*up leaves the f16 range (> 65504): without the per-row L2 rescale
    of src/moe.rs:292-313 the f16-staged down projection would overflow."""
    from maxuna_b200.moe import MoeBlock

    blk = MoeBlock.random(256, 256, 8, 3, seed=91, device=dev, weight_std=0.25)
    host = blk.host_layer(orc)
    x = (np.random.default_rng(92).standard_normal((96, 256)) * 120.0).astype(np.float32)
    out = blk.forward(torch.from_numpy(x).to(dev), path="prefill")
    torch.cuda.synchronize()
    blk.check_device_flag()
    want, _, _ = host.forward(x)
    assert np.abs(want).max() > 65504.0          # the case really is out of f16 range
    got = out.cpu().numpy()
    assert np.isfinite(got).all()
    assert orc.rel_l2(got, want) < 2e-3


@pytest.mark.parametrize("entry", ["prefill", "rows", "tokens", "shared"])
def test_prefill_entries_clear_the_device_flag(dev, entry):
    """The grouped-GEMM entries must work on scratch that was never initialised: with the workspace filled
    with 0xFF the device flag still reads clean after the call."""
    from maxuna_b200._native import check, lib
    from maxuna_b200.gguf import stream_ptr
    from maxuna_b200.moe import MoeBlock

    blk = MoeBlock.random(256, 512, 8, 3, seed=95, device=dev, weight_std=0.25)
    t = 70
    x = torch.randn(t, 256, device=dev)
    out = torch.empty(t, 256, device=dev)
    L = lib()
    if entry == "prefill":
        n = L.lmoe_layer_workspace_bytes(blk.handle, t)
        ws = torch.full((n,), 0xFF, dtype=torch.uint8, device=dev)
        check(L.lmoe_moe_forward_prefill(blk.handle, x.data_ptr(), t, out.data_ptr(), None, None, ws.data_ptr(), n, stream_ptr()))
    elif entry == "rows":
        n = L.lmoe_rows_workspace_bytes(blk.handle, t)
        ws = torch.full((n,), 0xFF, dtype=torch.uint8, device=dev)
        ids = torch.randint(0, 8, (t,), dtype=torch.int32, device=dev)
        w = torch.ones(t, device=dev)
        check(L.lmoe_experts_forward_rows(blk.handle, x.data_ptr(), ids.data_ptr(), w.data_ptr(), t, out.data_ptr(),
                                          ws.data_ptr(), n, stream_ptr()))
    elif entry == "tokens":
        n = L.lmoe_tokens_workspace_bytes(blk.handle, t, 3)
        ws = torch.full((n,), 0xFF, dtype=torch.uint8, device=dev)
        ids = torch.stack([torch.randperm(8, device=dev)[:3] for _ in range(t)]).to(torch.int32).contiguous()
        w = torch.ones(t, 3, device=dev)
        xh = x.to(torch.float16)
        check(L.lmoe_experts_forward_tokens_f16(blk.handle, xh.data_ptr(), ids.data_ptr(), w.data_ptr(), t, 3, out.data_ptr(),
                                                ws.data_ptr(), n, stream_ptr()))
    else:
        n = L.lmoe_rows_workspace_bytes(blk.handle, t)
        ws = torch.full((n,), 0xFF, dtype=torch.uint8, device=dev)
        check(L.lmoe_shared_forward(blk.handle, x.data_ptr(), t, out.data_ptr(), ws.data_ptr(), n, stream_ptr()))
    torch.cuda.synchronize()
    check(L.lmoe_check_device_flag(ws.data_ptr(), stream_ptr()))
    assert torch.isfinite(out).all()


def test_second_decode_call_in_flight_is_refused(dev, zipf_block):
    """One decode call at a time per layer handle: a call on a second stream while the first is still
    running is an error, not silent corruption; after the first has finished the second stream may call."""
    from maxuna_b200._native import lib

    blk = zipf_block
    L = lib()
    x = torch.randn(4, H, device=dev)
    out = torch.empty(4, H, device=dev)
    ws = blk.workspace(4)
    torch.cuda.synchronize()
    s1, s2 = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    with torch.cuda.stream(s1):
        torch.cuda._sleep(400_000_000)           # keeps stream 1 busy for a fraction of a second
    rc1 = L.lmoe_moe_forward_decode(blk.handle, x.data_ptr(), 4, out.data_ptr(), None, None, ws.data_ptr(), ws.numel(), s1.cuda_stream)
    rc2 = L.lmoe_moe_forward_decode(blk.handle, x.data_ptr(), 4, out.data_ptr(), None, None, ws.data_ptr(), ws.numel(), s2.cuda_stream)
    msg = L.lmoe_last_error()
    torch.cuda.synchronize()
    assert rc1 == 0
    assert rc2 == -1 and b"in flight" in msg
    rc3 = L.lmoe_moe_forward_decode(blk.handle, x.data_ptr(), 4, out.data_ptr(), None, None, ws.data_ptr(), ws.numel(), s2.cuda_stream)
    torch.cuda.synchronize()
    assert rc3 == 0


def test_decode_entry_takes_more_than_64_tokens(orc, dev):
    """The mat-vec entry serves any token count in launches of 64 (LAGUNA_NO_MM_ID forces it everywhere)."""
    from maxuna_b200.moe import MoeBlock

    blk = MoeBlock.random(256, 256, 8, 3, seed=97, device=dev, weight_std=0.25)
    host = blk.host_layer(orc)
    x = np.random.default_rng(98).standard_normal((150, 256)).astype(np.float32)
    out, ids, _ = blk.forward(torch.from_numpy(x).to(dev), return_routing=True, path="decode")
    torch.cuda.synchronize()
    blk.check_device_flag()
    want, ids_o, _ = host.forward(x)
    assert np.array_equal(ids.cpu().numpy().astype(np.uint32), ids_o)
    assert orc.rel_l2(out.cpu().numpy(), want) < 2e-3


def test_lm_head_shape_plain_mv(orc, dev):
    """`ops::mul_mv` at the shape the model calls it on, once per decoded token (src/model.rs:388-403):
    Q6_K [100352 x 3072].  256 sampled rows against the oracle, the first and the last chunk among them, and
    every row finite; a second activation row checks the per-token loop."""
    from maxuna_b200 import ops
    from maxuna_b200.gguf import Q6_K, ExpertStack

    n_out, k = 100352, 3072
    st = ExpertStack.random(Q6_K, 1, n_out, k, std=0.02, seed=4242, device=dev, chunk_experts=1)
    gen = torch.Generator(device=dev)
    gen.manual_seed(9)
    x = torch.randn(2, k, generator=gen, device=dev)
    x[0, 100] = 40.0  # an outlier channel, as the hidden state has them
    w = st.buffer[st.base_off:st.base_off + st.nbytes]
    got = ops.mul_mv(w, Q6_K, n_out, k, x)
    assert bool(torch.isfinite(got).all())
    rows = np.unique(np.concatenate([np.arange(16), np.arange(n_out - 16, n_out),
                                     np.random.default_rng(3).choice(n_out, 224, replace=False)]))
    rb = (k // 256) * 210
    raw = w.view(n_out, rb)[torch.from_numpy(rows).to(dev)].cpu().numpy()
    want = orc.mul_mv(Q6_K, raw, len(rows), k, x.cpu().numpy())
    sub = got[:, torch.from_numpy(rows).to(dev)].cpu().numpy()
    assert orc.rel_l2(sub, want) < 1e-5
