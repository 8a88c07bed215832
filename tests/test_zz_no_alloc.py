"""`lmoe_route_noalloc`: routing for hosts that may not allocate device memory at call time
(their own pool owns the GPU, or they are inside a stream capture).  The entry point keeps its
logits scratch in a fixed array inside the library; this test calls it through the C ABI twice
in a row and requires the same expert ids and weights, bit for bit, as `lmoe_route` with a
caller workspace.  It lives in a file that pytest collects last."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_route_noalloc_matches_route_twice():
    from maxuna_b200 import _native
    from maxuna_b200.gguf import stream_ptr

    lib = _native.lib()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    gen = torch.Generator(device=dev)
    gen.manual_seed(2024)
    n_expert, hidden, top_k = 256, 3072, 10
    router = torch.randn(n_expert, hidden, generator=gen, device=dev) * 0.02
    bias = torch.rand(n_expert, generator=gen, device=dev) * 0.2 - 0.1
    for call, t in enumerate((16, 5, 100)):  # later calls reuse the array the earlier ones left dirty; 100 tokens take the tiled logits kernel
        x = torch.randn(t, hidden, generator=gen, device=dev)
        ids_a = torch.empty(t, top_k, dtype=torch.int32, device=dev)
        w_a = torch.empty(t, top_k, dtype=torch.float32, device=dev)
        ids_b, w_b = torch.empty_like(ids_a), torch.empty_like(w_a)
        nbytes = lib.lmoe_route_workspace_bytes(t, n_expert)
        ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        _native.check(lib.lmoe_route(router.data_ptr(), bias.data_ptr(), x.data_ptr(), t, hidden, n_expert, top_k, 2.5, 1,
                                     ids_a.data_ptr(), w_a.data_ptr(), ws.data_ptr(), nbytes, stream_ptr()))
        _native.check(lib.lmoe_route_noalloc(router.data_ptr(), bias.data_ptr(), x.data_ptr(), t, hidden, n_expert, top_k,
                                             2.5, 1, ids_b.data_ptr(), w_b.data_ptr(), stream_ptr()))
        torch.cuda.synchronize()
        assert torch.equal(ids_a, ids_b), f"call {call}: expert ids differ"
        assert np.array_equal(w_a.cpu().numpy().view(np.uint32), w_b.cpu().numpy().view(np.uint32)), f"call {call}"
    # beyond the built-in scratch: a clear error, nothing launched
    t_big = 32768 // n_expert + 1
    rc = lib.lmoe_route_noalloc(router.data_ptr(), bias.data_ptr(), router.data_ptr(), t_big, hidden, n_expert, top_k, 2.5, 1,
                                ids_a.data_ptr(), w_a.data_ptr(), stream_ptr())
    assert rc == -1 and b"exceeds the built-in scratch" in lib.lmoe_last_error()
    # a token count whose product with n_expert wraps around 64 bits is refused as well
    rc = lib.lmoe_route_noalloc(router.data_ptr(), bias.data_ptr(), router.data_ptr(), (1 << 54) + (1 << 31) - 1, hidden, 512, top_k,
                                2.5, 1, ids_a.data_ptr(), w_a.data_ptr(), stream_ptr())
    assert rc == -1 and b"exceeds the built-in scratch" in lib.lmoe_last_error()
    torch.cuda.synchronize()
