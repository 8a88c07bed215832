"""The C-ABI library without a GPU: it loads, exports every symbol the header
declares, and rejects bad arguments with an error code before touching CUDA."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "lmoe.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(lmoe_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_exported():
    from maxuna_b200 import _native

    lib = _native.lib()
    names = _declared()
    assert len(names) >= 25
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/lmoe.h but not exported"
    assert set(names) == set(_native.PROTOTYPES), set(names) ^ set(_native.PROTOTYPES)
    assert b"sm_100a" in lib.lmoe_version()


def test_argument_errors_without_cuda():
    from maxuna_b200 import _native

    lib = _native.lib()
    h = C.c_void_p()
    # bad dtype, bad k, size mismatch, misaligned base_off: errors, not crashes
    assert lib.lmoe_expert_stack_wrap(99, 1, 8, 256, 16, 8 * 144, 0, C.byref(h)) == -1
    assert b"dtype" in lib.lmoe_last_error()
    assert lib.lmoe_expert_stack_wrap(12, 1, 8, 100, 16, 8 * 144, 0, C.byref(h)) == -1
    assert b"multiple" in lib.lmoe_last_error()
    assert lib.lmoe_expert_stack_wrap(12, 1, 8, 256, 16, 7 * 144, 0, C.byref(h)) == -1
    assert lib.lmoe_expert_stack_wrap(12, 1, 8, 256, 16, 8 * 144, 8, C.byref(h)) == -1
    assert lib.lmoe_expert_stack_wrap(12, 4, 8, 256, 4096, 4 * 8 * 144, 0, C.byref(h)) == 0
    # mul_mv_id seam checks (src/ops/dispatch.rs:812-847 of the reference)
    fake = C.c_void_p(4096)
    assert lib.lmoe_mul_mv_id(h, fake, 1, 1, 128, fake, 1, 2, fake, None) == -1
    assert b"does not match expert stack k" in lib.lmoe_last_error()
    assert lib.lmoe_mul_mv_id(h, fake, 2, 1, 256, fake, 3, 2, fake, None) == -1
    assert b"ids t" in lib.lmoe_last_error()
    assert lib.lmoe_mul_mv_id(h, fake, 2, 3, 256, fake, 2, 2, fake, None) == -1
    assert b"x_per_row" in lib.lmoe_last_error()
    lib.lmoe_expert_stack_destroy(h)
    # combine guards (src/ops/dispatch.rs:294-305)
    assert lib.lmoe_combine(fake, None, fake, 1, 130, 8, fake, None) == -1
    assert lib.lmoe_combine(fake, None, fake, 1 << 20, 10, 3072, fake, None) == -1
    assert b"i32::MAX" in lib.lmoe_last_error()
    # routing guards
    assert lib.lmoe_route_from_logits(fake, None, 1, 1000, 10, 2.5, 1, fake, fake, None) == -1
    assert lib.lmoe_route_from_logits(fake, None, 1, 8, 9, 2.5, 1, fake, fake, None) == -1
    # workspace guard
    assert lib.lmoe_prepare_map0(fake, 16, 2, 4, fake, 8, None) == -4
    assert lib.lmoe_map0_scratch_bytes(256, 512) >= 256 * 4 + 256 * 512 * 4


def test_expert_parallel_argument_errors_without_cuda():
    from maxuna_b200 import _native

    lib = _native.lib()
    fake = C.c_void_p(4096)
    # n_expert must divide over the ranks, hidden a multiple of 8, buffers non-NULL and aligned
    assert lib.lmoe_ep_pack(fake, fake, fake, 4, 128, 2, 8, 3, fake, fake, fake, fake, fake, fake, 1 << 20, None) == -1
    assert b"divisible" in lib.lmoe_last_error()
    assert lib.lmoe_ep_pack(fake, fake, fake, 4, 100, 2, 8, 2, fake, fake, fake, fake, fake, fake, 1 << 20, None) == -1
    assert lib.lmoe_ep_pack(fake, fake, fake, 4, 128, 2, 8, 2, None, fake, fake, fake, fake, fake, 1 << 20, None) == -1
    assert lib.lmoe_ep_pack(C.c_void_p(4100), fake, fake, 4, 128, 2, 8, 2, fake, fake, fake, fake, fake, fake, 1 << 20, None) == -1
    assert b"aligned" in lib.lmoe_last_error()
    assert lib.lmoe_ep_pack(fake, fake, fake, 4, 128, 2, 8, 2, fake, fake, fake, fake, fake, fake, 16, None) == -4
    assert lib.lmoe_ep_pack_workspace_bytes(8, 4) >= 8 * 4 + 8 * 4 * 4
    assert lib.lmoe_ep_combine(None, fake, None, 4, 2, 128, fake, None) == -1
    assert lib.lmoe_ep_combine(fake, fake, None, 4, 0, 128, fake, None) == -1
    assert lib.lmoe_ep_combine(fake, fake, None, 0, 2, 128, fake, None) == 0
    assert lib.lmoe_experts_forward_rows_f16(None, fake, fake, fake, 4, fake, fake, 1 << 20, None) == -1


def test_peer_and_host_entry_argument_errors_without_cuda():
    """The peer-memory exchange and the host-buffer entries check their arguments before they touch the GPU."""
    from maxuna_b200 import _native

    lib = _native.lib()
    fake = C.c_void_p(4096)
    arr = (C.c_void_p * 2)(4096, 8192)
    assert lib.lmoe_peer_ctrl_bytes() >= 128 * 4
    assert lib.lmoe_peer_alloc(0, C.byref(C.c_void_p()), C.create_string_buffer(64)) == -1
    assert lib.lmoe_peer_open(None, C.byref(C.c_void_p())) == -1
    assert lib.lmoe_peer_put(None, 64, 2, 0, 0, arr, arr, fake, 0, None) == -1
    assert lib.lmoe_peer_put(fake, 64, 17, 0, 0, arr, arr, fake, 0, None) == -1          # more ranks than the kernel carries
    assert lib.lmoe_peer_put(fake, 64, 2, 2, 0, arr, arr, fake, 0, None) == -1           # rank outside the world
    assert lib.lmoe_peer_put(fake, 40, 2, 0, 0, arr, arr, fake, 0, None) == -1           # chunk not a multiple of 16
    assert b"16" in lib.lmoe_last_error()
    assert lib.lmoe_peer_put(fake, 64, 2, 0, 0, arr, arr, fake, 2, None) == -1           # direction is 0 or 1
    assert lib.lmoe_peer_wait(None, 2, 0, None) == -1
    assert lib.lmoe_peer_wait(fake, 0, 0, None) == -1
    for fn in (lib.lmoe_moe_forward_host, lib.lmoe_moe_forward_host_async):
        assert fn(None, fake, 1, fake, None, None, fake, 1 << 20, None) == -1
        assert b"layer" in lib.lmoe_last_error()


def test_host_mirror_rejects_cpu_tensors():
    import torch

    from maxuna_b200 import LmoeError, ops

    with pytest.raises(LmoeError):
        ops.silu_mul(torch.zeros(4), torch.zeros(4))
    with pytest.raises(LmoeError):
        ops.combine(torch.zeros(1, 2, 3), None, torch.zeros(1, 2))


def test_cpp_host_mirror_compiles_and_reports_errors(tmp_path):
    import shutil
    import subprocess

    from maxuna_b200 import _native

    _native.lib()
    gxx = shutil.which("g++")
    assert gxx, "g++ not found"
    exe = str(tmp_path / "host_errors")
    libdir = os.path.dirname(_native.lib_path())
    env = {k: v for k, v in os.environ.items() if k not in ("CC", "CXX")}
    subprocess.run([gxx, "-std=c++17", "-O1", os.path.join(ROOT, "tests", "cpp", "host_errors.cpp"), "-o", exe,
                    "-L" + libdir, "-llmoe", "-Wl,-rpath," + libdir], check=True, env=env)
    out = subprocess.run([exe], capture_output=True, text=True, env=env)
    assert out.returncode == 0 and out.stdout.strip() == "ok", out.stdout + out.stderr
