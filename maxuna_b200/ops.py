"""Host mirror of the reference's ``src/ops`` dispatch layer for the MoE path.

Same function names, argument meaning and error behaviour as the reference's
Rust wrappers; every function enqueues hand-written CUDA kernels through the C
ABI (``include/lmoe.h``) on the current torch stream and returns a fresh device
tensor, like the reference's ops return fresh Metal tensors.  Shape and dtype
mismatches raise :class:`LmoeError` before anything is launched.

  mul_mv_id          src/ops/mv_id.rs:37-45
  mul_mv             src/ops/mv_id.rs:54-56
  mul_mm_id          src/ops/mm_id.rs:16-18
  prepare_map0       src/ops/mm_id.rs:27-29
  mul_mm_id_shared   src/ops/mm_id.rs:32-39
  supported          src/ops/mm_id.rs:48-50
  silu_mul           src/ops/silu_mul.rs:14
  combine            src/ops/combine.rs:16
  route              src/moe.rs:62-71 (MoeBlock::route), 84-119
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from . import _native
from ._native import LmoeError, check, lib
from .gguf import ExpertStack, stream_ptr

MM_ID_MIN_SEQ_REFERENCE = 32  # src/ops/mod.rs:31: the reference's own crossover, for documentation


def mm_id_min_seq() -> int:
    """Token count from which the grouped GEMM is used (`lmoe_mm_id_min_seq`): 65 on B200 unless
    `LAGUNA_MM_ID_MIN_SEQ` / `LAGUNA_NO_MM_ID` (src/ops/mod.rs:24-60) say otherwise.  One value for the C
    entries that pick a path themselves and for the host mirrors, read once per process by the library."""
    return int(lib().lmoe_mm_id_min_seq())


def no_mm_id() -> bool:
    """`LAGUNA_NO_MM_ID`: presence-based, forces the mat-vec path everywhere."""
    return mm_id_min_seq() >= (1 << 62)


def _require(cond, msg):
    if not cond:
        raise LmoeError(-1, msg)


def _f32_dev(name, t: torch.Tensor):
    _require(isinstance(t, torch.Tensor), f"{name} must be a tensor")
    _require(t.is_cuda, f"{name} must be on a CUDA device")
    _require(t.dtype == torch.float32, f"{name} must be f32, got {t.dtype}")
    _require(t.is_contiguous(), f"{name} must be contiguous")


def _ids_dev(ids: torch.Tensor):
    _require(ids.is_cuda, "ids must be on a CUDA device")
    # torch has no first-class u32 arithmetic; int32 storage carries the same bits
    _require(ids.dtype in (torch.int32, torch.uint32), f"ids must be u32, got {ids.dtype}")
    _require(ids.is_contiguous(), "ids must be contiguous")
    _require(ids.dim() == 2, "ids must be rank-2 [t, top_k]")


def _x3(x):
    _f32_dev("x", x)
    _require(x.dim() == 3, "x must be rank-3 [t, x_per_row, k]")
    return x.shape


def mul_mv_id(stack: ExpertStack, x: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    """x ``[t, x_per_row, k]`` f32, ids ``[t, top_k]`` u32 -> ``[t, top_k, n_out]`` f32."""
    t, xpr, k = _x3(x)
    _ids_dev(ids)
    t_ids, top_k = ids.shape
    out = torch.empty(t_ids, top_k, stack.n_out, dtype=torch.float32, device=x.device)
    check(lib().lmoe_mul_mv_id(stack.handle, x.data_ptr(), t, xpr, k, ids.data_ptr(), t_ids, top_k,
                               out.data_ptr(), stream_ptr()))
    return out


def mul_mv(weight: torch.Tensor, dtype: int, n_out: int, k: int, x: torch.Tensor) -> torch.Tensor:
    """Plain quantized mat-vec: weight = raw ``[n_out, k]`` super-blocks, x ``[t, k]`` -> ``[t, n_out]``."""
    _f32_dev("x", x)
    _require(x.dim() == 2, "x must be rank-2 [t, k]")
    _require(x.shape[1] == k, f"x k ({x.shape[1]}) does not match weight k ({k})")
    _require(weight.is_cuda and weight.dtype == torch.uint8, "weight must be a CUDA uint8 buffer")
    out = torch.empty(x.shape[0], n_out, dtype=torch.float32, device=x.device)
    check(lib().lmoe_mul_mv(weight.data_ptr(), dtype, n_out, k, x.data_ptr(), x.shape[0], out.data_ptr(),
                            stream_ptr()))
    return out


@dataclass
class Map0Scratch:
    """`Map0Scratch`, src/ops/dispatch.rs:752-757: the buffer plus the geometry it was laid out for."""
    buffer: torch.Tensor
    n_expert: int
    t: int
    top_k: int

    def tpe(self) -> torch.Tensor:
        return self.buffer[: self.n_expert * 4].view(torch.int32)

    def ids_map(self) -> torch.Tensor:
        return self.buffer[self.n_expert * 4: self.n_expert * 4 * (1 + self.t)].view(torch.int32).view(self.n_expert, self.t)


def prepare_map0(n_expert: int, ids: torch.Tensor) -> Map0Scratch:
    _ids_dev(ids)
    t, top_k = ids.shape
    nbytes = lib().lmoe_map0_scratch_bytes(n_expert, t)
    buf = torch.empty(nbytes, dtype=torch.uint8, device=ids.device)
    check(lib().lmoe_prepare_map0(ids.data_ptr(), t, top_k, n_expert, buf.data_ptr(), nbytes, stream_ptr()))
    return Map0Scratch(buf, n_expert, t, top_k)


def supported(dtype: int, top_k: int) -> bool:
    return bool(lib().lmoe_mm_id_supported(dtype, top_k))


def mul_mm_id_shared(stack: ExpertStack, x: torch.Tensor, ids: torch.Tensor, scratch: Map0Scratch) -> torch.Tensor:
    t, xpr, k = _x3(x)
    _ids_dev(ids)
    t_ids, top_k = ids.shape
    out = torch.empty(t_ids, top_k, stack.n_out, dtype=torch.float32, device=x.device)
    ws_bytes = lib().lmoe_mm_id_workspace_bytes(stack.handle, t, top_k, xpr)
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=x.device)
    check(lib().lmoe_mul_mm_id_shared(stack.handle, x.data_ptr(), t, xpr, k, ids.data_ptr(), t_ids, top_k,
                                      scratch.buffer.data_ptr(), scratch.n_expert, scratch.t, scratch.top_k,
                                      out.data_ptr(), ws.data_ptr(), ws_bytes, stream_ptr()))
    return out


def mul_mm_id(stack: ExpertStack, x: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    t, xpr, k = _x3(x)
    _ids_dev(ids)
    t_ids, top_k = ids.shape
    out = torch.empty(t_ids, top_k, stack.n_out, dtype=torch.float32, device=x.device)
    ws_bytes = lib().lmoe_mm_id_workspace_bytes(stack.handle, t, top_k, xpr) + lib().lmoe_map0_scratch_bytes(stack.n_expert, t)
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=x.device)
    check(lib().lmoe_mul_mm_id(stack.handle, x.data_ptr(), t, xpr, k, ids.data_ptr(), t_ids, top_k, out.data_ptr(),
                               ws.data_ptr(), ws_bytes, stream_ptr()))
    return out


def silu_mul(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    _f32_dev("gate", gate)
    _f32_dev("up", up)
    _require(gate.shape == up.shape, f"silu_mul shape mismatch: gate {tuple(gate.shape)}, up {tuple(up.shape)}")
    _require(gate.device == up.device, "gate and up must be on the same device")
    out = torch.empty_like(gate)
    check(lib().lmoe_silu_mul(gate.data_ptr(), up.data_ptr(), gate.numel(), out.data_ptr(), stream_ptr()))
    return out


def combine(down: torch.Tensor, col_l2, weights: torch.Tensor) -> torch.Tensor:
    _f32_dev("down", down)
    _require(down.dim() == 3, "down must be rank-3 [seq, top_k, n_out]")
    seq, top_k, n_out = down.shape
    _f32_dev("weights", weights)
    _require(tuple(weights.shape) == (seq, top_k), f"weights shape {tuple(weights.shape)} must be [seq, top_k] = [{seq}, {top_k}]")
    l2p = None
    if col_l2 is not None:
        _f32_dev("col_l2", col_l2)
        _require(tuple(col_l2.shape) == (seq, top_k, 1), f"col_l2 shape {tuple(col_l2.shape)} must be [seq, top_k, 1] = [{seq}, {top_k}, 1]")
        l2p = col_l2.data_ptr()
    out = torch.empty(seq, n_out, dtype=torch.float32, device=down.device)
    check(lib().lmoe_combine(down.data_ptr(), l2p, weights.data_ptr(), seq, top_k, n_out, out.data_ptr(), stream_ptr()))
    return out


def route(router: torch.Tensor, bias, x: torch.Tensor, top_k: int, scale: float = 2.5, norm: bool = True):
    """router ``[n_expert, hidden]``, x ``[t, hidden]`` -> (ids ``[t, top_k]`` int32-as-u32, weights f32)."""
    _f32_dev("router", router)
    _f32_dev("x", x)
    _require(router.dim() == 2 and x.dim() == 2, "router must be [n_expert, hidden], x [t, hidden]")
    n_expert, hidden = router.shape
    _require(x.shape[1] == hidden, f"x hidden ({x.shape[1]}) does not match router hidden ({hidden})")
    t = x.shape[0]
    if bias is not None:
        _f32_dev("bias", bias)
        _require(bias.numel() == n_expert, "bias must have n_expert entries")
    ids = torch.empty(t, top_k, dtype=torch.int32, device=x.device)
    w = torch.empty(t, top_k, dtype=torch.float32, device=x.device)
    nbytes = lib().lmoe_route_workspace_bytes(t, n_expert)
    ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=x.device)
    check(lib().lmoe_route(router.data_ptr(), None if bias is None else bias.data_ptr(), x.data_ptr(), t, hidden,
                           n_expert, top_k, scale, int(norm), ids.data_ptr(), w.data_ptr(), ws.data_ptr(), nbytes,
                           stream_ptr()))
    return ids, w


def route_from_logits(logits: torch.Tensor, bias, top_k: int, scale: float = 2.5, norm: bool = True):
    _f32_dev("logits", logits)
    _require(logits.dim() == 2, "logits must be [t, n_expert]")
    t, n_expert = logits.shape
    ids = torch.empty(t, top_k, dtype=torch.int32, device=logits.device)
    w = torch.empty(t, top_k, dtype=torch.float32, device=logits.device)
    check(lib().lmoe_route_from_logits(logits.data_ptr(), None if bias is None else bias.data_ptr(), t, n_expert,
                                       top_k, scale, int(norm), ids.data_ptr(), w.data_ptr(), stream_ptr()))
    return ids, w
