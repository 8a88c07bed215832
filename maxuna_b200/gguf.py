"""`ExpertStack`: stacked per-expert weights kept in their quantized GGUF layout.

Mirror of the reference's ``ExpertStack`` (src/gguf.rs:247-276) and of
``Weights::expert_stack`` (src/gguf.rs:554-607): ``[n_expert, n_out, k]``
super-blocks, expert-major and contiguous, uploaded once and indexed by expert
id on the device.  No re-layout is done: the bytes in HBM are the bytes of the
GGUF tensor.
"""
from __future__ import annotations

import ctypes as C
import warnings

import numpy as np
import torch

from . import _native

Q4_K = 12
Q6_K = 14
QK_K = 256
TYPE_SIZE = {Q4_K: 144, Q6_K: 210}
DTYPE_NAME = {Q4_K: "Q4_K", Q6_K: "Q6_K"}


def stream_ptr(stream=None) -> int:
    s = torch.cuda.current_stream() if stream is None else stream
    return s.cuda_stream


class ExpertStack:
    """Device-resident quantized expert stack (src/gguf.rs:247-276).

    Fields keep the reference's names: ``dtype``, ``n_expert``, ``n_out``, ``k``,
    ``base_off``; ``buffer`` is the torch uint8 tensor that owns the bytes.
    """

    def __init__(self, buffer: torch.Tensor, dtype: int, n_expert: int, n_out: int, k: int, base_off: int = 0):
        if dtype not in TYPE_SIZE:
            raise _native.LmoeError(-1, f"unsupported expert dtype {dtype}")
        if buffer.dtype != torch.uint8 or not buffer.is_contiguous():
            raise _native.LmoeError(-1, "expert stack buffer must be a contiguous uint8 tensor")
        if not buffer.is_cuda:
            raise _native.LmoeError(-3, "expert stack has no device buffer; the fused MoE path requires CUDA")
        self.buffer, self.dtype, self.n_expert, self.n_out, self.k, self.base_off = buffer, dtype, n_expert, n_out, k, base_off
        nbytes = self.nbytes
        if buffer.numel() < base_off + nbytes:
            raise _native.LmoeError(-1, f"expert stack buffer holds {buffer.numel()} bytes, needs {base_off + nbytes}")
        h = C.c_void_p()
        _native.check(_native.lib().lmoe_expert_stack_wrap(dtype, n_expert, n_out, k, buffer.data_ptr(), nbytes,
                                                           base_off, C.byref(h)))
        self._h = h

    @property
    def nbytes(self) -> int:
        return self.n_expert * self.n_out * (self.k // QK_K) * TYPE_SIZE[self.dtype] if self.k % QK_K == 0 else -1

    @property
    def handle(self) -> C.c_void_p:
        return self._h

    def __del__(self):
        h = getattr(self, "_h", None)
        if h:
            try:
                _native.lib().lmoe_expert_stack_destroy(h)
            except Exception:  # interpreter shutdown: the library is already gone
                pass
            self._h = None

    # ---- construction -----------------------------------------------------
    @classmethod
    def from_bytes(cls, raw, dtype: int, n_expert: int, n_out: int, k: int, device="cuda", base_off: int = 0):
        """One upload of raw GGUF super-blocks (``expert_stack_classic``, src/gguf.rs:567-607)."""
        raw = np.ascontiguousarray(raw, dtype=np.uint8).reshape(-1)
        buf = torch.zeros(base_off + raw.size + 128, dtype=torch.uint8, device=device)
        with warnings.catch_warnings():
            # a read-only view of a mapped file is only read here: one host-to-device copy
            warnings.simplefilter("ignore", UserWarning)
            buf[base_off:base_off + raw.size] = torch.from_numpy(raw).to(device)
        return cls(buf, dtype, n_expert, n_out, k, base_off)

    @classmethod
    def quantize(cls, w: torch.Tensor, dtype: int):
        """Encode an f32 ``[n_expert, n_out, k]`` CUDA tensor on the device (synthetic stacks)."""
        assert w.is_cuda and w.dtype == torch.float32 and w.dim() == 3
        n_expert, n_out, k = w.shape
        w = w.contiguous()
        nblocks = w.numel() // QK_K
        buf = torch.zeros(nblocks * TYPE_SIZE[dtype] + 128, dtype=torch.uint8, device=w.device)
        _native.check(_native.lib().lmoe_quantize(dtype, w.data_ptr(), nblocks, buf.data_ptr(), stream_ptr()))
        return cls(buf, dtype, n_expert, n_out, k, 0)

    @classmethod
    def random(cls, dtype: int, n_expert: int, n_out: int, k: int, std: float = 0.02, seed: int = 0,
               device="cuda", chunk_experts: int = 32):
        """Seeded N(0, std) weights encoded on the device, ``chunk_experts`` at a time."""
        nb_e = n_out * (k // QK_K)
        ts = TYPE_SIZE[dtype]
        buf = torch.zeros(n_expert * nb_e * ts + 128, dtype=torch.uint8, device=device)
        gen = torch.Generator(device=device)
        gen.manual_seed(seed)
        for e0 in range(0, n_expert, chunk_experts):
            ne = min(chunk_experts, n_expert - e0)
            w = torch.randn(ne, n_out, k, generator=gen, device=device, dtype=torch.float32) * std
            dst = buf[e0 * nb_e * ts:]
            _native.check(_native.lib().lmoe_quantize(dtype, w.data_ptr(), ne * nb_e, dst.data_ptr(), stream_ptr()))
            torch.cuda.current_stream().synchronize()
        return cls(buf, dtype, n_expert, n_out, k, 0)

    # ---- views ------------------------------------------------------------
    def raw(self) -> np.ndarray:
        """The super-block bytes on the host (for the CPU checker)."""
        return self.buffer[self.base_off:self.base_off + self.nbytes].cpu().numpy()

    def dequantize(self) -> torch.Tensor:
        """f32 ``[n_expert, n_out, k]`` on the device (``QTensor::dequantize``)."""
        out = torch.empty(self.n_expert, self.n_out, self.k, dtype=torch.float32, device=self.buffer.device)
        _native.check(_native.lib().lmoe_dequantize(self.dtype, self.buffer.data_ptr() + self.base_off,
                                                    out.numel() // QK_K, out.data_ptr(), stream_ptr()))
        return out

    def slice_experts(self, first: int, count: int) -> "ExpertStack":
        """Zero-copy sub-stack of experts ``[first, first+count)`` (expert-parallel shards)."""
        per = self.n_out * (self.k // QK_K) * TYPE_SIZE[self.dtype]
        return ExpertStack(self.buffer, self.dtype, count, self.n_out, self.k, self.base_off + first * per)
