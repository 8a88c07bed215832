"""GGUF container reader for the MoE path: tensor directory, raw quantized bytes, `ExpertStack` upload.

Mirror of the part of the reference's loader that feeds the fused MoE block:
``Weights::expert_stack`` (src/gguf.rs:554-607: rank-3 ``[n_expert, n_out, k]`` stacks uploaded as the
file's bytes, no re-layout), ``QLinear`` for the shared expert (src/gguf.rs:207-242) and the tensor
names used by ``MoeBlock::new`` / ``FusedExperts::new`` / ``SharedExpert::new`` (src/moe.rs:43-44,
134-136, 336-338).  Only the container format is parsed here (GGUF v2/v3: header, key/value section,
tensor infos, aligned data section); the file is memory-mapped and tensor bytes are handed out as
zero-copy views, so a 75 GB checkpoint is never read into host memory as a whole.
"""
from __future__ import annotations

import mmap
import struct
from dataclasses import dataclass

import numpy as np
import torch

from .gguf import Q4_K, Q6_K, ExpertStack

GGUF_MAGIC = 0x46554747  # "GGUF" little endian
F32, F16 = 0, 1
# ggml type -> (elements per block, bytes per block)
BLOCK = {F32: (1, 4), F16: (1, 2), Q4_K: (256, 144), Q6_K: (256, 210), 8: (32, 34), 13: (256, 176)}
_SCALAR = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}
_STRING, _ARRAY = 8, 9


class GgufError(ValueError):
    pass


@dataclass
class TensorInfo:
    name: str
    shape: tuple      # outermost first (the reference's / candle's order; the file stores it reversed)
    ggml_type: int
    offset: int       # from the start of the data section
    nbytes: int


class _Cursor:
    def __init__(self, buf):
        self.buf, self.pos = buf, 0

    def take(self, fmt):
        size = struct.calcsize(fmt)
        if self.pos + size > len(self.buf):
            raise GgufError("GGUF file is truncated")
        v = struct.unpack_from(fmt, self.buf, self.pos)[0]
        self.pos += size
        return v

    def string(self):
        n = self.take("<Q")
        if self.pos + n > len(self.buf):
            raise GgufError("GGUF file is truncated inside a string")
        s = bytes(self.buf[self.pos:self.pos + n]).decode("utf-8", errors="replace")
        self.pos += n
        return s

    def value(self, vtype):
        if vtype in _SCALAR:
            return self.take(_SCALAR[vtype])
        if vtype == _STRING:
            return self.string()
        if vtype == _ARRAY:
            itype, count = self.take("<I"), self.take("<Q")
            if itype in _SCALAR and itype != 7:
                fmt = _SCALAR[itype][1]
                size = struct.calcsize("<" + fmt)
                if self.pos + size * count > len(self.buf):
                    raise GgufError("GGUF file is truncated inside an array")
                arr = np.frombuffer(self.buf, dtype=np.dtype("<" + fmt), count=count, offset=self.pos)
                self.pos += size * count
                return arr
            return [self.value(itype) for _ in range(count)]
        raise GgufError(f"unknown GGUF value type {vtype}")


class GgufFile:
    """A memory-mapped GGUF file: ``kv`` (metadata), ``tensors`` (name -> TensorInfo), raw tensor views."""

    def __init__(self, path: str):
        self.path = path
        self._f = open(path, "rb")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        c = _Cursor(self._mm)
        if len(self._mm) < 24 or c.take("<I") != GGUF_MAGIC:
            raise GgufError(f"{path}: not a GGUF file")
        self.version = c.take("<I")
        if self.version not in (2, 3):
            raise GgufError(f"{path}: GGUF version {self.version} is not supported (2 and 3 are)")
        n_tensors, n_kv = c.take("<Q"), c.take("<Q")
        self.kv = {}
        for _ in range(n_kv):
            key = c.string()
            self.kv[key] = c.value(c.take("<I"))
        self.alignment = int(self.kv.get("general.alignment", 32))
        self.tensors = {}
        for _ in range(n_tensors):
            name = c.string()
            n_dims = c.take("<I")
            ne = [c.take("<Q") for _ in range(n_dims)]
            ggml_type, offset = c.take("<I"), c.take("<Q")
            if ggml_type not in BLOCK:
                nbytes = -1        # a type this path never touches; reported when the tensor is asked for
            else:
                per, size = BLOCK[ggml_type]
                elems = int(np.prod(ne, dtype=np.int64)) if ne else 1
                if ne and ne[0] % per:
                    raise GgufError(f"{name}: innermost dimension {ne[0]} is not a multiple of the block size {per}")
                nbytes = elems // per * size
            self.tensors[name] = TensorInfo(name, tuple(reversed(ne)), ggml_type, offset, nbytes)
        self.data_offset = (c.pos + self.alignment - 1) // self.alignment * self.alignment
        for t in self.tensors.values():
            if t.nbytes >= 0 and self.data_offset + t.offset + t.nbytes > len(self._mm):
                raise GgufError(f"{t.name}: data runs past the end of the file")

    def close(self):
        self._mm.close()
        self._f.close()

    def info(self, name: str) -> TensorInfo:
        if name not in self.tensors:
            raise GgufError(f"tensor {name} not found in {self.path}")
        t = self.tensors[name]
        if t.nbytes < 0:
            raise GgufError(f"{name}: ggml type {t.ggml_type} is not supported")
        return t

    def raw(self, name: str) -> np.ndarray:
        """The tensor's bytes as a zero-copy uint8 view of the mapping."""
        t = self.info(name)
        return np.frombuffer(self._mm, dtype=np.uint8, count=t.nbytes, offset=self.data_offset + t.offset)

    def f32(self, name: str, device="cpu") -> torch.Tensor:
        """An F32 or F16 tensor as float32, in the reference's dimension order."""
        t = self.info(name)
        if t.ggml_type == F32:
            a = self.raw(name).view(np.float32)
        elif t.ggml_type == F16:
            a = self.raw(name).view(np.float16).astype(np.float32)
        else:
            raise GgufError(f"{name}: expected F32/F16, found ggml type {t.ggml_type}")
        return torch.from_numpy(np.array(a).reshape(t.shape)).to(device)

    def expert_stack(self, name: str, device="cuda") -> ExpertStack:
        """Rank-3 ``[n_expert, n_out, k]`` quantized stack, uploaded byte for byte (src/gguf.rs:567-607).
        A rank-2 ``[n_out, k]`` tensor (the shared expert's projections) becomes a one-expert stack."""
        t = self.info(name)
        if t.ggml_type not in (Q4_K, Q6_K):
            raise GgufError(f"{name}: ggml type {t.ggml_type} has no fused kernels (Q4_K and Q6_K do)")
        if len(t.shape) == 3:
            n_expert, n_out, k = t.shape
        elif len(t.shape) == 2:
            n_expert, (n_out, k) = 1, t.shape
        else:
            raise GgufError(f"{name} is not a rank-3 expert stack: {list(t.shape)}")
        return ExpertStack.from_bytes(self.raw(name), t.ggml_type, n_expert, n_out, k, device=device)

    # ---- the MoE block of one layer ---------------------------------------------------
    def moe_config(self, arch: str = "laguna") -> dict:
        """Routing hyper-parameters as the reference reads them (src/config.rs:124-129)."""
        kv = self.kv
        if f"{arch}.expert_used_count" not in kv:
            raise GgufError(f"{self.path}: metadata key {arch}.expert_used_count is missing")
        return {
            "n_expert_used": int(kv[f"{arch}.expert_used_count"]),
            "weights_scale": float(kv.get(f"{arch}.expert_weights_scale", 2.5)),
            "weights_norm": bool(kv.get(f"{arch}.expert_weights_norm", True)),
            "rms_eps": float(kv.get(f"{arch}.attention.layer_norm_rms_epsilon", 1e-6)),
        }

    def moe_block(self, layer: int, device="cuda", arch: str = "laguna", **overrides):
        """`MoeBlock::new` (src/moe.rs:41-60) for layer `layer`: router `ffn_gate_inp`, selection bias
        `exp_probs_b` (`.weight`, else `.bias`: src/gguf.rs:676-687), the three routed stacks
        `ffn_{gate,up,down}_exps` and, when present, the shared expert `ffn_{gate,up,down}_shexp`."""
        from .moe import MoeBlock

        cfg = {**self.moe_config(arch), **overrides}
        p = f"blk.{layer}."
        router = self.f32(p + "ffn_gate_inp.weight", device)
        bias_name = p + "exp_probs_b.weight" if p + "exp_probs_b.weight" in self.tensors else p + "exp_probs_b.bias"
        bias = self.f32(bias_name, device).reshape(-1)
        gate, up, down = (self.expert_stack(p + f"ffn_{n}_exps.weight", device) for n in ("gate", "up", "down"))
        if router.dim() != 2 or tuple(router.shape) != (gate.n_expert, gate.k):
            raise GgufError(f"{p}ffn_gate_inp.weight is {list(router.shape)}, expected [{gate.n_expert}, {gate.k}]")
        if bias.numel() != gate.n_expert:
            raise GgufError(f"{bias_name} has {bias.numel()} entries, expected {gate.n_expert}")
        shared = [None, None, None]
        if p + "ffn_gate_shexp.weight" in self.tensors:
            shared = [self.expert_stack(p + f"ffn_{n}_shexp.weight", device) for n in ("gate", "up", "down")]
        return MoeBlock(router, bias, gate, up, down, *shared, n_expert_used=cfg["n_expert_used"],
                        weights_scale=cfg["weights_scale"], weights_norm=cfg["weights_norm"])

    def ffn_norm(self, layer: int, device="cuda") -> torch.Tensor:
        """The RMS-norm weight applied before the block (`ffn_norm`, src/model.rs:340)."""
        return self.f32(f"blk.{layer}.ffn_norm.weight", device).reshape(-1)
