"""ctypes/numpy front-end of the CPU oracle (``lmoe_oracle.c``).

TEST INFRASTRUCTURE ONLY: imported by the test-suite, the smoke check and the
benchmark's CPU-baseline leg, never by the shipped package.  Each function
below names the C function it calls; that C function cites the reference
file:line it restates.
"""
from __future__ import annotations

import ctypes as C
import hashlib
import os
import subprocess

import numpy as np

Q4_K = 12  # ggml type ids
Q6_K = 14
QK_K = 256
TYPE_SIZE = {Q4_K: 144, Q6_K: 210}

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "liblmoe_oracle.so")
_lib = None


def _cpu_tag() -> str:
    """Identifies the host CPU's instruction set: the baseline unit is compiled with -march=native, so a
    library built on another machine must not be loaded here."""
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("flags"):
                    return hashlib.sha256(line.encode()).hexdigest()[:16]
    except OSError:
        pass
    return "unknown"


def build(force: bool = False) -> str:
    """Compile the oracle with gcc (``make -C oracle``); rebuilt when a source is newer or when the
    existing library was built for a different CPU."""
    srcs = [os.path.join(_HERE, n) for n in ("lmoe_oracle.c", "lmoe_cpu_baseline.c", "lmoe_oracle.h", "Makefile")]
    tag_file = os.path.join(_HERE, "_build", "cpu_tag.txt")
    tag = _cpu_tag()
    stale = (not os.path.exists(_SO) or any(os.path.getmtime(_SO) < os.path.getmtime(p) for p in srcs)
             or not os.path.exists(tag_file) or open(tag_file).read().strip() != tag)
    if force or stale:
        subprocess.run(["make", "-C", _HERE, "-B"], check=True, capture_output=True)
        with open(tag_file, "w") as f:
            f.write(tag)
    return _SO


class Layer(C.Structure):
    """Mirror of ``lmo_layer``."""

    _fields_ = [
        ("hidden", C.c_int), ("expert_ff", C.c_int), ("n_expert", C.c_int), ("top_k", C.c_int),
        ("scale", C.c_float), ("norm", C.c_int),
        ("router", C.c_void_p), ("bias", C.c_void_p),
        ("gate", C.c_void_p), ("up", C.c_void_p), ("down", C.c_void_p),
        ("sh_gate", C.c_void_p), ("sh_up", C.c_void_p), ("sh_down", C.c_void_p),
        ("gate_dtype", C.c_int), ("down_dtype", C.c_int),
    ]


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(_SO)
        _lib.lmo_h2f.restype = C.c_float
        _lib.lmo_h2f.argtypes = [C.c_uint16]
        _lib.lmo_f2h.restype = C.c_uint16
        _lib.lmo_f2h.argtypes = [C.c_float]
        _lib.lmo_sigmoid.restype = C.c_float
        _lib.lmo_sigmoid.argtypes = [C.c_float]
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _u8(a):
    return np.ascontiguousarray(a, dtype=np.uint8)


def _u32(a):
    return np.ascontiguousarray(a, dtype=np.uint32)


def quantize(dtype: int, x: np.ndarray) -> np.ndarray:
    """``lmo_quantize``: f32 ``[..., k]`` -> raw super-block bytes (1-D uint8)."""
    x = _f32(x)
    assert x.size % QK_K == 0
    nb = x.size // QK_K
    out = np.empty(nb * TYPE_SIZE[dtype], np.uint8)
    rc = lib().lmo_quantize(C.c_int(dtype), _p(x), C.c_int64(nb), _p(out))
    assert rc == 0
    return out


def dequantize(dtype: int, blocks: np.ndarray) -> np.ndarray:
    """``lmo_dequantize``: raw bytes -> f32 (1-D)."""
    blocks = _u8(blocks).reshape(-1)
    ts = TYPE_SIZE[dtype]
    assert blocks.size % ts == 0
    nb = blocks.size // ts
    out = np.empty(nb * QK_K, np.float32)
    rc = lib().lmo_dequantize(C.c_int(dtype), _p(blocks), C.c_int64(nb), _p(out))
    assert rc == 0
    return out


def route_logits(router: np.ndarray, x: np.ndarray) -> np.ndarray:
    """``lmo_route_logits``; router ``[E,H]``, x ``[T,H]`` -> ``[T,E]``."""
    router, x = _f32(router), _f32(x)
    e, h = router.shape
    t = x.shape[0]
    out = np.empty((t, e), np.float32)
    lib().lmo_route_logits(_p(router), _p(x), C.c_int(t), C.c_int(h), C.c_int(e), _p(out))
    return out


def rms_norm(x, weight, eps=1e-6) -> np.ndarray:
    """``lmo_rms_norm``: the reference's ``ffn_norm`` (src/model.rs:340), x ``[T,H]``, weight ``[H]``."""
    x, weight = _f32(x), _f32(weight)
    t, h = x.shape
    out = np.empty((t, h), np.float32)
    lib().lmo_rms_norm(_p(x), _p(weight), C.c_float(eps), C.c_int(t), C.c_int(h), _p(out))
    return out


def route_from_logits(logits, bias, top_k, scale=2.5, norm=True):
    """``lmo_route_from_logits`` -> (ids ``[T,K]`` u32, weights ``[T,K]`` f32)."""
    logits = _f32(logits)
    t, e = logits.shape
    bias = None if bias is None else _f32(bias)
    ids = np.empty((t, top_k), np.uint32)
    w = np.empty((t, top_k), np.float32)
    lib().lmo_route_from_logits(_p(logits), _p(bias), C.c_int(t), C.c_int(e), C.c_int(top_k),
                                C.c_float(scale), C.c_int(int(norm)), _p(ids), _p(w))
    return ids, w


def route(router, bias, x, top_k, scale=2.5, norm=True):
    """``lmo_route``: router matmul + routing decision."""
    return route_from_logits(route_logits(router, x), bias, top_k, scale, norm)


def mul_id(dtype, stack, n_expert, n_out, k, x, ids, accum64=False) -> np.ndarray:
    """``lmo_mul_id``: x ``[T, x_per_row, k]``, ids ``[T, top_k]`` -> ``[T, top_k, n_out]``."""
    stack, x, ids = _u8(stack).reshape(-1), _f32(x), _u32(ids)
    t, xpr, kx = x.shape
    assert kx == k and ids.shape[0] == t
    top_k = ids.shape[1]
    out = np.empty((t, top_k, n_out), np.float32)
    rc = lib().lmo_mul_id(C.c_int(dtype), _p(stack), C.c_int(n_expert), C.c_int(n_out), C.c_int(k), _p(x),
                          C.c_int(xpr), _p(ids), C.c_int(t), C.c_int(top_k), _p(out), C.c_int(int(accum64)))
    assert rc == 0, rc
    return out


def mul_mv(dtype, w, n_out, k, x) -> np.ndarray:
    """``lmo_mul_mv``: plain quantized mat-vec, x ``[T,k]`` -> ``[T,n_out]``."""
    w, x = _u8(w).reshape(-1), _f32(x)
    out = np.empty((x.shape[0], n_out), np.float32)
    rc = lib().lmo_mul_mv(C.c_int(dtype), _p(w), C.c_int(n_out), C.c_int(k), _p(x), C.c_int(x.shape[0]), _p(out))
    assert rc == 0
    return out


def silu_mul(gate, up) -> np.ndarray:
    """``lmo_silu_mul``."""
    gate, up = _f32(gate), _f32(up)
    out = np.empty_like(gate)
    lib().lmo_silu_mul(_p(gate), _p(up), C.c_int64(gate.size), _p(out))
    return out


def combine(down, col_l2, w) -> np.ndarray:
    """``lmo_combine``: down ``[S,K,N]``, col_l2 ``[S,K,1]`` or None, w ``[S,K]`` -> ``[S,N]``."""
    down, w = _f32(down), _f32(w)
    col_l2 = None if col_l2 is None else _f32(col_l2)
    s, k, n = down.shape
    out = np.empty((s, n), np.float32)
    lib().lmo_combine(_p(down), _p(col_l2), _p(w), C.c_int(s), C.c_int(k), C.c_int(n), _p(out))
    return out


def map0(ids, n_expert):
    """``lmo_map0`` -> (tpe ``[E]`` u32, ids_map ``[E,T]`` i32, unused entries = -1)."""
    ids = _u32(ids)
    t, k = ids.shape
    tpe = np.zeros(n_expert, np.uint32)
    m = np.full((n_expert, t), -1, np.int32)
    rc = lib().lmo_map0(_p(ids), C.c_int(t), C.c_int(k), C.c_int(n_expert), _p(tpe), _p(m))
    assert rc == 0
    return tpe, m


class HostLayer:
    """One MoE layer's weights on the host (numpy), as the oracle consumes them."""

    def __init__(self, hidden, expert_ff, n_expert, top_k, router, bias, gate, up, down,
                 sh_gate=None, sh_up=None, sh_down=None, scale=2.5, norm=True,
                 gate_dtype=Q4_K, down_dtype=Q6_K):
        self.hidden, self.expert_ff, self.n_expert, self.top_k = hidden, expert_ff, n_expert, top_k
        self.scale, self.norm = scale, norm
        self.router = _f32(router)
        self.bias = None if bias is None else _f32(bias)
        self.gate, self.up, self.down = _u8(gate).reshape(-1), _u8(up).reshape(-1), _u8(down).reshape(-1)
        self.sh_gate = None if sh_gate is None else _u8(sh_gate).reshape(-1)
        self.sh_up = None if sh_up is None else _u8(sh_up).reshape(-1)
        self.sh_down = None if sh_down is None else _u8(sh_down).reshape(-1)
        self.gate_dtype, self.down_dtype = gate_dtype, down_dtype

    def _struct(self) -> Layer:
        pv = lambda a: None if a is None else a.ctypes.data
        return Layer(self.hidden, self.expert_ff, self.n_expert, self.top_k, self.scale, int(self.norm),
                     pv(self.router), pv(self.bias), pv(self.gate), pv(self.up), pv(self.down),
                     pv(self.sh_gate), pv(self.sh_up), pv(self.sh_down), self.gate_dtype, self.down_dtype)

    def forward(self, x, accum64=False):
        """``lmo_moe_forward`` -> (out ``[T,H]``, ids ``[T,K]``, weights ``[T,K]``)."""
        x = _f32(x)
        t = x.shape[0]
        out = np.empty((t, self.hidden), np.float32)
        ids = np.empty((t, self.top_k), np.uint32)
        w = np.empty((t, self.top_k), np.float32)
        s = self._struct()
        rc = lib().lmo_moe_forward(C.byref(s), _p(x), C.c_int(t), _p(out), _p(ids), _p(w), C.c_int(int(accum64)))
        assert rc == 0
        return out, ids, w

    def experts_forward(self, x, ids, weights, accum64=False):
        """``lmo_experts_forward``: the `ExpertFfn` seam (src/moe.rs:19-21) -- caller-supplied routing,
        routed experts only; ids >= n_expert are empty slots."""
        x, ids, weights = _f32(x), _u32(ids), _f32(weights)
        t, k = ids.shape
        out = np.empty((t, self.hidden), np.float32)
        s = self._struct()
        rc = lib().lmo_experts_forward(C.byref(s), _p(x), _p(ids), _p(weights), C.c_int(t), C.c_int(k), _p(out),
                                       C.c_int(int(accum64)))
        assert rc == 0
        return out

    def forward_q8(self, x):
        """``lmo_moe_forward_q8``: the int8-activation CPU convention (timed baseline)."""
        x = _f32(x)
        out = np.empty((x.shape[0], self.hidden), np.float32)
        s = self._struct()
        rc = lib().lmo_moe_forward_q8(C.byref(s), _p(x), C.c_int(x.shape[0]), _p(out))
        assert rc == 0
        return out


def num_threads() -> int:
    return int(lib().lmo_num_threads())


def rel_l2(got, want) -> float:
    """Relative L2 error, src/ops/dispatch.rs:2303-2311 of the reference."""
    got = np.asarray(got, np.float64).ravel()
    want = np.asarray(want, np.float64).ravel()
    return float(np.sqrt(((got - want) ** 2).sum() / max((want ** 2).sum(), 1e-30)))


def pseudo_random(n: int, seed: int, lo: float, hi: float) -> np.ndarray:
    """The reference tests' xorshift generator, src/ops/dispatch.rs:2321-2332."""
    m = (1 << 64) - 1
    s = (seed * 0x9E3779B97F4A7C15 + 1) & m
    out = np.empty(n, np.float32)
    for i in range(n):
        s ^= (s << 13) & m
        s ^= s >> 7
        s ^= (s << 17) & m
        u = (s >> 11) / float(1 << 53)
        out[i] = np.float32(lo) + np.float32(hi - lo) * np.float32(u)
    return out


def random_ids(t, top_k, n_expert, seed) -> np.ndarray:
    """src/ops/dispatch.rs:2334-2339."""
    r = pseudo_random(t * top_k, seed, 0.0, float(n_expert))
    return (r.astype(np.int64) % n_expert).astype(np.uint32).reshape(t, top_k)


def distinct_ids(t, top_k, n_expert, seed) -> np.ndarray:
    """top_k distinct experts per token, src/ops/dispatch.rs:2346-2364."""
    m = (1 << 64) - 1
    s = (seed * 0x9E3779B97F4A7C15 + 1) & m
    out = np.empty((t, top_k), np.uint32)
    for i in range(t):
        chosen = []
        while len(chosen) < top_k:
            s ^= (s << 13) & m
            s ^= s >> 7
            s ^= (s << 17) & m
            e = s % n_expert
            if e not in chosen:
                chosen.append(e)
        out[i] = chosen
    return out
