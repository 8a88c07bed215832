"""Host mirror of the reference's ``src/moe.rs`` for the B200 backend.

  ExpertFfn       src/moe.rs:19-21   forward(x, ids, weights) -> [seq, hidden]
  MoeBlock        src/moe.rs:28-79   route -> experts -> + shared expert
  FusedExperts    src/moe.rs:194-324 op-by-op runner over ``ops`` (mv_id / mm_id)
  SharedExpert    src/moe.rs:327-345 the always-on SwiGLU expert
``MoeBlock.forward`` runs the whole block through the fused CUDA entry points
(``lmoe_moe_forward_decode`` / ``_prefill``); ``MoeBlock.forward_unfused``
follows the reference's op-by-op sequence and exists for op-level parity.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import ops
from ._native import LmoeError, check, lib
from .gguf import Q4_K, Q6_K, ExpertStack, stream_ptr

WEIGHTS_SUM_FLOOR = 6.103515625e-5  # src/moe.rs:14


class ExpertFfn:
    """`ExpertFfn`, src/moe.rs:19-21."""

    def forward(self, x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class FusedExperts(ExpertFfn):
    """`FusedExperts`, src/moe.rs:194-324: the stacks stay quantized, ids stay on the GPU."""

    def __init__(self, gate: ExpertStack, up: ExpertStack, down: ExpertStack):
        if not (gate.n_expert == up.n_expert == down.n_expert):
            raise LmoeError(-1, f"MoE expert stacks disagree on n_expert: gate={gate.n_expert}, "
                                f"up={up.n_expert}, down={down.n_expert}")
        self.gate, self.up, self.down = gate, up, down

    def forward(self, x, ids, weights, use_mm=None):
        """`use_mm`: None applies the `seq >= mm_id_min_seq()` rule of src/moe.rs:236-240; True / False force
        the grouped-GEMM or the mat-vec op chain."""
        seq, hidden = x.shape
        top_k = ids.shape[1]
        x = x.to(torch.float32)
        mm_supported = all(ops.supported(s.dtype, top_k) for s in (self.gate, self.up, self.down))
        use_mm = (seq >= ops.mm_id_min_seq() if use_mm is None else bool(use_mm)) and mm_supported
        map0 = ops.prepare_map0(self.gate.n_expert, ids) if use_mm else None

        def matmul(stack, xin):
            if map0 is not None:
                return ops.mul_mm_id_shared(stack, xin, ids, map0)
            return ops.mul_mv_id(stack, xin, ids)

        x_g = x.reshape(seq, 1, hidden).contiguous()
        gate = matmul(self.gate, x_g)
        up = matmul(self.up, x_g)
        act = ops.silu_mul(gate, up)
        w = weights.to(torch.float32)
        if use_mm:
            # the grouped GEMM stages the activation as f16: keep it in range with the
            # per-(token, slot) L2 rescale and undo it in the combine (src/moe.rs:292-313)
            col_l2 = act.square().sum(2, keepdim=True).sqrt().clamp(1e-8, 1e30)
            act_s = (act * 32768.0) / col_l2
            down = matmul(self.down, act_s.contiguous())
            return ops.combine(down, col_l2.contiguous(), w)
        down = matmul(self.down, act)
        return ops.combine(down, None, w)


class SharedExpert:
    """`SharedExpert`, src/moe.rs:327-345 + `swiglu`, src/moe.rs:369-374."""

    def __init__(self, gate: ExpertStack, up: ExpertStack, down: ExpertStack):
        self.gate, self.up, self.down = gate, up, down

    def forward(self, x):
        seq, hidden = x.shape
        zeros = torch.zeros(seq, 1, dtype=torch.int32, device=x.device)
        xg = x.reshape(seq, 1, hidden).contiguous()
        g = ops.mul_mv_id(self.gate, xg, zeros)
        u = ops.mul_mv_id(self.up, xg, zeros)
        h = ops.silu_mul(g, u)
        return ops.mul_mv_id(self.down, h, zeros).reshape(seq, hidden)


class MoeBlock:
    """`MoeBlock`, src/moe.rs:28-79.

    ``router`` is ``[n_expert, hidden]`` (the GGUF ``ffn_gate_inp`` orientation; the
    reference transposes it at load only to feed candle's matmul, src/moe.rs:43).
    """

    def __init__(self, router: torch.Tensor, exp_probs_b, gate: ExpertStack, up: ExpertStack, down: ExpertStack,
                 shared_gate: ExpertStack = None, shared_up: ExpertStack = None, shared_down: ExpertStack = None,
                 n_expert_used: int = 10, weights_scale: float = 2.5, weights_norm: bool = True):
        self.router = router.contiguous()
        self.exp_probs_b = None if exp_probs_b is None else exp_probs_b.contiguous()
        self.experts = FusedExperts(gate, up, down)
        self.shared = SharedExpert(shared_gate, shared_up, shared_down) if shared_gate is not None else None
        self.n_expert_used, self.weights_scale, self.weights_norm = n_expert_used, weights_scale, weights_norm
        self.hidden, self.expert_ff, self.n_expert = gate.k, gate.n_out, gate.n_expert
        h = C.c_void_p()
        hp = lambda s: None if s is None else s.handle
        check(lib().lmoe_layer_create(self.hidden, self.expert_ff, self.n_expert, n_expert_used, weights_scale,
                                      int(weights_norm), self.router.data_ptr(),
                                      None if self.exp_probs_b is None else self.exp_probs_b.data_ptr(),
                                      gate.handle, up.handle, down.handle, hp(shared_gate), hp(shared_up),
                                      hp(shared_down), C.byref(h)))
        self._h = h
        self._ws = None
        self._ws_tokens = 0

    def __del__(self):
        h = getattr(self, "_h", None)
        if h:
            try:
                lib().lmoe_layer_destroy(h)
            except Exception:  # interpreter shutdown: the library is already gone
                pass
            self._h = None

    @property
    def handle(self):
        return self._h

    # ---- synthetic layer ----------------------------------------------------
    @classmethod
    def random(cls, hidden=3072, expert_ff=1024, n_expert=256, top_k=10, seed=0, device="cuda", shared=True,
               weight_std=0.02, bias=None, gate_dtype=Q4_K, down_dtype=Q6_K):
        """Seeded synthetic layer: expert weights N(0, 0.02) encoded on the device,
        router N(0, 0.02), selection bias U(-0.1, 0.1) unless ``bias`` is given."""
        gen = torch.Generator(device=device)
        gen.manual_seed(seed * 7919 + 11)
        router = torch.randn(n_expert, hidden, generator=gen, device=device) * 0.02
        if bias is None:
            bias = torch.rand(n_expert, generator=gen, device=device) * 0.2 - 0.1
        mk = lambda dt, ne, no, k, s: ExpertStack.random(dt, ne, no, k, std=weight_std, seed=seed * 1000 + s, device=device)
        gate = mk(gate_dtype, n_expert, expert_ff, hidden, 1)
        up = mk(gate_dtype, n_expert, expert_ff, hidden, 2)
        down = mk(down_dtype, n_expert, hidden, expert_ff, 3)
        sg = su = sd = None
        if shared:
            sg = mk(gate_dtype, 1, expert_ff, hidden, 4)
            su = mk(gate_dtype, 1, expert_ff, hidden, 5)
            sd = mk(down_dtype, 1, hidden, expert_ff, 6)
        return cls(router, bias, gate, up, down, sg, su, sd, top_k)

    # ---- reference-shaped API ----------------------------------------------
    def route(self, x_normed: torch.Tensor):
        """`MoeBlock::route`, src/moe.rs:62-71 -> (ids [seq, top_k], weights [seq, top_k])."""
        return ops.route(self.router, self.exp_probs_b, x_normed.to(torch.float32).contiguous(),
                         self.n_expert_used, self.weights_scale, self.weights_norm)

    def forward_unfused(self, x_normed: torch.Tensor, use_mm=None) -> torch.Tensor:
        """The reference's op-by-op sequence, src/moe.rs:73-78."""
        x = x_normed.to(torch.float32).contiguous()
        ids, weights = self.route(x)
        routed = self.experts.forward(x, ids, weights, use_mm)
        if self.shared is None:
            return routed
        return routed + self.shared.forward(x)

    def workspace(self, tokens: int) -> torch.Tensor:
        if self._ws is None or tokens > self._ws_tokens:
            n = lib().lmoe_layer_workspace_bytes(self._h, tokens)
            self._ws = torch.zeros(n, dtype=torch.uint8, device=self.router.device)
            self._ws_tokens = tokens
        return self._ws

    def forward(self, x_normed: torch.Tensor, return_routing: bool = False, out: torch.Tensor = None,
                path: str = None):
        """`MoeBlock::forward`, src/moe.rs:73-78, through the fused CUDA entry points.  `path`: None picks
        the mat-vec kernel below `ops.mm_id_min_seq()` tokens and the grouped GEMM from there on (the same
        rule as `lmoe_moe_forward_host` / `lmoe_moe_layer_forward`); "decode" / "prefill" force one."""
        x = x_normed.to(torch.float32).contiguous()
        seq = x.shape[0]
        if x.dim() != 2 or x.shape[1] != self.hidden:
            raise LmoeError(-1, f"x must be [seq, {self.hidden}], got {tuple(x.shape)}")
        if out is None:
            out = torch.empty(seq, self.hidden, dtype=torch.float32, device=x.device)
        ids = w = None
        if return_routing:
            ids = torch.empty(seq, self.n_expert_used, dtype=torch.int32, device=x.device)
            w = torch.empty(seq, self.n_expert_used, dtype=torch.float32, device=x.device)
        ws = self.workspace(seq)
        if path not in (None, "decode", "prefill"):
            raise LmoeError(-1, f"path must be None, 'decode' or 'prefill', got {path!r}")
        prefill = path == "prefill" or (path is None and seq >= ops.mm_id_min_seq())
        fn = lib().lmoe_moe_forward_prefill if prefill else lib().lmoe_moe_forward_decode
        check(fn(self._h, x.data_ptr(), seq, out.data_ptr(), None if ids is None else ids.data_ptr(),
                 None if w is None else w.data_ptr(), ws.data_ptr(), ws.numel(), stream_ptr()))
        return (out, ids, w) if return_routing else out

    def experts_forward(self, x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, add_shared: bool = False):
        """`ExpertFfn::forward`, src/moe.rs:19-21, through the fused kernels (`lmoe_experts_forward`): the
        routing decision is the caller's; ids >= n_expert are empty slots."""
        x = x.to(torch.float32).contiguous()
        seq = x.shape[0]
        if x.dim() != 2 or x.shape[1] != self.hidden:
            raise LmoeError(-1, f"x must be [seq, {self.hidden}], got {tuple(x.shape)}")
        if tuple(ids.shape) != (seq, self.n_expert_used) or tuple(weights.shape) != (seq, self.n_expert_used):
            raise LmoeError(-1, f"ids / weights must be [{seq}, {self.n_expert_used}]")
        ids = ids.contiguous()
        weights = weights.to(torch.float32).contiguous()
        out = torch.empty(seq, self.hidden, dtype=torch.float32, device=x.device)
        n = lib().lmoe_experts_workspace_bytes(self._h, seq)
        if getattr(self, "_ews", None) is None or self._ews.numel() < n:
            self._ews = torch.empty(n, dtype=torch.uint8, device=x.device)
        check(lib().lmoe_experts_forward(self._h, x.data_ptr(), ids.data_ptr(), weights.data_ptr(), seq, int(add_shared),
                                         out.data_ptr(), self._ews.data_ptr(), self._ews.numel(), stream_ptr()))
        return out

    def layer_forward(self, ffn_inp: torch.Tensor, norm_weight: torch.Tensor, eps: float = 1e-6,
                      return_routing: bool = False):
        """`lmoe_moe_layer_forward`: ``ffn_inp + MoeBlock::forward(ffn_norm(ffn_inp))``, src/model.rs:340-350."""
        x = ffn_inp.to(torch.float32).contiguous()
        seq = x.shape[0]
        if x.dim() != 2 or x.shape[1] != self.hidden:
            raise LmoeError(-1, f"ffn_inp must be [seq, {self.hidden}], got {tuple(x.shape)}")
        g = norm_weight.to(torch.float32).contiguous()
        out = torch.empty(seq, self.hidden, dtype=torch.float32, device=x.device)
        ids = w = None
        if return_routing:
            ids = torch.empty(seq, self.n_expert_used, dtype=torch.int32, device=x.device)
            w = torch.empty(seq, self.n_expert_used, dtype=torch.float32, device=x.device)
        n = lib().lmoe_moe_layer_workspace_bytes(self._h, seq)
        if getattr(self, "_lws", None) is None or self._lws.numel() < n:
            self._lws = torch.zeros(n, dtype=torch.uint8, device=x.device)
        check(lib().lmoe_moe_layer_forward(self._h, x.data_ptr(), g.data_ptr(), eps, seq, out.data_ptr(),
                                           None if ids is None else ids.data_ptr(), None if w is None else w.data_ptr(),
                                           self._lws.data_ptr(), self._lws.numel(), stream_ptr()))
        return (out, ids, w) if return_routing else out

    def forward_host(self, x_host: torch.Tensor, out_host: torch.Tensor = None, sync: bool = True):
        """Host-buffer call (x and result in pinned host memory), `lmoe_moe_forward_host`; with ``sync=False``
        `lmoe_moe_forward_host_async`: the result is valid once the current stream has been synchronised."""
        assert not x_host.is_cuda and x_host.dtype == torch.float32 and x_host.is_contiguous()
        seq = x_host.shape[0]
        if out_host is None:
            out_host = torch.empty(seq, self.hidden, dtype=torch.float32).pin_memory()
        ws = self.workspace(seq)
        fn = lib().lmoe_moe_forward_host if sync else lib().lmoe_moe_forward_host_async
        check(fn(self._h, x_host.data_ptr(), seq, out_host.data_ptr(), None, None, ws.data_ptr(), ws.numel(), stream_ptr()))
        return out_host

    # ---- expert-parallel pieces (rows already dispatched to this GPU) -------------------
    def _rows_ws(self, rows: int) -> torch.Tensor:
        n = lib().lmoe_rows_workspace_bytes(self._h, rows)
        if getattr(self, "_rws", None) is None or self._rws.numel() < n:
            self._rws = torch.zeros(n, dtype=torch.uint8, device=self.router.device)
        return self._rws

    def experts_forward_rows(self, x: torch.Tensor, local_ids: torch.Tensor, row_w: torch.Tensor) -> torch.Tensor:
        """`lmoe_experts_forward_rows` (`_f16` for half-precision rows): y[r] = row_w[r] * FFN_{local_ids[r]}(x[r])."""
        f16 = x.dtype == torch.float16
        x = (x if f16 else x.to(torch.float32)).contiguous()
        rows = x.shape[0]
        out = torch.empty(rows, self.hidden, dtype=torch.float32, device=x.device)
        ws = self._rows_ws(rows)
        fn = lib().lmoe_experts_forward_rows_f16 if f16 else lib().lmoe_experts_forward_rows
        check(fn(self._h, x.data_ptr(), local_ids.contiguous().data_ptr(), row_w.contiguous().data_ptr(), rows,
                 out.data_ptr(), ws.data_ptr(), ws.numel(), stream_ptr()))
        return out

    def experts_forward_tokens(self, x: torch.Tensor, ids: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        """`lmoe_experts_forward_tokens_f16`: x [t, hidden] f16, ids / w [t, k] (id >= local expert count = empty
        slot) -> [t, hidden] f32, the slot-order sum of the weighted local experts of every token."""
        x = x.to(torch.float16).contiguous()
        t, k = ids.shape
        out = torch.empty(t, self.hidden, dtype=torch.float32, device=x.device)
        n = lib().lmoe_tokens_workspace_bytes(self._h, t, k)
        if getattr(self, "_tws", None) is None or self._tws.numel() < n:
            self._tws = torch.zeros(n, dtype=torch.uint8, device=self.router.device)
        check(lib().lmoe_experts_forward_tokens_f16(self._h, x.data_ptr(), ids.contiguous().data_ptr(),
                                                    w.contiguous().data_ptr(), t, k, out.data_ptr(),
                                                    self._tws.data_ptr(), self._tws.numel(), stream_ptr()))
        return out

    def shared_forward(self, x: torch.Tensor) -> torch.Tensor:
        """`lmoe_shared_forward`: the shared expert alone."""
        x = x.to(torch.float32).contiguous()
        out = torch.empty(x.shape[0], self.hidden, dtype=torch.float32, device=x.device)
        # a workspace of its own: the shared expert may run on a side stream beside the routed experts
        n = lib().lmoe_rows_workspace_bytes(self._h, x.shape[0])
        if getattr(self, "_sws", None) is None or self._sws.numel() < n:
            self._sws = torch.zeros(n, dtype=torch.uint8, device=self.router.device)
        ws = self._sws
        check(lib().lmoe_shared_forward(self._h, x.data_ptr(), x.shape[0], out.data_ptr(), ws.data_ptr(), ws.numel(),
                                        stream_ptr()))
        return out

    def shard(self, rank: int, world: int) -> "MoeBlock":
        """Zero-copy expert-parallel shard: experts [rank*E/world, (rank+1)*E/world), shared expert kept."""
        e = self.experts
        n = self.n_expert // world
        sh = self.shared
        return MoeBlock(self.router[rank * n:(rank + 1) * n], None, e.gate.slice_experts(rank * n, n),
                        e.up.slice_experts(rank * n, n), e.down.slice_experts(rank * n, n),
                        None if sh is None else sh.gate, None if sh is None else sh.up,
                        None if sh is None else sh.down, min(self.n_expert_used, n), self.weights_scale,
                        self.weights_norm)

    def check_device_flag(self):
        """Raise if any call on this block recorded a device flag: every workspace the block has used
        (block, layer, row-level, token-level and shared-expert entries) is inspected."""
        for name in ("_ws", "_lws", "_rws", "_tws", "_sws", "_ews"):
            ws = getattr(self, name, None)
            if ws is not None:
                check(lib().lmoe_check_device_flag(ws.data_ptr(), stream_ptr()))

    # ---- checker support ------------------------------------------------------
    def host_layer(self, orc):
        """The same weights as an ``oracle.HostLayer`` (tests and the CPU baseline only)."""
        e = self.experts
        sh = self.shared
        return orc.HostLayer(self.hidden, self.expert_ff, self.n_expert, self.n_expert_used,
                             self.router.cpu().numpy(),
                             None if self.exp_probs_b is None else self.exp_probs_b.cpu().numpy(),
                             e.gate.raw(), e.up.raw(), e.down.raw(),
                             None if sh is None else sh.gate.raw(), None if sh is None else sh.up.raw(),
                             None if sh is None else sh.down.raw(), self.weights_scale, self.weights_norm,
                             e.gate.dtype, e.down.dtype)
