"""Expert-parallel MoE block: experts sharded over ranks, tokens data-parallel.

The reference engine is single-GPU; this is new.  Rank r owns the routed experts
``[r*E/G, (r+1)*E/G)``; the router, its bias and the shared expert are replicated;
every rank routes its own tokens (the router is replicated, so expert ids are
identical to the single-GPU result by construction).  One exchange before the
experts (dispatch of routed rows) and one after (return of the weighted rows),
both ``torch.distributed.all_to_all_single`` (NCCL over NVLink on GPUs, gloo in
the CPU tests).  The source rank sums the K returned rows of a token in slot
order and adds the shared expert, exactly like the single-GPU path.

The expert math is supplied as two callables so that the host logic can be
exercised on CPU ranks:
  rows_fn(x_rows[payload dtype R,H], local_ids[i32 R], row_w[f32 R]) -> y[f32 R,H]
  shared_fn(x[f32 T,H]) -> y[f32 T,H]  (or None)
  combine_fn(y[f32 T,K,H]) -> out[f32 T,H], the slot-order sum (optional; a plain loop otherwise)
  pack_fn(x, ids, w) -> (rows, local_ids, row_w, row_pos, send_counts) and
  combine_rows_fn(rows_back, row_pos, shared_or_None, t) -> out: the device-side packing of the
  dispatch and the fused return-leg sum (`lmoe_ep_pack` / `lmoe_ep_combine`); optional, the torch
  index arithmetic of `plan` is used otherwise.
On GPUs the shared expert runs on a side stream while the dispatch is in flight.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


class ExpertParallelMoe:
    def __init__(self, route_fn, rows_fn, shared_fn, n_expert: int, top_k: int, group=None,
                 payload_dtype=torch.float16, combine_fn=None, pack_fn=None, combine_rows_fn=None):
        self.route_fn, self.rows_fn, self.shared_fn = route_fn, rows_fn, shared_fn
        self.combine_fn = combine_fn
        self.pack_fn, self.combine_rows_fn = pack_fn, combine_rows_fn
        self._side = None
        self.n_expert, self.top_k = n_expert, top_k
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if n_expert % self.world:
            raise ValueError(f"n_expert ({n_expert}) must divide over {self.world} ranks")
        self.e_local = n_expert // self.world
        self.payload_dtype = payload_dtype
        self.last_stats = {}

    # -- the exchange plan (pure index arithmetic; covered by the CPU tests) --------
    def plan(self, ids: torch.Tensor):
        """ids [T,K] -> (order, send_counts): rows sorted by destination rank, stably."""
        flat = ids.reshape(-1).to(torch.int64)
        dest = flat // self.e_local
        order = torch.sort(dest, stable=True).indices
        send_counts = torch.bincount(dest, minlength=self.world)
        return order, send_counts

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        t, h = x.shape
        k = self.top_k
        ids, w = self.route_fn(x)                       # [T,K] int32 (u32 bits), [T,K] f32
        dev = x.device
        packed = self.pack_fn is not None and self.combine_rows_fn is not None
        if packed:
            xs, meta_ids, meta_w, row_pos, send_counts = self.pack_fn(x, ids, w)
        else:
            order, send_counts = self.plan(ids)
        # counts exchange (G x G int64)
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=self.group)
        sc, rc = send_counts.tolist(), recv_counts.tolist()
        n_send, n_recv = sum(sc), sum(rc)
        # the shared expert needs nothing from the exchange: on GPUs it runs beside it
        shared = None
        if self.shared_fn is not None and x.is_cuda:
            if self._side is None:
                self._side = torch.cuda.Stream(device=dev)
            self._side.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(self._side):
                shared = self.shared_fn(x)
        if not packed:
            # dispatch payloads: activations (f16 on the wire: the grouped GEMM consumes f16 operands
            # rounded the same way), local expert id, routing weight
            tok = order // k
            xs = x.to(self.payload_dtype).index_select(0, tok)
            meta_ids = (ids.reshape(-1).to(torch.int64).index_select(0, order) % self.e_local).to(torch.int32)
            meta_w = w.reshape(-1).index_select(0, order).contiguous()
        xr = torch.empty(n_recv, h, dtype=xs.dtype, device=dev)
        dist.all_to_all_single(xr, xs, rc, sc, group=self.group)
        # expert id and routing weight travel together: one [rows, 2] array of 32-bit words
        meta = torch.stack([meta_ids.view(torch.int32), meta_w.view(torch.int32)], dim=1)
        meta_r = torch.empty(n_recv, 2, dtype=torch.int32, device=dev)
        dist.all_to_all_single(meta_r, meta, rc, sc, group=self.group)
        ir = meta_r[:, 0].contiguous()
        wr = meta_r[:, 1].contiguous().view(torch.float32)
        # local experts on the received rows
        yr = self.rows_fn(xr, ir, wr) if n_recv else torch.empty(0, h, dtype=torch.float32, device=dev)
        # combine exchange: rows go back to where they came from, in the order they were sent
        ys = torch.empty(n_send, h, dtype=torch.float32, device=dev)
        dist.all_to_all_single(ys, yr.contiguous(), sc, rc, group=self.group)
        if shared is not None:
            torch.cuda.current_stream(dev).wait_stream(self._side)
        elif self.shared_fn is not None:
            shared = self.shared_fn(x)
        if packed:
            out = self.combine_rows_fn(ys, row_pos, shared, t)
        else:
            y = torch.empty(t * k, h, dtype=torch.float32, device=dev)
            y.index_copy_(0, order, ys)
            y3 = y.view(t, k, h)
            if self.combine_fn is not None:
                out = self.combine_fn(y3)
            else:
                out = torch.zeros(t, h, dtype=torch.float32, device=dev)
                for s_ in range(k):                     # fixed slot order, like the single-GPU combine
                    out += y3[:, s_]
            if shared is not None:
                out += shared
        self.last_stats = {"rows_sent": n_send, "rows_received": n_recv,
                           "remote_rows_sent": n_send - sc[self.rank]}
        return out


def make_gpu_ep_block(full_router, bias, local_block, n_expert, top_k, scale=2.5, norm=True, group=None):
    """Bind the exchange logic to the CUDA entry points of a local `MoeBlock` shard."""
    from . import ops

    def route_fn(x):
        return ops.route(full_router, bias, x, top_k, scale, norm)

    def combine_fn(y3):
        # the fused slot-order sum with unit weights (multiplying by 1.0 changes nothing)
        return ops.combine(y3, None, torch.ones(y3.shape[0], y3.shape[1], dtype=torch.float32, device=y3.device))

    from ._native import check, lib
    from .gguf import stream_ptr

    world = dist.get_world_size(group)
    state = {}

    def pack_fn(x, ids, w):
        t, h = x.shape
        dev = x.device
        n = t * top_k
        rows = torch.empty(n, h, dtype=torch.float16, device=dev)
        local_ids = torch.empty(n, dtype=torch.int32, device=dev)
        row_w = torch.empty(n, dtype=torch.float32, device=dev)
        row_pos = torch.empty(n, dtype=torch.int32, device=dev)
        counts = torch.empty(world, dtype=torch.int64, device=dev)
        need = lib().lmoe_ep_pack_workspace_bytes(n_expert, t)
        if state.get("ws") is None or state["ws"].numel() < need:
            state["ws"] = torch.empty(need, dtype=torch.uint8, device=dev)
        check(lib().lmoe_ep_pack(x.contiguous().data_ptr(), ids.contiguous().data_ptr(), w.contiguous().data_ptr(), t, h, top_k,
                                 n_expert, world, rows.data_ptr(), local_ids.data_ptr(), row_w.data_ptr(), row_pos.data_ptr(),
                                 counts.data_ptr(), state["ws"].data_ptr(), state["ws"].numel(), stream_ptr()))
        return rows, local_ids, row_w, row_pos, counts

    def combine_rows_fn(ys, row_pos, shared, t):
        out = torch.empty(t, ys.shape[1], dtype=torch.float32, device=ys.device)
        check(lib().lmoe_ep_combine(ys.contiguous().data_ptr(), row_pos.data_ptr(), shared.data_ptr() if shared is not None else None,
                                    t, top_k, ys.shape[1], out.data_ptr(), stream_ptr()))
        return out

    return ExpertParallelMoe(route_fn, local_block.experts_forward_rows,
                             local_block.shared_forward if local_block.shared is not None else None,
                             n_expert, top_k, group, combine_fn=combine_fn, pack_fn=pack_fn,
                             combine_rows_fn=combine_rows_fn)
