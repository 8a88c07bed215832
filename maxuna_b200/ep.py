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
  tokens_fn(x[payload dtype N,H], ids[i32 N,K], w[f32 N,K]) -> y[f32 N,H]: the token-level form.  When it
  is given, a token travels to a rank ONCE however many of its K experts live there (ids of the other ranks'
  experts are replaced by the empty-slot id `e_local`), the rank returns one row per token, already summed
  over its local experts in slot order, and the source adds the ranks' rows in rank order, then the shared
  expert.  With K = 10 experts over 2 ranks that is 5x fewer rows each way than the row-level exchange; the
  sum is grouped by rank instead of running in slot order, so it differs from the single-GPU result by f32
  rounding only.  sum_ranks_fn(rows_back, pos[i32 T,G], shared_or_None, t) -> out is the fused form of the
  final sum (`lmoe_ep_combine` with one slot per rank); optional.
On GPUs the shared expert runs on a side stream while the dispatch is in flight.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


class ExpertParallelMoe:
    def __init__(self, route_fn, rows_fn, shared_fn, n_expert: int, top_k: int, group=None,
                 payload_dtype=torch.float16, combine_fn=None, pack_fn=None, combine_rows_fn=None,
                 tokens_fn=None, sum_ranks_fn=None):
        self.route_fn, self.rows_fn, self.shared_fn = route_fn, rows_fn, shared_fn
        self.tokens_fn, self.sum_ranks_fn = tokens_fn, sum_ranks_fn
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

    def plan_tokens(self, ids: torch.Tensor):
        """ids [T,K] -> (tok, dst, send_counts): the (token, destination rank) pairs with at least one of the
        token's experts on that rank, sorted by rank, then token."""
        dest = ids.to(torch.int64) // self.e_local
        mask = torch.zeros(ids.shape[0], self.world, dtype=torch.bool, device=ids.device)
        mask.scatter_(1, dest, True)
        pairs = mask.t().nonzero()                       # row-major over [G,T]: by rank, then by token
        return pairs[:, 1], pairs[:, 0], mask.sum(0)

    def _start_shared(self, x):
        """The shared expert needs nothing from the exchange: on GPUs it runs beside it."""
        if self.shared_fn is None or not x.is_cuda:
            return None
        if self._side is None:
            self._side = torch.cuda.Stream(device=x.device)
        self._side.wait_stream(torch.cuda.current_stream(x.device))
        with torch.cuda.stream(self._side):
            return self.shared_fn(x)

    def _forward_tokens(self, x, ids, w):
        t, h = x.shape
        k, dev = self.top_k, x.device
        tok, dst, send_counts = self.plan_tokens(ids)
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=self.group)
        sc, rc = send_counts.tolist(), recv_counts.tolist()
        n_send, n_recv = sum(sc), sum(rc)
        shared = self._start_shared(x)
        # payloads: the token's activations once per destination; its K (local id, weight) pairs with the
        # other ranks' experts blanked
        xs = x.to(self.payload_dtype).index_select(0, tok)
        ids_t = ids.to(torch.int64).index_select(0, tok)
        mine = (ids_t // self.e_local) == dst[:, None]
        lid = torch.where(mine, ids_t - dst[:, None] * self.e_local, self.e_local).to(torch.int32)
        wt = torch.where(mine, w.index_select(0, tok), 0.0)
        meta = torch.stack([lid, wt.contiguous().view(torch.int32)], dim=2).contiguous()     # [N,K,2] words
        xr = torch.empty(n_recv, h, dtype=xs.dtype, device=dev)
        dist.all_to_all_single(xr, xs, rc, sc, group=self.group)
        meta_r = torch.empty(n_recv, k, 2, dtype=torch.int32, device=dev)
        dist.all_to_all_single(meta_r, meta, rc, sc, group=self.group)
        ir = meta_r[:, :, 0].contiguous()
        wr = meta_r[:, :, 1].contiguous().view(torch.float32)
        yr = self.tokens_fn(xr, ir, wr) if n_recv else torch.empty(0, h, dtype=torch.float32, device=dev)
        ys = torch.empty(n_send, h, dtype=torch.float32, device=dev)
        dist.all_to_all_single(ys, yr.contiguous(), sc, rc, group=self.group)
        if shared is not None:
            torch.cuda.current_stream(dev).wait_stream(self._side)
        elif self.shared_fn is not None:
            shared = self.shared_fn(x)
        if self.sum_ranks_fn is not None:
            pos = torch.full((t, self.world), -1, dtype=torch.int32, device=dev)
            pos[tok, dst] = torch.arange(n_send, dtype=torch.int32, device=dev)
            out = self.sum_ranks_fn(ys, pos, shared, t)
        else:
            out = torch.zeros(t, h, dtype=torch.float32, device=dev)
            o = 0
            for g in range(self.world):                  # rank order; a token appears once per rank
                out.index_add_(0, tok[o:o + sc[g]], ys[o:o + sc[g]])
                o += sc[g]
            if shared is not None:
                out += shared
        self.last_stats = {"rows_sent": n_send, "rows_received": n_recv,
                           "remote_rows_sent": n_send - sc[self.rank]}
        return out

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        t, h = x.shape
        k = self.top_k
        ids, w = self.route_fn(x)                       # [T,K] int32 (u32 bits), [T,K] f32
        if self.tokens_fn is not None:
            return self._forward_tokens(x, ids, w)
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
        shared = self._start_shared(x)
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


def make_gpu_ep_block(full_router, bias, local_block, n_expert, top_k, scale=2.5, norm=True, group=None,
                      token_level=True):
    """Bind the exchange logic to the CUDA entry points of a local `MoeBlock` shard.  `token_level` picks
    the exchange that sends a token once per destination rank (needs Q4_K gate/up and Q6_K down experts);
    False keeps the row-level exchange, whose sum runs in slot order like the single-GPU path."""
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

    def sum_ranks_fn(ys, pos, shared, t):
        out = torch.empty(t, ys.shape[1], dtype=torch.float32, device=ys.device)
        check(lib().lmoe_ep_combine(ys.contiguous().data_ptr(), pos.data_ptr(), shared.data_ptr() if shared is not None else None,
                                    t, world, ys.shape[1], out.data_ptr(), stream_ptr()))
        return out

    return ExpertParallelMoe(route_fn, local_block.experts_forward_rows,
                             local_block.shared_forward if local_block.shared is not None else None,
                             n_expert, top_k, group, combine_fn=combine_fn, pack_fn=pack_fn,
                             combine_rows_fn=combine_rows_fn,
                             tokens_fn=local_block.experts_forward_tokens if token_level else None,
                             sum_ranks_fn=sum_ranks_fn if token_level else None)


class ExpertParallelDecode:
    """Expert-parallel batched decode of one MoE layer (BASELINE config 5: 64 sequences over the ranks).

    Rank r owns the routed experts ``[r*E/G, (r+1)*E/G)`` and ``t_loc`` of the ``T = G*t_loc`` tokens; router,
    bias and shared expert are replicated.  The step is latency-bound, so it uses two fixed-size collectives and
    no host round trip:
      1. all-gather of the normed hidden states: every rank sees all T rows;
      2. every rank routes all T tokens itself (the router is replicated, so the decision is identical on all
         ranks and bit-identical to the single-GPU one) and keeps the slots of its own experts;
      3. one launch of the fused mat-vec kernel streams each local expert that any token selected ONCE, for all
         T tokens, and the shared expert for the rank's own tokens;
      4. all-to-all of the partial rows ([G, t_loc, H]: chunk s goes to the owner of tokens s); the owner adds
         the G partial rows of a token in rank order, then the residual.
    The expert math comes in as callables so that the host logic runs on CPU ranks in the tests:
      norm_fn(x[t_loc,H]) -> [t_loc,H];  route_fn(x[T,H]) -> (ids[T,K] int32, w[T,K] f32);
      localize_fn(ids, first, count) -> local ids (empty slot = count);
      experts_fn(x[T,H], ids_local, w, shared_first, shared_count) -> partial rows [T,H] f32;
      sum_fn(parts[G*t_loc,H], residual[t_loc,H]) -> [t_loc,H] (rank-order sum + residual).
    """

    def __init__(self, norm_fn, route_fn, localize_fn, experts_fn, sum_fn, n_expert: int, group=None, exchange=None):
        self.norm_fn, self.route_fn, self.localize_fn = norm_fn, route_fn, localize_fn
        self.experts_fn, self.sum_fn = experts_fn, sum_fn
        self.group = group
        self.exchange = exchange  # a `PeerExchange`: both exchanges as stores into the peers' memory instead of NCCL
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if n_expert % self.world:
            raise ValueError(f"n_expert ({n_expert}) must divide over {self.world} ranks")
        self.e_local = n_expert // self.world

    def forward(self, ffn_inp: torch.Tensor) -> torch.Tensor:
        """ffn_inp [t_loc, H] (this rank's tokens; t_loc equal on all ranks) -> ffn_inp + block(norm(ffn_inp))."""
        t_loc, h = ffn_inp.shape
        g = self.world
        normed = self.norm_fn(ffn_inp)
        if self.exchange is not None:
            x_all = self.exchange.gather(normed.contiguous())
        else:
            x_all = torch.empty(g * t_loc, h, dtype=normed.dtype, device=normed.device)
            dist.all_gather_into_tensor(x_all, normed.contiguous(), group=self.group)
        ids, w = self.route_fn(x_all)
        ids_local = self.localize_fn(ids, self.rank * self.e_local, self.e_local)
        part = self.experts_fn(x_all, ids_local, w, self.rank * t_loc, t_loc)
        if self.exchange is not None:
            recv = self.exchange.scatter(part.contiguous())
        else:
            recv = torch.empty_like(part)
            dist.all_to_all_single(recv, part.contiguous(), group=self.group)
        return self.sum_fn(recv, ffn_inp)


def make_gpu_ep_decode(router, bias, norm_weight, local_block, n_expert, top_k, scale=2.5, norm=True, eps=1e-6,
                       group=None, exchange=None):
    """Bind `ExpertParallelDecode` to the CUDA entry points of a local `MoeBlock` shard (`MoeBlock.shard`):
    `lmoe_rms_norm`, `lmoe_route` on the full replicated router, `lmoe_ep_localize_ids`,
    `lmoe_experts_forward_ep`, `lmoe_ep_combine`."""
    from . import ops
    from ._native import check, lib
    from .gguf import stream_ptr

    world = dist.get_world_size(group)
    state = {}

    def norm_fn(x):
        out = torch.empty_like(x)
        check(lib().lmoe_rms_norm(x.data_ptr(), norm_weight.data_ptr(), eps, x.shape[0], x.shape[1], out.data_ptr(), stream_ptr()))
        return out

    def route_fn(x_all):
        return ops.route(router, bias, x_all, top_k, scale, norm)

    def localize_fn(ids, first, count):
        out = torch.empty_like(ids)
        check(lib().lmoe_ep_localize_ids(ids.data_ptr(), ids.numel(), first, count, out.data_ptr(), stream_ptr()))
        return out

    def experts_fn(x_all, ids_local, w, sh_first, sh_count):
        t = x_all.shape[0]
        out = torch.empty(t, x_all.shape[1], dtype=torch.float32, device=x_all.device)
        n = lib().lmoe_experts_workspace_bytes(local_block.handle, t)
        if state.get("ws") is None or state["ws"].numel() < n:
            state["ws"] = torch.empty(n, dtype=torch.uint8, device=x_all.device)
        check(lib().lmoe_experts_forward_ep(local_block.handle, x_all.data_ptr(), ids_local.data_ptr(), w.data_ptr(), t,
                                            sh_first, sh_count, out.data_ptr(), state["ws"].data_ptr(), state["ws"].numel(),
                                            stream_ptr()))
        return out

    def sum_fn(parts, residual):
        t_loc, h = residual.shape
        key = (t_loc, str(parts.device))
        if state.get("pos_key") != key:
            # row of rank s's partial for token i inside the received buffer: s * t_loc + i
            state["pos"] = (torch.arange(world, dtype=torch.int32, device=parts.device)[None, :] * t_loc +
                            torch.arange(t_loc, dtype=torch.int32, device=parts.device)[:, None]).contiguous()
            state["pos_key"] = key
        out = torch.empty(t_loc, h, dtype=torch.float32, device=parts.device)
        check(lib().lmoe_ep_combine(parts.data_ptr(), state["pos"].data_ptr(), residual.data_ptr(), t_loc, world, h,
                                    out.data_ptr(), stream_ptr()))
        return out

    return ExpertParallelDecode(norm_fn, route_fn, localize_fn, experts_fn, sum_fn, n_expert, group, exchange)


class ExpertParallelPrefill:
    """Expert-parallel prefill of one MoE layer without any host round trip (BASELINE config 4).

    Rank r owns experts ``[r*E/G, (r+1)*E/G)`` and ``t_loc`` tokens (the same count on every rank).  Instead of
    compacting per-destination token lists - which needs the counts on the host before the payload exchange can
    be sized - every rank receives every token: fixed-size collectives, sized by the shapes alone.
      1. all-gather of the f16 activations, in `waves` slices of the local tokens, queued first (they do not
         depend on routing); route the rank's own tokens meanwhile (replicated router: ids identical to the
         single-GPU result);
      2. all-gather of the (id, weight) words, in the same slices;
      3. per wave: localise the ids (other ranks' experts -> empty slot) and run the token-level grouped GEMMs
         over all G*n tokens of the wave: a token without a local expert costs nothing but a zero output row;
      4. per wave: all-to-all of the partial rows ([G, n, H] f32: chunk s belongs to rank s's tokens);
      5. the shared expert of the rank's own tokens runs while the last partial rows travel; the owner then adds
         the G partial rows of a token in rank order and the shared expert's row.
    The collectives of wave i+1 (gather) and i-1 (return) run on the communicator's stream while wave i
    multiplies.  (Keeping 8 or 16 SMs free of the persistent GEMM kernels for the collectives' kernels was measured
    on 8 GPUs and did not pay: 1.92 ms with none, 1.94 / 1.97 ms with 8 / 16.)  Callables as in `ExpertParallelMoe` / `ExpertParallelDecode`:
      route_fn(x) -> (ids, w);  localize_fn(ids, first, count);  tokens_fn(x16[N,H], ids_local[N,K], w[N,K]) -> [N,H] f32;
      shared_fn(x) -> [t_loc,H] or None;  sum_fn(parts[G*n,H], shared_or_None[n,H]) -> [n,H].
    """

    def __init__(self, route_fn, localize_fn, tokens_fn, shared_fn, sum_fn, n_expert: int, top_k: int, group=None,
                 payload_dtype=torch.float16, waves: int = 0):
        self.route_fn, self.localize_fn, self.tokens_fn = route_fn, localize_fn, tokens_fn
        self.shared_fn, self.sum_fn = shared_fn, sum_fn
        self.n_expert, self.top_k, self.group = n_expert, top_k, group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if n_expert % self.world:
            raise ValueError(f"n_expert ({n_expert}) must divide over {self.world} ranks")
        self.e_local = n_expert // self.world
        self.payload_dtype = payload_dtype
        self.waves = waves
        self.profile = False      # set to record per-phase CUDA-event times of the next forward in `last_phases`
        self.last_phases = None
        self.last_stats = {}

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        t_loc, h = x.shape
        g, k, dev = self.world, self.top_k, x.device
        # by default: one wave for small inputs, else two (measured on 4 and 8 GPUs at 16384 tokens: two waves
        # hide part of the exchange; four stream the local experts' weights too often to pay)
        n_waves = self.waves if self.waves > 0 else (1 if t_loc < 2048 else 2)
        n_waves = max(1, min(n_waves, t_loc))
        marks = []                                         # (name, event) on the compute stream, when profiling

        def mark(name):
            if self.profile and x.is_cuda:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                marks.append((name, ev))

        mark("start")
        bounds = [(t_loc * i // n_waves, t_loc * (i + 1) // n_waves) for i in range(n_waves)]
        # The activation rows do not depend on routing: the first wave's all-gather is queued before the router runs.
        # After it the order on the communicator's stream is (id, weight) words of wave 0, rows of wave 1, words of
        # wave 1, ...: a wave waits for nothing that belongs to a later one.
        x16 = x.to(self.payload_dtype)

        def gather_rows(a, b):
            xa = torch.empty(g * (b - a), h, dtype=x16.dtype, device=dev)
            return xa, dist.all_gather_into_tensor(xa, x16[a:b].contiguous(), group=self.group, async_op=True)

        first = gather_rows(*bounds[0])
        ids, w = self.route_fn(x)
        mark("route")
        meta = torch.cat([ids.view(torch.int32), w.contiguous().view(torch.int32)], dim=1).contiguous()  # [t_loc, 2K] words
        gathers = []
        for i, (a, b) in enumerate(bounds):
            xa, h1 = first if i == 0 else gather_rows(a, b)
            ma = torch.empty(g * (b - a), 2 * k, dtype=torch.int32, device=dev)
            h2 = dist.all_gather_into_tensor(ma, meta[a:b].contiguous(), group=self.group, async_op=True)
            gathers.append((xa, ma, h1, h2))
        returns = []
        for (a, b), (xa, ma, h1, h2) in zip(bounds, gathers):
            h1.wait()
            h2.wait()
            mark("gathered")
            ids_all = ma[:, :k].contiguous()
            w_all = ma[:, k:].contiguous().view(torch.float32)
            part = self.tokens_fn(xa, self.localize_fn(ids_all, self.rank * self.e_local, self.e_local), w_all)
            mark("experts")
            recv = torch.empty_like(part)
            hr = dist.all_to_all_single(recv, part, group=self.group, async_op=True)
            returns.append((recv, hr, part))
        # the shared expert of the rank's own tokens runs while the last partial rows travel
        shared = self.shared_fn(x) if self.shared_fn is not None else None
        mark("shared")
        out = torch.empty(t_loc, h, dtype=torch.float32, device=dev)
        for (a, b), (recv, hr, _) in zip(bounds, returns):
            hr.wait()
            mark("returned")
            out[a:b] = self.sum_fn(recv, None if shared is None else shared[a:b])
            mark("summed")
        self.last_stats = {"waves": n_waves, "tokens_gathered": g * t_loc, "rows_returned": (g - 1) * t_loc}
        if marks:
            # milliseconds on the compute stream between consecutive marks: the time a wait takes is the part of
            # the collective that the preceding compute did not hide
            torch.cuda.synchronize(dev)
            self.last_phases = [(name, marks[i - 1][1].elapsed_time(ev)) for i, (name, ev) in enumerate(marks) if i > 0]
        return out


def make_gpu_ep_prefill(full_router, bias, local_block, n_expert, top_k, scale=2.5, norm=True, group=None, waves=0):
    """Bind `ExpertParallelPrefill` to the CUDA entry points of a local `MoeBlock` shard: `lmoe_route`,
    `lmoe_ep_localize_ids`, `lmoe_experts_forward_tokens_f16`, `lmoe_shared_forward`, `lmoe_ep_combine`."""
    from . import ops
    from ._native import check, lib
    from .gguf import stream_ptr

    world = dist.get_world_size(group)
    state = {}

    def route_fn(x):
        return ops.route(full_router, bias, x, top_k, scale, norm)

    def localize_fn(ids, first, count):
        out = torch.empty_like(ids)
        check(lib().lmoe_ep_localize_ids(ids.data_ptr(), ids.numel(), first, count, out.data_ptr(), stream_ptr()))
        return out

    def sum_fn(parts, shared):
        n = parts.shape[0] // world
        hdim = parts.shape[1]
        key = (n, str(parts.device))
        if state.get("pos_key") != key:
            state["pos"] = (torch.arange(world, dtype=torch.int32, device=parts.device)[None, :] * n +
                            torch.arange(n, dtype=torch.int32, device=parts.device)[:, None]).contiguous()
            state["pos_key"] = key
        out = torch.empty(n, hdim, dtype=torch.float32, device=parts.device)
        sh = None if shared is None else shared.contiguous()
        check(lib().lmoe_ep_combine(parts.data_ptr(), state["pos"].data_ptr(), None if sh is None else sh.data_ptr(), n, world,
                                    hdim, out.data_ptr(), stream_ptr()))
        return out

    return ExpertParallelPrefill(route_fn, localize_fn, local_block.experts_forward_tokens,
                                 local_block.shared_forward if local_block.shared is not None else None, sum_fn,
                                 n_expert, top_k, group, waves=waves)


class _RawCuda:
    """A device range as an object torch can wrap without copying (`__cuda_array_interface__`)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


class PeerExchange:
    """The two exchanges of an expert-parallel decode step over peer memory instead of NCCL collectives:
    `lmoe_peer_put` / `lmoe_peer_wait` on buffers every rank maps from every other rank (CUDA IPC).

    ``gather(x)``: x [n, H] of this rank -> [G*n, H] with every rank's rows (an all-gather);
    ``scatter(parts)``: parts [G*n, H], chunk s for rank s -> [G*n, H], chunk s from rank s (an all-to-all).
    Both return views of the receive buffers: they are overwritten by the next call of the same kind, which is safe
    inside a decode step (a rank sends its next rows only after it has received everybody's previous ones).
    The only host-side collective is the exchange of the 64-byte handles at construction."""

    def __init__(self, max_rows: int, hidden: int, group=None, dtype=torch.float32):
        import ctypes as C

        from ._native import check, lib
        self._lib, self._check, self._C = lib(), check, C
        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.dtype, self.hidden, self.max_rows = dtype, hidden, max_rows
        item = torch.empty(0, dtype=dtype).element_size()
        self.chunk_cap = max_rows * hidden * item                      # bytes one rank may send to one rank
        sizes = {"gather": self.world * self.chunk_cap, "scatter": self.world * self.chunk_cap,
                 "ctrl": int(self._lib.lmoe_peer_ctrl_bytes())}
        self._own, handles = {}, {}
        for name, nbytes in sizes.items():
            p, h = C.c_void_p(), C.create_string_buffer(64)
            check(self._lib.lmoe_peer_alloc(nbytes, C.byref(p), h))
            self._own[name], handles[name] = p.value, h.raw
        everyone = [None] * self.world
        dist.all_gather_object(everyone, handles, group=group)
        self._opened = []
        self._ptrs = {name: [0] * self.world for name in sizes}
        for s in range(self.world):
            for name in sizes:
                if s == self.rank:
                    self._ptrs[name][s] = self._own[name]
                else:
                    p = C.c_void_p()
                    check(self._lib.lmoe_peer_open(everyone[s][name], C.byref(p)))
                    self._ptrs[name][s] = p.value
                    self._opened.append(p.value)
        arr = C.c_void_p * self.world
        self._arr = {name: arr(*self._ptrs[name]) for name in sizes}
        dev = torch.device("cuda", torch.cuda.current_device())
        self._recv = {name: torch.as_tensor(_RawCuda(self._own[name], sizes[name]), device=dev) for name in ("gather", "scatter")}
        self._ctrl = torch.as_tensor(_RawCuda(self._own["ctrl"], sizes["ctrl"]), device=dev).view(torch.int32)
        dist.barrier(group=group)                                       # every rank has mapped every buffer

    def _exchange(self, src: torch.Tensor, name: str, per_rank: int, direction: int) -> torch.Tensor:
        from .gguf import stream_ptr
        n = src.shape[0] // self.world if per_rank else src.shape[0]
        chunk = n * self.hidden * src.element_size()
        assert src.is_contiguous() and src.dtype == self.dtype and src.shape[-1] == self.hidden and chunk <= self.chunk_cap
        st = stream_ptr()
        self._check(self._lib.lmoe_peer_put(src.data_ptr(), chunk, self.world, self.rank, per_rank, self._arr[name],
                                            self._arr["ctrl"], self._own["ctrl"], direction, st))
        self._check(self._lib.lmoe_peer_wait(self._own["ctrl"], self.world, direction, st))
        return self._recv[name][: self.world * chunk].view(self.dtype).view(self.world * n, self.hidden)

    def gather(self, x: torch.Tensor) -> torch.Tensor:
        return self._exchange(x, "gather", 0, 0)

    def scatter(self, parts: torch.Tensor) -> torch.Tensor:
        return self._exchange(parts, "scatter", 1, 1)

    def timed_out(self) -> int:
        """Word 40 of the control block: non-zero when a wait gave up (bit 0x2, plus 0x100 << rank per missing rank)."""
        return int(self._ctrl[40].item())

    def close(self):
        dist.barrier(group=self.group)
        torch.cuda.synchronize()
        for p in self._opened:
            self._lib.lmoe_peer_close(p)
        self._opened = []
        dist.barrier(group=self.group)
        for p in self._own.values():
            self._lib.lmoe_peer_free(p)
        self._own = {}
