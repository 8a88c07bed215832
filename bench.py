#!/usr/bin/env python
"""Benchmark of the MoE hot path on B200.

Metric (BASELINE.json): MoE-layer decode tok/s, with achieved HBM GB/s against the
measured peak.  Workload at N=1 = BASELINE config 2: one MoE FFN layer (hidden
3072, 256 routed experts + 1 shared, top-10, Q4_K gate/up, Q6_K down), decode
batch sweep B = 1/2/4/8/16 with independent N(0,1) hidden states.  One "step" is
one pass over the sweep (31 tokens, five launches of the fused decode kernel).
Every launch uses a different layer copy out of `--layers` (default 8, 12.6 GB
of weights, far beyond the 126 MB L2) and a different hidden-state batch, so
weights come from HBM, not from cache.

  value     device-resident inputs, CUDA-event timed, whole job (all ranks)
  e2e       same sweep through the C-ABI host-buffer call (pinned host x in,
            host result out, copies inside the timed region): the asynchronous
            entry with one stream synchronisation per step; `sync_every_call`
            is the synchronous entry
  roofline  decode kernel: algorithmic bytes / event-timed launch duration
  cpu_baseline  the CPU restatement of the reference's CPU path (int8-activation
            k-quant dot products), all host threads, bounded sample
  prefill   config 3 (N = 1: 4096 tokens, with parity sample, e2e, CPU leg and a
            16384-token anchor) or config 4 (N > 1: 16384 tokens expert parallel,
            with parity sample and per-phase times)
  stack     config 5: 48 layers, 64-sequence batched decode and 2048-token prefill
            (expert parallel under torchrun)
  lm_head   the vocabulary-projection mat-vec, Q6_K [100352 x 3072]

`--impl reference` times that CPU restatement alone (the reference is Rust +
Metal and cannot be built or run here).
With N>1 (torchrun) every rank runs an independent replica of the sweep (decode
at batch <= 16 does not shard; weak scaling).
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# torchrun exports OMP_NUM_THREADS=1 to its workers; the CPU arm (rank 0 only) is meant to use
# every host core, so the variable is reset before the OpenMP runtime of the CPU code starts.
if os.environ.get("TORCHELASTIC_RUN_ID") is not None and os.environ.get("RANK", "0") == "0":
    os.environ["OMP_NUM_THREADS"] = str(len(os.sched_getaffinity(0)))

H, F, E, K = 3072, 1024, 256, 10
SWEEP = (1, 2, 4, 8, 16)
EXPERT_BYTES = 2 * F * (H // 256) * 144 + H * (F // 256) * 210  # 6 119 424
ROUTER_BYTES = E * H * 4
WORKLOAD = "config2: single MoE layer decode sweep B=1/2/4/8/16 (31 tokens per step)"
# DRAM traffic of one decode sweep (B = 1, 2, 4, 8, 16) from an ncu capture of the five launches
# (dram__bytes_read.sum + dram__bytes_write.sum: 72.3 + 136.0 + 224.6 + 412.8 + 705.8 MB; the algorithmic figure is
# the mean over the three sweeps of that run).  The figure belongs to the kernel source it was captured on: when
# csrc/decode.cu has changed since, the line reports null.
NCU_TRAFFIC = {"bytes_per_sweep": 1.5516e9, "algorithmic_bytes_of_that_sweep": 1.4648e9,
               "decode_cu_sha256_16": "462102bd0ae44431"}
NVSMI_Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
           "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
           "clocks_event_reasons.sw_power_cap")


def algorithmic_bytes(n_distinct: int, batch: int) -> int:
    """Bytes one decode launch must move: each distinct routed expert once, the shared
    expert, the router, the bias, activations in and out."""
    return n_distinct * EXPERT_BYTES + EXPERT_BYTES + ROUTER_BYTES + E * 4 + batch * (H * 4 + H * 4)


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 10 ms; every row carries the host time at which it
    was read, so the rows that fall inside the timed region can be told from those of the loaded windows
    around it (warm-up before, per-batch timing loops after)."""

    def __init__(self, gpu_index: int):
        self.rows = []
        self.proc = None
        self.gpu = gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={NVSMI_Q}", "--format=csv,noheader,nounits",
                                          "-lms", "10", "-i", str(self.gpu)], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.perf_counter(), [c.strip() for c in line.split(",")]))

    def stop(self, t0=None, t1=None):
        """Summary over the rows read in [t0, t1] (the timed region); when the region was too short to
        hold a sample, over every row read while the GPU was under load, and `window` says so."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"], "samples": 0}
        time.sleep(0.03)
        self.proc.terminate()
        rows = [r for r in self.rows if len(r[1]) >= 9 and r[1][1].replace(".", "").isdigit()]
        inside = [r for r in rows if t0 is not None and t0 <= r[0] <= t1 + 0.02]
        window = "timed region"
        if not inside:
            inside, window = rows, "warm-up, timed region and per-batch loops (the timed region is shorter than one sample period)"
        sm = [float(r[1][1]) for r in inside]
        mx = [float(r[1][2]) for r in inside if r[1][2].replace(".", "").isdigit()]
        reasons = set()
        for _, r in inside:
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "window": window, "period_ms": 10}


def build_host_layer(orc, seed=0):
    """Config-1/2 layer on the host for the CPU arm: N(0,0.02) weights through the oracle's encoder."""
    rng = np.random.default_rng(seed)

    def stack(dt, ne, n_out, k):
        out = np.empty(ne * n_out * (k // 256) * orc.TYPE_SIZE[dt], np.uint8)
        per = n_out * (k // 256) * orc.TYPE_SIZE[dt]
        for e in range(ne):
            w = (rng.standard_normal(n_out * k, dtype=np.float32) * np.float32(0.02))
            out[e * per:(e + 1) * per] = orc.quantize(dt, w)
        return out

    return orc.HostLayer(H, F, E, K, router=(rng.standard_normal((E, H)) * 0.02).astype(np.float32),
                         bias=rng.uniform(-0.1, 0.1, E).astype(np.float32),
                         gate=stack(orc.Q4_K, E, F, H), up=stack(orc.Q4_K, E, F, H), down=stack(orc.Q6_K, E, H, F),
                         sh_gate=stack(orc.Q4_K, 1, F, H), sh_up=stack(orc.Q4_K, 1, F, H),
                         sh_down=stack(orc.Q6_K, 1, H, F))


def cpu_time_sweep(host, xs, batches, budget_s):
    """Time the int8-activation CPU path over `batches`; stops early past the budget.
    Returns (tokens, seconds)."""
    tok, t0 = 0, time.perf_counter()
    for b in batches:
        host.forward_q8(xs[b])
        tok += b
        if time.perf_counter() - t0 > budget_s:
            break
    return tok, time.perf_counter() - t0


def run_reference(args, rank, world):
    """`--impl reference`: the CPU restatement of the reference's CPU path, rank 0 only."""
    if rank != 0:
        return
    from oracle import oracle as orc

    orc.build()
    host = build_host_layer(orc, seed=0)
    rng = np.random.default_rng(1)
    xs = {b: rng.standard_normal((b, H)).astype(np.float32) for b in SWEEP}
    # bounded sample: size each step so steps+warmup end in about two minutes
    tok, sec = cpu_time_sweep(host, xs, (1,), 1e9)
    per_tok = sec / tok
    total = args.steps + args.warmup
    max_tok_per_step = max(1, int(120.0 / total / per_tok))
    batches = []
    for b in SWEEP:
        if sum(batches) + b <= max_tok_per_step:
            batches.append(b)
    if not batches:
        batches = [1]
    for _ in range(args.warmup):
        cpu_time_sweep(host, xs, batches, 1e9)
    t0 = time.perf_counter()
    toks = 0
    for _ in range(args.steps):
        n, _ = cpu_time_sweep(host, xs, batches, 1e9)
        toks += n
    sec = time.perf_counter() - t0
    val = toks / sec
    cores = orc.num_threads()
    sample = f"decode batches {batches} of the sweep per step ({sum(batches)} tokens), one layer"
    print(json.dumps({
        "impl": "reference", "metric": "moe_layer_decode_tok_per_s", "value": val, "unit": "tok/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "i8xq4/q6 -> f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "hidden": H, "expert_ff": F,
                   "n_expert": E, "top_k": K, "shared_expert": True, "sample": sample},
        "cpu_baseline": {"value": val, "unit": "tok/s", "cores": cores, "kind": "port", "sample": sample,
                         "build": "int8-activation k-quant dots, -O3 -march=native, 256-bit integer SIMD where the host has it, OpenMP"},
        "e2e": {"value": val, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "CPU restatement of the reference's CPU k-quant path (the reference itself is Rust + Metal: not buildable here)",
    }))


def zipf_bias(n_expert, seed, device):
    """Selection bias that skews per-expert token counts: Zipf(s=1.1) over a seeded shuffle."""
    import torch

    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(n_expert, generator=g)
    z = 1.0 / (torch.arange(1, n_expert + 1, dtype=torch.float32) ** 1.1)
    b = torch.empty(n_expert)
    b[perm] = (z / z.max()) * 0.3 - 0.1
    return b.to(device)


def _time_gpu(run, steps, warmup, world, dev):
    """Mean milliseconds of `run()` over `steps` calls after `warmup`: CUDA events on the current stream,
    barrier + synchronize on both sides, max over ranks."""
    import torch
    import torch.distributed as dist

    for _ in range(warmup):
        run()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        run()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    if world > 1:
        tt = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms = float(tt[0])
    return ms


def prefill_parity(blk, x, out, ids, n_sample, seed):
    """Outside every timed region: a token sample of a prefill result against the CPU oracle (routing
    decision bit for bit, block output in relative L2), plus the count of tokens whose 10th and 11th
    selection scores lie within 1e-6 of each other in float64 (the ones f32 noise could re-rank)."""
    import torch

    from oracle import oracle as orc

    orc.build()
    host = blk.host_layer(orc)
    t = x.shape[0]
    rng = np.random.default_rng(seed)
    sample = np.sort(rng.choice(t, min(n_sample, t), replace=False))
    xs = x[torch.from_numpy(sample).to(x.device)].cpu().numpy()
    want, ids_o, _ = host.forward(xs)
    got = out[torch.from_numpy(sample).to(out.device)].cpu().numpy()
    ids_g = ids[torch.from_numpy(sample).to(ids.device)].cpu().numpy().astype(np.uint32)
    logits = orc.route_logits(host.router, x.cpu().numpy()).astype(np.float64)
    sel = 1.0 / (1.0 + np.exp(-logits)) + (0.0 if host.bias is None else host.bias.astype(np.float64))
    part = -np.sort(-sel, axis=1)
    return {"tokens": int(len(sample)), "ids_exact": bool(np.array_equal(ids_g, ids_o)),
            "rel_l2": orc.rel_l2(got, want), "against": "CPU oracle (dequantize -> f32 dot)",
            "near_ties_lt_1e-6": int(np.count_nonzero(part[:, K - 1] - part[:, K] < 1e-6)), "of_tokens": int(t)}


def measure_prefill(dev, rank, world, steps=8, warmup=3, tokens=None, checks=True, ep_mode="dense", ep_waves=0):
    """Prefill of one MoE layer: N=1 -> config 3 (4096 tokens, Zipf-skewed routing, one GPU), plus the
    16384-token single-GPU run that anchors the expert-parallel scaling curve; N>1 -> config 4 (16384 tokens
    split over the ranks, experts sharded 256/N per GPU, all-to-all dispatch / combine), uniform and Zipf.
    Each result carries a parity check of a token sample made outside the timed region."""
    import torch
    import torch.distributed as dist

    from maxuna_b200 import _native
    from maxuna_b200.ep import make_gpu_ep_block, make_gpu_ep_prefill
    from maxuna_b200.moe import MoeBlock

    lib = _native.lib()
    res = {}
    t_total = tokens if tokens else (4096 if world == 1 else 16384)
    cases = [("zipf", t_total)] if world == 1 else [("uniform", t_total), ("zipf", t_total)]
    if world == 1 and not tokens:
        cases.append(("zipf_t16384", 16384))
    for name, t_case in cases:
        zipf = name.startswith("zipf")
        bias = zipf_bias(E, 3, dev) if zipf else None
        blk = MoeBlock.random(H, F, E, K, seed=4242, device=dev, bias=bias)
        gen = torch.Generator(device=dev)
        gen.manual_seed(99 + rank)
        t_loc = t_case // world
        x = torch.randn(t_loc, H, generator=gen, device=dev)
        out = torch.empty(t_loc, H, device=dev)
        entry = {"tokens": t_case, "seed_layer": 4242, "seed_tokens": 99, "bias": "zipf(1.1), seed 3" if zipf else "U(-0.1, 0.1)"}
        if world == 1:
            ids = torch.empty(t_loc, K, dtype=torch.int32, device=dev)
            ws = blk.workspace(t_loc)
            stream = torch.cuda.current_stream().cuda_stream

            def run():
                _native.check(lib.lmoe_moe_forward_prefill(blk.handle, x.data_ptr(), t_loc, out.data_ptr(), ids.data_ptr(), None,
                                                           ws.data_ptr(), ws.numel(), stream))
            ep = None
            entry["path"] = "lmoe_moe_forward_prefill: router, expert-sorted gather, tcgen05 grouped GEMMs, slot-order sum"
        else:
            if ep_mode == "tokens":
                ep = make_gpu_ep_block(blk.router, blk.exp_probs_b, blk.shard(rank, world), E, K)
                entry["path"] = "expert parallel, compacted token-level exchange (ExpertParallelMoe: counts on the host)"
            else:
                ep = make_gpu_ep_prefill(blk.router, blk.exp_probs_b, blk.shard(rank, world), E, K, waves=ep_waves)
                entry["path"] = ("expert parallel, fixed-size exchange (ExpertParallelPrefill: all-gather of f16 rows, "
                                 "all-to-all of f32 partial rows, waves overlapped with the grouped GEMMs)")

            def run():
                out.copy_(ep.forward(x))
        ms = _time_gpu(run, steps, warmup, world, dev)
        flops = t_case * (K + 1) * 18874368
        entry.update({"ms": ms, "tflops": flops / ms / 1e9, "tok_per_s": t_case / ms * 1e3})
        if checks:
            if world == 1:
                if rank == 0:
                    entry["parity"] = prefill_parity(blk, x, out, ids, 32, 7)
            else:
                # the same tokens through the single-GPU block on this rank (it holds the full layer): a sample
                # of the expert-parallel result must agree to f32 rounding (the sums are grouped by rank)
                n_s = min(256, t_loc)
                ref, ids_ref, _ = blk.forward(x[:n_s], return_routing=True, path="prefill")
                ep.profile = True                          # per-phase CUDA-event times of this (untimed) call
                got = ep.forward(x)[:n_s]
                ep.profile = False
                torch.cuda.synchronize()
                d = (got.double() - ref.double()).pow(2).sum().sqrt() / ref.double().pow(2).sum().sqrt()
                tt = torch.tensor([float(d)], device=dev, dtype=torch.float64)
                dist.all_reduce(tt, op=dist.ReduceOp.MAX)
                entry["parity"] = {"tokens": n_s * world, "rel_l2": float(tt[0]),
                                   "against": "the single-GPU grouped-GEMM block on the same tokens, max over ranks",
                                   "ids_exact": True, "ids_note": "every rank routes its own tokens with the replicated router"}
                if getattr(ep, "last_phases", None):
                    entry["phases_ms"] = ep.last_phases
                entry["rows"] = dict(ep.last_stats)
        if checks and world == 1 and rank == 0 and t_case == t_total:
            # end to end through the host-buffer entry (pinned x in, result out, copies inside the timed region)
            xh = x.cpu().pin_memory()
            oh = torch.empty(t_loc, H).pin_memory()
            n_ws = lib.lmoe_layer_workspace_bytes(blk.handle, t_loc)
            wsh = torch.empty(n_ws, dtype=torch.uint8, device=dev)
            stream = torch.cuda.current_stream().cuda_stream

            def host_call():
                _native.check(lib.lmoe_moe_forward_host(blk.handle, xh.data_ptr(), t_loc, oh.data_ptr(), None, None, wsh.data_ptr(),
                                                        n_ws, stream))
            for _ in range(2):
                host_call()
            t0 = time.perf_counter()
            for _ in range(4):
                host_call()
            e2e_ms = (time.perf_counter() - t0) / 4 * 1e3
            entry["e2e"] = {"ms": e2e_ms, "tflops": flops / e2e_ms / 1e9, "unit": "TFLOP/s", "h2d_bytes_per_step": t_loc * H * 4,
                            "d2h_bytes_per_step": t_loc * H * 4}
            # bounded CPU leg: the int8-activation port on 16 of these tokens
            from oracle import oracle as orc

            host = blk.host_layer(orc)
            xs_cpu = x[:16].cpu().numpy()
            host.forward_q8(xs_cpu[:1])
            t0 = time.perf_counter()
            host.forward_q8(xs_cpu)
            sec = time.perf_counter() - t0
            entry["cpu_baseline"] = {"value": 16 * (K + 1) * 18874368 / sec / 1e12, "unit": "TFLOP/s", "cores": orc.num_threads(),
                                     "kind": "port", "sample": "16 tokens of this prefill through the int8-activation CPU path"}
        res[name] = entry
        del blk, ep
        torch.cuda.empty_cache()
    return res


def measure_lm_head(dev, steps=20, warmup=5):
    """The plain quantized mat-vec at the model's lm_head shape (`ops::mul_mv`, src/ops/mv_id.rs:54-56 of the
    reference, called from src/model.rs:388-403): Q6_K [100352 x 3072], 253 MB per token, one token.  Timed with
    CUDA events over weights that do not fit L2; a sample of rows is checked against the CPU oracle."""
    import torch

    from maxuna_b200 import _native
    from maxuna_b200.gguf import Q6_K, ExpertStack, stream_ptr
    from oracle import oracle as orc

    lib = _native.lib()
    n_out, k = 100352, H
    copies = 2                                                       # 2 x 253 MB rotated: nothing stays in L2
    stacks = [ExpertStack.random(Q6_K, 1, n_out, k, std=0.02, seed=900 + i, device=dev, chunk_experts=1) for i in range(copies)]
    gen = torch.Generator(device=dev)
    gen.manual_seed(77)
    x = torch.randn(1, k, generator=gen, device=dev)
    out = torch.empty(1, n_out, device=dev)

    def run(i=[0]):
        st = stacks[i[0] % copies]
        i[0] += 1
        _native.check(lib.lmoe_mul_mv(st.buffer.data_ptr() + st.base_off, Q6_K, n_out, k, x.data_ptr(), 1, out.data_ptr(), stream_ptr()))

    ms = _time_gpu(run, steps, warmup, 1, dev)
    nbytes = n_out * (k // 256) * 210
    # parity: the last launch used stack (steps + warmup - 1) % copies; check 64 sampled rows of it
    st = stacks[(steps + warmup - 1) % copies]
    rows = np.sort(np.random.default_rng(5).choice(n_out, 64, replace=False))
    rb = (k // 256) * 210
    raw = st.buffer[st.base_off:st.base_off + st.nbytes].view(n_out, rb)[torch.from_numpy(rows).to(dev)].cpu().numpy()
    want = orc.mul_mv(Q6_K, raw, 64, k, x.cpu().numpy())[0]
    got = out[0, torch.from_numpy(rows).to(dev)].cpu().numpy()
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    peak = float(json.load(open(peaks_path))["hbm_gbs"]) if os.path.exists(peaks_path) else 6650.0
    return {"workload": "lm_head-shaped plain mat-vec: Q6_K [100352 x 3072], one token", "us": ms * 1e3,
            "gb_per_s": nbytes / ms / 1e6, "frac_of_peak": nbytes / ms / 1e6 / peak, "bytes": nbytes,
            "parity": {"rows": 64, "rel_l2": orc.rel_l2(got, want), "against": "CPU oracle (dequantize -> f32 dot)"}}


def measure_stack(dev, rank, world, n_layers, steps=3, warmup=3, graph=False, peer=False):
    """The expert portion of a Laguna-shaped model (BASELINE config 5): a residual stack of `n_layers` MoE
    layers, x <- x + block_l(rms_norm_l(x)); batched decode of 64 sequences (one token each) and a 2048-token
    prefill.
    One GPU: every layer whole on the device (48 layers are 75.5 GB and fit one B200), through
    `lmoe_moe_layer_forward`; for the 64-token step the grouped-GEMM path (what the reference's `seq >= 32` rule
    would pick) is timed beside the mat-vec kernel.
    N GPUs: expert parallel - rank r holds experts [r*256/N, (r+1)*256/N) of every layer (router, bias, norm and
    shared expert replicated) and 64/N sequences / 2048/N prefill tokens; decode through
    `ExpertParallelDecode` (all-gather, one fused mat-vec launch per layer, all-to-all of the partial rows),
    prefill through `ExpertParallelPrefill` (the same exchange around the grouped GEMMs).  A two-layer copy of the stack that every
    rank also holds whole gives the parity figure (expert-parallel result against the single-GPU layer entry)."""
    import torch
    import torch.distributed as dist

    from maxuna_b200 import _native
    from maxuna_b200.ep import make_gpu_ep_decode, make_gpu_ep_prefill
    from maxuna_b200.gguf import Q4_K, Q6_K, ExpertStack
    from maxuna_b200.moe import MoeBlock

    lib = _native.lib()
    gen = torch.Generator(device=dev)
    gen.manual_seed(5)
    stream = torch.cuda.current_stream().cuda_stream
    res = {"layers": n_layers, "n_gpus": world,
           "weights_gb_per_gpu": n_layers * ((E // world + 1) * EXPERT_BYTES + ROUTER_BYTES) / 1e9}

    def timed(fn, tokens):
        ms = _time_gpu(fn, steps, warmup, world, dev)
        return {"tokens": tokens, "ms_per_pass": ms, "tok_per_s": tokens / ms * 1e3, "us_per_layer": ms * 1e3 / n_layers}

    def graphed(fn, tokens):
        """The same pass recorded once as a CUDA graph and replayed (`maxuna_b200.graphs.GraphedCall`): no host work
        per launch.  Every rank must get through the capture before any rank replays."""
        from maxuna_b200.graphs import GraphedCall
        try:
            gc = GraphedCall(fn)
            ok = 1.0
        except Exception as e:  # noqa: BLE001 - reported in the result, the eager figure stands
            gc, ok, err = None, 0.0, f"{type(e).__name__}: {e}"[:300]
        if world > 1:
            tt = torch.tensor([ok], device=dev, dtype=torch.float64)
            dist.all_reduce(tt, op=dist.ReduceOp.MIN)
            ok = float(tt[0])
        if ok < 1.0:
            return {"error": err if gc is None else "capture failed on another rank"}
        r = timed(gc.replay, tokens)
        r["how"] = "one CUDA graph per pass, replayed"
        return r

    if world == 1:
        layers = [MoeBlock.random(H, F, E, K, seed=7000 + i, device=dev) for i in range(n_layers)]
        norms = [0.5 + torch.rand(H, generator=gen, device=dev) for _ in layers]
        need = max(lib.lmoe_moe_layer_workspace_bytes(layers[0].handle, 2048), lib.lmoe_moe_layer_workspace_bytes(layers[0].handle, 64))
        ws = torch.zeros(need, dtype=torch.uint8, device=dev)

        def layer_path(x, bufs):
            stream = torch.cuda.current_stream().cuda_stream   # the capture stream when a graph is being recorded
            for i, ly in enumerate(layers):
                a, b = bufs[i & 1], bufs[(i & 1) ^ 1]
                src = x if i == 0 else a
                _native.check(lib.lmoe_moe_layer_forward(ly.handle, src.data_ptr(), norms[i].data_ptr(), 1e-6, x.shape[0],
                                                         b.data_ptr(), None, None, ws.data_ptr(), ws.numel(), stream))

        def gemm_path(x, bufs, normed):
            t = x.shape[0]
            for i, ly in enumerate(layers):
                a, b = bufs[i & 1], bufs[(i & 1) ^ 1]
                src = x if i == 0 else a
                _native.check(lib.lmoe_rms_norm(src.data_ptr(), norms[i].data_ptr(), 1e-6, t, H, normed.data_ptr(), stream))
                _native.check(lib.lmoe_moe_forward_prefill(ly.handle, normed.data_ptr(), t, b.data_ptr(), None, None,
                                                          ws.data_ptr(), ws.numel(), stream))
                b.add_(src)

        for name, t, fn in (("decode64", 64, layer_path), ("decode64_grouped_gemm", 64, gemm_path),
                            ("prefill2048", 2048, layer_path)):
            x = torch.randn(t, H, generator=gen, device=dev)
            bufs = [torch.empty(t, H, device=dev), torch.empty(t, H, device=dev)]
            extra = (torch.empty(t, H, device=dev),) if fn is gemm_path else ()
            res[name] = timed(lambda: fn(x, bufs, *extra), t)
            if graph and name == "decode64":
                res["decode64_graph"] = graphed(lambda: fn(x, bufs), t)
        return res

    # ---- expert parallel ----
    n_loc = E // world

    def shard_layer(i):
        """This rank's part of layer i: replicated router / bias / shared expert (same seed on every rank), own experts."""
        g = torch.Generator(device=dev)
        g.manual_seed(7000 + i)
        router = torch.randn(E, H, generator=g, device=dev) * 0.02
        bias = torch.rand(E, generator=g, device=dev) * 0.2 - 0.1
        mk = lambda dt, ne, no, k, sd: ExpertStack.random(dt, ne, no, k, std=0.02, seed=sd, device=dev)
        base = (7000 + i) * 100
        blk = MoeBlock(router[rank * n_loc:(rank + 1) * n_loc], None, mk(Q4_K, n_loc, F, H, base + 10 * rank + 1),
                       mk(Q4_K, n_loc, F, H, base + 10 * rank + 2), mk(Q6_K, n_loc, H, F, base + 10 * rank + 3),
                       mk(Q4_K, 1, F, H, base + 94), mk(Q4_K, 1, F, H, base + 95), mk(Q6_K, 1, H, F, base + 96), K)
        return router, bias, blk

    parts = [shard_layer(i) for i in range(n_layers)]
    norms = [0.5 + torch.rand(H, generator=gen, device=dev) for _ in parts]
    dec = [make_gpu_ep_decode(r, b, nw, blk, E, K) for (r, b, blk), nw in zip(parts, norms)]
    pre = [make_gpu_ep_prefill(r, b, blk, E, K) for (r, b, blk) in parts]

    t_loc = 64 // world
    xg = torch.Generator(device=dev)
    xg.manual_seed(50 + rank)
    x64 = torch.randn(t_loc, H, generator=xg, device=dev)

    def decode_pass():
        x = x64
        for step in dec:
            x = step.forward(x)
        return x

    res["decode64"] = timed(decode_pass, 64)
    if graph:
        res["decode64_graph"] = graphed(decode_pass, 64)
    if peer:
        # the two exchanges of a layer as stores into the other ranks' memory (lmoe_peer_put / lmoe_peer_wait)
        from maxuna_b200.ep import PeerExchange
        px = PeerExchange(t_loc, H)
        dec_nccl = dec
        dec = [make_gpu_ep_decode(r, b, nw, blk, E, K, exchange=px) for (r, b, blk), nw in zip(parts, norms)]
        res["decode64_peer"] = timed(decode_pass, 64)
        if graph:
            res["decode64_peer_graph"] = graphed(decode_pass, 64)
        import gc
        gc.collect()                       # recorded graphs hold the peer pointers: drop them before unmapping
        torch.cuda.synchronize()
        res["decode64_peer"]["wait_timeouts"] = px.timed_out()
        px.close()
        dec = dec_nccl
    p_loc = 2048 // world
    x2k = torch.randn(p_loc, H, generator=xg, device=dev)
    normed = torch.empty_like(x2k)

    def prefill_pass():
        x = x2k
        for ep, nw in zip(pre, norms):
            _native.check(lib.lmoe_rms_norm(x.data_ptr(), nw.data_ptr(), 1e-6, p_loc, H, normed.data_ptr(), stream))
            x = ep.forward(normed) + x
        return x

    res["prefill2048"] = timed(prefill_pass, 2048)
    del parts, dec, pre
    torch.cuda.empty_cache()
    # ---- parity: two layers that every rank also holds whole ----
    fulls = [MoeBlock.random(H, F, E, K, seed=7100 + i, device=dev) for i in range(2)]
    pn = [0.5 + torch.rand(H, generator=gen, device=dev) for _ in fulls]
    steps_p = [make_gpu_ep_decode(f.router, f.exp_probs_b, nw, f.shard(rank, world), E, K) for f, nw in zip(fulls, pn)]
    x, ref = x64, x64
    for step, f, nw in zip(steps_p, fulls, pn):
        x = step.forward(x)
        ref = f.layer_forward(ref, nw, 1e-6)
    torch.cuda.synchronize()
    tt = torch.tensor([float((x - ref).norm() / ref.norm()), float((x - ref).abs().max())], device=dev, dtype=torch.float64)
    dist.all_reduce(tt, op=dist.ReduceOp.MAX)
    res["parity"] = {"tokens": 64, "layers": 2, "rel_l2": float(tt[0]), "max_abs_diff": float(tt[1]),
                     "against": "the single-GPU layer entry on the same tokens and weights, max over ranks"}
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=50)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--layers", type=int, default=8, help="layer copies rotated through (working set >> L2)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-prefill", action="store_true", help="skip the prefill (grouped GEMM) measurement")
    ap.add_argument("--prefill-only", action="store_true", help="profiling aid: run only the prefill measurement and print it")
    ap.add_argument("--prefill-tokens", type=int, default=0, help="profiling aid: token count of the prefill measurement")
    ap.add_argument("--stack-layers", type=int, default=0,
                    help="run only the residual stack of this many MoE layers (48 = the model's expert portion; expert "
                         "parallel under torchrun) and print it")
    ap.add_argument("--ep-mode", default="dense", choices=["dense", "tokens"],
                    help="expert-parallel prefill exchange: fixed-size (all-gather / all-to-all) or compacted token lists")
    ap.add_argument("--ep-waves", type=int, default=0, help="waves of the fixed-size exchange (0 = by size)")
    ap.add_argument("--stack-graph", action="store_true", help="with --stack-layers: also time the decode pass replayed as one CUDA graph")
    ap.add_argument("--stack-peer", action="store_true", help="with --stack-layers under torchrun: also time the decode pass with peer-memory exchanges")
    ap.add_argument("--no-stack", action="store_true", help="skip the config-5 stack and the lm_head measurements of the default run")
    ap.add_argument("--lm-head-only", action="store_true", help="profiling aid: run only the lm_head-shaped mat-vec and print it")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import torch
    import torch.distributed as dist

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the MoE path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    from maxuna_b200 import _native
    from maxuna_b200.moe import MoeBlock

    _native.lib()
    if args.stack_layers > 0:
        st = measure_stack(dev, rank, world, args.stack_layers, steps=max(1, min(args.steps, 5)), warmup=min(args.warmup, 3),
                           graph=args.stack_graph, peer=args.stack_peer)
        if rank == 0:
            print(json.dumps({"stack": st}))
        if world > 1:
            dist.destroy_process_group()
        return
    if args.lm_head_only:
        if rank == 0:
            print(json.dumps({"lm_head": measure_lm_head(dev, steps=max(3, min(args.steps, 50)), warmup=args.warmup)}))
        if world > 1:
            dist.destroy_process_group()
        return
    if args.prefill_only:
        res = measure_prefill(dev, rank, world, steps=max(1, min(args.steps, 8)), warmup=args.warmup,
                              tokens=args.prefill_tokens or None, ep_mode=args.ep_mode, ep_waves=args.ep_waves)
        if rank == 0:
            print(json.dumps({"prefill_only": res}))
        if world > 1:
            dist.destroy_process_group()
        return
    layers = [MoeBlock.random(H, F, E, K, seed=100 * rank + i, device=dev) for i in range(args.layers)]
    n_x = 64
    gen = torch.Generator(device=dev)
    gen.manual_seed(1234 + rank)
    xs = {b: [torch.randn(b, H, generator=gen, device=dev) for _ in range(n_x)] for b in SWEEP}
    outs = {b: torch.empty(b, H, device=dev) for b in SWEEP}
    ws = [ly.workspace(max(SWEEP)) for ly in layers]
    n_launch = args.steps * len(SWEEP)
    ids_log = torch.zeros(n_launch, max(SWEEP) * K, dtype=torch.int32, device=dev)
    lib = _native.lib()
    stream = torch.cuda.current_stream().cuda_stream

    def launch(i, b, log_row=None):
        ly = layers[i % args.layers]
        x = xs[b][i % n_x]
        idp = None if log_row is None else ids_log[log_row].data_ptr()
        _native.check(lib.lmoe_moe_forward_decode(ly.handle, x.data_ptr(), b, outs[b].data_ptr(), idp, None,
                                                  ws[i % args.layers].data_ptr(), ws[i % args.layers].numel(), stream))

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- warm-up (the clock sampler starts first: nvidia-smi needs a moment before its first row) ----
    sampler = ClockSampler(local_rank)
    sampler.start()
    i = 0
    for _ in range(args.warmup):
        for b in SWEEP:
            launch(i, b)
            i += 1
    barrier()

    # ---- timed region: K sweeps, device-resident inputs ----
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t_region0 = time.perf_counter()
    e0.record()
    row = 0
    for _ in range(args.steps):
        for b in SWEEP:
            launch(i, b, row)
            i += 1
            row += 1
    e1.record()
    barrier()
    t_region1 = time.perf_counter()
    ms = e0.elapsed_time(e1)

    # ---- per-batch timing (same rotation), for the sweep table and the roofline: at least 0.2 s per size ----
    per_b = {}
    for b in SWEEP:
        n = max(50, args.steps // 2, int(0.2 / (ms * 1e-3 / args.steps / len(SWEEP))))
        barrier()
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a0.record()
        for _ in range(n):
            launch(i, b)
            i += 1
        a1.record()
        torch.cuda.synchronize()
        per_b[b] = a0.elapsed_time(a1) / n * 1e-3  # seconds per launch
    clocks = sampler.stop(t_region0, t_region1)

    # distinct experts per launch from the logged routing decisions
    ids_host = ids_log.cpu().numpy()
    distinct = {b: [] for b in SWEEP}
    for r in range(n_launch):
        b = SWEEP[r % len(SWEEP)]
        distinct[b].append(len(np.unique(ids_host[r, : b * K])))
    mean_u = {b: float(np.mean(distinct[b])) for b in SWEEP}
    bytes_sweep = sum(algorithmic_bytes(1, b) - EXPERT_BYTES + mean_u[b] * EXPERT_BYTES for b in SWEEP)
    launch_s = sum(per_b[b] for b in SWEEP)
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        peak_gbs, peak_src = float(json.load(open(peaks_path))["hbm_gbs"]), "measured"
    else:
        peak_gbs, peak_src = 6650.0, "fallback"
    achieved = bytes_sweep / launch_s / 1e9
    decode_hash = hashlib.sha256(open(os.path.join(ROOT, "maxuna_b200", "csrc", "decode.cu"), "rb").read()).hexdigest()[:16]
    if decode_hash == NCU_TRAFFIC["decode_cu_sha256_16"]:
        traffic = NCU_TRAFFIC["bytes_per_sweep"]
        traffic_src = ("constant: dram__bytes_read.sum + dram__bytes_write.sum of the five launches of one sweep in an ncu "
                       f"capture of this kernel source (decode.cu sha256 {decode_hash}); algorithmic bytes of that sweep: "
                       f"{NCU_TRAFFIC['algorithmic_bytes_of_that_sweep']:.4g}")
    else:
        traffic = None
        traffic_src = "no ncu capture of this kernel source yet (decode.cu changed since the last one)"
    sweep_tab = []
    for b in SWEEP:
        by = algorithmic_bytes(1, b) - EXPERT_BYTES + mean_u[b] * EXPERT_BYTES
        sweep_tab.append({"batch": b, "us_per_launch": per_b[b] * 1e6, "tok_per_s": b / per_b[b],
                          "distinct_experts": mean_u[b], "gb_per_s": by / per_b[b] / 1e9,
                          "frac_of_peak": by / per_b[b] / 1e9 / peak_gbs})

    # ---- end to end: host buffers through the C ABI ----
    # A step is one sweep: its five calls take their inputs from pinned host memory and leave their results in pinned
    # host memory.  Headline: the asynchronous entry (like the reference's ops, which return before the GPU has run
    # them), the stream synchronised once per step, when the step's results are read.  Beside it the synchronous
    # entry, which waits for the GPU inside every call.
    xh = {b: [x.cpu().pin_memory() for x in xs[b][:8]] for b in SWEEP}
    oh = {b: torch.empty(b, H).pin_memory() for b in SWEEP}
    e2e_steps = max(20, args.steps // 10)

    def host_call(j, b, fn):
        ly = layers[j % args.layers]
        _native.check(fn(ly.handle, xh[b][j % 8].data_ptr(), b, oh[b].data_ptr(), None, None,
                         ws[j % args.layers].data_ptr(), ws[j % args.layers].numel(), stream))

    def e2e_run(fn, sync_each_step):
        j = 0
        for _ in range(3):
            for b in SWEEP:
                host_call(j, b, fn)
                j += 1
        torch.cuda.synchronize()
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            for b in SWEEP:
                host_call(j, b, fn)
                j += 1
            if sync_each_step:
                torch.cuda.current_stream().synchronize()
        torch.cuda.synchronize()
        return time.perf_counter() - t0

    e2e_sync_s = e2e_run(lib.lmoe_moe_forward_host, False)          # synchronises inside every call
    e2e_s = e2e_run(lib.lmoe_moe_forward_host_async, True)

    # ---- max over ranks ----
    tokens_per_step = sum(SWEEP)
    if world > 1:
        tt = torch.tensor([ms, e2e_s, e2e_sync_s], device=dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms, e2e_s, e2e_sync_s = float(tt[0]), float(tt[1]), float(tt[2])
    value = world * tokens_per_step * args.steps / (ms * 1e-3)
    e2e_val = world * tokens_per_step * e2e_steps / e2e_s

    # ---- CPU baseline (rank 0, N=1 only, bounded sample) ----
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        from oracle import oracle as orc

        host = layers[0].host_layer(orc)
        xs_cpu = {b: xs[b][0].cpu().numpy() for b in SWEEP}
        cpu_time_sweep(host, xs_cpu, (1,), 1e9)
        tok, sec = cpu_time_sweep(host, xs_cpu, SWEEP + SWEEP + SWEEP, 20.0)
        cpu = {"value": tok / sec, "unit": "tok/s", "cores": orc.num_threads(), "kind": "port",
               "sample": f"{tok} tokens of the decode sweep on layer 0 (int8-activation k-quant dots, OpenMP)",
               "build": "-O3 -march=native, 256-bit integer SIMD where the host has it"}

    prefill = None
    if not args.no_prefill:
        del layers, ws
        torch.cuda.empty_cache()
        prefill = measure_prefill(dev, rank, world, tokens=args.prefill_tokens or None, ep_mode=args.ep_mode, ep_waves=args.ep_waves)

    stack = None
    if not args.no_stack:
        # config 5: all 48 layers; expert parallel under torchrun, whole on the device on one GPU (75.5 GB)
        if prefill is None:
            del layers, ws
        torch.cuda.empty_cache()
        stack = measure_stack(dev, rank, world, 48, steps=3, warmup=3)

    lm_head = measure_lm_head(dev) if (rank == 0 and world == 1 and not args.no_stack) else None

    if rank == 0:
        line = {
            "metric": "moe_layer_decode_tok_per_s", "value": value, "unit": "tok/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "q4_K/q6_K (u8 fields) x s8 activation digits (3 digits = 21 bits up to 8 tokens, 2 digits = 15 bits beyond) -> s32 -> f32",
            "data": "synthetic",
            "config": {"workload": WORKLOAD,
                       "hidden": H, "expert_ff": F, "n_expert": E, "top_k": K, "shared_expert": True,
                       "layers_rotated": args.layers,
                       "l2": f"inputs larger than L2: {args.layers} layer copies ({args.layers * 1.573:.1f} GB), "
                             "a different copy and hidden-state batch every launch",
                       "parallelism": "replicas" if world > 1 else "single GPU"},
            "gpu_launches": args.steps * len(SWEEP),
            "e2e": {"value": e2e_val, "unit": "tok/s",
                    "h2d_bytes_per_step": tokens_per_step * H * 4, "d2h_bytes_per_step": tokens_per_step * H * 4,
                    "steps": e2e_steps,
                    "mode": "lmoe_moe_forward_host_async: five host-buffer calls per step, stream synchronised once per step",
                    "sync_every_call": {"value": world * tokens_per_step * e2e_steps / e2e_sync_s, "unit": "tok/s",
                                        "mode": "lmoe_moe_forward_host: stream synchronised inside each of the five calls"}},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak_gbs, "unit": "GB/s",
                         "frac": achieved / peak_gbs, "traffic": traffic, "peak_source": peak_src,
                         "traffic_source": traffic_src,
                         "kernel": "moe_decode_kernel", "algorithmic_bytes_per_sweep": bytes_sweep},
            "provenance": {"library": lib.lmoe_version().decode(), "decode_path": "moe_decode_kernel: fused routing + indexed "
                           "mat-vecs + SwiGLU + combine + shared expert, one cooperative launch per batch",
                           "mm_id_min_seq": int(lib.lmoe_mm_id_min_seq()),
                           "seeds": {"layers": [100 * rank + i for i in range(args.layers)], "hidden_states": 1234 + rank},
                           "decode_cu_sha256_16": decode_hash},
            "sweep": sweep_tab,
            "clocks": clocks,
        }
        if cpu is not None:
            line["cpu_baseline"] = cpu
        if prefill is not None:
            peaks = json.load(open(peaks_path)) if os.path.exists(peaks_path) else {"bf16_tflops": 1590.0}
            line["prefill"] = {
                "workload": ("config3: 4096-token prefill of one layer, Zipf-skewed routing, 1 GPU (zipf_t16384: the "
                             "16384 tokens of config4 on one GPU, the anchor of the expert-parallel curve)" if world == 1 else
                             f"config4: 16384-token expert-parallel prefill over {world} GPUs (256/{world} experts per GPU, "
                             "all-to-all dispatch and combine)"),
                "unit": "TFLOP/s", "flops_per_token": (K + 1) * 18874368,
                "peak_tflops": peaks.get("bf16_tflops"), "results": prefill,
                "frac_of_peak": {k: v["tflops"] / (peaks.get("bf16_tflops") * world) for k, v in prefill.items()},
            }
        if lm_head is not None:
            line["lm_head"] = lm_head
        if stack is not None:
            stack["workload"] = ("config5: residual stack of MoE layers, 64-sequence batched decode and 2048-token prefill" +
                                 (f", expert parallel over {world} GPUs" if world > 1 else
                                  ", one GPU (all 48 layers resident: 75.5 GB)"))
            line["stack"] = stack
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
