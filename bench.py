#!/usr/bin/env python
"""Benchmark of the GGUF quantized-linear decode path (Q4_K / Q4_0 GEMV sweep) on B200.

One "step" is one pass over the whole decode sweep: batch 1, 4 and 16 activation rows, Q4_0 and Q4_K weights,
shapes (K->N) 3840->3840, 3840->15360, 15360->3840, 5120->17408, 17408->5120, fp32 in / fp32 out.  The step
streams 350 MB of distinct packed weights per batch size (larger than L2; two sets of weights), in an order that puts at
least 350 MB of other traffic between two uses of the same matrix, so no launch finds its weights in L2.  The timed
steps replay two CUDA graphs each (the roofline kernel's two launches, then the rest) with one event between them.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line.  `value` is algorithmic bytes per second over the timed steps with inputs resident in
HBM; `e2e` is the same sweep through the host-buffer C-ABI call (activations copied in, results copied out,
every call); `roofline` covers the Q4_K decode kernel at batch 1 and 4; `cpu_baseline` times the CPU oracle
(a port of the reference's CPU path) on the host cores.  With N > 1 every matrix is tensor-parallel: up-projections
are split by output rows, down-projections by 256-aligned input columns with an NCCL all-reduce of the partials.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SHAPES = [(3840, 3840), (3840, 15360), (15360, 3840), (5120, 17408), (17408, 5120)]  # (K, N)
BATCHES = [1, 4, 16]
Q4_0, Q4_K = 2, 12
FORMATS = [(Q4_K, "q4_k"), (Q4_0, "q4_0")]
METRIC = "Q4_K/Q4_0 decode GEMV sweep, algorithmic HBM GB/s"
BPW = 0.5625
# DRAM bytes (read + write) over algorithmic bytes of one captured launch of the roofline kernel (ncu, the Q4_K batch-1
# block of five matrices: 177.70 MB read + 3.91 MB written for 175.83 MB algorithmic)
NCU_TRAFFIC_RATIO = (177.70 + 3.91) / 175.83


def algorithmic_bytes(k: int, n: int, m: int) -> int:
    """Packed weight bytes (original GGUF packing) + fp32 activations in + fp32 results out."""
    return int(n * k * BPW) + m * k * 4 + m * n * 4


def read_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return float(p["hbm_gbs"]), float(p.get("bf16_tflops", 1590.0)), "measured"
    return 6650.0, 1590.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = "clocks.sm,clocks.max.sm,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index: int):
        self.index = index
        self.rows = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 7:
                continue
            try:
                sm.append(float(r[0]))
                smax.append(float(r[1]))
            except ValueError:
                continue
            for name, v in zip(names, r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(smax) if smax else None, "samples": len(sm), "reasons": sorted(reasons),
                "window": "every 20 ms from before ~0.25 s (several GPUs: 600) of untimed steps of the same work, through the warm-up, to the end of the timed steps"}


def run_ours(args):
    import torch
    import torch.distributed as dist

    from zllm_b200.backend import B200Context
    from zllm_b200.dist import shard_plan

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    if world > 1:
        import datetime
        import faulthandler

        # a collective that never completes must end the run with a traceback, not sit on the GPUs
        faulthandler.dump_traceback_later(args.watchdog, exit=True)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank), timeout=datetime.timedelta(seconds=120))
    ctx = B200Context(local_rank)
    if world > 1 and not args.nccl_reduce:
        ctx.dist_init(slot_bytes=4 << 20)  # peer group of the node: exchange buffers mapped over CUDA IPC
    if args.no_pdl:
        ctx.set_option("disable_pdl", 1)
    if args.f16_gemv:
        ctx.set_option("force_f16_gemv", 1)
    if args.fused_gemm:
        ctx.set_option("force_fused_gemm", 1)
    if args.narrow_tiles:
        ctx.set_option("narrow_gemv_tiles", 1)
    device = torch.device("cuda", local_rank)
    hbm_peak, _, peak_kind = read_peaks()
    if args.only_prefill:
        m, k, n = args.only_prefill, 5120, 17408
        full = torch.randn((n, k), device=device, dtype=torch.float32) * 0.02
        w = ctx.prepare_weight(Q4_K, ctx.quantize(Q4_K, full), n, k)
        del full
        x = torch.randn((m, k), device=device, dtype=torch.float32).to(torch.bfloat16)
        for _ in range(max(args.steps, 1)):
            y = ctx.linear(x, w)
        ctx.sync()
        print(json.dumps({"only_prefill": m, "launches": ctx.launch_count}))
        return

    if args.only_kquant:
        print(json.dumps({"only_kquant": bench_kquant_decode(ctx, device, read_peaks()[0]), "launches": ctx.launch_count}))
        return

    if args.only_moe:
        out = bench_moe(ctx, device, args, world, rank, only=args.only_moe)
        print(json.dumps({"only_moe": args.only_moe, "moe": out, "launches": ctx.launch_count}))
        return

    # ---- synthetic inputs: N(0, 0.02) weights quantised on the device, N(0, 1) activations, seed 0
    gen = torch.Generator(device=device)
    # two sets of the ten matrices: batch 1 and 16 use set 0, batch 4 uses set 1, so that the two Q4_K blocks that open a
    # step (batch 1, batch 4) do not share a byte
    case_sets = []  # per set: (fmt_name, fmt, k, n, mode, weight, k_local, n_local)
    for wset in range(2):
        cases = []
        for fmt, name in FORMATS:
            for si, (k, n) in enumerate(SHAPES):
                gen.manual_seed(1000 * fmt + si + 100000 * wset)
                full = torch.randn((n, k), generator=gen, device=device, dtype=torch.float32) * 0.02
                mode, (r0, r1), (c0, c1) = shard_plan(k, n, world, rank)
                local = full[r0:r1, c0:c1].contiguous()
                del full
                packed = ctx.quantize(fmt, local)
                w = ctx.prepare_weight(fmt, packed, r1 - r0, c1 - c0)
                del local, packed
                cases.append((name, fmt, k, n, mode, w, (c0, c1), (r0, r1)))
        case_sets.append(cases)
    cases = case_sets[0]
    xs = {}
    for k in sorted({k for k, _ in SHAPES}):
        gen.manual_seed(77 + k)
        xs[k] = torch.randn((max(BATCHES), k), generator=gen, device=device, dtype=torch.float32)
    ctx.sync()
    torch.cuda.synchronize()

    # Step order.  The two blocks of the roofline kernel come first (Q4_K batch 1 on set 0, Q4_K batch 4 on set 1), then
    # Q4_0 batch 1 (set 0), Q4_0 batch 4 (set 1), Q4_K batch 16 (set 0), Q4_0 batch 16 (set 0): at least 350 MB of other
    # weights stream between two uses of a matrix, so no launch finds its weights in L2.
    order = [(1, Q4_K), (4, Q4_K), (1, Q4_0), (4, Q4_0), (16, Q4_K), (16, Q4_0)]
    plan = []
    for m, fmt in order:
        for case in case_sets[1 if m == 4 else 0]:
            if case[1] == fmt:
                plan.append((m, case))
    if args.only:
        oname, oshape, om = args.only.split(":")
        ok, on = (int(v) for v in oshape.split("x"))
        plan = [(m, c) for m, c in plan if c[0] == oname and c[2] == ok and c[3] == on and m == int(om)]
        if not plan:
            raise SystemExit(f"--only {args.only}: no such case")
    if args.only_block:
        oname, om = args.only_block.split(":")
        plan = [(m, c) for m, c in plan if c[0] == oname and m == int(om)]
        if not plan:
            raise SystemExit(f"--only-block {args.only_block}: no such block")
    outs = {}
    for m, case in plan:
        name, fmt, k, n, mode, w, (c0, c1), (r0, r1) = case
        outs[(m, name, k, n)] = torch.empty((m, r1 - r0), device=device, dtype=torch.float32)
    x_local = {}
    for m, case in plan:
        name, fmt, k, n, mode, w, (c0, c1), (r0, r1) = case
        x_local[(m, k, c0, c1)] = xs[k][:m, c0:c1].contiguous()

    import ctypes as C

    from zllm_b200 import ffi

    def launch(m, case, collective=True):
        name, fmt, k, n, mode, w, (c0, c1), (r0, r1) = case
        x = x_local[(m, k, c0, c1)]
        y = outs[(m, name, k, n)]
        if mode == "row" and world > 1 and not args.nccl_reduce:
            ffi.call("zq_linear_row_parallel", ctx.handle, w.handle, C.c_void_p(x.data_ptr()), ffi.F32, m, C.c_void_p(y.data_ptr()), ffi.F32, None)
            return
        ffi.call("zq_linear", ctx.handle, w.handle, C.c_void_p(x.data_ptr()), ffi.F32, m, C.c_void_p(y.data_ptr()), ffi.F32, None)
        if mode == "row" and collective and world > 1:
            dist.all_reduce(y)

    # A block is one (batch, format) group: five distinct matrices, 175 MB of packed weights.  By default a block is ONE
    # zq_linear_batch call (the work-list decode kernel: one record pass + one persistent launch for the five
    # matrices); --per-call issues one zq_linear per matrix instead.  No matrix appears twice in a block, and the
    # blocks in between stream 175-350 MB of other weights, so no launch finds its weights in L2.
    # CUDA graphs keep the host out of the timed region (a Python/ctypes call costs more than a 5 us kernel).
    # Collectives are never captured: with several GPUs the all-reduces of a block's K-split matrices are launched
    # from the host right after the block's graph.  Events around the Q4_K batch-1 and batch-4 blocks (the headline
    # kernel) are recorded inside the timed region.
    blocks = []
    for m, fmt in order:
        members = [(mm, case) for mm, case in plan if mm == m and case[1] == fmt]
        if members:
            blocks.append((m, fmt, members))
    head = [bi for bi, (m, fmt, _) in enumerate(blocks) if fmt == Q4_K and m <= 4]  # the roofline kernel's blocks: the first ones of a step
    job_arrays = []
    for m, fmt, members in blocks:
        arr = (ffi.ZqLinearJob * len(members))()
        for i, (mm, case) in enumerate(members):
            name, _, k, n, mode, w, (c0, c1), (r0, r1) = case
            arr[i].w = w.handle.value
            arr[i].w_up = None
            arr[i].dev_x = x_local[(mm, k, c0, c1)].data_ptr()
            arr[i].m = mm
            arr[i].dev_y = outs[(mm, name, k, n)].data_ptr()
            arr[i].dev_residual = None
            # K-split matrices: the partial results of the ranks are summed by the library's own peer-store reduce kernel
            arr[i].flags = ffi.JOB_ROW_PARALLEL if (mode == "row" and world > 1 and not args.nccl_reduce) else 0
        job_arrays.append(arr)
    # --nccl-reduce (A/B aid): the partials are summed by a host-launched NCCL all-reduce after the block instead
    reduce_after = [[outs[(mm, case[0], case[2], case[3])] for mm, case in members if case[4] == "row" and args.nccl_reduce] for _, _, members in blocks]

    def launch_block(bi):
        m, fmt, members = blocks[bi]
        if args.per_call:
            for mm, case in members:
                launch(mm, case, collective=False)
        else:
            ffi.call("zq_linear_batch", ctx.handle, job_arrays[bi], len(members), ffi.F32, ffi.F32)

    for bi in range(len(blocks)):  # eager pass: sizes every internal buffer before capture
        launch_block(bi)
    torch.cuda.synchronize()
    graphs = []  # one graph per block
    launches_per_graph = []
    if not args.no_graph:
        side = torch.cuda.Stream(device=device)
        try:
            for bi in range(len(blocks)):
                g = torch.cuda.CUDAGraph()
                n0 = ctx.launch_count
                with torch.cuda.graph(g, stream=side):
                    ctx.set_stream(torch.cuda.current_stream(device).cuda_stream)
                    launch_block(bi)
                graphs.append(g)
                launches_per_graph.append(ctx.launch_count - n0)
            # A step as TWO graphs: the roofline kernel's blocks (Q4_K batch 1 and 4), then the rest, each chained by
            # programmatic dependent launch with no host launch inside; one CUDA event between the two.
            step_graph = None
            if not args.nccl_reduce and not args.per_call and head == list(range(len(head))) and len(head) < len(blocks):
                step_graph = []
                for part in (head, [bi for bi in range(len(blocks)) if bi not in head]):
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, stream=side):
                        ctx.set_stream(torch.cuda.current_stream(device).cuda_stream)
                        for bi in part:
                            launch_block(bi)
                    step_graph.append(g)
        except Exception as exc:
            graphs = []
            step_graph = None
            sys.stderr.write(f"bench: graph capture failed ({exc}); launching from the host\n")
        ctx.set_stream(torch.cuda.current_stream(device).cuda_stream)
    else:
        step_graph = None

    def step(events=None, head_events=None):
        if events is None and step_graph is not None:  # the headline form: two graph replays per step
            if head_events is not None:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
            step_graph[0].replay()
            if head_events is not None:
                e1.record()
                head_events.append((e0, e1))
            step_graph[1].replay()
            return
        for bi, (m, fmt, members) in enumerate(blocks):
            mark = events is not None
            if mark:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
            if graphs:
                graphs[bi].replay()
            else:
                launch_block(bi)
            if world > 1:
                for y in reduce_after[bi]:
                    dist.all_reduce(y)
            if mark:
                e1.record()
                events.append((bi, e0, e1))

    step_bytes = sum(algorithmic_bytes(case[2], case[3], m) for m, case in plan)
    q4k_kernel_bytes = sum(algorithmic_bytes(case[2], case[3], m) for m, case in plan if case[1] == Q4_K and m <= 4)
    # launches of the roofline kernel per step: one per Q4_K batch-1/-4 block (work list), or one per matrix (--per-call)
    q4k_kernel_launches = sum(1 for m, case in plan if case[1] == Q4_K and m <= 4) if args.per_call else sum(1 for m, fmt, _ in blocks if fmt == Q4_K and m <= 4)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # The timed region of a default run lasts a few milliseconds, less than one period of the clock sampler, so the
    # sampler runs from here on: through ~0.25 s of untimed steps of the very same work (not counted as warm-up steps),
    # the warm-up steps and the timed steps.
    sampler = ClockSampler(local_rank)
    if rank == 0 and not args.no_clocks:
        sampler.start()
    if not args.no_clocks:
        if world > 1:
            # every rank must issue the same number of steps (the row-parallel reduces pair up across ranks), so the
            # settle phase is a fixed count here, not a time
            for _ in range(30):
                for _ in range(20):
                    step()
                torch.cuda.synchronize()
        else:
            settle = time.perf_counter()
            while time.perf_counter() - settle < 0.25:
                for _ in range(20):
                    step()
                torch.cuda.synchronize()
    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    launches_before = ctx.launch_count
    events = []
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    head_events = [] if step_graph is not None else None
    t0.record()
    for _ in range(args.steps):
        step(None if step_graph is not None else events, head_events)
    t1.record()
    barrier()
    ctx.sync()
    elapsed_ms = t0.elapsed_time(t1)
    head_ms = sum(a.elapsed_time(b) for a, b in head_events) if head_events else None
    launches = ctx.launch_count - launches_before
    per_block_pass_ms = elapsed_ms
    if step_graph is not None:
        # Second pass over the very same K steps, block by block (one graph per block, CUDA events on the launching
        # stream around each): the per-block report.  Not part of the timed region.
        barrier()
        p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        p0.record()
        for _ in range(args.steps):
            step(events)
        p1.record()
        barrier()
        ctx.sync()
        per_block_pass_ms = p0.elapsed_time(p1)
    block_ms = [0.0] * len(blocks)
    for bi, a, b in events:
        block_ms[bi] += a.elapsed_time(b)
    kernel_ms = sum(t for t, (m, fmt, _) in zip(block_ms, blocks) if fmt == Q4_K and m <= 4)
    per_block_kernel_ms = kernel_ms
    if head_ms is not None:  # the roofline kernel's launches as timed inside the timed region (first graph of every step)
        kernel_ms = head_ms
    # every block of the step on its own (this rank's CUDA events; see "per_block_pass")
    blocks_report = [{"batch": m, "format": "q4_k" if fmt == Q4_K else "q4_0", "us": round(t / max(args.steps, 1) * 1e3, 2),
                      "gbs": round(sum(algorithmic_bytes(c[2], c[3], mm) for mm, c in members) / (t / max(args.steps, 1) * 1e-3) / 1e9 / max(world, 1), 1) if t > 0 else None}
                     for t, (m, fmt, members) in zip(block_ms, blocks)]
    if graphs:  # replayed launches do not pass through the library's counter: count what each graph captured
        launches = sum(launches_per_graph) * args.steps
    clocks = sampler.stop() if rank == 0 and not args.no_clocks else None
    if world > 1:
        t = torch.tensor([elapsed_ms, kernel_ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms, kernel_ms = float(t[0]), float(t[1])
        lt = torch.tensor([launches], device=device, dtype=torch.int64)
        dist.all_reduce(lt)
        launches = int(lt[0])
    ms_per_step = elapsed_ms / args.steps
    value = step_bytes / (ms_per_step * 1e-3) / 1e9
    achieved = q4k_kernel_bytes * args.steps / (kernel_ms * 1e-3) / 1e9 / max(world, 1) if kernel_ms > 0 else 0.0

    # ---- end to end through the host-buffer entry point (activations H2D, results D2H, every call)
    e2e = None
    if world == 1 and not args.no_e2e:
        import numpy as np

        # inputs and outputs live in pinned host memory (the library copies from / to page-locked buffers directly and
        # stages pageable ones through its own pinned arena)
        hx_t = {k: xs[k].cpu().pin_memory() for k in xs}
        hy_t = {key: torch.zeros(tuple(v.shape), dtype=torch.float32).pin_memory() for key, v in outs.items()}
        hx = {k: t.numpy() for k, t in hx_t.items()}
        hy = {key: t.numpy() for key, t in hy_t.items()}

        host_jobs = [(hx[case[2]][:m], case[5], hy[(m, case[0], case[2], case[3])]) for m, case in plan]
        host_arr = (ffi.ZqLinearHostJob * len(host_jobs))()
        for i, (xh, w, yh) in enumerate(host_jobs):
            host_arr[i].w, host_arr[i].host_x, host_arr[i].m, host_arr[i].host_y = w.handle.value, xh.ctypes.data, xh.shape[0], yh.ctypes.data

        def host_step(bracket):
            # one step = every matrix of the sweep through the host-buffer entry.  Bracketed (Backend::begin_batch /
            # finish_batch of the reference): one zq_linear_host_batch call = begin, zq_linear_host per matrix, finish,
            # so the calls only enqueue and the step waits once.  Unbracketed: zq_linear_host waits inside every call.
            if bracket:
                ffi.call("zq_linear_host_batch", ctx.handle, host_arr, len(host_jobs), ffi.F32, ffi.F32)
                return
            for xh, w, yh in host_jobs:
                ctx.linear_host(xh, w, yh)

        def time_host(bracket):
            host_step(bracket)
            n = max(1, min(args.steps, 20))
            torch.cuda.synchronize()
            h0 = time.perf_counter()
            for _ in range(n):
                host_step(bracket)
            torch.cuda.synchronize()
            return (time.perf_counter() - h0) / n

        t_call, t_batch = time_host(False), time_host(True)
        e2e = {  # h2d: an input shared by several matrices of the bracket travels once
            "value": round(step_bytes / t_batch / 1e9, 2), "unit": "GB/s",
            "h2d_bytes_per_step": sum(m * k * 4 for m, k in {(m, case[2]) for m, case in plan}), "d2h_bytes_per_step": sum(m * case[3] * 4 for m, case in plan),
            "ms_per_step": round(t_batch * 1e3, 3), "api": "zq_linear_host_batch = zq_batch_begin, zq_linear_host per matrix (H2D from pinned host memory starts, the layer is recorded; layers launched as work-list batches once a launch-worth is pending, D2H to pinned host memory), zq_batch_finish (the rest, one wait)",
            "per_call_wait": {"value": round(step_bytes / t_call / 1e9, 2), "ms_per_step": round(t_call * 1e3, 3), "api": "zq_linear_host waiting inside every call"},
        }

    parity = None
    if world > 1 and not args.nccl_reduce:
        parity = {"tp_row_split_max_rel_error": tp_parity(ctx, device, world, rank), "ep_moe_max_rel_error": ep_parity(device, world, rank, local_rank, experts_per_rank=16), "bound": 2e-3,
                  "ep_moe_prefill_path_max_rel_error": ep_parity(device, world, rank, local_rank), "prefill_path_chain_bound": 4e-3,
                  "what": "TP: Q4_K 1024x4096, 4 rows, K-split over the ranks + peer-store reduce; EP: 64 tokens, 16 experts per rank (owners on the decode path, as in the "
                          "64-token case) and 16 experts in all (owners on the prefill path: two tensor-core GEMMs per expert with an f16 intermediate, each within 2e-3 of the "
                          "CPU matmul on its own input, the chain of the two within 4e-3); all against float64 references on the bit-exact dequantised weights"}
    launch_desc = ("two CUDA graphs per step (Q4_K batch 1+4, then the other four blocks; zq_linear_batch calls chained by programmatic dependent launch)" if step_graph is not None
                   else "one CUDA graph per block" if graphs else "host launches")
    # free the sweep's weights before the larger side measurements
    extras = {}
    if not args.no_extras:
        del graphs, step_graph, cases, case_sets, plan, blocks, job_arrays
        torch.cuda.empty_cache()
        if world == 1 and args.extras in ("all", "prefill"):
            extras["prefill_gemm"] = bench_prefill(ctx, device, args)
        if world == 1 and args.extras in ("all", "prefill"):
            extras["kquant_decode"] = bench_kquant_decode(ctx, device, hbm_peak)
        if world == 1 and args.extras in ("all", "configs"):
            sustained = hbm_peak
            peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
            sustained_tf = float(json.load(open(peaks_path)).get("bf16_tflops_sustained", 1387.8)) if os.path.exists(peaks_path) else 1400.0
            extras["config0_minicpm5_decode_step"] = bench_config0(ctx, device, hbm_peak)
            extras["config3_iq4nl_q8_0"] = bench_config3(ctx, device, hbm_peak, sustained_tf)
        if args.extras in ("all", "moe"):
            extras["moe"] = bench_moe(ctx, device, args, world, rank)
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    cpu = cpu_baseline_sample() if world == 1 and not args.no_cpu else None
    line = {
        "metric": METRIC, "value": round(value, 2), "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "u4 x s16 (two s8 limbs) -> s32, f32 scales", "data": "synthetic",
        "config": {"workload": "configs[1]: decode GEMV sweep, batch 1/4/16, Q4_0+Q4_K, 5 shapes, fp32 in/out", "l2": "inputs larger than L2: 350 MB of distinct weights between reuses",
                   "parallelism": f"tp{world}" if world > 1 else "single", "bytes_per_step": step_bytes, "launch": launch_desc, "launches_per_step": launches // max(args.steps, 1) // max(world, 1)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 2), "peak": hbm_peak, "unit": "GB/s", "frac": round(achieved / hbm_peak, 4),
                     # ncu, 5120x17408 batch-1 launch: dram read+write = 50.21 MB for 50.23 MB algorithmic; scaled by bytes
                     "traffic": int(q4k_kernel_bytes // max(q4k_kernel_launches, 1) * NCU_TRAFFIC_RATIO), "traffic_kind": "ncu capture of one launch, scaled by algorithmic bytes",
                     "kernel": "zq::gemv_i8_kernel<Q4_K, 1 column tile> (batch 1 and 4, one launch per matrix)" if args.per_call else "zq::gemv_wl_kernel<Q4_K, 1 column tile> (batch 1 and 4; one launch per block of five matrices, timed together with its record pass)", "peak_kind": peak_kind, "launches": q4k_kernel_launches * args.steps,
                     "timing": ("CUDA events inside the timed region around the first graph of every step = the Q4_K batch-1 and batch-4 launches (with their record passes), chained by programmatic dependent launch" if head_ms is not None else "CUDA events around each block inside the timed region"),
                     "per_block_pass": {"what": "the same launches timed one graph per block with an event pair each, in a second pass after the timed region", "achieved": round(q4k_kernel_bytes * args.steps / (per_block_kernel_ms * 1e-3) / 1e9 / max(world, 1), 2) if per_block_kernel_ms > 0 else None,
                                        "ms_per_step": round(per_block_pass_ms / args.steps, 4)},
                     "bytes_per_launch_avg": q4k_kernel_bytes // max(q4k_kernel_launches, 1)},
        "gpu_launches": launches, "clocks": clocks, "e2e": e2e, "cpu_baseline": cpu,
        "blocks": blocks_report, "parity": parity,
    }
    line.update(extras)
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def tp_parity(ctx, device, world, rank):
    """Correctness of the multi-GPU path on the hardware it runs on, outside any timed region: one K-split matrix
    (Q4_K, 1024 x 4096, 4 rows; every rank quantises its 256-aligned column slice, the blocks being independent the
    slices concatenate to the full quantised weight) through the row-parallel entry, against a float64 product with
    the library's (bit-exact) dequantisation of the SAME weight as one matrix.  Returns max_i |a_i - e_i| / max(|e_i|, rms(e)), the largest over the ranks."""
    import torch
    import torch.distributed as dist

    from zllm_b200.dist import shard_plan

    n, k, m = 1024, 4096, 4
    gen = torch.Generator(device=device)
    gen.manual_seed(4242)
    full = torch.randn((n, k), generator=gen, device=device, dtype=torch.float32) * 0.02
    x = torch.randn((m, k), generator=gen, device=device, dtype=torch.float32)
    units = k // 256
    base, extra = divmod(units, world)
    lo = rank * base + min(rank, extra)
    hi = lo + base + (1 if rank < extra else 0)
    c0, c1 = lo * 256, hi * 256
    w_local = ctx.prepare_weight(Q4_K, ctx.quantize(Q4_K, full[:, c0:c1].contiguous()), n, c1 - c0)
    w_full = ctx.prepare_weight(Q4_K, ctx.quantize(Q4_K, full), n, k)
    got = ctx.linear_row_parallel(x[:, c0:c1].contiguous(), w_local)
    want = x.double() @ ctx.dequantize(w_full).double().T  # float64 product with the exact dequantised values
    ctx.sync()
    rms = want.double().pow(2).mean().sqrt()
    err = ((got.double() - want.double()).abs() / torch.maximum(want.double().abs(), rms)).max()
    t = torch.tensor([float(err)], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    w_local.release()
    w_full.release()
    return float(t[0])


def ep_parity(device, world, rank, local_rank, experts_per_rank=None):
    """Correctness of the expert-parallel MoE forward on the hardware it runs on, outside any timed region: experts
    (Q4_K, hidden 512, FFN 256, top-4, one shared expert) over the ranks, 64 tokens data-parallel, against the same
    layer in float64 on the library's (bit-exact) dequantised weights, for this rank's tokens.  Largest error over the
    ranks.  With 16 experts per rank the owners run the decode path (integer-MMA kernels, f32 intermediate), as the
    64-token case of the bench does; with 16 experts in all they run the prefill path (tensor-core GEMMs, f16
    intermediate between the two GEMMs of an expert)."""
    import torch
    import torch.distributed as dist

    from zllm_b200.backend import B200Context, MoeExperts, moe_forward, moe_forward_ep, moe_route
    from zllm_b200.dist import expert_range

    E, K, H, I, M = (experts_per_rank * world if experts_per_rank else 16), 4, 512, 256, 64
    c = B200Context(local_rank)
    c.dist_init(slot_bytes=1 << 20)
    c.moe_ep_init(M // world, H, K, E, dtype=torch.bfloat16)
    gen = torch.Generator(device=device)

    def make(rows, cols, seed):
        gen.manual_seed(seed)
        full = torch.randn((rows, cols), generator=gen, device=device, dtype=torch.float32) * 0.03
        return c.prepare_weight(Q4_K, c.quantize(Q4_K, full), rows, cols)

    gates = [make(I, H, 100 + 3 * e) for e in range(E + 1)]
    ups = [make(I, H, 101 + 3 * e) for e in range(E + 1)]
    downs = [make(H, I, 102 + 3 * e) for e in range(E + 1)]
    lo, hi = expert_range(E, world, rank)
    local_table = MoeExperts(c, gates[lo:hi], ups[lo:hi], downs[lo:hi])
    shared = (gates[E], ups[E], downs[E])
    gen.manual_seed(55)
    x_all = torch.randn((M, H), generator=gen, device=device, dtype=torch.float32).to(torch.bfloat16)
    router = torch.randn((E, H), generator=gen, device=device, dtype=torch.float32) / (H ** 0.5)
    per = M // world
    x = x_all[rank * per:(rank + 1) * per].contiguous()
    ids, w = moe_route(c, x, router, K, 1.0, True)
    got = moe_forward_ep(c, local_table, x, ids, w, shared=shared, out_dtype=torch.float32)
    c.sync()
    # float64 reference from the library's (bit-exact) dequantised values
    dq = lambda lst: [c.dequantize(wgt).double() for wgt in lst]
    Wg, Wu, Wd = dq(gates), dq(ups), dq(downs)
    xd = x.double()

    def expert(e, rows):
        g, u = rows @ Wg[e].T, rows @ Wu[e].T
        return (g / (1.0 + torch.exp(-g)) * u) @ Wd[e].T

    want = expert(E, xd)
    for t in range(per):
        for j in range(K):
            want[t] += float(w[t, j]) * expert(int(ids[t, j]), xd[t:t + 1])[0]
    rms = want.double().pow(2).mean().sqrt()
    err = ((got.double() - want.double()).abs() / torch.maximum(want.double().abs(), rms)).max()
    t = torch.tensor([float(err)], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dist.barrier()
    del local_table
    for wgt in gates + ups + downs:
        wgt.release()
    c.close()
    return float(t[0])


def _time_ms(fn, reps):
    import torch

    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps


def _graph_time_us(ctx, device, fn, reps=20):
    """Average time of one fn() call: captured once in a CUDA graph (after an eager pass that sizes the library's
    buffers), replayed `reps` times between CUDA events."""
    import torch

    fn()
    torch.cuda.synchronize()
    side = torch.cuda.Stream(device=device)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=side):
        ctx.set_stream(torch.cuda.current_stream(device).cuda_stream)
        fn()
    ctx.set_stream(torch.cuda.current_stream(device).cuda_stream)
    for _ in range(3):
        g.replay()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(reps):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps * 1e3


def bench_config0(ctx, device, hbm_peak):
    """configs[0]: the decode step of a 1B-class dense decoder (MiniCPM5-1B Q4_K_M shape): hidden 1536, q/o 1536 -> 1536,
    k/v 1536 -> 512, gate/up 1536 -> 3840, down 3840 -> 1536, Q4_K from N(0, 0.02), one f32 N(0, 1) row, seed 0; LM head
    Q8_0 with a synthetic vocabulary of 32 768 rows (the reference reads the vocabulary from the model file).  24
    layers of distinct weights (326 MB: larger than L2) are walked in turn.  Reported: latency of every projection on
    its own (one zq_linear per call), and of the layer's linear work as the fused operators issue it: RMSNorm + q/k/v
    (zq_rmsnorm_linear, one decode launch), o + residual, RMSNorm + gate/up + SiLU and down + residual (zq_gated_mlp).
    Attention itself is not part of this path and is left out."""
    import ctypes as C

    import torch

    from zllm_b200 import ffi

    hidden, kv, ffn, layers, vocab = 1536, 512, 3840, 24, 32768
    shapes = {"q": (hidden, hidden), "k": (kv, hidden), "v": (kv, hidden), "o": (hidden, hidden), "gate": (ffn, hidden), "up": (ffn, hidden), "down": (hidden, ffn)}
    gen = torch.Generator(device=device)
    weights = []
    for l in range(layers):
        layer = {}
        for i, (name, (rows, cols)) in enumerate(shapes.items()):
            gen.manual_seed(l * 16 + i)
            full = torch.randn((rows, cols), generator=gen, device=device, dtype=torch.float32) * 0.02
            layer[name] = ctx.prepare_weight(Q4_K, ctx.quantize(Q4_K, full), rows, cols)
        weights.append(layer)
    gen.manual_seed(999)
    head_full = torch.randn((vocab, hidden), generator=gen, device=device, dtype=torch.float32) * 0.02
    head = ctx.prepare_weight(8, ctx.quantize(8, head_full), vocab, hidden)
    del head_full
    gen.manual_seed(0)
    x = torch.randn((1, hidden), generator=gen, device=device, dtype=torch.float32)
    xf = torch.randn((1, ffn), generator=gen, device=device, dtype=torch.float32)
    norm_w = torch.ones(hidden, device=device, dtype=torch.float32)
    out = {"layers_walked": layers, "unit": "us", "weights": "Q4_K (N(0, 0.02) through the reference's encoder), LM head Q8_0 x 32768 rows (synthetic vocabulary)"}
    per = {}
    for name, (rows, cols) in shapes.items():
        src = xf if cols == ffn else x
        y = torch.empty((1, rows), device=device, dtype=torch.float32)

        def each(name=name, src=src, y=y, rows=rows):
            for l in range(layers):
                ffi.call("zq_linear", ctx.handle, weights[l][name].handle, C.c_void_p(src.data_ptr()), ffi.F32, 1, C.c_void_p(y.data_ptr()), ffi.F32, None)

        us = _graph_time_us(ctx, device, each) / layers
        nbytes = int(rows * cols * BPW) + cols * 4 + rows * 4
        per[name] = {"us": round(us, 2), "gbs": round(nbytes / us / 1e3, 1)}
    out["per_projection"] = per
    yq, yk, yv = (torch.empty((1, r), device=device, dtype=torch.float32) for r in (hidden, kv, kv))
    yo, ymlp = torch.empty((1, hidden), device=device, dtype=torch.float32), torch.empty((1, hidden), device=device, dtype=torch.float32)
    y3 = (C.c_void_p * 3)(yq.data_ptr(), yk.data_ptr(), yv.data_ptr())

    def step():
        for l in range(layers):
            w = weights[l]
            w3 = (C.c_void_p * 3)(w["q"].handle, w["k"].handle, w["v"].handle)
            ffi.call("zq_rmsnorm_linear", ctx.handle, w3, 3, C.c_void_p(x.data_ptr()), ffi.F32, 1, C.c_void_p(norm_w.data_ptr()), C.c_float(1e-6), C.c_float(0.0), y3, ffi.F32)
            ffi.call("zq_linear", ctx.handle, w["o"].handle, C.c_void_p(yq.data_ptr()), ffi.F32, 1, C.c_void_p(yo.data_ptr()), ffi.F32, C.c_void_p(x.data_ptr()))
            ffi.call("zq_gated_mlp", ctx.handle, w["gate"].handle, w["up"].handle, w["down"].handle, C.c_void_p(yo.data_ptr()), ffi.F32, 1, C.c_void_p(ymlp.data_ptr()), ffi.F32, C.c_void_p(yo.data_ptr()))

    n0 = ctx.launch_count
    step()
    launches = (ctx.launch_count - n0) // layers
    us_layer = _graph_time_us(ctx, device, step) / layers
    layer_bytes = sum(int(r * c * BPW) for r, c in shapes.values())
    out["fused_layer"] = {"us": round(us_layer, 2), "launches": launches, "weight_bytes": layer_bytes, "gbs": round(layer_bytes / us_layer / 1e3, 1),
                          "roofline": {"bound": "hbm", "achieved": round(layer_bytes / us_layer / 1e3, 1), "peak": hbm_peak, "unit": "GB/s", "frac": round(layer_bytes / us_layer / 1e3 / hbm_peak, 4),
                                       "note": "13.6 MB per layer stream in 2 us at peak: the layer is bound by its launches, not by bandwidth"}}
    yh = torch.empty((1, vocab), device=device, dtype=torch.float32)
    us_head = _graph_time_us(ctx, device, lambda: ffi.call("zq_linear", ctx.handle, head.handle, C.c_void_p(x.data_ptr()), ffi.F32, 1, C.c_void_p(yh.data_ptr()), ffi.F32, None))
    head_bytes = int(vocab * hidden * 1.0625)
    out["lm_head_q8_0"] = {"us": round(us_head, 2), "gbs": round(head_bytes / us_head / 1e3, 1), "note": "53 MB: fits in L2 when replayed back to back"}
    for layer in weights:
        for w in layer.values():
            w.release()
    head.release()
    torch.cuda.empty_cache()
    return out


def bench_config3(ctx, device, hbm_peak, sustained_tflops):
    """configs[3]: mixed formats: IQ4_NL for the FFN (gate/up 3840 -> 15360, down 15360 -> 3840), Q8_0 for the attention
    projections (q, k, v, o taken as 3840 -> 3840: the head geometry is not given).  Decode with one f32 row (four
    layers of distinct weights, 650 MB, walked in turn) and prefill with 4 096 bf16 tokens (one layer)."""
    import ctypes as C

    import torch

    from zllm_b200 import ffi

    IQ4_NL, Q8_0 = 20, 8
    hidden, ffn, layers = 3840, 15360, 4
    shapes = [("q", Q8_0, hidden, hidden), ("k", Q8_0, hidden, hidden), ("v", Q8_0, hidden, hidden), ("o", Q8_0, hidden, hidden), ("gate", IQ4_NL, ffn, hidden), ("up", IQ4_NL, ffn, hidden), ("down", IQ4_NL, hidden, ffn)]
    bpw = {Q8_0: 1.0625, IQ4_NL: 0.5625}
    gen = torch.Generator(device=device)
    weights = []
    for l in range(layers):
        layer = {}
        for i, (name, fmt, rows, cols) in enumerate(shapes):
            gen.manual_seed(7000 + l * 16 + i)
            full = torch.randn((rows, cols), generator=gen, device=device, dtype=torch.float32) * 0.02
            layer[name] = ctx.prepare_weight(fmt, ctx.quantize(fmt, full), rows, cols)
            del full
        weights.append(layer)
    gen.manual_seed(1)
    x = torch.randn((1, hidden), generator=gen, device=device, dtype=torch.float32)
    xf = torch.randn((1, ffn), generator=gen, device=device, dtype=torch.float32)
    out = {"formats": "attention q/k/v/o Q8_0 3840->3840 (assumed geometry), FFN IQ4_NL 3840->15360 / 15360->3840"}
    dec, total_us, total_bytes = {}, 0.0, 0
    for name, fmt, rows, cols in shapes:
        src = xf if cols == ffn else x
        y = torch.empty((1, rows), device=device, dtype=torch.float32)

        def each(name=name, src=src, y=y):
            for l in range(layers):
                ffi.call("zq_linear", ctx.handle, weights[l][name].handle, C.c_void_p(src.data_ptr()), ffi.F32, 1, C.c_void_p(y.data_ptr()), ffi.F32, None)

        us = _graph_time_us(ctx, device, each) / layers
        nbytes = int(rows * cols * bpw[fmt]) + cols * 4 + rows * 4
        dec[name] = {"us": round(us, 2), "gbs": round(nbytes / us / 1e3, 1)}
        total_us += us
        total_bytes += nbytes
    dec["all_seven"] = {"us": round(total_us, 2), "gbs": round(total_bytes / total_us / 1e3, 1)}
    dec["roofline"] = {"bound": "hbm", "achieved": round(total_bytes / total_us / 1e3, 1), "peak": hbm_peak, "unit": "GB/s", "frac": round(total_bytes / total_us / 1e3 / hbm_peak, 4),
                       "kernels": "integer-MMA decode kernel, one launch per matrix (IQ4_NL: codebook looked up with byte permutes)"}
    out["decode_m1"] = dec
    m = 4096
    xb = torch.randn((m, hidden), generator=gen, device=device, dtype=torch.float32).to(torch.bfloat16)
    xfb = torch.randn((m, ffn), generator=gen, device=device, dtype=torch.float32).to(torch.bfloat16)
    pre, total_ms, total_flop = {}, 0.0, 0.0
    for name, fmt, rows, cols in shapes:
        src = xfb if cols == ffn else xb
        y = torch.empty((m, rows), device=device, dtype=torch.bfloat16)
        fn = lambda name=name, src=src, y=y: ffi.call("zq_linear", ctx.handle, weights[0][name].handle, C.c_void_p(src.data_ptr()), ffi.BF16, m, C.c_void_p(y.data_ptr()), ffi.BF16, None)
        fn()
        ms = _time_ms(fn, 3)
        flop = 2.0 * m * rows * cols
        pre[name] = {"ms": round(ms, 3), "tflops": round(flop / ms / 1e9, 1)}
        total_ms += ms
        total_flop += flop
        del y
    pre["all_seven"] = {"ms": round(total_ms, 3), "tflops": round(total_flop / total_ms / 1e9, 1)}
    pre["roofline"] = {"bound": "tensor", "achieved": round(total_flop / total_ms / 1e9, 1), "peak": sustained_tflops, "unit": "TFLOP/s", "frac": round(total_flop / total_ms / 1e9 / sustained_tflops, 4),
                       "kernels": "f16 operand pass (dequantise to the workspace) + tcgen05 GEMM: these block-32 formats have no fused prefill kernel"}
    out["prefill_m4096"] = pre
    for layer in weights:
        for w in layer.values():
            w.release()
    torch.cuda.empty_cache()
    return out


def bench_kquant_decode(ctx, device, hbm_peak=6545.9):
    """Q5_K and Q6_K, one activation row, 5120 -> 17408 (integer-MMA decode kernel, one launch per matrix): four
    distinct weights (245 / 292 MB, larger than L2) used in turn; GB/s of GGUF bytes."""
    import numpy as np
    import torch

    from zllm_b200 import Q5_K, Q6_K
    from zllm_b200.ffi import BLOCK

    k, n = 5120, 17408
    out = {"shape": "5120->17408, 1 row, f32 in/out", "unit": "GB/s"}
    x = torch.randn((1, k), device=device, dtype=torch.float32)
    for fmt, name in ((Q5_K, "q5_k"), (Q6_K, "q6_k")):
        e, b = BLOCK[fmt]
        scale = torch.from_numpy(np.frombuffer(np.float16(3e-4).tobytes(), dtype=np.uint8).copy()).to(device)
        weights = []
        for i in range(4):
            packed = torch.randint(0, 256, (n * k // e, b), device=device, dtype=torch.uint8)
            off = 208 if fmt == Q6_K else 0
            packed[:, off:off + 2] = scale
            if fmt == Q5_K:
                packed[:, 2:4] = scale
            weights.append(ctx.prepare_weight(fmt, packed.reshape(-1), n, k))
            del packed

        def sweep():
            for w in weights:
                ctx.linear(x, w)

        sweep()
        ms = _time_ms(sweep, 5) / len(weights)
        gbs = n * k // e * b / ms / 1e6
        out[name] = {"us_per_launch": round(ms * 1e3, 2), "gbs": round(gbs, 1), "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": hbm_peak, "unit": "GB/s", "frac": round(gbs / hbm_peak, 4)}}
        del weights
    out["kernel"] = "zq::gemv_i8_kernel<Q5_K / Q6_K, 1 column tile>"
    return out


def bench_prefill(ctx, device, args):
    """configs[2]: Q4_K 5120->17408 and 17408->5120, bf16 activations and outputs, f32 accumulate, a stack of
    64 distinct (up, down) pairs (6.4 GB packed) timed end to end.  Every layer takes fixed N(0,1) inputs (chaining
    un-normalised outputs would overflow), so the stack is 128 independent GEMMs over 128 distinct weights."""
    import ctypes as C

    import torch

    from zllm_b200 import ffi

    layers = args.stack_layers
    k, n = 5120, 17408
    gen = torch.Generator(device=device)
    ups, downs = [], []
    for l in range(layers):
        for lst, (rows, cols) in ((ups, (n, k)), (downs, (k, n))):
            gen.manual_seed(5000 + 2 * l + (lst is downs))
            full = torch.randn((rows, cols), generator=gen, device=device, dtype=torch.float32) * 0.02
            lst.append(ctx.prepare_weight(Q4_K, ctx.quantize(Q4_K, full), rows, cols))
            del full
    _, tensor_peak, kind = read_peaks()
    sustained = tensor_peak
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        sustained = float(json.load(open(path)).get("bf16_tflops_sustained", tensor_peak))
    out = {"unit": "TFLOP/s", "stack_layers": layers, "weights": "Q4_K 5120x17408 + 17408x5120 per layer", "activations": "bf16 in, bf16 out, f32 accumulate", "operands": "f16"}
    launches0 = ctx.launch_count
    for m in (512, 4096, 16384):
        gen.manual_seed(31 + m)
        x = torch.randn((m, k), generator=gen, device=device, dtype=torch.float32).to(torch.bfloat16)
        h0 = torch.randn((m, n), generator=gen, device=device, dtype=torch.float32).to(torch.bfloat16)
        h = torch.empty((m, n), device=device, dtype=torch.bfloat16)
        y = torch.empty((m, k), device=device, dtype=torch.bfloat16)

        def stack():
            for l in range(layers):
                ffi.call("zq_linear", ctx.handle, ups[l].handle, C.c_void_p(x.data_ptr()), ffi.BF16, m, C.c_void_p(h.data_ptr()), ffi.BF16, None)
                ffi.call("zq_linear", ctx.handle, downs[l].handle, C.c_void_p(h0.data_ptr()), ffi.BF16, m, C.c_void_p(y.data_ptr()), ffi.BF16, None)

        stack()
        ms = _time_ms(stack, 2 if m >= 4096 else 4)
        flops = layers * 2 * 2.0 * m * k * n
        out[f"m{m}"] = {"ms_per_stack": round(ms, 3), "tflops": round(flops / ms / 1e9, 1)}
        del x, h0, h, y
    # end to end through the host-buffer entry: one up-projection at 4 096 tokens, bf16 rows in page-locked host memory in
    # and out (the copies cross PCIe inside the timed region)
    if not args.no_e2e:
        m = 4096
        hx = torch.randn((m, k), dtype=torch.float32).to(torch.bfloat16).pin_memory()
        hy = torch.empty((m, n), dtype=torch.bfloat16).pin_memory()

        def host_call():
            ffi.call("zq_linear_host", ctx.handle, ups[0].handle, C.c_void_p(hx.data_ptr()), ffi.BF16, m, C.c_void_p(hy.data_ptr()), ffi.BF16)

        host_call()
        t0 = time.perf_counter()
        for _ in range(5):
            host_call()
        dt = (time.perf_counter() - t0) / 5
        out["e2e"] = {"value": round(2.0 * m * k * n / dt / 1e12, 1), "unit": "TFLOP/s", "ms": round(dt * 1e3, 3), "h2d_bytes_per_step": m * k * 2, "d2h_bytes_per_step": m * n * 2,
                      "api": "zq_linear_host, Q4_K 5120->17408 at 4096 tokens, bf16 in / out in page-locked host memory (waits inside the call)"}
        del hx, hy
    if not args.no_cpu:
        out["cpu_baseline"] = cpu_prefill_sample()
    best = out["m16384"]["tflops"]
    out["roofline"] = {"bound": "tensor", "achieved": best, "peak": sustained, "unit": "TFLOP/s", "frac": round(best / sustained, 4), "peak_kind": kind + " (sustained bf16)", "kernel": "zq::gemm_kernel (tcgen05, M=16384, incl. operand dequantisation)"}
    out["gpu_launches"] = ctx.launch_count - launches0
    for w in ups + downs:
        w.release()
    torch.cuda.empty_cache()
    return out


def bench_moe(ctx, device, args, world, rank, only=None):
    """configs[4]: 256 experts, top-8, hidden 7168, expert FFN 2048 (Q4_K), one shared expert, softmax top-k router,
    bf16 activations; 64 tokens (decode) and 8192 tokens (prefill).  With N ranks the experts are expert-parallel
    (256/N per rank), tokens data-parallel (total fixed), routed rows cross ranks with one all-to-all each way."""
    import torch
    import torch.distributed as dist

    from zllm_b200.backend import MoeExperts, moe_forward, moe_forward_ep, moe_route
    from zllm_b200.dist import expert_parallel_forward, expert_range

    E, K, H, I = 256, 8, 7168, 2048
    lo, hi = expert_range(E, world, rank)
    gen = torch.Generator(device=device)

    def make(rows, cols, seed):
        gen.manual_seed(seed)
        full = torch.randn((rows, cols), generator=gen, device=device, dtype=torch.float32) * 0.02
        w = ctx.prepare_weight(Q4_K, ctx.quantize(Q4_K, full), rows, cols)
        del full
        return w

    gates = [make(I, H, 9000 + 3 * e) for e in range(lo, hi)]
    ups = [make(I, H, 9001 + 3 * e) for e in range(lo, hi)]
    downs = [make(H, I, 9002 + 3 * e) for e in range(lo, hi)]
    table = MoeExperts(ctx, gates, ups, downs)
    shared = (make(I, H, 8000), make(I, H, 8001), make(H, I, 8002))
    gen.manual_seed(8100)
    router = torch.randn((E, H), generator=gen, device=device, dtype=torch.float32) / (H ** 0.5)
    expert_bytes = 3 * int(I * H * BPW)
    native_ep = world > 1 and not args.nccl_reduce
    if native_ep:
        ctx.moe_ep_init(8192 // world, H, K, E, dtype=torch.bfloat16)  # exchange buffers for the larger of the two batches
    out = {"experts": E, "top_k": K, "hidden": H, "intermediate": I, "weights": "Q4_K", "parallelism": f"ep{world}" if world > 1 else "single", "exchange": ("peer-memory stores (zq_moe_forward_ep)" if native_ep else "NCCL all-to-all from the host") if world > 1 else None, "router": "softmax top-k, renormalised over the selected experts"}
    for name, m_total in (("decode_m64", 64), ("prefill_m8192", 8192)):
        if only and only != name:
            continue
        m = m_total // world
        gen.manual_seed(8200 + m_total)
        x_all = torch.randn((m_total, H), generator=gen, device=device, dtype=torch.float32).to(torch.bfloat16)
        x = x_all[rank * m:(rank + 1) * m].contiguous()

        def run_local(rows, local_ids, route_w):
            n = rows.shape[0]
            return moe_forward(ctx, table, rows, local_ids.view(n, 1).contiguous(), route_w.view(n, 1).contiguous(), out_dtype=torch.float32)

        def forward():
            ids, w = moe_route(ctx, x, router, K, 1.0, True)
            if world == 1:
                return moe_forward(ctx, table, x, ids, w, shared=shared, out_dtype=torch.bfloat16), ids
            if native_ep:  # dispatch, experts and combine inside the library, over peer memory
                return moe_forward_ep(ctx, table, x, ids, w, shared=shared, out_dtype=torch.bfloat16), ids
            routed = expert_parallel_forward(x, ids, w, E, run_local)
            sh = ctx.gated_mlp(x, *shared, out_dtype=torch.float32)
            return (routed + sh).to(torch.bfloat16), ids

        y, ids = forward()
        distinct = int(torch.unique(ids).numel())
        if world > 1:
            dist.barrier()
        ms = _time_ms(lambda: forward(), 3)
        if world > 1:
            t = torch.tensor([ms], device=device, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t[0])
        flops = (m_total * K + m_total) * 3 * 2.0 * H * I
        entry = {"tokens": m_total, "ms": round(ms, 3), "tflops": round(flops / ms / 1e9, 2)}
        if m_total == 64:
            entry["distinct_experts_hit_rank0"] = distinct
            entry["weight_gbs_rank0"] = round((distinct + 1) * expert_bytes / ms / 1e6, 1)
        if world == 1 and not args.no_e2e:
            # end to end through the public API: token rows from page-locked host memory, router, experts, result rows back
            hx = x.cpu().pin_memory()
            hy = torch.empty((m, H), dtype=torch.bfloat16).pin_memory()

            def host_forward():
                xd = hx.to(device, non_blocking=True)
                ids_d, w_d = moe_route(ctx, xd, router, K, 1.0, True)
                yd = moe_forward(ctx, table, xd, ids_d, w_d, shared=shared, out_dtype=torch.bfloat16)
                ctx.sync()
                hy.copy_(yd, non_blocking=True)
                torch.cuda.synchronize()

            host_forward()
            t0 = time.perf_counter()
            for _ in range(3):
                host_forward()
            dt = (time.perf_counter() - t0) / 3
            entry["e2e"] = {"value": round(flops / dt / 1e12, 2), "unit": "TFLOP/s", "ms": round(dt * 1e3, 3), "h2d_bytes_per_step": m * H * 2, "d2h_bytes_per_step": m * H * 2,
                            "api": "moe_route + moe_forward (zq_moe_route_softmax_topk, zq_moe_forward) on rows copied from / to page-locked host memory inside the timed region"}
            del hx, hy
        out[name] = entry
        del x_all, x, y
    if world == 1 and rank == 0 and not args.no_cpu:
        out["cpu_baseline"] = cpu_moe_sample()
    return out


def _random_q4k_bytes(rng, rows, cols):
    """Random Q4_K bytes with small finite scales: CPU time does not depend on the values."""
    import numpy as np

    data = rng.integers(0, 256, size=(rows * cols // 256, 144), dtype=np.uint8)
    data[:, 0:2] = np.frombuffer(np.float16(0.01).tobytes(), dtype=np.uint8)
    data[:, 2:4] = np.frombuffer(np.float16(0.01).tobytes(), dtype=np.uint8)
    return data.reshape(-1)


def cpu_prefill_sample():
    """ggml_quant::matmul (src/kernel/cpu/ggml_quant.rs:280-315) on the host cores: Q4_K 5120->17408 at 16 tokens."""
    import numpy as np

    from oracle import oracle as orc

    orc.set_threads(0)
    k, n, m = 5120, 17408, 16
    rng = np.random.default_rng(0)
    data = _random_q4k_bytes(rng, n, k)
    x = rng.standard_normal((m, k)).astype(np.float32)
    orc.linear(Q4_K, data, n, k, x)  # untimed: page in, start the worker threads
    t0 = time.perf_counter()
    passes = 0
    while passes < 3 or time.perf_counter() - t0 < 4.0:
        orc.linear(Q4_K, data, n, k, x)
        passes += 1
    dt = time.perf_counter() - t0
    return {"value": round(2.0 * m * n * k * passes / dt / 1e12, 4), "unit": "TFLOP/s", "cores": orc.threads(), "kind": "port", "sample": f"Q4_K 5120->17408 at {m} tokens, {passes} passes after one warm-up pass", "seconds": round(dt, 2)}


def cpu_moe_sample():
    """The CPU MoE path (src/kernel/cpu/moe.rs:122-138: per token, per routed expert, three matvecs) on the host cores:
    8 experts of the configured shape, every token routed to all 8, 4 tokens."""
    import numpy as np

    from oracle import oracle as orc

    orc.set_threads(0)
    E, K, H, I, m = 8, 8, 7168, 2048, 4
    rng = np.random.default_rng(0)
    gates = [(Q4_K, _random_q4k_bytes(rng, I, H), I, H) for _ in range(E)]
    ups = [(Q4_K, _random_q4k_bytes(rng, I, H), I, H) for _ in range(E)]
    downs = [(Q4_K, _random_q4k_bytes(rng, H, I), H, I) for _ in range(E)]
    x = rng.standard_normal((m, H)).astype(np.float32)
    ids = np.tile(np.arange(E, dtype=np.uint32), (m, 1))
    w = np.full((m, K), 1.0 / K, dtype=np.float32)
    orc.moe_forward(gates, ups, downs, x, ids, w)
    t0 = time.perf_counter()
    passes = 0
    while passes < 2 or time.perf_counter() - t0 < 4.0:
        orc.moe_forward(gates, ups, downs, x, ids, w)
        passes += 1
    dt = time.perf_counter() - t0
    flops = m * K * 3 * 2.0 * H * I * passes
    return {"value": round(flops / dt / 1e12, 5), "unit": "TFLOP/s", "tokens_per_s": round(m * passes / dt, 2), "cores": orc.threads(), "kind": "port",
            "sample": f"{E} experts of the configured shape, {m} tokens each routed to all {K}, {passes} passes after one warm-up pass", "seconds": round(dt, 2)}


def _cpu_sweep(batches, repeat_seed=0):
    """The decode sweep on the CPU oracle (ggml_quant::matvec for one row, ::matmul for several)."""
    import numpy as np

    from oracle import oracle as orc

    rng = np.random.default_rng(repeat_seed)
    work = []
    for fmt, name in FORMATS:
        for k, n in SHAPES:
            e, b = orc.BLOCK[fmt]
            # random packed bytes with small finite scales: CPU time does not depend on the values
            data = rng.integers(0, 256, size=(n * k // e, b), dtype=np.uint8)
            data[:, 0:2] = np.frombuffer(np.float16(0.01).tobytes(), dtype=np.uint8)
            if fmt == Q4_K:
                data[:, 2:4] = np.frombuffer(np.float16(0.01).tobytes(), dtype=np.uint8)
            work.append((fmt, k, n, data.reshape(-1)))
    xs = {k: rng.standard_normal((max(batches), k)).astype(np.float32) for k, _ in SHAPES}
    return orc, work, xs


def cpu_baseline_sample():
    """Times the CPU oracle on a bounded sample of the same sweep (batch 1 and 4 of every matrix)."""
    batches = [1, 4]
    orc, work, xs = _cpu_sweep(batches)
    orc.set_threads(0)
    cores = orc.threads()
    def one_pass():
        done = 0
        for m in batches:
            for fmt, k, n, data in work:
                orc.linear(fmt, data, n, k, xs[k][:m])
                done += algorithmic_bytes(k, n, m)
        return done

    one_pass()  # untimed: page in the weights, start the worker threads
    t0 = time.perf_counter()
    total, passes = 0, 0
    while passes < 3 or time.perf_counter() - t0 < 10.0:  # about 10 s of CPU work
        total += one_pass()
        passes += 1
    dt = time.perf_counter() - t0
    return {"value": round(total / dt / 1e9, 3), "unit": "GB/s", "cores": cores, "kind": "port", "sample": f"batch 1 and 4 of all 10 matrices, {passes} passes after one warm-up pass",
            "seconds": round(dt, 2)}


def run_reference(args):
    """Reference arm: the reference's own CPU algorithm for this path (C port in oracle/; the Rust original cannot
    be built here), all host threads, same sweep and metric.  Rank 0 only."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    orc, work, xs = _cpu_sweep(BATCHES)
    orc.set_threads(0)
    cores = orc.threads()

    def step():
        for m in BATCHES:
            for fmt, k, n, data in work:
                orc.linear(fmt, data, n, k, xs[k][:m])

    step_bytes = sum(algorithmic_bytes(k, n, m) for m in BATCHES for _, k, n, _ in work)
    # --steps and --warmup are honoured as given; only a run that would pass four minutes is cut short (and says so in
    # "steps"): a full sweep step takes ~0.2 s on 16 cores
    warm = max(args.warmup, 0)
    t_first = time.perf_counter()
    for _ in range(warm):
        step()
    est = (time.perf_counter() - t_first) / warm if warm else 0.2
    steps = max(1, min(args.steps, int(240.0 / max(est, 1e-3))))
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = time.perf_counter() - t0
    value = round(step_bytes * steps / dt / 1e9, 3)
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": steps, "warmup": warm, "ms_per_step": round(dt / steps * 1e3, 2),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "configs[1]: decode GEMV sweep, batch 1/4/16, Q4_0+Q4_K, 5 shapes, fp32 in/out", "bytes_per_step": step_bytes},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": cores, "kind": "port", "sample": f"{steps} full sweep step(s) on the host cores"},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg")
    ap.add_argument("--watchdog", type=int, default=480, help="multi-GPU runs: seconds after which a stuck run dumps tracebacks and exits")
    ap.add_argument("--no-extras", action="store_true", help="skip the prefill-GEMM and MoE side measurements")
    ap.add_argument("--extras", default="all", choices=["all", "prefill", "moe", "configs"], help="which side measurements to run")
    ap.add_argument("--nccl-reduce", action="store_true", help="several GPUs: sum the K-split partials with a host-launched NCCL all-reduce instead of the library's peer-store reduce (A/B aid)")
    ap.add_argument("--per-call", action="store_true", help="one zq_linear call (and launch) per matrix instead of one zq_linear_batch call per block (A/B aid)")
    ap.add_argument("--no-graph", action="store_true", help="launch every kernel from the host instead of replaying CUDA graphs")
    ap.add_argument("--no-clocks", action="store_true", help="do not sample clocks with nvidia-smi")
    ap.add_argument("--no-pdl", action="store_true", help="launch decode kernels without programmatic dependent launch (A/B aid)")
    ap.add_argument("--narrow-tiles", action="store_true", help="integer-MMA decode, up to 4 rows: 64-row tiles, two CTAs per SM (A/B aid)")
    ap.add_argument("--fused-gemm", action="store_true", help="Q4_K prefill on the kernel that dequantises inside the GEMM at every token count (A/B aid)")
    ap.add_argument("--f16-gemv", action="store_true", help="decode on the f16 warp-MMA kernels instead of the integer-MMA kernel (A/B aid)")
    ap.add_argument("--stack-layers", type=int, default=64, help="layers of the prefill GEMM stack (configs[2] names 64)")
    ap.add_argument("--only-prefill", type=int, default=0, help="profiling aid: run only a few prefill GEMMs (Q4_K 5120->17408) at this token count and exit")
    ap.add_argument("--only-kquant", action="store_true", help="profiling aid: run only the Q5_K / Q6_K one-row decode measurement and exit")
    ap.add_argument("--only-moe", default=None, choices=["decode_m64", "prefill_m8192"], help="profiling aid: run only this MoE case and exit")
    ap.add_argument("--only-block", default=None, help="restrict the sweep to one block of five matrices, e.g. q4_k:1 (format:batch); for profiling")
    ap.add_argument("--only", default=None, help="restrict the sweep to one case, e.g. q4_k:5120x17408:1 (format:KxN:batch); for profiling")
    ap.add_argument("--timeline", action="store_true", help="profiling aid for runs on several GPUs (where ncu is not used): record rank 0's kernels with the torch profiler (CUPTI) and print the last ones, with start offsets and durations, to stderr")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.timeline:
        run_with_timeline(args)
    else:
        run_ours(args)


def run_with_timeline(args):
    """The same run under the torch profiler; rank 0 prints the kernels of the library that ran last (one forward of
    --only-moe, or the last steps of the sweep) as `+start_us duration_us name` lines on stderr.  Times under a profiler
    are for attribution, never bench values."""
    import torch
    from torch.profiler import ProfilerActivity, profile

    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        run_ours(args)
    if int(os.environ.get("RANK", "0")) != 0:
        return
    events = [e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA and "zq::" in e.name]
    events.sort(key=lambda e: e.time_range.start)
    tail = events[-48:]
    if not tail:
        sys.stderr.write("timeline: no kernels of the library were recorded\n")
        return
    t0 = tail[0].time_range.start
    for e in tail:
        sys.stderr.write(f"+{e.time_range.start - t0:10.1f} {e.time_range.end - e.time_range.start:9.1f} us  {e.name[:110]}\n")


if __name__ == "__main__":
    main()
