#!/usr/bin/env python
"""Benchmark of the inference forward path on B200: the wide-MLP configuration.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (synthetic, seeded): X [65536, 4096] bf16 ~ N(0,1); 4 x (FC 4096->4096, bf16 weights ~ N(0, 1/4096),
fp32 bias, fp32 accumulation, ReLU); FC 4096->1000; softmax.  One step = one forward pass over the whole
batch; with N GPUs the batch is split evenly over the ranks (strong scaling) and the probabilities are
gathered on rank 0.  Prints ONE JSON line on rank 0.

`value` is samples/s with the inputs already resident in HBM; `e2e` is the same forward pass called with
pinned HOST buffers (host->device copy of X and device->host copy of the probabilities inside the timed
region).  `--impl reference` times the reference's own scalar CPU kernels on a bounded slice of the same
workload, one slice per host thread.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path[:0] = [ROOT, os.path.join(ROOT, "tests")]

BATCH, WIDTH, CLASSES, LAYERS, SEED = 65536, 4096, 1000, 4, 1003
METRIC, UNIT = "inference samples/sec", "samples/s"


def config(n_gpus, rows_per_rank):
    return {"workload": "wide MLP forward (BASELINE configs[2]): X[65536,4096] bf16 -> 4x(FC 4096->4096 + bias + ReLU) "
                        "-> FC 4096->1000 + bias -> softmax",
            "global_batch": BATCH, "rows_per_gpu": rows_per_rank, "parallelism": f"dp{n_gpus} (batch split; Gather to rank 0 by peer copies over NVLink, overlapped with the next step)",
            "l2": "inputs larger than L2 (X 512 MiB, activations 512 MiB per layer); no flush needed"}


def peaks():
    try:
        p = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        return float(p["bf16_tflops_sustained"]), "measured (MEASURED_PEAKS.json bf16_tflops_sustained)"
    except Exception:
        return 1400.0, "fallback (sustained figure of the profiling recipe)"


class ClockSampler:
    """Samples SM clock and throttle reasons while the timed region runs (read-only NVML queries)."""

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml as nv
            nv.nvmlInit()
            self.nv = nv
            self.h = nv.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = nv.nvmlDeviceGetMaxClockInfo(self.h, nv.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {"hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
                 "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
                 "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
                 "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4)}
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for k, bit in names.items():
                    if mask & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            self._stop.wait(0.05)

    def __enter__(self):
        if self.nv:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thread:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["nvml unavailable"]}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}


def make_inputs(torch, device, rows, row0):
    """Seeded synthetic tensors of the configuration, generated on the device.  Weights are identical on
    every rank (same seed); each rank draws its own rows of X."""
    g = torch.Generator(device=device).manual_seed(SEED)
    ws, bs = [], []
    for i in range(LAYERS + 1):
        n = WIDTH if i < LAYERS else CLASSES
        ws.append((torch.randn((WIDTH, n), generator=g, device=device) / WIDTH ** 0.5).to(torch.bfloat16).float())
        bs.append(torch.randn(n, generator=g, device=device) * 0.01)
    gx = torch.Generator(device=device).manual_seed(SEED * 1000 + row0)
    x = torch.randn((rows, WIDTH), generator=gx, device=device).to(torch.bfloat16)
    return x, ws, bs


class CpuArm:
    """The CPU implementation on `threads` slices of `rows_per_thread` rows each, one forward pass per slice,
    slices run concurrently (the reference's own batch split; its kernels are single-threaded)."""

    def __init__(self, rows_per_thread, threads, kind_pref="reference"):
        import numpy as np

        import cases
        from oracle import oracle as orc
        self.cases = cases
        self.impl = orc.Reference() if (kind_pref == "reference" and orc.Reference.available()) else orc.Oracle()
        if self.impl.kind == "port":
            self.impl.set_threads(1)  # parallelism comes from the slices, as for the reference
        self.threads, self.rows = threads, rows_per_thread * threads
        c = cases.config3_wide_mlp(batch=self.rows, width=WIDTH, classes=CLASSES, layers=LAYERS, seed=SEED)
        self.slices = [dict(c, x=np.ascontiguousarray(c["x"][i * rows_per_thread:(i + 1) * rows_per_thread]))
                       for i in range(threads)]

    def step(self):
        """One pass over all slices; returns seconds."""
        ts = [threading.Thread(target=self.cases.wide_mlp_forward, args=(self.impl, s)) for s in self.slices]
        t0 = time.perf_counter()
        for t in ts:
            t.start()
        for t in ts:
            t.join()
        return time.perf_counter() - t0


def run_reference(args, rank, world):
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    rows_per_thread = 32
    arm = CpuArm(rows_per_thread, threads)
    for _ in range(min(args.warmup, 1)):
        arm.step()
    total = sum(arm.step() for _ in range(args.steps))
    value = arm.rows * args.steps / total
    sample = (f"{arm.rows} rows per step ({rows_per_thread} per thread x {threads} threads) of the 65536-row batch, "
              "full-width layers")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": min(args.warmup, 1), "ms_per_step": 1e3 * total / args.steps, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config(args.gpus, BATCH // max(1, args.gpus)),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": arm.impl.kind, "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0}))


def run_ours(args, rank, world, local_rank):
    import torch
    import torch.distributed as dist

    import swcompiler_b200 as swc
    from swcompiler_b200.programs import WideMlpProgram

    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    rows = BATCH // world
    row0 = rank * rows
    be = swc.Backend(local_rank, swc.TC_BF16)
    x, ws, bs = make_inputs(torch, device, rows, row0)
    prog = WideMlpProgram(be, ws, bs, max_rows=rows)
    del ws
    # Two output buffers: with more than one GPU the Gather of step s (NCCL, on its own stream, through the
    # library's swcb200_gather) runs while the tensor cores work on step s+1.
    probs2 = [torch.empty((rows, CLASSES), dtype=torch.float32, device=device) for _ in range(2 if world > 1 else 1)]
    probs = probs2[0]
    comm = gathered = None
    if world > 1:
        from swcompiler_b200 import parallel as par

        def exchange(uid):
            box = [uid]
            dist.broadcast_object_list(box, src=0)
            return box[0]

        comm_stream = torch.cuda.Stream(device)
        comm = par.NcclComm(swc.Backend(local_rank, swc.TC_BF16, stream=comm_stream), rank, world, exchange)
        if rank == 0:
            gathered = torch.empty((BATCH, CLASSES), dtype=torch.float32, device=device)
        # The Gather: peer copies on the copy engines (swcb200_gather_rows), so that it takes no SM from the
        # persistent GEMMs of the next step; SWCB200_BENCH_GATHER=nccl selects the send/recv path instead.
        use_rows = os.environ.get("SWCB200_BENCH_GATHER", "rows") != "nccl"
        if use_rows:
            comm.gather_rows_setup(gathered, rows * CLASSES * 4, root=0)
    main_stream = torch.cuda.current_stream(device)
    gather_done = [None, None]
    counter = [0]

    def step(on_launch=None):
        s = counter[0]
        counter[0] += 1
        out = probs2[s % len(probs2)]
        if gather_done[s % 2] is not None:
            main_stream.wait_event(gather_done[s % 2])  # the buffer's previous Gather has read it
        prog.forward(x, out, on_launch=on_launch)
        if world > 1:
            ready = torch.cuda.Event()
            ready.record(main_stream)
            comm.be.torch_stream.wait_event(ready)
            if use_rows:
                comm.gather_rows(out)
            else:
                dst = C.c_void_p(gathered.data_ptr()) if rank == 0 else C.c_void_p(0)
                comm.be._call("gather", C.c_void_p(out.data_ptr()), dst, (C.c_size_t * 2)(BATCH, CLASSES), C.c_int(2),
                              C.c_int(0), C.c_int(swc.F32), C.c_int(0))
            done = torch.cuda.Event()
            done.record(comm.be.torch_stream)
            gather_done[s % 2] = done

    def drain():
        if world > 1:
            main_stream.wait_stream(comm.be.torch_stream)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()

    # ---- timed region: K steps, device-timed, per-launch events for the dominant kernel
    nl = prog.launches_per_forward
    ev = [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(nl)]
          for _ in range(args.steps)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = be.launches
    with ClockSampler(local_rank) as clocks:
        barrier()
        e0.record()
        for s in range(args.steps):
            step(on_launch=lambda i, when, s=s: ev[s][i][when].record())
        drain()
        e1.record()
        barrier()
    launches = be.launches - launches0 # the Gather is a copy-engine transfer, not a launch
    be.sync()  # also surfaces a device-side timeout status, if any
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    value = BATCH * args.steps / (ms * 1e-3)

    # dominant kernel: the hidden-layer FC launches (4 per step)
    fc_ms = [ev[s][i][0].elapsed_time(ev[s][i][1]) for s in range(args.steps) for i in range(LAYERS)]
    fc_avg_ms = sum(fc_ms) / len(fc_ms)
    flops_per_launch = 2.0 * rows * WIDTH * WIDTH
    achieved = flops_per_launch / (fc_avg_ms * 1e-3) / 1e12
    peak, peak_src = peaks()
    per_kernel_ms = [sum(ev[s][i][0].elapsed_time(ev[s][i][1]) for s in range(args.steps)) / args.steps for i in range(nl)]

    e2e_value = e2e_ms = None
    e2e_steps = max(3, min(args.steps, 10))
    x_host = probs_host = None
    if not args.skip_e2e:
        e2e_value, e2e_ms, x_host, probs_host = run_e2e(torch, dist, prog, x, probs, world, device, rows, e2e_steps,
                                                        barrier)

    cpu = None
    if rank == 0 and world == 1 and not args.skip_cpu_baseline:
        threads = os.cpu_count() or 1
        arm = CpuArm(64, threads)
        dt = arm.step()
        cpu = {"value": arm.rows / dt, "unit": UNIT, "cores": threads, "kind": arm.impl.kind,
               "sample": f"{arm.rows} rows (64 per thread x {threads} threads) of the 65536-row batch, one pass, {dt:.1f} s"}

    if rank == 0:
        e2e = None if e2e_value is None else {
            "value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": x_host.numel() * 2 * world,
            "d2h_bytes_per_step": probs_host.numel() * 4 * world, "ms_per_step": e2e_ms / e2e_steps}
        print(json.dumps({
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16 (fp32 accumulate)", "data": "synthetic", "config": config(world, rows),
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                         "traffic": 32e6 + 127.6e6 * rows / 8192, "traffic_source": "ncu dram bytes of the 8192-row launch (159.6 MB), row-proportional part scaled; profiles/fc_tc_pair_kernel__config3_layer.md", "kernel": "fc_tc_pair_kernel (FC 4096->4096 + bias + ReLU, one launch)",
                         "launch_ms": fc_avg_ms, "flops_per_launch": flops_per_launch, "peak_source": peak_src},
            "per_launch_ms": per_kernel_ms,
            "cpu_baseline": cpu, "e2e": e2e,
            "gpu_launches": launches, "clocks": clocks.summary()}))
    if world > 1:
        barrier()
        comm.close()
        dist.destroy_process_group()


def run_fcpair(args, rank, world, local_rank):
    """Model-parallel FC pair (BASELINE configs[3]): X[8192,8192] bf16 replicated; FC1 8192->32768 split by output
    columns -> ReLU; FC2 32768->8192 split by input rows; fp32 partial sums joined by an NCCL all-reduce.  One step =
    one forward pass over the 8192 rows; the rows go through in `--chunks` chunks so that the all-reduce of one chunk
    (communication stream) overlaps the tensor-core work of the next."""
    import torch
    import torch.distributed as dist

    import swcompiler_b200 as swc
    from swcompiler_b200 import parallel as par
    from swcompiler_b200.programs import FcPairProgram

    M, K, N1, N2 = args.fcpair_rows, 8192, 32768, 8192
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    be = swc.Backend(local_rank, swc.TC_BF16)

    def exchange(uid):
        box = [uid]
        if world > 1:
            dist.broadcast_object_list(box, src=0)
        return box[0]

    comm = par.NcclComm(swc.Backend(local_rank, swc.TC_BF16, stream=torch.cuda.Stream(device)), rank, world, exchange)
    g = torch.Generator(device=device).manual_seed(1004)
    x = torch.randn((M, K), generator=g, device=device).to(torch.bfloat16)
    # the rank's shards are drawn directly (same law as the full matrices; the full 512 MiB + 512 MiB fp32 weights
    # are never materialised): W1[:, cols of this rank] ~ N(0, 1/K), W2[rows of this rank, :] ~ N(0, 1/N1)
    gs = torch.Generator(device=device).manual_seed(1004 * 100 + rank)
    n1s = N1 // world

    w1s = (torch.randn((K, n1s), generator=gs, device=device) / K ** 0.5)
    w2s = (torch.randn((n1s, N2), generator=gs, device=device) / N1 ** 0.5)
    prog = FcPairProgram(be, comm, w1s, w2s, max_rows=M, sharded=True)
    del w1s, w2s
    chunks = args.chunks

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        prog.forward(x, chunks=chunks)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = be.launches
    with ClockSampler(local_rank) as clocks:
        barrier()
        e0.record()
        for _ in range(args.steps):
            prog.forward(x, chunks=chunks)
        e1.record()
        barrier()
    be.sync()
    comm.be.sync()
    ms = e0.elapsed_time(e1)
    # the two GEMMs alone (no all-reduce), for the roofline of the dominant kernel
    g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    import swcompiler_b200._lib as L
    g0.record()
    for _ in range(args.steps):
        be.fc_bf16(x, prog.wp1, None, L.ACT_RELU, out=prog.h)
    g1.record()
    torch.cuda.synchronize()
    fc1_ms = g0.elapsed_time(g1) / args.steps
    if world > 1:
        t = torch.tensor([ms, fc1_ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, fc1_ms = float(t[0].item()), float(t[1].item())
    launches = be.launches - launches0 - args.steps
    flops_fc1 = 2.0 * M * n1s * K
    peak, peak_src = peaks()
    if rank == 0:
        step_ms = ms / args.steps
        total_flops = 2.0 * M * N1 * (K + N2)
        print(json.dumps({
            "metric": METRIC, "value": M / (step_ms * 1e-3), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": step_ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16 (fp32 accumulate, fp32 all-reduce)", "data": "synthetic",
            "config": {"workload": "model-parallel FC pair (BASELINE configs[3]): X[8192,8192] bf16 -> FC 8192->32768 "
                                   "(column split) -> ReLU -> FC 32768->8192 (row split) -> all-reduce(sum)",
                       "global_batch": M, "parallelism": f"mp{world}", "chunks": chunks,
                       "l2": "weights (1 GiB / p per rank) larger than L2; no flush needed"},
            "job_tflops": total_flops / (step_ms * 1e-3) / 1e12,
            "roofline": {"bound": "tensor", "achieved": flops_fc1 / (fc1_ms * 1e-3) / 1e12, "peak": peak, "unit": "TFLOP/s",
                         "frac": flops_fc1 / (fc1_ms * 1e-3) / 1e12 / peak, "traffic": None,
                         "kernel": "fc_tc_pair_kernel (FC1 shard 8192 x 32768/p x 8192 + ReLU, one launch, timed alone)",
                         "launch_ms": fc1_ms, "flops_per_launch": flops_fc1, "peak_source": peak_src},
            "allreduce_bytes_per_rank": M * N2 * 4, "cpu_baseline": None, "e2e": None,
            "gpu_launches": launches, "clocks": clocks.summary()}))
    barrier()
    comm.close()
    if world > 1:
        dist.destroy_process_group()


def run_resstage(args, rank, world, local_rank):
    """ResNet-style stage (BASELINE configs[4]): [256,56,56,64] bf16 NHWC -> 3 x (Conv3x3+BN+ReLU, Conv3x3+BN+Add+ReLU) ->
    MaxPool 2x2/2, every Conv-BN-[Add]-ReLU chain one tensor-core launch.  The batch is split evenly over the ranks
    (every op is per-image, no collective inside the stage); the pooled outputs are gathered on rank 0 by peer copies."""
    import torch
    import torch.distributed as dist

    import swcompiler_b200 as swc
    from swcompiler_b200.programs import ResStageProgram

    N, HW, CH, BLOCKS = 256, 56, 64, 3
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    n = N // world
    be = swc.Backend(local_rank, swc.TC_BF16)
    g = torch.Generator(device=device).manual_seed(1005)
    convs = [dict(w=torch.randn((CH, 3, 3, CH), generator=g, device=device) * (2.0 / (9 * CH)) ** 0.5,
                  b=torch.zeros(CH, device=device)) for _ in range(2 * BLOCKS)]
    bns = [dict(scale=torch.rand(CH, generator=g, device=device) + 0.5, bias=torch.randn(CH, generator=g, device=device) * 0.1,
                mean=torch.randn(CH, generator=g, device=device) * 0.1, var=torch.rand(CH, generator=g, device=device) + 0.5,
                eps=1e-5) for _ in range(2 * BLOCKS)]
    gx = torch.Generator(device=device).manual_seed(1005 * 1000 + rank)
    x = torch.randn((n, HW, HW, CH), generator=gx, device=device).to(torch.bfloat16)
    prog = ResStageProgram(be, convs, bns, max_batch=n, hw=HW, ch=CH)
    comm = gathered = None
    if world > 1:
        from swcompiler_b200 import parallel as par

        def exchange(uid):
            box = [uid]
            dist.broadcast_object_list(box, src=0)
            return box[0]

        comm = par.NcclComm(swc.Backend(local_rank, swc.TC_BF16, stream=torch.cuda.Stream(device)), rank, world, exchange)
        if rank == 0:
            gathered = torch.empty((N, HW // 2, HW // 2, CH), dtype=torch.bfloat16, device=device)
        comm.gather_rows_setup(gathered, n * (HW // 2) * (HW // 2) * CH * 2, root=0)
    main_stream = torch.cuda.current_stream(device)

    def step(on_launch=None):
        out = prog.forward(x, on_launch=on_launch)
        if world > 1:
            ready = torch.cuda.Event()
            ready.record(main_stream)
            comm.be.torch_stream.wait_event(ready)
            comm.gather_rows(out)
            main_stream.wait_stream(comm.be.torch_stream)  # one pooled buffer: the next pass may overwrite it

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    nl = prog.launches_per_forward
    ev = [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(nl)]
          for _ in range(args.steps)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = be.launches
    with ClockSampler(local_rank) as clocks:
        barrier()
        e0.record()
        for s in range(args.steps):
            step(on_launch=lambda i, when, s=s: ev[s][i][when].record())
        e1.record()
        barrier()
    launches = be.launches - launches0
    be.sync()
    ms = e0.elapsed_time(e1)
    conv_ms = [ev[s][i][0].elapsed_time(ev[s][i][1]) for s in range(args.steps) for i in range(nl - 1)]
    conv_avg = sum(conv_ms) / len(conv_ms)
    if world > 1:
        t = torch.tensor([ms, conv_avg], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, conv_avg = float(t[0].item()), float(t[1].item())
    flops = 2.0 * n * HW * HW * CH * 9 * CH
    try:
        peak, peak_src = float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops"]), \
            "measured (MEASURED_PEAKS.json bf16_tflops, burst: the launches are short)"
    except Exception:
        peak, peak_src = 1590.0, "fallback (burst figure of the profiling recipe)"
    if rank == 0:
        step_ms = ms / args.steps
        achieved = flops / (conv_avg * 1e-3) / 1e12
        print(json.dumps({
            "metric": METRIC, "value": N / (step_ms * 1e-3), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": step_ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16 (fp32 accumulate)", "data": "synthetic",
            "config": {"workload": "ResNet-style conv stage (BASELINE configs[4]): [256,56,56,64] bf16 NHWC, 3 residual blocks "
                                   "of two 3x3 64->64 convolutions with BN / skip / ReLU fused, then MaxPool 2x2/2",
                       "global_batch": N, "images_per_gpu": n, "parallelism": f"dp{world} (batch split; pooled outputs gathered on rank 0)",
                       "l2": "activations (103 MB per tensor at 256 images) larger than L2 at 1 and 2 GPUs; smaller beyond"},
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                         "traffic": None, "kernel": "conv_tc_kernel (3x3 64->64 + BN [+ skip] + ReLU, one launch)",
                         "launch_ms": conv_avg, "flops_per_launch": flops, "peak_source": peak_src},
            "cpu_baseline": None, "e2e": None, "gpu_launches": launches, "clocks": clocks.summary()}))
    barrier()
    if world > 1:
        comm.close()
        dist.destroy_process_group()


def run_e2e(torch, dist, prog, x, probs, world, device, rows, e2e_steps, barrier):
    """End to end with host buffers (rank-local slice): H2D of X, forward, D2H of the probabilities."""
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    x_host = torch.empty((rows, WIDTH), dtype=torch.bfloat16).pin_memory()
    x_host.copy_(x.cpu())
    probs_host = torch.empty((rows, CLASSES), dtype=torch.float32).pin_memory()
    x_dev = torch.empty_like(x)
    for _ in range(2):
        prog.forward_host(x_host, probs_host, x_dev, probs)
    barrier()
    e0.record()
    for _ in range(e2e_steps):
        prog.forward_host(x_host, probs_host, x_dev, probs)  # every rank returns its rows to its own host buffer
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([e2e_ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    e2e_value = BATCH * e2e_steps / (e2e_ms * 1e-3)
    return e2e_value, e2e_ms, x_host, probs_host


def main():
    global BATCH
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=BATCH, help="rows in the whole job (smaller only for profiler captures)")
    ap.add_argument("--skip-cpu-baseline", action="store_true", help="leave the CPU sample out (profiler captures)")
    ap.add_argument("--skip-e2e", action="store_true", help="leave the host-buffer pass out (profiler captures)")
    ap.add_argument("--workload", default="widemlp", choices=["widemlp", "fcpair", "resstage"],
                    help="widemlp: the data-parallel wide MLP (default, the headline); fcpair: the model-parallel FC pair; "
                         "resstage: the batch-split ResNet-style conv stage")
    ap.add_argument("--chunks", type=int, default=4, help="fcpair: row chunks per forward (all-reduce overlap)")
    ap.add_argument("--fcpair-rows", type=int, default=8192, help="fcpair: rows of X")
    args = ap.parse_args()
    BATCH = args.batch
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
    elif args.workload == "fcpair":
        run_fcpair(args, rank, world, local_rank)
    elif args.workload == "resstage":
        run_resstage(args, rank, world, local_rank)
    else:
        run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
