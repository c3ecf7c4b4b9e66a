#!/usr/bin/env python
"""Benchmark of the inference forward path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload all|widemlp|...]

Headline workload (synthetic, seeded): the wide MLP -- X [65536, 4096] bf16 ~ N(0,1); 4 x (FC 4096->4096, bf16 weights
~ N(0, 1/4096), fp32 bias, fp32 accumulation, ReLU); FC 4096->1000; softmax.  One step = one forward pass over the
whole batch; with N GPUs the batch is split evenly over the ranks (strong scaling) and the probabilities are gathered
on rank 0.  Rank 0 prints ONE JSON line.

`value` is samples/s with the inputs already resident in HBM; `e2e` is the same program called with pinned HOST
buffers (host->device copy of X, the Gather, and the device->host copy of the gathered probabilities inside the timed
region).  `--impl reference` times the reference's own scalar CPU kernels on a bounded slice of the same workload,
one slice per host thread.

With `--workload all` (the default) the same line also carries, under `workloads`, the other configurations --
`resstage` (the batch-split ResNet-style conv stage), `fcpair` (the model-parallel FC pair, 2 GPUs and more) and
`latency` (the two small latency-bound networks, 1 GPU) -- and under `ops` every kernel of the table timed alone
against its own roofline (1 GPU).  At more than one GPU every gathered / reduced result is checked on rank 0 against a
recomputation from the known seeds (`gather_check`).
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
            "precision": "bf16 operands and stored activations, fp32 accumulation (the split-activation mode is reported under workloads.widemlp_split)",
            "l2": "inputs larger than L2 (X 512 MiB, activations 512 MiB per layer); no flush needed"}


def peaks():
    try:
        p = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        return {"sustained": float(p["bf16_tflops_sustained"]), "burst": float(p["bf16_tflops"]), "hbm": float(p["hbm_gbs"]),
                "source": "measured (MEASURED_PEAKS.json)"}
    except Exception:
        return {"sustained": 1400.0, "burst": 1590.0, "hbm": 6650.0, "source": "fallback (figures of the profiling recipe)"}


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
            self._stop.wait(0.02)

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


class Env:
    """One process per GPU: device, the process group (more than one rank) and the few collective helpers of the bench."""

    def __init__(self, rank, world, local_rank):
        import torch
        import torch.distributed as dist
        self.torch, self.dist = torch, dist
        self.rank, self.world, self.local_rank = rank, world, local_rank
        torch.cuda.set_device(local_rank)
        self.device = torch.device("cuda", local_rank)
        if world > 1:
            dist.init_process_group("nccl", device_id=self.device)

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, values):
        if self.world == 1:
            return [float(v) for v in values]
        t = self.torch.tensor([float(v) for v in values], device=self.device)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return [float(v) for v in t.tolist()]

    def gather_floats(self, values):
        """Every rank's list on rank 0 (a list of lists), None elsewhere."""
        if self.world == 1:
            return [[float(v) for v in values]]
        t = self.torch.tensor([float(v) for v in values], device=self.device)
        outs = [self.torch.empty_like(t) for _ in range(self.world)]
        self.dist.all_gather(outs, t)
        return [[float(v) for v in o.tolist()] for o in outs] if self.rank == 0 else None

    def exchange(self, uid):
        box = [uid]
        if self.world > 1:
            self.dist.broadcast_object_list(box, src=0)
        return box[0]

    def comm(self, swc):
        """A communicator of the kernel library on a stream of its own."""
        from swcompiler_b200 import parallel as par
        stream = self.torch.cuda.Stream(self.device)
        return par.NcclComm(swc.Backend(self.local_rank, swc.TC_BF16, stream=stream), self.rank, self.world, self.exchange)

    def close(self):
        if self.world > 1:
            self.barrier()
            self.dist.destroy_process_group()


def make_weights(torch, device):
    """Seeded synthetic weights of the configuration, generated on the device; identical on every rank."""
    g = torch.Generator(device=device).manual_seed(SEED)
    ws, bs = [], []
    for i in range(LAYERS + 1):
        n = WIDTH if i < LAYERS else CLASSES
        ws.append((torch.randn((WIDTH, n), generator=g, device=device) / WIDTH ** 0.5).to(torch.bfloat16).float())
        bs.append(torch.randn(n, generator=g, device=device) * 0.01)
    return ws, bs


def make_rows(torch, device, rows, row0):
    """The rows [row0, row0 + rows) of X: each rank draws its own slice from a seed that names its first row."""
    gx = torch.Generator(device=device).manual_seed(SEED * 1000 + row0)
    return torch.randn((rows, WIDTH), generator=gx, device=device).to(torch.bfloat16)


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


# ---------------------------------------------------------------------------------------------------------------------
# wide MLP (the headline)

def run_widemlp(env, args, split=False):
    """Returns the JSON record of the wide-MLP benchmark (rank 0; None elsewhere).  `split`: hidden activations are
    stored as two bf16 terms (value and rounding remainder) and every layer multiplies both, see fc_tcgen05.cu."""
    torch, dist = env.torch, env.dist
    import swcompiler_b200 as swc
    from swcompiler_b200.programs import WideMlpProgram

    world, rank, device = env.world, env.rank, env.device
    rows = BATCH // world
    row0 = rank * rows
    be = swc.Backend(env.local_rank, swc.TC_BF16)
    ws, bs = make_weights(torch, device)
    x = make_rows(torch, device, rows, row0)
    prog = WideMlpProgram(be, ws, bs, max_rows=rows, split=split)
    del ws
    # Two output buffers: with more than one GPU the Gather of step s runs while the tensor cores work on step s+1.
    probs2 = [torch.empty((rows, CLASSES), dtype=torch.float32, device=device) for _ in range(2 if world > 1 else 1)]
    comm = gathered = None
    use_rows = os.environ.get("SWCB200_BENCH_GATHER", "rows") != "nccl"
    if world > 1:
        comm = env.comm(swc)
        if rank == 0:
            gathered = torch.empty((BATCH, CLASSES), dtype=torch.float32, device=device)
        # The Gather: peer copies on the copy engines (swcb200_gather_rows), so that it takes no SM from the
        # persistent GEMMs of the next step; SWCB200_BENCH_GATHER=nccl selects the send/recv path instead.
        if use_rows:
            comm.gather_rows_setup(gathered, rows * CLASSES * 4, root=0)
    main_stream = torch.cuda.current_stream(device)
    gather_done = [None, None]
    counter = [0]

    def gather(out):
        ready = torch.cuda.Event()
        ready.record(main_stream)
        comm.be.torch_stream.wait_event(ready)
        if use_rows:
            comm.gather_rows(out)
        else:
            dst = C.c_void_p(gathered.data_ptr()) if rank == 0 else C.c_void_p(0)
            comm.be._call("gather", C.c_void_p(out.data_ptr()), dst, (C.c_size_t * 2)(BATCH, CLASSES), C.c_int(2),
                          C.c_int(0), C.c_int(swc.F32), C.c_int(0))

    def step(on_launch=None):
        s = counter[0]
        counter[0] += 1
        out = probs2[s % len(probs2)]
        if gather_done[s % 2] is not None:
            main_stream.wait_event(gather_done[s % 2])  # the buffer's previous Gather has read it
        prog.forward(x, out, on_launch=on_launch)
        if world > 1:
            gather(out)
            done = torch.cuda.Event()
            done.record(comm.be.torch_stream)
            gather_done[s % 2] = done

    def drain():
        if world > 1:
            main_stream.wait_stream(comm.be.torch_stream)

    for _ in range(max(args.warmup, 3)):
        step()
    env.barrier()

    # ---- timed region: K steps, device-timed, per-launch events for the dominant kernel
    nl = prog.launches_per_forward
    ev = [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(nl)]
          for _ in range(args.steps)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = be.launches
    with ClockSampler(env.local_rank) as clocks:
        env.barrier()
        e0.record()
        for s in range(args.steps):
            step(on_launch=lambda i, when, s=s: ev[s][i][when].record())
        drain()
        e1.record()
        env.barrier()
    launches = be.launches - launches0  # the Gather is a copy-engine transfer, not a launch
    be.sync()  # also surfaces a device-side timeout status, if any
    ms = env.max_over_ranks([e0.elapsed_time(e1)])[0]
    value = BATCH * args.steps / (ms * 1e-3)

    # dominant kernel: the hidden-layer FC launches (4 per step)
    fc_ms = [ev[s][i][0].elapsed_time(ev[s][i][1]) for s in range(args.steps) for i in range(LAYERS)]
    fc_avg_ms = sum(fc_ms) / len(fc_ms)
    flops_per_launch = 2.0 * rows * WIDTH * WIDTH * (1.0 if not split else 1.75)  # split: layers 2-4 multiply two terms
    achieved = flops_per_launch / (fc_avg_ms * 1e-3) / 1e12
    pk = peaks()
    per_kernel_ms = [sum(ev[s][i][0].elapsed_time(ev[s][i][1]) for s in range(args.steps)) / args.steps for i in range(nl)]

    check = None
    if world > 1:
        check = check_gather_widemlp(env, prog, gathered, rows)

    e2e = None
    if not args.skip_e2e and not split:
        e2e = run_e2e(env, args, prog, x, probs2, comm, gathered, rows)

    cpu = None
    if rank == 0 and world == 1 and not args.skip_cpu_baseline and not split:
        threads = os.cpu_count() or 1
        arm = CpuArm(64, threads)
        dt = arm.step()
        cpu = {"value": arm.rows / dt, "unit": UNIT, "cores": threads, "kind": arm.impl.kind,
               "sample": f"{arm.rows} rows (64 per thread x {threads} threads) of the 65536-row batch, one pass, {dt:.1f} s"}

    rec = None
    if rank == 0:
        # DRAM traffic of one hidden-layer launch by its operands: A and C once (rows x 4096 bf16 each), the packed
        # weight once (32 MiB); an ncu capture of an 8192-row launch measured 3 % less than this count.  Not measured here.
        traffic_model = 2.0 * rows * WIDTH * 2 + WIDTH * WIDTH * 2
        rec = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16 (fp32 accumulate)" + (", hidden activations as two bf16 terms" if split else ""), "data": "synthetic",
            "config": config(world, rows),
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": pk["sustained"], "unit": "TFLOP/s",
                         "frac": achieved / pk["sustained"], "traffic": None if split else traffic_model,
                         "traffic_source": "operand bytes of one launch (A + C + packed weight), not measured in this run",
                         "kernel": "fc_tc_pair_kernel (FC 4096->4096 + bias + ReLU, one launch)",
                         "launch_ms": fc_avg_ms, "flops_per_launch": flops_per_launch,
                         "peak_source": pk["source"] + " bf16_tflops_sustained"},
            "per_launch_ms": per_kernel_ms, "cpu_baseline": cpu, "e2e": e2e, "gather_check": check,
            "gpu_launches": launches, "clocks": clocks.summary()}
    if world > 1:
        env.barrier()
        comm.close()
    del prog, probs2, x, gathered
    torch.cuda.empty_cache()
    return rec


def check_gather_widemlp(env, prog, gathered, rows, samples=48):
    """Rank 0 draws every rank's slice of X again from its seed, pushes `samples` rows of each through the forward
    pass and compares them with what the Gather of the last step left in its buffer."""
    torch = env.torch
    env.barrier()
    if env.rank != 0:
        return None
    worst, n = 0.0, 0
    out = torch.empty((samples, CLASSES), dtype=torch.float32, device=env.device)
    for r in range(env.world):
        xr = make_rows(torch, env.device, rows, r * rows)
        idx = torch.linspace(0, rows - 1, samples, device=env.device).long()
        prog.forward(xr[idx].contiguous(), out)
        prog.be.sync()
        got = gathered[r * rows + idx]
        worst = max(worst, float((got - out).abs().max().item()))
        n += samples
        del xr
    return {"rows": n, "max_abs": worst, "ok": bool(worst <= 1e-6), "what": "gathered probabilities vs the same rows recomputed on rank 0"}


def run_e2e(env, args, prog, x, probs2, comm, gathered, rows):
    """End to end with host buffers: every rank copies its rows of X in from pinned host memory while earlier chunks
    compute, and copies its probabilities out, chunk by chunk, into its rows of ONE result array in host memory.  With
    more than one GPU that array is a shared-memory segment every rank has mapped and registered with CUDA: the Gather
    of the results on the host is carried by all the GPUs' copy engines at once instead of funnelling through rank 0's
    link."""
    torch = env.torch
    world, rank, device = env.world, env.rank, env.device
    steps = max(3, min(args.steps, 10))
    x_host = torch.empty((rows, WIDTH), dtype=torch.bfloat16).pin_memory()
    x_host.copy_(x.cpu())
    x_dev = torch.empty_like(x)
    chunk = min(4096, max(1024, rows // 8))  # short first copy-in and last copy-out; the copies, not the GEMMs, set the pace
    main = torch.cuda.current_stream(device)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    shm_path = None
    if world == 1:
        result = torch.empty((BATCH, CLASSES), dtype=torch.float32).pin_memory()
    else:
        # the result array: a file in /dev/shm created by rank 0, mapped by everyone, page-locked for CUDA by everyone
        nbytes = BATCH * CLASSES * 4
        if rank == 0:
            import tempfile
            st = os.statvfs("/dev/shm") if os.path.isdir("/dev/shm") else None
            where = "/dev/shm" if st and st.f_bavail * st.f_frsize > 2 * nbytes else tempfile.gettempdir()
            shm_path = os.path.join(where, f"swcb200_bench_{os.getpid()}")
        shm_path = env.exchange(shm_path)
        if rank == 0:
            with open(shm_path, "wb") as f:
                f.truncate(nbytes)
        env.barrier()
        result = torch.from_file(shm_path, shared=True, size=BATCH * CLASSES, dtype=torch.float32).view(BATCH, CLASSES)
        err = torch.cuda.cudart().cudaHostRegister(result.data_ptr(), nbytes, 0)
        if int(err) != 0:
            raise RuntimeError(f"cudaHostRegister of the shared result array failed ({err})")
    mine = result[rank * rows:(rank + 1) * rows]

    def one():
        prog.forward_host(x_host, mine, x_dev, probs2[0], chunk_rows=chunk)
    out_bytes = BATCH * CLASSES * 4

    def finish():
        pass  # forward_host has made the main stream wait for the last copy-out

    for _ in range(2):
        one()
    finish()
    env.barrier()
    e0.record()
    for _ in range(steps):
        one()
    finish()
    e1.record()
    env.barrier()
    e2e_ms = env.max_over_ranks([e0.elapsed_time(e1)])[0]

    # what the host links give each rank when every rank copies at once (plain pinned copies, no compute)
    def copy_gbs(dst, src, nbytes):
        c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        env.barrier()
        c0.record()
        for _ in range(3):
            dst.copy_(src, non_blocking=True)
        c1.record()
        torch.cuda.synchronize()
        return 3 * nbytes / (c0.elapsed_time(c1) * 1e-3) / 1e9
    h2d = copy_gbs(x_dev, x_host, x_host.numel() * 2)
    probe_host = torch.empty((rows, CLASSES), dtype=torch.float32).pin_memory()
    d2h = copy_gbs(probe_host, probs2[0], rows * CLASSES * 4)
    links = env.gather_floats([h2d, d2h])
    # the gathered result on the host against this rank's probabilities on the device (every rank checks its rows)
    torch.cuda.synchronize()
    same = bool(torch.equal(mine, probs2[0].cpu()))
    all_same = env.max_over_ranks([0.0 if same else 1.0])[0] == 0.0
    env.barrier()
    if world > 1:
        torch.cuda.cudart().cudaHostUnregister(result.data_ptr())
        del mine, result
        env.barrier()
        if rank == 0:
            os.unlink(shm_path)
    if rank != 0:
        return None
    return {"value": BATCH * steps / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": x_host.numel() * 2 * world,
            "d2h_bytes_per_step": out_bytes, "ms_per_step": e2e_ms / steps, "steps": steps, "chunk_rows": chunk,
            "program": "H2D of each rank's rows in chunks overlapped with compute; chunked D2H of its probabilities into its rows of "
                       "one result array in host memory" + ("" if world == 1 else " (a shared-memory segment all ranks map: the Gather happens over every GPU's host link at once)"),
            "result_on_host_matches_device": all_same,
            "host_link_GBps_all_ranks_copying": {"h2d_per_rank": [l[0] for l in links], "d2h_per_rank": [l[1] for l in links],
                                                  "h2d_sum": sum(l[0] for l in links), "d2h_sum": sum(l[1] for l in links)}}


# ---------------------------------------------------------------------------------------------------------------------
# model-parallel FC pair

def run_fcpair(env, args):
    """Model-parallel FC pair (BASELINE configs[3]): X[8192,8192] bf16 replicated; FC1 8192->32768 split by output
    columns -> ReLU; FC2 32768->8192 split by input rows; fp32 partial sums joined by an NCCL all-reduce.  One step =
    one forward pass over the 8192 rows; the rows go through in `--chunks` chunks so that the all-reduce of one chunk
    (communication stream) overlaps the tensor-core work of the next."""
    torch = env.torch
    import swcompiler_b200 as swc
    import swcompiler_b200._lib as L
    from swcompiler_b200.programs import FcPairProgram

    world, rank, device = env.world, env.rank, env.device
    M, K, N1, N2 = args.fcpair_rows, 8192, 32768, 8192
    be = swc.Backend(env.local_rank, swc.TC_BF16)
    comm = env.comm(swc)
    x = torch.randn((M, K), generator=torch.Generator(device=device).manual_seed(1004), device=device).to(torch.bfloat16)
    n1s = N1 // world

    def shards(r):
        # a rank's shards are drawn directly (same law as the full matrices, which are never materialised):
        # W1[:, cols of rank r] ~ N(0, 1/K), W2[rows of rank r, :] ~ N(0, 1/N1)
        gs = torch.Generator(device=device).manual_seed(1004 * 100 + r)
        w1 = torch.randn((K, n1s), generator=gs, device=device) / K ** 0.5
        w2 = torch.randn((n1s, N2), generator=gs, device=device) / N1 ** 0.5
        return w1, w2

    w1s, w2s = shards(rank)
    prog = FcPairProgram(be, comm, w1s, w2s, max_rows=M, sharded=True)
    del w1s, w2s
    chunks = args.chunks

    def timed(fn, steps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        env.barrier()
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        env.barrier()
        return e0.elapsed_time(e1) / steps

    comm_sms = args.comm_sms if world > 1 else 0
    for _ in range(max(args.warmup, 3)):
        prog.forward(x, chunks=chunks, comm_sms=comm_sms)
    launches0 = be.launches
    with ClockSampler(env.local_rank) as clocks:
        step_ms = timed(lambda: prog.forward(x, chunks=chunks, comm_sms=comm_sms), args.steps)
    launches = be.launches - launches0
    be.sync()
    comm.be.sync()
    serial_ms = timed(lambda: prog.forward(x, chunks=1), args.steps)          # no overlap: GEMMs, then one all-reduce
    fc1_ms = timed(lambda: be.fc_bf16(x, prog.wp1, None, L.ACT_RELU, out=prog.h), args.steps)   # the dominant kernel alone
    step_ms, serial_ms, fc1_ms = env.max_over_ranks([step_ms, serial_ms, fc1_ms])

    # check on rank 0: sampled rows against relu(X W1) W2 with every rank's shards drawn again (fp32 matmul of the
    # bf16-rounded operands; the hidden activation rounded to bf16 as the program stores it)
    shared_ms = timed(lambda: prog.forward(x, chunks=chunks), args.steps)      # chunked, GEMMs on every SM
    shared_ms = env.max_over_ranks([shared_ms])[0]
    y = prog.forward(x, chunks=chunks, comm_sms=comm_sms)
    be.sync()
    comm.be.sync()
    # The join done by FC2's own epilogue over peer memory (no collective kernel): every rank ends up with its row
    # block of the sum; the copy engines then carry the blocks to rank 0 (the reference's Reduce leaves the result on
    # the master).  Timed with and without that last Gather.
    peer_ms = peer_root_ms = None
    peer_err = None
    if world > 1 and M % world == 0:
        prog.peer_setup()
        y_root = torch.empty((M, N2), dtype=torch.float32, device=device) if rank == 0 else None
        comm.gather_rows_setup(y_root, (M // world) * N2 * 4, root=0)
        ms_stream, cs_stream = be.torch_stream, comm.be.torch_stream

        copied = [None, None]
        npass = [0]

        def peer_to_root():
            # the Gather of pass s runs on the communication stream beside pass s + 1; the two result buffers alternate
            s_ = npass[0] & 1
            npass[0] += 1
            if copied[s_] is not None:
                ms_stream.wait_event(copied[s_])   # the copy of two passes ago has read this buffer
            own = prog.forward_peer(x)
            ready = torch.cuda.Event()
            ready.record(ms_stream)
            cs_stream.wait_event(ready)
            comm.gather_rows(own)
            done = torch.cuda.Event()
            done.record(cs_stream)
            copied[s_] = done

        for _ in range(3):
            peer_to_root()
        ms_stream.wait_stream(cs_stream)
        peer_ms = timed(lambda: prog.forward_peer(x), args.steps)
        if prog._peer_pass & 1:
            prog.forward_peer(x)       # keep the program's and the bench's buffer parity in step

        def peer_root_steps():
            peer_to_root()

        def timed_drained(fn, steps):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            env.barrier()
            e0.record()
            for _ in range(steps):
                fn()
            ms_stream.wait_stream(cs_stream)   # the last Gather is inside the timed region
            e1.record()
            env.barrier()
            return e0.elapsed_time(e1) / steps
        npass[0] = 0
        copied[0] = copied[1] = None
        peer_root_ms = timed_drained(peer_root_steps, args.steps)
        peer_ms, peer_root_ms = env.max_over_ranks([peer_ms, peer_root_ms])
        peer_to_root()
        ms_stream.wait_stream(cs_stream)
        env.barrier()
        if rank == 0:
            peer_err = float((y_root - y).abs().max().item())
        env.barrier()
        comm.gather_rows_release()
    check = None
    if rank == 0:
        idx = torch.linspace(0, M - 1, 64, device=device).long()
        xs = x[idx].float()
        ref = torch.zeros((64, N2), device=device)
        for r in range(world):
            w1, w2 = shards(r)
            h = torch.relu(xs @ w1.to(torch.bfloat16).float()).to(torch.bfloat16).float()
            ref += h @ w2.to(torch.bfloat16).float()
            del w1, w2
        err = float((y[idx] - ref).abs().max().item())
        check = {"rows": 64, "max_abs": err, "ok": bool(err <= 2e-2), "what": "all-reduced output vs relu(X W1) W2 from the seeds"}
        if peer_err is not None:
            check["peer_join_vs_allreduce_max_abs"] = peer_err
            check["ok"] = bool(check["ok"] and peer_err <= 1e-3)
    env.barrier()
    flops_fc1 = 2.0 * M * n1s * K
    pk = peaks()
    rec = None
    if rank == 0:
        total_flops = 2.0 * M * N1 * (K + N2)
        variants = {"one all-reduce after the GEMMs": serial_ms, "all-reduce of row chunks beside the next chunk's GEMMs": shared_ms,
                    f"the same with {comm_sms} SMs left to the all-reduce": step_ms}
        if peer_root_ms is not None:
            variants["peer join (FC2's epilogue stores into the owners' memory), blocks gathered on rank 0"] = peer_root_ms
        best = min(variants, key=variants.get)
        best_ms = variants[best]
        rec = {
            "metric": METRIC, "value": M / (best_ms * 1e-3), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "value_variant": best, "ms_per_step_by_variant": variants,
            "ms_per_step": best_ms, "ms_per_step_no_overlap": serial_ms, "ms_per_step_chunked_all_sms": shared_ms,
            "ms_per_step_chunked_gemms_leave_sms": step_ms,
            "ms_per_step_peer_join": peer_ms, "ms_per_step_peer_join_to_root": peer_root_ms,
            "variants": "the all-reduce variants leave the result on every rank; peer_join leaves every rank its row block of the sum "
                        "(FC2's epilogue stores partial row blocks into their owners' memory over NVLink, the ranks meet, each adds "
                        "its p slots in rank order); peer_join_to_root adds the copy-engine Gather of the blocks to rank 0, where the "
                        "reference's Reduce leaves the result (the Gather of one pass runs beside the next pass)",
            "scaling": "strong",
            "dtype": "bf16 (fp32 accumulate, fp32 all-reduce)", "data": "synthetic",
            "config": {"workload": "model-parallel FC pair (BASELINE configs[3]): X[8192,8192] bf16 -> FC 8192->32768 "
                                   "(column split) -> ReLU -> FC 32768->8192 (row split) -> Reduce(sum) to rank 0",
                       "global_batch": M, "parallelism": f"mp{world}", "chunks": chunks,
                       "comm_sms": comm_sms,
                       "l2": "weights (1 GiB / p per rank) larger than L2; no flush needed"},
            "job_tflops": total_flops / (best_ms * 1e-3) / 1e12,
            "roofline": {"bound": "tensor", "achieved": flops_fc1 / (fc1_ms * 1e-3) / 1e12, "peak": pk["sustained"], "unit": "TFLOP/s",
                         "frac": flops_fc1 / (fc1_ms * 1e-3) / 1e12 / pk["sustained"], "traffic": None,
                         "kernel": "fc_tc_pair_kernel (FC1 shard 8192 x 32768/p x 8192 + ReLU, one launch, timed alone)",
                         "launch_ms": fc1_ms, "flops_per_launch": flops_fc1, "peak_source": pk["source"] + " bf16_tflops_sustained"},
            "allreduce_bytes_per_rank": M * N2 * 4, "gather_check": check,
            "gpu_launches": launches, "clocks": clocks.summary()}
    env.barrier()
    comm.close()
    del prog, x
    torch.cuda.empty_cache()
    return rec


# ---------------------------------------------------------------------------------------------------------------------
# ResNet-style conv stage

def run_resstage(env, args):
    """ResNet-style stage (BASELINE configs[4]): [256,56,56,64] bf16 NHWC -> 3 x (Conv3x3+BN+ReLU, Conv3x3+BN+Add+ReLU) ->
    MaxPool 2x2/2, every Conv-BN-[Add]-ReLU chain one tensor-core launch.  The batch is split evenly over the ranks
    (every op is per-image, no collective inside the stage); the pooled outputs are gathered on rank 0 by peer copies."""
    torch = env.torch
    import swcompiler_b200 as swc
    from swcompiler_b200.programs import ResStageProgram

    world, rank, device = env.world, env.rank, env.device
    N, HW, CH, BLOCKS = 256, 56, 64, 3
    n = N // world
    main_stream = torch.cuda.Stream(device)  # a stream of its own: the forward pass is captured into a CUDA graph
    torch.cuda.set_stream(main_stream)
    be = swc.Backend(env.local_rank, swc.TC_BF16, stream=main_stream)
    g = torch.Generator(device=device).manual_seed(1005)
    convs = [dict(w=torch.randn((CH, 3, 3, CH), generator=g, device=device) * (2.0 / (9 * CH)) ** 0.5,
                  b=torch.zeros(CH, device=device)) for _ in range(2 * BLOCKS)]
    bns = [dict(scale=torch.rand(CH, generator=g, device=device) + 0.5, bias=torch.randn(CH, generator=g, device=device) * 0.1,
                mean=torch.randn(CH, generator=g, device=device) * 0.1, var=torch.rand(CH, generator=g, device=device) + 0.5,
                eps=1e-5) for _ in range(2 * BLOCKS)]

    def images(r):
        gx = torch.Generator(device=device).manual_seed(1005 * 1000 + r)
        return torch.randn((n, HW, HW, CH), generator=gx, device=device).to(torch.bfloat16)

    x = images(rank)
    prog = ResStageProgram(be, convs, bns, max_batch=n, hw=HW, ch=CH)
    comm = gathered = None
    if world > 1:
        comm = env.comm(swc)
        if rank == 0:
            gathered = torch.empty((N, HW // 2, HW // 2, CH), dtype=torch.bfloat16, device=device)
        comm.gather_rows_setup(gathered, n * (HW // 2) * (HW // 2) * CH * 2, root=0)
    replay, pooled = prog.capture(x)

    # One step: the stage's seven launches as ONE graph launch (eager only for the per-launch event timing below: at
    # 2 GPUs and more a launch is 10-30 us long and seven calls through Python take longer than the kernels).
    def step(on_launch=None):
        if on_launch is None:
            replay()
            out = pooled
        else:
            out = prog.forward(x, on_launch=on_launch)
        if world > 1:
            ready = torch.cuda.Event()
            ready.record(main_stream)
            comm.be.torch_stream.wait_event(ready)
            comm.gather_rows(out)
            main_stream.wait_stream(comm.be.torch_stream)  # one pooled buffer: the next pass may overwrite it

    # the launches are short and are measured against the burst peak: start from a rested GPU, not from the clocks the
    # power-limited workloads before this one settled on, and give the clocks a few milliseconds of work to come up
    torch.cuda.synchronize()
    time.sleep(1.5)
    for _ in range(max(args.warmup, 10)):
        step()
    env.barrier()
    steps = max(args.steps, 20)  # a step is well under a millisecond
    nl = prog.launches_per_forward
    ev = [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(nl)] for _ in range(steps)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(env.local_rank) as clocks:
        env.barrier()
        e0.record()
        for s in range(steps):
            step()
        e1.record()
        env.barrier()
        # the same steps once more, launch by launch with an event on either side of each: the kernels' own durations.
        # A spinning kernel is queued ahead of every step so that the step's launches are all enqueued by the time
        # the first one starts; otherwise, with launches this short, an event pair would also span the host's time
        # between two calls.
        for s in range(steps):
            torch.cuda._sleep(2_000_000)
            step(on_launch=lambda i, when, s=s: ev[s][i][when].record())
    launches = steps * nl  # kernels inside the timed region: every replay launches the captured seven
    be.sync()
    per_launch = [sum(ev[s][i][0].elapsed_time(ev[s][i][1]) for s in range(steps)) / steps for i in range(nl)]
    convs_timed = per_launch if prog.fuse_pool else per_launch[:-1]  # the MaxPool rides in the last convolution's epilogue, or is the last launch
    conv_avg = sum(convs_timed) / len(convs_timed)
    ms, conv_avg = env.max_over_ranks([e0.elapsed_time(e1), conv_avg])

    # check on rank 0: the first image of every rank through a plain fp32 convolution chain (torch, as the checker),
    # activations rounded to bf16 where the program stores them, against the gathered pooled tensor
    check = None
    if world > 1:
        env.barrier()
    if rank == 0:
        import torch.nn.functional as F
        worst, scale = 0.0, 0.0
        bf = lambda t: t.to(torch.bfloat16).float()

        def conv_bn(h, i):
            w = bf(convs[i]["w"]).permute(0, 3, 1, 2)  # [oC,kh,kw,iC] -> [oC,iC,kh,kw]
            y = F.conv2d(h, w, convs[i]["b"], padding=1)
            b = bns[i]
            a = b["scale"] / torch.sqrt(b["var"] + b["eps"])
            return y * a.view(1, -1, 1, 1) + (b["bias"] - b["mean"] * a).view(1, -1, 1, 1)

        prev = torch.backends.cudnn.allow_tf32
        torch.backends.cudnn.allow_tf32 = False
        for r in range(world):
            h = images(r)[:1].float().permute(0, 3, 1, 2)
            for blk in range(BLOCKS):
                t = bf(torch.relu(conv_bn(h, 2 * blk)))
                h = bf(torch.relu(conv_bn(t, 2 * blk + 1) + h))
            ref = F.max_pool2d(h, 2).permute(0, 2, 3, 1)
            got = (gathered[r * n] if world > 1 else prog.pooled[0]).float()
            worst = max(worst, float((got - ref[0]).abs().max().item()))
            scale = max(scale, float(ref.abs().max().item()))
        torch.backends.cudnn.allow_tf32 = prev
        check = {"images": world, "max_abs": worst, "max_activation": scale, "ok": bool(worst <= 0.02 * scale),
                 "what": "pooled output of each rank's first image vs an fp32 convolution chain with the same rounding points"}
    flops = 2.0 * n * HW * HW * CH * 9 * CH
    pk = peaks()
    rec = None
    if rank == 0:
        step_ms = ms / steps
        achieved = flops / (conv_avg * 1e-3) / 1e12
        rec = {
            "metric": METRIC, "value": N / (step_ms * 1e-3), "unit": UNIT, "n_gpus": world, "steps": steps,
            "ms_per_step": step_ms, "scaling": "strong", "dtype": "bf16 (fp32 accumulate)", "data": "synthetic",
            "config": {"workload": "ResNet-style conv stage (BASELINE configs[4]): [256,56,56,64] bf16 NHWC, 3 residual blocks "
                                   "of two 3x3 64->64 convolutions with BN / skip / ReLU fused, then MaxPool 2x2/2 (in the last convolution's epilogue)",
                       "global_batch": N, "images_per_gpu": n, "parallelism": f"dp{world} (batch split; pooled outputs gathered on rank 0)",
                       "l2": "activations (103 MB per tensor at 256 images) larger than L2 at 1 and 2 GPUs; smaller beyond"},
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": pk["burst"], "unit": "TFLOP/s", "frac": achieved / pk["burst"],
                         "traffic": 2.5 * n * HW * HW * CH * 2,
                         "traffic_source": "operand bytes of one launch, mean of the six (input + output, and the skip tensor in every "
                                           "second one), not measured in this run; an ncu capture of the 256-image launch without a "
                                           "skip tensor read 103 MB and wrote 55 MB (the rest of the output was still in L2)",
                         "kernel": "conv_rows_kernel (3x3 64->64 + BN [+ skip] + ReLU, one launch; mean of the stage's six)",
                         "launch_ms": conv_avg, "flops_per_launch": flops,
                         "frac_of_sustained": achieved / pk["sustained"],
                         "peak_source": pk["source"] + " bf16_tflops (burst: the launches are short; frac_of_sustained is the "
                                        "same against bf16_tflops_sustained, the clocks these back-to-back steps run at)"},
            "per_launch_ms": per_launch, "gather_check": check, "gpu_launches": launches, "clocks": clocks.summary(),
            "timing": "value: graph replays (one CUDA-graph launch per step); per_launch_ms and the roofline: the same steps "
                      "issued call by call right after (behind a spinning kernel, so that they are queued before they run), one "
                      "CUDA event on either side of every launch"}
    env.barrier()
    if world > 1:
        comm.close()
    del prog, x, gathered, replay, pooled
    torch.cuda.set_stream(torch.cuda.default_stream(device))
    torch.cuda.empty_cache()
    return rec


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
    ap.add_argument("--workload", default="all", choices=["all", "widemlp", "widemlp_split", "fcpair", "resstage", "latency", "ops"],
                    help="all: the wide-MLP headline with every other workload appended under `workloads` / `ops`; "
                         "widemlp: the headline alone; the others: that workload's record alone")
    ap.add_argument("--chunks", type=int, default=4, help="fcpair: row chunks per forward (all-reduce overlap)")
    ap.add_argument("--fcpair-rows", type=int, default=8192, help="fcpair: rows of X")
    ap.add_argument("--comm-sms", type=int, default=16,
                    help="fcpair: SMs the GEMMs leave free for the all-reduce of the previous chunk to run beside them")
    args = ap.parse_args()
    BATCH = args.batch
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        return run_reference(args, rank, world)
    env = Env(rank, world, local_rank)
    w = args.workload

    def guarded(name, fn):
        """An appended workload must not take the headline down with it: a failure is reported in its place."""
        try:
            return fn()
        except Exception as e:  # noqa: BLE001
            return {"error": f"{name}: {type(e).__name__}: {e}"[:400]}

    rec = None
    if w in ("all", "widemlp"):
        rec = run_widemlp(env, args)
    elif w == "widemlp_split":
        rec = run_widemlp(env, args, split=True)
    elif w == "fcpair":
        rec = run_fcpair(env, args)
    elif w == "resstage":
        rec = run_resstage(env, args)
    elif w in ("latency", "ops"):
        if rank == 0:
            from swcompiler_b200 import opbench
            rec = {"latency": opbench.latency_rows()} if w == "latency" else {"ops": opbench.op_rows()}
    if w == "all":
        extra = {"resstage": guarded("resstage", lambda: run_resstage(env, args))}
        if world > 1:
            extra["fcpair"] = guarded("fcpair", lambda: run_fcpair(env, args))
        extra["widemlp_split"] = guarded("widemlp_split", lambda: _brief(run_widemlp(env, args, split=True)))
        ops = None
        if world == 1:
            from swcompiler_b200 import opbench
            extra["latency"] = guarded("latency", lambda: opbench.latency_rows())
            ops = guarded("ops", lambda: opbench.op_rows())
        if rank == 0:
            rec["workloads"] = extra
            if ops is not None:
                rec["ops"] = ops
    if rank == 0 and rec is not None:
        print(json.dumps(rec))
    env.close()


def _brief(rec):
    """The split-precision run of the wide MLP, reduced to what differs from the headline."""
    if rec is None:
        return None
    keep = ("value", "unit", "ms_per_step", "dtype", "roofline", "per_launch_ms", "gather_check", "gpu_launches")
    return {k: rec[k] for k in keep if k in rec}


if __name__ == "__main__":
    main()
