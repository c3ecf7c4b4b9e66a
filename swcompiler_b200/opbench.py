"""Per-kernel roofline measurements on one GPU:  python -m swcompiler_b200.opbench [--only NAME] [--iters N]

Times every kernel of the table at the sizes the benchmark configurations give it (config 5 stage
[256,56,56,64], config 3 activations [65536,4096] and logits [65536,1000]), with CUDA events on the
launching stream after warm-up, inputs larger than L2, and prints one JSON line per kernel:
achieved GB/s (algorithmic bytes / time) or TFLOP/s, and the fraction of the measured peak.
"""
from __future__ import annotations

import argparse
import json
import os

import torch

import swcompiler_b200 as swc

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _peaks():
    try:
        p = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        return float(p["hbm_gbs"]), float(p["bf16_tflops"]), "measured"
    except Exception:
        return 6650.0, 1590.0, "fallback"


def _time(fn, iters, rest=0.0):
    """`rest` seconds of idle time first: a tensor-bound kernel is to be measured as a burst, on its own, not at the
    clocks the power limit has settled on after the kernels measured before it."""
    if rest:
        import time
        torch.cuda.synchronize()
        time.sleep(rest)
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    if rest:
        # after a rest the clocks take a few milliseconds of work to come back up: short kernels get more warm-up
        # launches (about 3 ms worth, 20 at most), long ones none beyond the three above
        import time
        t0 = time.perf_counter()
        fn()
        torch.cuda.synchronize()
        dt = max(time.perf_counter() - t0, 1e-6)
        for _ in range(min(20, int(3e-3 / dt))):
            fn()
        torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters * 1e-3


def latency_rows(iters=50):
    """The two configurations that are bound by launch latency, not by any roofline (52 and 182 MFLOP per forward):
    X[64,784] -> FC 784->512 -> Tanh -> FC 512->10 -> Softmax, and [32,28,28,1] -> Conv5x5 1->16 -> ReLU -> MaxPool ->
    Conv5x5 16->32 -> ReLU -> MaxPool -> FC 1568->10 -> Softmax.  One table call per op node, strict fp32 kernels and
    the tensor-core mode of the same entry points; microseconds per forward pass and samples per second, launched call
    by call and replayed as a CUDA graph (the form the generator prints with graph_replays)."""
    import time
    torch.cuda.synchronize()
    time.sleep(2.0)   # not at the clocks a power-limited workload measured just before has left behind
    dev = torch.device("cuda", torch.cuda.current_device())
    g = torch.Generator(device=dev).manual_seed(1001)
    rn = lambda *shape, s=1.0: torch.randn(shape, generator=g, device=dev) * s
    x1, w0, b0, w1, b1 = torch.rand((64, 784), generator=g, device=dev), rn(784, 512, s=0.05), torch.zeros(512, device=dev), \
        rn(512, 10, s=0.05), torch.zeros(10, device=dev)
    x2 = torch.rand((32, 28, 28, 1), generator=g, device=dev)
    cw0, cb0 = rn(16, 5, 5, 1, s=(2 / 25) ** 0.5), torch.zeros(16, device=dev)
    cw1, cb1 = rn(32, 5, 5, 16, s=(2 / 400) ** 0.5), torch.zeros(32, device=dev)
    fw, fb = rn(1568, 10, s=0.02), torch.zeros(10, device=dev)
    k5, s1, p2, k2, s2, p0 = (5, 5), (1, 1), (2, 2, 2, 2), (2, 2), (2, 2), (0, 0, 0, 0)
    rows = []
    stream = torch.cuda.Stream(dev)
    for mode, name in ((swc.STRICT_F32, "strict fp32"), (swc.TC_BF16, "tensor-core mode")):
        with torch.cuda.stream(stream):
            be = swc.Backend(dev.index, mode, stream=stream)

            def mlp():
                return be.mlp_forward(x1, w0, b0, w1, b1)

            def lenet():
                h = be.maxpool_f(be.relu_f(be.conv2d_f(x2, cw0, cb0, k5, s1, p2)), k2, s2, p0)
                h = be.maxpool_f(be.relu_f(be.conv2d_f(h, cw1, cb1, k5, s1, p2)), k2, s2, p0)
                return be.matrixSoftmax_f(be.fc(h, fw, fb))

            for label, fn, batch in (("MLP 784-512-10, batch 64", mlp, 64), ("LeNet-style conv net, batch 32", lenet, 32)):
                n0 = be.launches
                fn()
                per_forward = be.launches - n0
                t = _time(fn, iters, rest=0.3)
                # the same calls captured once and replayed: what remains is the kernels' own time
                stream.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=stream):
                    fn()
                tg = _time(graph.replay, iters, rest=0.3)
                rows.append({"config": label, "mode": name, "us_per_forward": t * 1e6, "samples_per_s": batch / t,
                             "graph_us_per_forward": tg * 1e6, "graph_samples_per_s": batch / tg,
                             "launches_per_forward": per_forward})
            if mode == swc.TC_BF16:
                # the program the fusion planner prints for the MLP: weights packed once at load, one launch per FC layer
                # (matmul + bias + tanh), bf16 between them
                wp0, wp1 = be.pack_weight_bf16(w0), be.pack_weight_bf16(w1)

                def mlp_fused():
                    h = be.fc_bf16(be.cast_f32_to_bf16(x1), wp0, b0, swc.ACT_TANH)
                    return be.matrixSoftmax_f(be.fc_bf16(h, wp1, b1, swc.ACT_NONE, torch.float32))

                n0 = be.launches
                mlp_fused()
                per_forward = be.launches - n0
                t = _time(mlp_fused, iters)
                stream.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=stream):
                    mlp_fused()
                tg = _time(graph.replay, iters)
                rows.append({"config": "MLP 784-512-10, batch 64", "mode": "fused bf16 program (packed weights, one launch per FC layer)",
                             "us_per_forward": t * 1e6, "samples_per_s": 64 / t, "graph_us_per_forward": tg * 1e6,
                             "graph_samples_per_s": 64 / tg, "launches_per_forward": per_forward})
            be.sync()
    return rows


def latency(iters):
    for r in latency_rows(iters):
        print(json.dumps(r))


def op_rows(iters=20, only=None):
    """One row per kernel at the benchmark configurations' sizes: achieved GB/s or TFLOP/s and the fraction of the
    measured peak (see the module docstring)."""
    rows = []
    hbm, tflops, src = _peaks()
    be = swc.Backend(torch.cuda.current_device(), swc.STRICT_F32)
    dev = be.device
    g = torch.Generator(device=dev).manual_seed(0)
    stage = (256, 56, 56, 64)
    x = torch.randn(stage, generator=g, device=dev)
    y = torch.randn(stage, generator=g, device=dev)
    out = torch.empty_like(x)
    E = x.numel()
    C = stage[3]
    vec = [torch.rand(C, generator=g, device=dev) + 0.5 for _ in range(4)]
    pooled = torch.empty((256, 28, 28, 64), device=dev)
    logits = torch.randn((65536, 1000), generator=g, device=dev)
    probs = torch.empty_like(logits)
    act = torch.randn((32768, 4096), generator=g, device=dev)  # 512 MiB fp32
    act_out = torch.empty_like(act)
    bias = torch.randn(4096, generator=g, device=dev)
    xb = x.to(torch.bfloat16)
    pooled_b = torch.empty((256, 28, 28, 64), device=dev, dtype=torch.bfloat16)

    mem_ops = [
        ("relu_f", 8 * E, lambda: be.relu_f(x, out=out)),
        ("vecAdd_f", 12 * E, lambda: be.vecAdd_f(x, y, out=out)),
        ("batchnormalization_f", 8 * E + 16 * C, lambda: be.batchnormalization_f(x, vec[0], vec[1], vec[2], vec[3], 1e-5, out=out)),
        ("maxpool_f 2x2/2", 5 * E, lambda: be.maxpool_f(x, (2, 2), (2, 2), (0, 0, 0, 0), out=pooled)),
        ("maxpool_bf16 2x2/2", 2.5 * E, lambda: be.maxpool_bf16(xb, (2, 2), (2, 2), (0, 0, 0, 0), out=pooled_b)),
        ("batchedadd_f [32768,4096]", 8 * act.numel() + 4 * 4096, lambda: be.batchedadd_f(act, bias, out=act_out)),
        ("matrixTanh_f strict [32768,4096]", 8 * act.numel(), lambda: be.matrixTanh_f(act, out=act_out)),
        ("matrixSoftmax_f strict [65536,1000]", 8 * logits.numel(), lambda: be.matrixSoftmax_f(logits, out=probs)),
        ("argMax_i top1 [65536,1000]", 4 * logits.numel(), lambda: be.argMax_i(logits, 1)),
        ("cast_f32_to_bf16", 6 * E, lambda: be.cast_f32_to_bf16(x, out=xb)),
    ]
    for name, nbytes, fn in mem_ops:
        if only and only not in name:
            continue
        t = _time(fn, iters)
        rows.append(({"kernel": name, "bound": "hbm", "us": t * 1e6, "achieved": nbytes / t / 1e9, "unit": "GB/s",
                          "peak": hbm, "frac": nbytes / t / 1e9 / hbm, "peak_source": src, "bytes": nbytes}))
    be.set_precision(swc.TC_BF16)
    for name, nbytes, fn in [
        ("matrixTanh_f fast [32768,4096]", 8 * act.numel(), lambda: be.matrixTanh_f(act, out=act_out)),
        ("matrixSoftmax_f fast [65536,1000]", 8 * logits.numel(), lambda: be.matrixSoftmax_f(logits, out=probs)),
    ]:
        if only and only not in name:
            continue
        t = _time(fn, iters)
        rows.append(({"kernel": name, "bound": "hbm", "us": t * 1e6, "achieved": nbytes / t / 1e9, "unit": "GB/s",
                          "peak": hbm, "frac": nbytes / t / 1e9 / hbm, "peak_source": src, "bytes": nbytes}))
    del act, act_out, logits, probs

    # tensor-core FC shapes (bf16, fp32 accumulate): config 3 hidden layer and last layer, config 4 per-GPU shards at p = 8
    for (m, n, k) in [(65536, 4096, 4096), (65536, 1000, 4096), (8192, 4096, 8192), (8192, 8192, 4096)]:
        name = f"fc_bf16 {m}x{n}x{k}"
        if only and only not in name:
            continue
        a = torch.randn((m, k), generator=g, device=dev).to(torch.bfloat16)
        wp = (torch.randn((n, k), generator=g, device=dev) / k ** 0.5).to(torch.bfloat16)
        b = torch.randn(n, generator=g, device=dev)
        o = torch.empty((m, n), device=dev, dtype=torch.bfloat16)
        t = _time(lambda: be.fc_bf16(a, wp, b, swc.ACT_RELU, out=o), iters, rest=1.0)
        fl = 2.0 * m * n * k
        rows.append(({"kernel": name, "bound": "tensor", "us": t * 1e6, "achieved": fl / t / 1e12, "unit": "TFLOP/s",
                          "peak": tflops, "frac": fl / t / 1e12 / tflops, "peak_source": src + " (burst)", "flops": fl}))
        del a, wp, o
    # config 5: 3x3 64->64 convolution on [256,56,56,64] with the fused epilogue, and the whole stage
    if not only or "conv" in only or "stage" in only:
        from .programs import ResStageProgram
        n, hw, ch = 256, 56, 64
        xin = torch.randn((n, hw, hw, ch), generator=g, device=dev).to(torch.bfloat16)
        convs = [dict(w=torch.randn((ch, 3, 3, ch), generator=g, device=dev) * (2.0 / (9 * ch)) ** 0.5,
                      b=torch.zeros(ch, device=dev)) for _ in range(6)]
        bns = [dict(scale=torch.rand(ch, generator=g, device=dev) + 0.5, bias=torch.randn(ch, generator=g, device=dev) * 0.1,
                    mean=torch.randn(ch, generator=g, device=dev) * 0.1, var=torch.rand(ch, generator=g, device=dev) + 0.5,
                    eps=1e-5) for _ in range(6)]
        prog = ResStageProgram(be, convs, bns, max_batch=n, hw=hw, ch=ch)
        o = torch.empty_like(xin)
        fl = 2.0 * n * hw * hw * ch * 9 * ch
        for name, fn in [
            ("conv2d_bf16 3x3 64->64 [256,56,56,64] +BN+ReLU",
             lambda: be.conv2d_bf16(xin, prog.fp[0], prog.cb[0], (3, 3), (1, 1), (1, 1, 1, 1), bn=prog.bn[0], relu=True, out=o)),
            ("conv2d_bf16 3x3 64->64 [256,56,56,64] +BN+Add+ReLU",
             lambda: be.conv2d_bf16(xin, prog.fp[1], prog.cb[1], (3, 3), (1, 1), (1, 1, 1, 1), bn=prog.bn[1], residual=xin,
                                    relu=True, out=o)),
        ]:
            t = _time(fn, iters, rest=1.5)
            rows.append(({"kernel": name, "bound": "tensor", "us": t * 1e6, "achieved": fl / t / 1e12, "unit": "TFLOP/s",
                              "peak": tflops, "frac": fl / t / 1e12 / tflops, "peak_source": src + " (burst)", "flops": fl,
                              "hbm_GBps": (2 * xin.numel() * 2) / t / 1e9}))
        t = _time(lambda: prog.forward(xin), iters, rest=1.5)
        rows.append(({"kernel": "res stage forward (config 5): 6 fused convs + maxpool, batch 256", "bound": "tensor",
                          "us": t * 1e6, "achieved": prog.flops(n) / t / 1e12, "unit": "TFLOP/s", "peak": tflops,
                          "frac": prog.flops(n) / t / 1e12 / tflops, "peak_source": src + " (burst)",
                          "samples_per_s": n / t, "launches": prog.launches_per_forward}))
    be.sync()
    return rows


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default=None)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--latency", action="store_true",
                    help="the two small configurations (MLP batch 64, LeNet-style net batch 32): microseconds per forward")
    args = ap.parse_args()
    if args.latency:
        return latency(args.iters)
    for r in op_rows(args.iters, args.only):
        print(json.dumps(r))


if __name__ == "__main__":
    main()
