"""CPU, world_size 2 over gloo: the host-side tiling logic of partitioned graphs (Scatter / Gather / Reduce /
Transform semantics, batch split, the model-parallel FC pair) against the un-partitioned computation."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from swcompiler_b200 import parallel as par


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, fn, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        fn(rank, world)
        ret[rank] = "ok"
    except Exception as e:  # surfaced to the parent
        import traceback
        ret[rank] = traceback.format_exc()
    finally:
        dist.destroy_process_group()


def run_ranks(fn, world=2):
    mgr = mp.get_context("spawn").Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), fn, ret), nprocs=world, join=True)
    assert all(ret.get(r) == "ok" for r in range(world)), dict(ret)


def _scatter_gather(rank, world):
    comm = par.TorchComm()
    g = torch.Generator().manual_seed(1)
    full = torch.randn((4, 6, 8), generator=g)
    for axis in (0, 1, 2, -1):
        local = comm.scatter(full if rank == 0 else None, full.shape, axis)
        assert torch.equal(local, par.take_shard(full, axis, rank, world))
        back = comm.gather(local, full.shape, axis)
        if rank == 0:
            assert torch.equal(back, full)
        else:
            assert back is None


def _transform(rank, world):
    comm = par.TorchComm()
    full = torch.arange(8 * 12, dtype=torch.float32).reshape(8, 12)
    for pre in (0, 1, -1):
        for post in (0, 1, -1):
            local = par.take_shard(full, pre, rank, world)
            out = comm.transform(local, full.shape, pre, post)
            assert torch.equal(out, par.take_shard(full, post, rank, world)), (pre, post)
    # partial sums: every rank holds a full-size addend
    part = full * (rank + 1)
    total = full * sum(range(1, world + 1))
    for post in (0, 1, -1):
        assert torch.equal(comm.transform(part, full.shape, par.PARTIAL, post), par.take_shard(total, post, rank, world))
    r = comm.reduce_sum(part)
    assert (rank != 0 and r is None) or torch.equal(r, total)
    assert torch.equal(comm.allgather(par.take_shard(full, 0, rank, world)), full)


def _transform_nd(rank, world):
    """Tensors with four dimensions (NHWC activations): every split axis to every other, to replicated, and from
    replicated or partial sums."""
    comm = par.TorchComm()
    full = torch.arange(2 * 4 * 6 * 8, dtype=torch.float32).reshape(2, 4, 6, 8)
    for pre in (0, 1, 2, 3, -1):
        for post in (0, 1, 2, 3, -1):
            out = comm.transform(par.take_shard(full, pre, rank, world), full.shape, pre, post)
            assert torch.equal(out, par.take_shard(full, post, rank, world)), (pre, post)
    part = full * (rank + 1)
    total = full * sum(range(1, world + 1))
    for post in (0, 2, 3, -1):
        assert torch.equal(comm.transform(part, full.shape, par.PARTIAL, post), par.take_shard(total, post, rank, world))


def _fc_pair(rank, world):
    """FC1 by output columns -> ReLU -> FC2 by input rows -> Reduce equals the un-partitioned chain (up to the
    order of the final sum)."""
    comm = par.TorchComm()
    g = torch.Generator().manual_seed(2)
    x = torch.randn((16, 32), generator=g, dtype=torch.float64)
    w1 = torch.randn((32, 48), generator=g, dtype=torch.float64)
    w2 = torch.randn((48, 24), generator=g, dtype=torch.float64)
    st = par.strategy_fc_pair(world)
    assert st["fc1"] == (-1, 1, 1) and st["fc2"] == (1, 0, -2)
    xs = comm.scatter(x if rank == 0 else None, x.shape, st["fc1"][0], dtype=torch.float64)
    w1s = comm.scatter(w1 if rank == 0 else None, w1.shape, st["fc1"][1], dtype=torch.float64)
    w2s = comm.scatter(w2 if rank == 0 else None, w2.shape, st["fc2"][1], dtype=torch.float64)
    h = torch.relu(xs @ w1s)                      # column shard [16, 48/p]
    y_part = h @ w2s                               # full-size partial sum
    y = comm.allreduce_sum(y_part)
    assert torch.allclose(y, torch.relu(x @ w1) @ w2, rtol=1e-12, atol=1e-12)


def _batch_split(rank, world):
    """Data-parallel: each rank runs the whole chain on its rows; gathering axis 0 gives the full result."""
    comm = par.TorchComm()
    g = torch.Generator().manual_seed(3)
    x = torch.randn((8, 5), generator=g)
    w = torch.randn((5, 7), generator=g)
    r0, n = par.split_rows(x.shape[0], world, rank)
    xs = comm.scatter(x if rank == 0 else None, x.shape, 0)
    assert torch.equal(xs, x[r0:r0 + n])
    ws = comm.scatter(w if rank == 0 else None, w.shape, -1)
    y = comm.gather(torch.softmax(xs @ ws, dim=1), (8, 7), 0)
    if rank == 0:
        assert torch.equal(y, torch.softmax(x @ w, dim=1))


def _emitted_programs(rank, world):
    """The partitioned programs B200Codegen emitted, call by call (tests/emitted_interp.py): compute by the CPU oracle,
    Scatter / Gather / Reduce / Transform by TorchComm over gloo, one interpreter per rank.  Checks the generator's
    reading of the reference's tiling labels -- axes, tile shapes, master-only guards, load-time scatters."""
    import sys
    here = os.path.dirname(os.path.abspath(__file__))
    sys.path[:0] = [os.path.dirname(here), here]
    import tempfile

    from codegen_util import EMITTED
    from emitted_interp import Interp
    from oracle import oracle as orc
    o = orc.Oracle()
    o.set_threads(1)
    golden = np.load(os.path.join(here, "golden", "ref_outputs.npz"))
    mnist = os.path.join(here, "golden", "mnist8")
    comm = par.TorchComm()
    for which, tol in (("mlp8_dp2", 0.0), ("mlp8_mp2", 1e-6), ("mlp8_dp2_fused", 2e-2)):
        out = Interp(o, mnist, rank, world, comm).run(os.path.join(EMITTED, which + "_Graph.cpp"))
        if rank == 0:
            assert out["top3"][:, 0].tolist() == [5, 0, 4, 1, 9, 2, 1, 3], which
            assert np.abs(out["data4"] - golden["mnist8__probs"]).max() <= tol, which
        else:
            assert out == {}, which   # only the master prints
    r = np.random.default_rng(404)
    x = r.standard_normal((64, 256)).astype(np.float32)
    w1 = (r.standard_normal((256, 512)) / 16).astype(np.float32)
    w2 = (r.standard_normal((512, 128)) / 22.6).astype(np.float32)
    with tempfile.TemporaryDirectory() as d:
        for name, arr in (("fp_x.bin", x), ("fp_w1.bin", w1), ("fp_w2.bin", w2)):
            arr.tofile(os.path.join(d, name))
        out = Interp(o, d, rank, world, comm).run(os.path.join(EMITTED, "fcpair_mp2_Graph.cpp"))
        fused = Interp(o, d, rank, world, comm)
        out_fused = fused.run(os.path.join(EMITTED, "fcpair_mp2_fused_Graph.cpp"))
    # with the planner the Reduce is printed as the join over peer memory: the GEMM stores row blocks into their owners'
    # slots, the ranks meet, each owner adds its slots in rank order and the master gathers the blocks
    assert fused.calls.count("fc_bf16_scatter_rows") == 1 and "reduce_sum" not in fused.calls
    i = fused.calls.index("fc_bf16_scatter_rows")
    assert fused.calls[i:i + 4] == ["fc_bf16_scatter_rows", "allreduce_sum", "sum_slots", "gather"]
    if rank == 0:
        want = o.matrixMatrixMul_f(o.relu_f(o.matrixMatrixMul_f(x, w1)), w2)
        assert np.allclose(out["y"], want, rtol=1e-5, atol=1e-5)
        import cases
        rb = cases.bf16_round
        part = [o.matrixMatrixMul_f(rb(o.relu_f(o.matrixMatrixMul_f(rb(x), rb(w1[:, c * 256:(c + 1) * 256])))),
                                    rb(w2[c * 256:(c + 1) * 256])) for c in range(2)]
        assert np.array_equal(out_fused["y"], part[0] + part[1])      # same rounding points, same order of the two terms
        assert np.abs(out_fused["y"] - want).max() <= 2e-2
    else:
        assert out_fused == {}
    # batch-split residual block: BatchNormalization and ElementAdd carry no tiling descriptor in the reference, so its
    # passes gather their inputs to the master, run them there (printed inside `if (rank == 0)`) and scatter again
    from codegen_util import resblock_inputs, resblock_oracle
    t = resblock_inputs()
    with tempfile.TemporaryDirectory() as d:
        for name, arr in t.items():
            arr.tofile(os.path.join(d, name))
        out = Interp(o, d, rank, world, comm).run(os.path.join(EMITTED, "resblock_dp2_Graph.cpp"))
    if rank == 0:
        assert np.array_equal(out["probs"], resblock_oracle(o, t))      # every op is per-sample: bit for bit


@pytest.mark.parametrize("fn", [_scatter_gather, _transform, _transform_nd, _fc_pair, _batch_split, _emitted_programs])
def test_two_ranks_gloo(fn):
    run_ranks(fn, 2)


def _fuzz_program(rank, world):
    import sys
    here = os.path.dirname(os.path.abspath(__file__))
    sys.path[:0] = [os.path.dirname(here), here]
    from codegen_util import resblock_inputs, resblock_oracle
    from emitted_interp import Interp
    from oracle import oracle as orc
    o = orc.Oracle()
    o.set_threads(1)
    prog = os.environ["SWC_FUZZ_PROGRAM"]
    mlp = "mlp8" in os.path.basename(prog)
    files = os.path.join(here, "golden", "mnist8") if mlp else os.path.dirname(prog)
    out = Interp(o, files, rank, world, par.TorchComm()).run(prog)
    if rank != 0:
        return
    if mlp:
        assert out["top3"][:, 0].tolist() == [5, 0, 4, 1, 9, 2, 1, 3]
    else:
        want = resblock_oracle(o, resblock_inputs())
        assert np.allclose(out["probs"], want, rtol=1e-4, atol=1e-5), np.abs(out["probs"] - want).max()


@pytest.mark.skipif(not os.path.exists(os.path.join(__import__("codegen_util").reference_root(), "include", "SWC.h")),
                    reason="no reference checkout")
@pytest.mark.parametrize("which", ["mlp8_rp2", "mlp8_rp2_fused", "resblock_rp2"])
def test_whatever_partitioning_the_reference_draws(which, tmp_path):
    """The reference's ParallelLabelingPass picks each op's strategy from std::random_device: every run of the generator
    gives another mix of batch, column, row and spatial splits with their Scatter / Gather / Reduce / Transform nodes
    (4-D re-tilings included).  Two draws are emitted here and interpreted on two gloo ranks; whatever was drawn, the
    un-partitioned result must come out.  One family of draws is left out: a convolution split by INPUT channels adds
    its bias on every rank before the Reduce in the reference's scheme, so the bias is counted once per rank."""
    import re
    import subprocess

    from codegen_util import resblock_inputs
    from swcompiler_b200.codegen import build_codegen as bc
    exe = bc.build(__import__("codegen_util").reference_root())
    done = 0
    for draw in range(12):
        d = tmp_path / str(draw)
        d.mkdir()
        if which.startswith("resblock"):
            for name, arr in resblock_inputs().items():
                arr.tofile(str(d / name))
        r = subprocess.run([exe, which, str(d), "x"], cwd=os.path.dirname(exe), capture_output=True, text=True)
        assert r.returncode == 0, r.stderr[-2000:]
        prog = str(d / (which + "_Graph.cpp"))
        if re.search(r"swcb200_scatter\(ctx, conv\d_w, \w+, \w+, 4, 3,", open(prog).read()):
            continue
        os.environ["SWC_FUZZ_PROGRAM"] = prog
        run_ranks(_fuzz_program, 2)
        done += 1
        if done == 2:
            break
    assert done >= 1


def test_shapes_and_costs():
    assert par.shard_dims((8, 12), 1, 4) == (8, 3) and par.shard_dims((8, 12), -1, 4) == (8, 12)
    with pytest.raises(ValueError):
        par.shard_dims((8, 10), 1, 4)
    assert par.split_rows(65536, 8, 3) == (3 * 8192, 8192)
    assert par.allreduce_wire_bytes(1 << 20, 4, 8) == 2 * 7 / 8 * 4 * (1 << 20)
    assert par.comm_cost_bytes((8, 8), -1, 0, 2) == 0 and par.comm_cost_bytes((8, 8), 0, 1, 2) == 128
