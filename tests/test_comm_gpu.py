"""GPU, 2 ranks (one process per GPU): the kernel library's NCCL entry points -- Scatter / Gather / Reduce /
Transform -- against the un-partitioned tensors, and the model-parallel FC pair on tensor cores against the
single-GPU result.  Skipped on a box with one GPU."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _setup(rank, world, comm_stream=False):
    import torch.distributed as dist

    import swcompiler_b200 as swc
    from swcompiler_b200 import parallel as par
    torch.cuda.set_device(rank)
    be = swc.Backend(rank, swc.TC_BF16)
    cbe = swc.Backend(rank, swc.TC_BF16, stream=torch.cuda.Stream()) if comm_stream else be

    def exchange(uid):
        box = [uid]
        dist.broadcast_object_list(box, src=0)
        return box[0]

    return be, par.NcclComm(cbe, rank, world, exchange), par


def _collectives(rank, world):
    be, comm, par = _setup(rank, world)
    dev = be.device
    g = torch.Generator(device=dev).manual_seed(1)
    full = torch.randn((4, 6, 8), generator=g, device=dev)
    for axis in (0, 1, 2, -1):
        local = comm.scatter(full if rank == 0 else None, full.shape, axis)
        be.sync()
        assert torch.equal(local, par.take_shard(full, axis, rank, world)), axis
        back = comm.gather(local, full.shape, axis)
        be.sync()
        assert rank != 0 or torch.equal(back, full), axis
    m = torch.arange(8 * 12, dtype=torch.float32, device=dev).reshape(8, 12)
    for pre in (0, 1, -1):
        for post in (0, 1, -1):
            out = comm.transform(par.take_shard(m, pre, rank, world), m.shape, pre, post)
            be.sync()
            assert torch.equal(out, par.take_shard(m, post, rank, world)), (pre, post)
    part, total = m * (rank + 1), m * sum(range(1, world + 1))
    for post in (0, 1, -1):
        out = comm.transform(part, m.shape, par.PARTIAL, post)
        be.sync()
        assert torch.equal(out, par.take_shard(total, post, rank, world)), post
    r = comm.reduce_sum(part)
    a = comm.allreduce_sum(part)
    ag = comm.allgather(par.take_shard(m, 0, rank, world))
    be.sync()
    assert (rank != 0 or torch.equal(r, total)) and torch.equal(a, total) and torch.equal(ag, m)
    # kernel-free Gather along axis 0 (peer copies into root's buffer)
    import torch.distributed as dist
    rows = torch.full((3, 5), float(rank + 1), device=dev)
    dst = torch.zeros((3 * world, 5), device=dev) if rank == 0 else None
    comm.gather_rows_setup(dst, rows.numel() * 4, root=0)
    for _ in range(2):
        comm.gather_rows(rows)
    be.sync()
    dist.barrier()
    if rank == 0:
        want = torch.cat([torch.full((3, 5), float(r + 1), device=dev) for r in range(world)])
        assert torch.equal(dst, want)
    dist.barrier()
    comm.gather_rows_release()
    # bf16 and int32 payloads
    b = torch.randn((16, 64), generator=g, device=dev).to(torch.bfloat16)
    lb = comm.scatter(b if rank == 0 else None, b.shape, 1, dtype=torch.bfloat16)
    be.sync()
    assert torch.equal(lb, par.take_shard(b, 1, rank, world))
    comm.close()


def _transform_nd(rank, world):
    """swcb200_transform on 4-D tensors: every split axis to every other, to and from replicated, from partial sums."""
    be, comm, par = _setup(rank, world)
    full = torch.arange(2 * 4 * 6 * 8, dtype=torch.float32, device=be.device).reshape(2, 4, 6, 8)
    for pre in (0, 1, 2, 3, -1):
        for post in (0, 1, 2, 3, -1):
            out = comm.transform(par.take_shard(full, pre, rank, world), full.shape, pre, post)
            be.sync()
            assert torch.equal(out, par.take_shard(full, post, rank, world)), (pre, post)
    part, total = full * (rank + 1), full * sum(range(1, world + 1))
    for post in (0, 2, 3, -1):
        out = comm.transform(part, full.shape, par.PARTIAL, post)
        be.sync()
        assert torch.equal(out, par.take_shard(total, post, rank, world)), post
    comm.close()


def _fc_pair(rank, world):
    """X[512,1024] -> FC 1024->2048 (column split) -> ReLU -> FC 2048->768 (row split) -> all-reduce."""
    import torch.distributed as dist

    import swcompiler_b200 as swc
    from swcompiler_b200.programs import FcPairProgram
    be, comm, par = _setup(rank, world, comm_stream=True)
    dev = be.device
    g = torch.Generator(device=dev).manual_seed(5)
    x = torch.randn((512, 1024), generator=g, device=dev).to(torch.bfloat16)
    w1 = (torch.randn((1024, 2048), generator=g, device=dev) / 32).to(torch.bfloat16).float()
    w2 = (torch.randn((2048, 768), generator=g, device=dev) / 45).to(torch.bfloat16).float()
    prog = FcPairProgram(be, comm, w1, w2, max_rows=512)
    torch.cuda.synchronize()
    y = prog.forward(x)
    torch.cuda.synchronize()
    y = y.clone()
    y2 = prog.forward(x, chunks=4)
    torch.cuda.synchronize()
    y2 = y2.clone()
    ref = torch.relu(x.float() @ w1).to(torch.bfloat16).float() @ w2
    assert (y - ref).abs().max().item() <= 2e-2
    assert (y2 - ref).abs().max().item() <= 2e-2
    y3 = prog.forward(x, chunks=4, comm_sms=16)      # the GEMMs leave 16 SMs to the all-reduce of the previous chunk
    torch.cuda.synchronize()
    assert torch.equal(y3, y2)
    # the join done by FC2's own epilogue over peer memory: this rank's row block, twice in a row
    prog.peer_setup()
    rows = 512 // world
    for _ in range(2):
        own = prog.forward_peer(x)
        torch.cuda.synchronize()
        dist.barrier()
        mine = y[rank * rows:(rank + 1) * rows]
        # the same p partial blocks added in rank order instead of NCCL's order: equal to rounding of an fp32 sum
        assert (own - mine).abs().max().item() <= 1e-5 * float(mine.abs().max().item()) + 1e-6
        assert (own - ref[rank * rows:(rank + 1) * rows]).abs().max().item() <= 2e-2
    comm.close()


def test_two_gpus_transform_of_4d_tensors():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    from test_parallel_cpu import run_ranks
    run_ranks(_transform_nd, 2)


@pytest.mark.parametrize("fn", [_collectives, _fc_pair])
def test_two_gpus(fn):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    from test_parallel_cpu import run_ranks
    run_ranks(fn, 2)
