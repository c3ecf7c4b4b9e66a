"""Partitioned graphs on the GPUs of one box: the reference's tiling labels and the Scatter / Gather /
Reduce / Transform nodes its parallel lowering inserts (src/parallel/ParallelPattern.h:35-172,
src/codegen/ParallelCodegen.cpp:457-896), one process per GPU.

Two interchangeable communicators with the same methods:

* ``TorchComm`` -- over ``torch.distributed`` (NCCL on GPUs, gloo on CPU for the host-logic tests);
* ``NcclComm``  -- over the C-ABI entry points of the kernel library (``swcb200_scatter`` ...), which is
  what a generated program links against.

Tiling convention: splitting a tensor of shape ``dims`` along ``axis`` over p ranks views it as ``outer``
rows of ``inner`` elements (outer = prod(dims[:axis]), inner = prod(dims[axis:])); rank r owns the block
[r*inner/p, (r+1)*inner/p) of every row and stores it packed.  axis -1 = replicated, -2 = partial sum.
"""
from __future__ import annotations

import ctypes as C
import math

import torch
import torch.distributed as dist

from . import _lib as L

REPLICATE, PARTIAL = -1, -2


def shard_dims(dims, axis: int, p: int):
    """Shape of one rank's packed shard."""
    dims = tuple(int(d) for d in dims)
    if axis < 0:
        return dims
    if dims[axis] % p:
        # the tiling pass only ever picks axes with dim % p == 0 (src/pass/ParallelLabelingPass.h:95-135)
        raise ValueError(f"dims[{axis}] = {dims[axis]} is not divisible by {p} ranks")
    return dims[:axis] + (dims[axis] // p,) + dims[axis + 1:]


def take_shard(full: torch.Tensor, axis: int, rank: int, p: int) -> torch.Tensor:
    """The packed shard of `full` that `rank` owns."""
    if axis < 0:
        return full
    n = full.shape[axis] // p
    return full.narrow(axis, rank * n, n).contiguous()


def strategy_fc_pair(p: int):
    """Strategy labels of the model-parallel FC -> ReLU -> FC chain, as the reference's tiling pass writes them
    (src/parallel/parallelGen.cpp:23-84; [inputs..., outputs...] axis per operand, the labels the sample program
    the fcpair_mp2 sample of gen_driver.cpp was lowered from): FC1 split by output columns, ReLU on the column shard,
    FC2 split by input rows with a partial-sum output that a Reduce node joins."""
    return {"fc1": (REPLICATE, 1, 1), "relu": (1, 1), "fc2": (1, 0, PARTIAL), "join": "reduce"}


class TorchComm:
    """Scatter / Gather / Reduce / Transform over torch.distributed."""

    def __init__(self, group=None):
        self.group = group
        self.rank = dist.get_rank(group)
        self.nranks = dist.get_world_size(group)

    def scatter(self, full, dims, axis, root=0, dtype=torch.float32, device=None):
        """Root holds `full` (others pass None); every rank returns its packed shard (axis -1: a copy)."""
        p, sd = self.nranks, shard_dims(dims, axis, self.nranks)
        device = device or (full.device if full is not None else torch.device("cpu"))
        out = torch.empty(sd, dtype=dtype, device=device)
        if axis < 0:
            if self.rank == root:
                out.copy_(full)
            dist.broadcast(out, src=root, group=self.group)
            return out
        ops = []
        if self.rank == root:
            for r in range(p):
                piece = take_shard(full, axis, r, p)
                if r == root:
                    out.copy_(piece)
                else:
                    ops.append(dist.P2POp(dist.isend, piece, r, self.group))
        else:
            ops.append(dist.P2POp(dist.irecv, out, root, self.group))
        if ops:
            for w in dist.batch_isend_irecv(ops):
                w.wait()
        return out

    def gather(self, local, dims, axis, root=0):
        """Inverse of scatter: root returns the full tensor, the others None."""
        p = self.nranks
        if axis < 0:
            return local if self.rank == root else None
        ops, pieces = [], None
        if self.rank == root:
            pieces = [torch.empty_like(local) for _ in range(p)]
            pieces[root] = local
            for r in range(p):
                if r != root:
                    ops.append(dist.P2POp(dist.irecv, pieces[r], r, self.group))
        else:
            ops.append(dist.P2POp(dist.isend, local.contiguous(), root, self.group))
        if ops:
            for w in dist.batch_isend_irecv(ops):
                w.wait()
        return torch.cat(pieces, dim=axis) if self.rank == root else None

    def reduce_sum(self, local, root=0):
        out = local.clone()
        dist.reduce(out, dst=root, op=dist.ReduceOp.SUM, group=self.group)
        return out if self.rank == root else None

    def allreduce_sum(self, local, out=None):
        if out is None:
            out = local.clone()
        elif out is not local:
            out.copy_(local)
        dist.all_reduce(out, op=dist.ReduceOp.SUM, group=self.group)
        return out

    def allgather(self, local):
        outs = [torch.empty_like(local) for _ in range(self.nranks)]
        dist.all_gather(outs, local.contiguous(), group=self.group)
        return torch.cat(outs, dim=0)

    def transform(self, local, dims, pre, post):
        """Re-tile a tensor of un-partitioned shape `dims` from tiling `pre` to tiling `post` (see module docstring);
        any number of dimensions."""
        p, r = self.nranks, self.rank
        if pre == post:
            return local
        if pre == REPLICATE:
            return take_shard(local, post, r, p)
        if pre == PARTIAL:
            full = self.allreduce_sum(local)
            return full if post == REPLICATE else take_shard(full, post, r, p)
        if post == REPLICATE:
            outs = [torch.empty_like(local) for _ in range(p)]
            dist.all_gather(outs, local.contiguous(), group=self.group)
            return torch.cat(outs, dim=pre)
        # split i -> split j: all-to-all of the sub-boxes (i in the sender's range, j in the receiver's)
        send = [take_shard(local, post, q, p) for q in range(p)]
        recv = [torch.empty_like(send[0]) for _ in range(p)]
        ops = []
        for q in range(p):
            if q == r:
                recv[q].copy_(send[q])
            else:
                ops.append(dist.P2POp(dist.isend, send[q], q, self.group))
                ops.append(dist.P2POp(dist.irecv, recv[q], q, self.group))
        if ops:
            for w in dist.batch_isend_irecv(ops):
                w.wait()
        return torch.cat(recv, dim=pre)


_DT = {torch.float32: L.F32, torch.bfloat16: L.BF16, torch.int32: L.I32}


class NcclComm:
    """The same operations through the kernel library's NCCL entry points, on the backend's stream.
    The 128-byte NCCL id is created on rank 0 and handed to the other ranks by `exchange`, a callable
    `bytes_or_None -> bytes` (for example a torch.distributed object broadcast, or a file)."""

    def __init__(self, backend, rank: int, nranks: int, exchange):
        self.be, self.rank, self.nranks = backend, rank, nranks
        lib = backend.lib
        nccl = _find_libnccl()
        if nccl:
            lib.swcb200_comm_load(C.c_char_p(nccl.encode()))
        uid = None
        if rank == 0:
            buf = C.create_string_buffer(128)
            rc = lib.swcb200_comm_unique_id(buf)
            if rc != L.OK:
                raise L.SwcError(rc, "comm_unique_id")
            uid = buf.raw
        uid = exchange(uid)
        backend._call("comm_init", C.c_char_p(uid), C.c_int(nranks), C.c_int(rank))

    def close(self):
        self.be._call("comm_destroy")

    def _dims(self, dims):
        return (C.c_size_t * len(dims))(*[int(d) for d in dims])

    def scatter(self, full, dims, axis, root=0, dtype=torch.float32, device=None):
        out = torch.empty(shard_dims(dims, axis, self.nranks), dtype=dtype, device=self.be.device)
        src = C.c_void_p(full.data_ptr()) if full is not None else C.c_void_p(0)
        self.be._call("scatter", src, C.c_void_p(out.data_ptr()), self._dims(dims), C.c_int(len(dims)), C.c_int(axis),
                      C.c_int(_DT[dtype]), C.c_int(root))
        return out

    def gather(self, local, dims, axis, root=0):
        out = torch.empty(tuple(dims), dtype=local.dtype, device=self.be.device) if self.rank == root else None
        dst = C.c_void_p(out.data_ptr()) if out is not None else C.c_void_p(0)
        self.be._call("gather", C.c_void_p(local.data_ptr()), dst, self._dims(dims), C.c_int(len(dims)), C.c_int(axis),
                      C.c_int(_DT[local.dtype]), C.c_int(root))
        return out

    def gather_rows_setup(self, dst_on_root, bytes_per_rank: int, root=0):
        """Collective.  Prepares the kernel-free Gather along axis 0: root passes its destination tensor (from
        the ordinary CUDA allocator), the others None."""
        dst = C.c_void_p(dst_on_root.data_ptr()) if dst_on_root is not None else C.c_void_p(0)
        self.be._call("gather_rows_setup", dst, C.c_size_t(bytes_per_rank), C.c_int(root))

    def gather_rows(self, local):
        """One copy-engine transfer of this rank's block into root's buffer, on the backend's stream.  Root may
        read the result after every rank has synchronised its stream and the ranks have met at a barrier."""
        self.be._call("gather_rows", C.c_void_p(local.data_ptr()))

    def peer_slots_setup(self, local_slots):
        """Collective.  `local_slots` [p, rows/p, cols] fp32 is this rank's slot array (slot r receives rank r's partial
        block); returns the ctypes table of every rank's array as this rank addresses it, for `Backend.fc_bf16_scatter_rows`."""
        table = (C.c_void_p * L.MAX_PEERS)()
        self.be._call("peer_slots_setup", C.c_void_p(local_slots.data_ptr()), table)
        return table

    def peer_slots_release(self):
        self.be._call("peer_slots_release")

    def gather_rows_release(self):
        self.be._call("gather_rows_release")

    def reduce_sum(self, local, root=0):
        out = torch.empty_like(local) if self.rank == root else None
        dst = C.c_void_p(out.data_ptr()) if out is not None else C.c_void_p(0)
        self.be._call("reduce_sum", C.c_void_p(local.data_ptr()), dst, C.c_size_t(local.numel()),
                      C.c_int(_DT[local.dtype]), C.c_int(root))
        return out

    def allreduce_sum(self, local, out=None):
        out = out if out is not None else torch.empty_like(local)
        self.be._call("allreduce_sum", C.c_void_p(local.data_ptr()), C.c_void_p(out.data_ptr()),
                      C.c_size_t(local.numel()), C.c_int(_DT[local.dtype]))
        return out

    def allgather(self, local):
        out = torch.empty((local.shape[0] * self.nranks,) + tuple(local.shape[1:]), dtype=local.dtype,
                          device=self.be.device)
        self.be._call("allgather", C.c_void_p(local.data_ptr()), C.c_void_p(out.data_ptr()),
                      C.c_size_t(local.numel()), C.c_int(_DT[local.dtype]))
        return out

    def transform(self, local, dims, pre, post):
        shape = tuple(dims) if post == REPLICATE else shard_dims(dims, post, self.nranks)
        out = torch.empty(shape, dtype=local.dtype, device=self.be.device)
        self.be._call("transform", C.c_void_p(local.data_ptr()), C.c_void_p(out.data_ptr()), self._dims(dims),
                      C.c_int(len(dims)), C.c_int(pre), C.c_int(post), C.c_int(_DT[local.dtype]))
        return out


def _find_libnccl():
    """The NCCL that ships with torch (so both use one copy), if it can be located."""
    import glob
    import os
    import sys
    for base in sys.path:
        hits = glob.glob(os.path.join(base, "nvidia", "nccl", "lib", "libnccl.so.2"))
        if hits:
            return hits[0]
    return None


def split_rows(total: int, p: int, rank: int):
    """Even batch split of the data-parallel strategy: (first row, row count) of `rank`."""
    if total % p:
        raise ValueError(f"{total} rows are not divisible by {p} ranks")
    n = total // p
    return rank * n, n


def allreduce_wire_bytes(count: int, elem: int, p: int) -> float:
    """Bytes each GPU sends in a ring all-reduce of `count` elements: 2 (p-1)/p * count * elem."""
    return 2.0 * (p - 1) / p * count * elem if p > 1 else 0.0


def comm_cost_bytes(dims, pre, post, p, elem=4):
    """Bytes that cross the network for one re-tiling, in the spirit of the reference's communication cost
    model (src/op/comSizeModel.cpp:16-79): none for -1 -> j, an all-to-all for i -> j, a reduce for -2."""
    n = math.prod(dims) * elem
    if pre == post or pre == REPLICATE:
        return 0.0
    if pre == PARTIAL:
        return allreduce_wire_bytes(math.prod(dims), elem, p) * p
    if post == REPLICATE:
        return n * (p - 1)
    return n * (p - 1) / p
