"""Forward programs: the sequence of kernel-table calls the code generator would emit for a graph,
with the tensors of its arena held resident in HBM.

The reference's generator writes a C++ main() that allocates one arena, loads weights, and calls one
kernel per op node in topological order (src/codegen/Codegen.cpp:288-356, :1035-1077).  These
classes are that emitted program for the benchmark graphs, issued through the C-ABI library: weights
are packed once at construction (load time), activations live in pre-allocated buffers, and
`forward` only launches kernels.
"""
from __future__ import annotations

import torch

from . import _lib as L
from .kernels import Backend


class WideMlpProgram:
    """x[B,width] bf16 -> `layers` x (FC width->width, +bias, ReLU) -> FC width->classes, +bias -> Softmax.

    Tensor-core path with bf16 storage: each hidden layer is ONE launch (matmul + bias + ReLU + bf16 store),
    the last FC writes fp32 logits, softmax is a separate bandwidth-bound launch.  A batch larger than
    `chunk_rows` is processed chunk by chunk through the same two activation buffers.

    `split`: hidden activations are kept as two bf16 terms (value and rounding remainder) and every layer behind
    the first multiplies both by its weights (`Backend.fc_bf16(a_lo=, out_lo=)`): the precision of the stored
    activations goes from 8 to 16 bits of mantissa at about 1.75 times the tensor-core time of the pass.
    """

    def __init__(self, be: Backend, weights, biases, max_rows: int, split: bool = False):
        self.be = be
        self.split = split
        self.wp = [be.pack_weight_bf16(w) if w.dtype == torch.float32 else w for w in weights]  # [n, k] bf16
        self.bias = [b.contiguous() for b in biases]
        self.width = self.wp[0].shape[1]
        self.classes = self.wp[-1].shape[0]
        self.max_rows = max_rows
        self.h = [torch.empty((max_rows, self.width), dtype=torch.bfloat16, device=be.device) for _ in range(2)]
        self.h_lo = [torch.empty_like(t) for t in self.h] if split else None
        self.logits = torch.empty((max_rows, self.classes), dtype=torch.float32, device=be.device)
        self.launches_per_forward = len(self.wp) + 1
        be.sync()

    def flops(self, rows: int) -> float:
        return float(sum(2.0 * rows * w.shape[0] * w.shape[1] for w in self.wp))

    def forward(self, x_bf16: torch.Tensor, probs_out: torch.Tensor, on_launch=None) -> torch.Tensor:
        """x_bf16 [rows, width] on device -> probs_out [rows, classes] fp32 on device.  `on_launch(i, when)` is
        called before (when=0) and after (when=1) the i-th launch, for per-kernel event timing."""
        rows = x_bf16.shape[0]
        if rows > self.max_rows:
            raise ValueError("batch exceeds the activation buffers")
        be, h, h_lo = self.be, x_bf16, None   # the input is bf16 to begin with: one term
        last = len(self.wp) - 1
        for i, (wp, b) in enumerate(zip(self.wp, self.bias)):
            if on_launch:
                on_launch(i, 0)
            if i < last:
                out = self.h[i & 1][:rows]
                out_lo = self.h_lo[i & 1][:rows] if self.split else None
                be.fc_bf16(h, wp, b, L.ACT_RELU, out=out, a_lo=h_lo, out_lo=out_lo)
                h, h_lo = out, out_lo
            else:
                logits = self.logits[:rows]
                be.fc_bf16(h, wp, b, L.ACT_NONE, out=logits, a_lo=h_lo)
            if on_launch:
                on_launch(i, 1)
        if on_launch:
            on_launch(last + 1, 0)
        be.matrixSoftmax_f(logits, out=probs_out)
        if on_launch:
            on_launch(last + 1, 1)
        return probs_out

    def forward_host(self, x_host: torch.Tensor, probs_host: torch.Tensor, x_dev: torch.Tensor,
                     probs_dev: torch.Tensor, chunk_rows: int = 8192) -> torch.Tensor:
        """End to end with pinned HOST buffers.  The batch is cut into row chunks and three streams work as a
        pipeline: chunk i+1 is copied in and chunk i-1 is copied out (both on copy engines) while the tensor
        cores work on chunk i.  Every op is per-sample, so chunking the rows changes no result.  On return the
        backend's stream has been made to wait for the last device->host copy.  With `probs_host` None the
        probabilities stay on the device (a Gather follows)."""
        rows = x_host.shape[0]
        main = self.be.torch_stream or torch.cuda.current_stream(self.be.device)
        if not hasattr(self, "_io_streams"):
            self._io_streams = (torch.cuda.Stream(self.be.device), torch.cuda.Stream(self.be.device))
        s_in, s_out = self._io_streams
        start = torch.cuda.Event()
        start.record(main)
        s_in.wait_event(start)   # buffers of an earlier call are free once the main stream got here
        s_out.wait_event(start)
        for r0 in range(0, rows, chunk_rows):
            r1 = min(rows, r0 + chunk_rows)
            with torch.cuda.stream(s_in):
                x_dev[r0:r1].copy_(x_host[r0:r1], non_blocking=True)
                arrived = torch.cuda.Event()
                arrived.record(s_in)
            main.wait_event(arrived)
            self.forward(x_dev[r0:r1], probs_dev[r0:r1])
            if probs_host is not None:
                done = torch.cuda.Event()
                done.record(main)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(done)
                    probs_host[r0:r1].copy_(probs_dev[r0:r1], non_blocking=True)
        main.wait_stream(s_out)
        return probs_host


class FcPairProgram:
    """Model-parallel FC -> ReLU -> FC on p GPUs (the strategy of `parallel.strategy_fc_pair`).

    FC1's weight is split by output columns, so each rank computes a column shard of the hidden activation
    and applies ReLU locally; FC2's weight is split by input rows, so each rank's product is a full-size
    partial sum, joined by a sum over ranks (the reference's Reduce node, an NCCL all-reduce here).  X is
    replicated.  With `chunks` > 1 the rows are processed in chunks: the all-reduce of chunk i runs on the
    communication context's stream while the tensor cores work on chunk i+1.
    """

    def __init__(self, be: Backend, comm, w1, w2, max_rows: int, sharded: bool = False):
        """`w1` [k, n1] and `w2` [n1, n2] are the full matrices (each rank keeps its shard), or, with
        `sharded`, already this rank's shards [k, n1/p] and [n1/p, n2] (the full matrices never exist)."""
        from . import parallel as par
        self.be, self.comm = be, comm
        p, r = comm.nranks, comm.rank
        w1s = w1 if sharded else par.take_shard(w1, 1, r, p)      # [k, n1/p]
        w2s = w2 if sharded else par.take_shard(w2, 0, r, p)      # [n1/p, n2]
        self.wp1 = be.pack_weight_bf16(w1s)         # [n1/p, k]
        self.wp2 = be.pack_weight_bf16(w2s)         # [n2, n1/p]
        self.k, self.n1s, self.n2 = w1s.shape[0], w1s.shape[1], w2s.shape[1]
        self.h = torch.empty((max_rows, self.n1s), dtype=torch.bfloat16, device=be.device)
        self.y_part = torch.empty((max_rows, self.n2), dtype=torch.float32, device=be.device)
        self.y = torch.empty((max_rows, self.n2), dtype=torch.float32, device=be.device)
        self.max_rows = max_rows
        be.sync()

    def flops(self, rows: int) -> float:
        """Per rank."""
        return 2.0 * rows * self.n1s * (self.k + self.n2)

    def forward(self, x_bf16: torch.Tensor, chunks: int = 1, comm_sms: int = 0) -> torch.Tensor:
        """`comm_sms` > 0 (with chunks > 1): the GEMMs leave that many SMs free, on which the all-reduce of the previous
        chunk can run at the same time (a persistent GEMM CTA fills its SM's shared memory, so a collective kernel
        launched beside it otherwise waits for the GEMM to drain)."""
        rows = x_bf16.shape[0]
        be = self.be
        chunks = max(1, chunks)
        be.set_sm_limit(0 if chunks == 1 or comm_sms <= 0 else self._sm_total() - comm_sms)
        step = (rows + chunks - 1) // chunks
        ms, cs = be.torch_stream, self.comm.be.torch_stream
        overlap = ms is not None and cs is not None and cs != ms
        if overlap:
            start = torch.cuda.Event()
            start.record(ms)
            cs.wait_event(start)  # y of an earlier forward may still be read on the main stream
        for r0 in range(0, rows, step):
            r1 = min(rows, r0 + step)
            be.fc_bf16(x_bf16[r0:r1], self.wp1, None, L.ACT_RELU, out=self.h[r0:r1])
            be.fc_bf16(self.h[r0:r1], self.wp2, None, L.ACT_NONE, out=self.y_part[r0:r1])
            if overlap:
                ready = torch.cuda.Event()
                ready.record(ms)
                cs.wait_event(ready)
            self.comm.allreduce_sum(self.y_part[r0:r1], out=self.y[r0:r1])
        if overlap:
            done = torch.cuda.Event()
            done.record(cs)
            ms.wait_event(done)
        be.set_sm_limit(0)
        return self.y[:rows]

    def _sm_total(self) -> int:
        return torch.cuda.get_device_properties(self.be.device).multi_processor_count

    # ---- the join done by FC2's own epilogue over peer memory
    def peer_setup(self):
        """Collective.  Slot arrays for `forward_peer`: every rank owns max_rows / p rows of the output.  Two sets of
        slots, used by alternate passes."""
        import ctypes as C
        p = self.comm.nranks
        if self.max_rows % p:
            raise ValueError("the rows do not split evenly over the ranks")
        self.slots = torch.empty((2, p, self.max_rows // p, self.n2), dtype=torch.float32, device=self.be.device)
        self.y_own = torch.empty((2, self.max_rows // p, self.n2), dtype=torch.float32, device=self.be.device)  # alternate passes
        self.word = torch.zeros(1, dtype=torch.float32, device=self.be.device)
        first = self.comm.peer_slots_setup(self.slots)
        half = self.slots[0].numel() * 4
        second = (C.c_void_p * len(first))(*[(v + half) if v else None for v in first])
        self.slot_tables = (first, second)
        self._peer_pass = 0

    def forward_peer(self, x_bf16: torch.Tensor) -> torch.Tensor:
        """FC1 -> ReLU -> FC2 with the partial sums joined WITHOUT a collective kernel: FC2's epilogue stores every
        row block straight into the slot array of the rank that owns it (peer stores over NVLink, overlapped with the
        tensor-core work), the ranks meet (a one-word all-reduce), and each rank adds the p slots of its own block in
        rank order.  Returns this rank's block of the result, [rows / p, n2] (one of two buffers, alternating, so that
        a copy of it may still be under way while the next pass runs); rank r owns rows [r * rows/p, (r+1) * rows/p).

        Alternate passes use alternate slot sets, which is what makes one meeting point per pass enough: the FC2 that
        overwrites a set again (two passes later) starts, on any rank, only after the meeting point of the pass in
        between, and every rank reaches that one only after it has added up its slots of this pass."""
        rows = x_bf16.shape[0]
        if rows != self.max_rows:
            raise ValueError("forward_peer works on the row count the slots were set up for")
        be, comm = self.be, self.comm
        ms, cs = be.torch_stream, comm.be.torch_stream
        s = self._peer_pass & 1
        self._peer_pass += 1
        be.fc_bf16(x_bf16, self.wp1, None, L.ACT_RELU, out=self.h)
        be.fc_bf16_scatter_rows(self.h, self.wp2, self.slot_tables[s], comm.nranks, comm.rank, self.n2)
        ready = torch.cuda.Event()
        ready.record(ms)
        cs.wait_event(ready)
        comm.allreduce_sum(self.word, out=self.word)   # completes once every rank's FC2, peer stores included, is done
        met = torch.cuda.Event()
        met.record(cs)
        ms.wait_event(met)
        be.sum_slots(self.slots[s], self.y_own[s])
        return self.y_own[s]


class ResStageProgram:
    """ResNet-style stage, NHWC bf16 storage: `blocks` x (Conv3x3-BN-ReLU-Conv3x3-BN-Add(skip)-ReLU), MaxPool 2x2/2.

    Each Conv -> BatchNormalization [-> ElementAdd] -> Relu chain of the graph is ONE tensor-core launch (the
    batch-norm becomes a per-channel affine map in the epilogue, the skip tensor is added there too); the
    pool is one bandwidth-bound launch, or, where the row-interleaved convolution kernel runs, part of the last
    convolution's epilogue.  2 * blocks (+ 1) launches per forward instead of 7 * blocks + 1.
    """

    def __init__(self, be: Backend, convs, bns, max_batch: int, hw: int, ch: int, fuse_pool: bool | None = None):
        """`fuse_pool`: the final MaxPool inside the last convolution's launch (default: wherever that kernel takes
        the shape: 64 channels and an even image size)."""
        self.be = be
        self.fuse_pool = (ch == 64 and hw % 2 == 0) if fuse_pool is None else fuse_pool
        self.fp = [be.pack_filter_bf16(c["w"]) for c in convs]
        self.cb = [c["b"].contiguous() for c in convs]
        self.bn = [(b["scale"], b["bias"], b["mean"], b["var"], float(b["eps"])) for b in bns]
        shape = (max_batch, hw, hw, ch)
        self.buf = [torch.empty(shape, dtype=torch.bfloat16, device=be.device) for _ in range(3)]
        self.pooled = torch.empty((max_batch, hw // 2, hw // 2, ch), dtype=torch.bfloat16, device=be.device)
        self.launches_per_forward = len(self.fp) + (0 if self.fuse_pool else 1)
        self.hw, self.ch = hw, ch
        be.sync()

    def flops(self, batch: int) -> float:
        return float(len(self.fp)) * 2.0 * batch * self.hw * self.hw * self.ch * 9 * self.ch

    def capture(self, x_bf16: torch.Tensor):
        """The forward pass on `x_bf16`, captured once into a CUDA graph: returns (replay, pooled output).  One graph
        launch per pass instead of 2 * blocks + 1 calls through the library, which matters once a pass is short (a
        few tens of microseconds per launch when the batch is split over several GPUs).  The backend must have been
        made on a stream that can be captured (not the legacy default stream); the plain run first lets the library
        do its first-call set-up outside the capture."""
        stream = self.be.torch_stream
        if stream is None:
            raise ValueError("capture needs a backend made on a torch stream")
        with torch.cuda.stream(stream):
            self.forward(x_bf16)
            stream.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                out = self.forward(x_bf16)
        self._graph = graph  # keeps the captured buffers' owner alive
        return graph.replay, out

    def forward(self, x_bf16: torch.Tensor, on_launch=None) -> torch.Tensor:
        n = x_bf16.shape[0]
        k3, s1, p1 = (3, 3), (1, 1), (1, 1, 1, 1)
        be, cur = self.be, x_bf16
        free = [b[:n] for b in self.buf]
        li = 0
        blocks = len(self.fp) // 2
        for blk in range(blocks):
            t, o = [b for b in free if b.data_ptr() != cur.data_ptr()][:2]
            if on_launch:
                on_launch(li, 0)
            be.conv2d_bf16(cur, self.fp[2 * blk], self.cb[2 * blk], k3, s1, p1, bn=self.bn[2 * blk], relu=True, out=t)
            if on_launch:
                on_launch(li, 1)
                on_launch(li + 1, 0)
            last = self.fuse_pool and blk == blocks - 1   # the stage's MaxPool rides in this launch's epilogue
            be.conv2d_bf16(t, self.fp[2 * blk + 1], self.cb[2 * blk + 1], k3, s1, p1, bn=self.bn[2 * blk + 1],
                           residual=cur, relu=True, out=self.pooled[:n] if last else o, pool=last)
            if on_launch:
                on_launch(li + 1, 1)
            li += 2
            cur = o
        if self.fuse_pool:
            return self.pooled[:n]
        if on_launch:
            on_launch(li, 0)
        out = be.maxpool_bf16(cur, (2, 2), (2, 2), (0, 0, 0, 0), out=self.pooled[:n])
        if on_launch:
            on_launch(li, 1)
        return out
