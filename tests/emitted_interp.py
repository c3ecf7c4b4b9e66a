"""Test infrastructure: runs the call sequence of a program B200Codegen emitted, on the CPU.

The emitted C++ is read as text: the `const size_t name[] = {...}` shape arrays, the `load_to_device` lines and the
`SWC_CHECK(swcb200_*(ctx, ...))` calls of main(), in order, with `if (rank == 0) { ... }` blocks honoured.  Every
table call is carried out by the CPU oracle on numpy arrays (bf16 entry points: operands rounded to bf16, fp32
accumulation), and the communication calls by `swcompiler_b200.parallel.TorchComm` over gloo when there is more than
one rank.  What this checks is the GENERATOR: call order, operand names, shapes, leading dimensions, axes, guards,
the storage plan of the fusion planner.  It says nothing about the CUDA kernels, which the GPU tests cover.
"""
import os
import re

import numpy as np

import cases

_CALL = re.compile(r"SWC_CHECK\(swcb200_(\w+)\((.*)\)\);")
_DIMS = re.compile(r"const size_t (\w+)\[\] = \{([^}]*)\};")
_LOAD = re.compile(r"load_to_device<(\w+)>\((\w+), (\d+), (\d+), \"([^\"]+)\", host_stage\);")
_PRINT = re.compile(r"print_device<(\w+)>\(\"(\w+)\", (\w+), (\d+), (\d+), host_stage\);")
_ALIAS = re.compile(r"^(\w+) = (\w+);$")   # a view (Reshape): the child names the parent's storage
_FILL = re.compile(r"fill_device<(\w+)>\((\w+), (\d+), \(\w+\)([-\d.e+]+), host_stage\);")
_LOADER = re.compile(r"RecordLoader loader\(\"([^\"]+)\", (true|false), (\d+), (\d+), (\d+)\);")
_SLOT = re.compile(r"^(\w+) = \1_slot\[s\];$")
_EPI = re.compile(r"const swcb200_conv_epilogue (\w+) = \{([^}]*)\};")


def _tanh(x):
    return (1.0 - 2.0 / (np.exp(2.0 * x.astype(np.float64)) + 1.0)).astype(np.float32)


class Interp:
    def __init__(self, oracle, files_dir, rank=0, nranks=1, comm=None):
        self.o, self.dir, self.rank, self.nranks, self.comm = oracle, files_dir, rank, nranks, comm
        self.t, self.dims, self.epi, self.printed, self.calls = {}, {}, {}, {}, []

    # ---- helpers
    def _get(self, name):
        name = name.strip().lstrip("&")
        if name in ("nullptr", "NULL"):
            return None
        return self.t.get(name)   # a master-only tensor off the master: None

    def _int(self, s):
        return int(s.strip().rstrip("f"))

    def run(self, path):
        text = open(path).read()
        lines = [l.strip() for l in text[text.index("int main("):].splitlines()]
        i = 0
        while i < len(lines):
            line = lines[i]
            m = _LOADER.search(line)
            if m:   # streaming evaluation: run the loop body once per batch the record file can fill
                start = next(j for j in range(i, len(lines)) if lines[j].startswith("for (int s = 0; have;"))
                end = next(j for j in range(start, len(lines)) if lines[j].startswith("SWC_CHECK(swcb200_sync(ctx)"))
                body = lines[start + 1:end - 1]
                fed = [_SLOT.match(l).group(1) for l in body if _SLOT.match(l)]   # label tensor, then data tensor
                samples, batch, size = int(m.group(3)), int(m.group(4)), int(m.group(5))
                raw = open(os.path.join(self.dir, m.group(1)), "rb").read()
                rec = 1 + size * (4 if m.group(2) == "true" else 1)
                self.batches = 0
                for b0 in range(0, samples - batch + 1, batch):
                    recs = [raw[(b0 + k) * rec:(b0 + k + 1) * rec] for k in range(batch)]
                    assert all(len(r) == rec for r in recs), "record file shorter than the sample count"
                    self.t[fed[0]] = np.array([np.frombuffer(r[:1], np.int8)[0] for r in recs], np.int32)
                    self.t[fed[1]] = np.concatenate([np.frombuffer(r[1:], np.float32) if m.group(2) == "true"
                                                     else np.frombuffer(r[1:], np.int8).astype(np.float32) for r in recs])
                    self._block(body)
                    self.batches += 1
                i = end
                continue
            if line == "auto forward = [&]() {":   # CUDA-graph form: the forward pass as a closure, run plainly then replayed
                end = next(j for j in range(i, len(lines)) if lines[j] == "};")
                self.forward_body, self.forward_runs = lines[i + 1:end], 0
                i = end + 1
                continue
            if line == "forward();" or line.startswith("for (int rep = 0;") and "cudaGraphLaunch" in line:
                reps = int(re.search(r"rep < (\d+)", line).group(1)) if line.startswith("for (int rep") else 1
                for _ in range(reps):
                    self._block(self.forward_body)
                    self.forward_runs += 1
                i += 1
                continue
            i = self._block(lines, i, single=True)
        return self.printed

    def _block(self, lines, i=0, single=False):
        """Executes lines[i:] (or, with single, one statement or one `if (rank == 0) {...}` block); returns the next index."""
        while i < len(lines):
            line = lines[i]
            if line == "if (rank == 0) {":
                j = i + 1
                while lines[j] != "}":
                    if self.rank == 0:
                        self._line(lines[j])
                    j += 1
                i = j + 1
            else:
                self._line(line)
                i += 1
            if single:
                break
        return i

    def _line(self, line):
        m = _DIMS.search(line)
        if m:
            self.dims[m.group(1)] = tuple(int(v) for v in m.group(2).split(","))
            return
        m = _EPI.search(line)
        if m:
            self.epi[m.group(1)] = [v.strip() for v in m.group(2).split(",")]
            return
        m = _LOAD.search(line)
        if m:
            dt = np.float32 if m.group(1) == "float" else np.int32
            a = np.fromfile(os.path.join(self.dir, m.group(5)), dtype=dt)
            self.t[m.group(2)] = a[int(m.group(4)):int(m.group(4)) + int(m.group(3))].copy()
            return
        m = _FILL.search(line)
        if m:
            dt = np.float32 if m.group(1) == "float" else np.int32
            self.t[m.group(2)] = np.full(int(m.group(3)), float(m.group(4)), dt)
            return
        m = _PRINT.search(line)
        if m:
            self.printed[m.group(2)] = self.t[m.group(3)].reshape(int(m.group(4)), int(m.group(5)))
            return
        m = _ALIAS.match(line)
        if m and m.group(2) in self.t:
            self.t[m.group(1)] = self.t[m.group(2)]
            return
        m = _CALL.search(line)
        if m:
            args = [a.strip() for a in m.group(2).split(",")][1:]   # drop ctx
            self.calls.append(m.group(1))
            getattr(self, "op_" + m.group(1), self._ignore)(*args)

    def _ignore(self, *a):
        pass

    # ---- fp32 table
    def op_matrixMatrixMul_f(self, m, n, k, a, lda, b, ldb, c, ldc):
        m, n, k = int(m), int(n), int(k)
        assert int(lda) == k and int(ldb) == n and int(ldc) == n
        self.t[c] = self.o.matrixMatrixMul_f(self._get(a).reshape(m, k), self._get(b).reshape(k, n)).reshape(-1)

    def op_batchedadd_f(self, dest, batch, sl, rows, cols):
        self.t[dest] = self.o.batchedadd_f(self._get(batch).reshape(int(rows), int(cols)), self._get(sl)).reshape(-1)

    def op_matrixTanh_f(self, m, n, a, lda, b, ldb):
        self.t[b] = self.o.matrixTanh_f(self._get(a).reshape(int(m), int(n))).reshape(-1)

    def op_matrixSoftmax_f(self, m, n, a, lda, b, ldb):
        self.t[b] = self.o.matrixSoftmax_f(self._get(a).reshape(int(m), int(n))).reshape(-1)

    def op_argMax_i(self, a, idx, m, n, k):
        self.t[idx] = self.o.argMax_i(self._get(a).reshape(int(m), int(n)), int(k)).reshape(-1).astype(np.int32)

    def op_accuracy_i(self, pred, label, accum, m, n):
        self.t[accum] = self.o.accuracy_i(self._get(pred).reshape(int(m), int(n)), self._get(label), self._get(accum))

    def op_relu_f(self, src, dst, size):
        self.t[dst] = self.o.relu_f(self._get(src)[:int(size)])

    def op_vecAdd_f(self, size, a, b, c):
        self.t[c] = self.o.vecAdd_f(self._get(a)[:int(size)], self._get(b)[:int(size)])

    def op_conv2d_f(self, out, x, f, b, od, idm, fd, bd, kd, sd, pd, group):
        y = self.o.conv2d_f(self._get(x).reshape(self.dims[idm]), self._get(f).reshape(self.dims[fd]), self._get(b),
                            self.dims[kd], self.dims[sd], self.dims[pd])
        assert y.shape == self.dims[od]
        self.t[out] = y.reshape(-1)

    def op_batchnormalization_f(self, out, x, mean, var, scale, bias, idm, eps):
        self.t[out] = self.o.batchnormalization_f(self._get(x).reshape(self.dims[idm]), self._get(mean), self._get(var),
                                                  self._get(scale), self._get(bias), float(eps.rstrip("f"))).reshape(-1)

    def op_maxpool_f(self, x, out, idm, od, kd, sd, pd):
        y = self.o.maxpool_f(self._get(x).reshape(self.dims[idm]), self.dims[kd], self.dims[sd], self.dims[pd])
        assert y.shape == self.dims[od]
        self.t[out] = y.reshape(-1)

    # ---- bf16 storage entry points: bf16-rounded operands, fp32 arithmetic
    def op_avgpool_f(self, x, out, idm, od, kd, sd, pd):
        xv = self._get(x).reshape(self.dims[idm.strip()])
        self.t[out.strip()] = self.o.avgpool_f(xv, self.dims[kd.strip()], self.dims[sd.strip()], self.dims[pd.strip()]).reshape(-1)

    def op_cast_f32_to_bf16(self, src, dst, count):
        self.t[dst] = cases.bf16_round(self._get(src)[:int(count)])

    def op_cast_bf16_to_f32(self, src, dst, count):
        self.t[dst] = self._get(src)[:int(count)].copy()

    def op_pack_weight_bf16(self, w, k, n, ldb, wp):
        assert int(ldb) == int(n)
        self.t[wp] = np.ascontiguousarray(cases.bf16_round(self._get(w).reshape(int(k), int(n))).T).reshape(-1)   # [n, k]

    def op_pack_filter_bf16(self, f, fd, fp):
        self.t[fp] = cases.bf16_round(self._get(f))

    def op_fc_bf16(self, m, n, k, a, lda, wp, ldw, bias, act, c, c_dtype, ldc):
        m, n, k = int(m), int(n), int(k)
        assert int(lda) == k and int(ldw) == k and int(ldc) == n
        y = self.o.matrixMatrixMul_f(self._get(a).reshape(m, k), np.ascontiguousarray(self._get(wp).reshape(n, k).T))
        if self._get(bias) is not None:
            y = self.o.batchedadd_f(y, self._get(bias))
        y = {"SWCB200_ACT_NONE": lambda v: v, "SWCB200_ACT_RELU": lambda v: np.maximum(v, 0), "SWCB200_ACT_TANH": _tanh}[act](y)
        self.t[c] = (cases.bf16_round(y) if c_dtype == "SWCB200_BF16" else y).reshape(-1)

    def op_conv2d_bf16(self, out, x, fp, b, od, idm, fd, kd, sd, pd, ep):
        y = self.o.conv2d_f(self._get(x).reshape(self.dims[idm]), self._get(fp).reshape(self.dims[fd]), self._get(b),
                            self.dims[kd], self.dims[sd], self.dims[pd])
        fields = self.epi[ep.lstrip("&")]
        scale, bias, mean, var, eps, res, relu = fields[:7]
        pool = len(fields) > 7 and int(fields[7])
        if scale != "nullptr":
            y = self.o.batchnormalization_f(y, self._get(mean), self._get(var), self._get(scale), self._get(bias),
                                            float(eps.rstrip("f")))
        if res != "nullptr":
            y = y + self._get(res).reshape(y.shape)
        if int(relu):
            y = np.maximum(y, 0)
        assert y.shape == self.dims[od]
        if pool:   # MaxPool 2x2 / 2 as the epilogue's last step
            n, h, w, c = y.shape
            y = self.o.maxpool_f(np.ascontiguousarray(y.astype(np.float32)), (2, 2), (2, 2), (0, 0, 0, 0))
            assert y.shape == (n, h // 2, w // 2, c)
        self.t[out] = cases.bf16_round(y.astype(np.float32)).reshape(-1)

    def op_maxpool_bf16(self, x, out, idm, od, kd, sd, pd):
        self.op_maxpool_f(x, out, idm, od, kd, sd, pd)

    # ---- communication
    def _torch(self, a, dtype):
        import torch
        return None if a is None else torch.from_numpy(np.ascontiguousarray(a)).to(dtype)

    def _dt(self, name):
        import torch
        return torch.int32 if name == "SWCB200_I32" else torch.float32

    def op_scatter(self, src, dst, dims, ndim, axis, dt, root):
        d = self.dims[dims]
        assert len(d) == int(ndim) and int(root) == 0
        full = self._get(src)
        assert (full is not None) == (self.rank == 0)
        full = None if full is None else self._torch(full.reshape(d), self._dt(dt))
        self.t[dst] = self.comm.scatter(full, d, int(axis), dtype=self._dt(dt)).numpy().reshape(-1)

    def op_gather(self, src, dst, dims, ndim, axis, dt, root):
        d = self.dims[dims]
        from swcompiler_b200.parallel import shard_dims
        local = self._torch(self._get(src).reshape(shard_dims(d, int(axis), self.nranks)), self._dt(dt))
        out = self.comm.gather(local, d, int(axis))
        if self.rank == 0:
            self.t[dst] = out.numpy().reshape(-1)

    def op_reduce_sum(self, src, dst, count, dt, root):
        out = self.comm.reduce_sum(self._torch(self._get(src)[:int(count)], self._dt(dt)))
        if self.rank == 0:
            self.t[dst] = out.numpy()

    # ---- the Reduce join over peer memory: each rank's slot array holds, for the rows it owns, every rank's partial sums
    def _sym(self, v):
        return {"nprocs": self.nranks, "rank": self.rank}.get(v.strip(), None) if not v.strip().isdigit() else int(v)

    def op_peer_slots_setup(self, local, table):
        self.slot_tables = getattr(self, "slot_tables", {})
        self.slot_tables[table] = local           # the table's entry for this rank is the local array; peers hold theirs

    def op_fc_bf16_scatter_rows(self, m, n, k, a, lda, wp, ldw, table, nranks, rank, ld_slot):
        import torch
        m, n, k = int(m), int(n), int(k)
        assert self._sym(nranks) == self.nranks and self._sym(rank) == self.rank and int(ld_slot) == n and m % self.nranks == 0
        part = self.o.matrixMatrixMul_f(self._get(a).reshape(m, k), np.ascontiguousarray(self._get(wp).reshape(n, k).T))
        parts = self.comm.allgather(torch.from_numpy(np.ascontiguousarray(part))).numpy().reshape(self.nranks, m, n)
        rows = m // self.nranks
        mine = [p[self.rank * rows:(self.rank + 1) * rows] for p in parts]   # slot r: rank r's partial sums of my rows
        self.t[self.slot_tables[table]] = np.concatenate([b.reshape(-1) for b in mine]).astype(np.float32)

    def op_allreduce_sum(self, src, dst, count, dt):
        v = self._get(src)
        v = np.zeros(int(count), np.float32) if v is None else v[:int(count)]
        self.t[dst] = self.comm.allreduce_sum(self._torch(v, self._dt(dt))).numpy()

    def op_sum_slots(self, slots, stride, nslots, out, count):
        stride, count, nslots = int(stride), int(count), self._sym(nslots)
        s = self._get(slots)
        acc = s[:count].copy()
        for r in range(1, nslots):                 # rank order, one rounding per addition
            acc = (acc + s[r * stride:r * stride + count]).astype(np.float32)
        self.t[out] = acc

    def op_transform(self, src, dst, dims, ndim, pre, post, dt):
        d = self.dims[dims]
        from swcompiler_b200.parallel import shard_dims
        pre, post = int(pre), int(post)
        shape = d if pre < 0 else shard_dims(d, pre, self.nranks)
        self.t[dst] = self.comm.transform(self._torch(self._get(src).reshape(shape), self._dt(dt)), d, pre, post).numpy().reshape(-1)
