"""Failure detection, tested without faulting any GPU.

Host side (CPU, no GPU): the bounded wait over a communicator's collectives (`swcb200_comm_watch`) runs its polling
loop against a stand-in NCCL library (tests/fake_nccl.c) whose asynchronous error state either stays "in progress" --
a peer that hangs: the loop must give up after the wall-clock limit with SWCB200_ERR_TIMEOUT and abort the
communicator -- or turns into an error -- a peer that died: SWCB200_ERR_NCCL and an abort, well before the limit.

Device side (GPU): a kernel waits, with the bounded wait every tensor-core kernel uses, on a barrier nothing arrives
at; the wait runs out after the context's limit, the kernel returns normally, `swcb200_sync` reports
SWCB200_ERR_TIMEOUT and the same context then runs the next kernel correctly.
"""
import os
import subprocess
import sys
import textwrap
import time

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _build_fake(tmp_path):
    so = os.path.join(str(tmp_path), "libfake_nccl.so")
    subprocess.run(["gcc", "-shared", "-fPIC", "-O1", "-o", so, os.path.join(ROOT, "tests", "fake_nccl.c")], check=True)
    return so


def _watch_in_child(so, timeout_ms, error_after):
    """The library caches the NCCL table it loaded for the life of the process, so each case runs in a child."""
    code = textwrap.dedent(f"""
        import ctypes as C, sys, time
        sys.path.insert(0, {ROOT!r})
        from swcompiler_b200 import _lib as L
        lib = L.lib()
        fake = C.CDLL({so!r})
        t0 = time.perf_counter()
        rc = lib.swcb200_comm_watch_selftest(C.c_char_p({so!r}.encode()), C.c_int({timeout_ms}))
        print(rc, fake.fake_nccl_aborts(), fake.fake_nccl_queries(), time.perf_counter() - t0)
    """)
    env = dict(os.environ, FAKE_NCCL_ERROR_AFTER=str(error_after))
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, timeout=60)
    assert r.returncode == 0, r.stderr
    rc, aborts, queries, secs = r.stdout.split()
    return int(rc), int(aborts), int(queries), float(secs)


def test_watch_gives_up_on_a_hung_peer_after_the_wall_clock_limit(tmp_path):
    from swcompiler_b200 import _lib as L
    so = _build_fake(tmp_path)
    rc, aborts, queries, secs = _watch_in_child(so, 300, 0)
    assert rc == L.ERR_TIMEOUT and aborts == 1
    assert 0.3 <= secs < 5.0 and queries > 10          # it polled for the whole limit, then stopped


def test_watch_reports_a_dead_peer_at_once(tmp_path):
    from swcompiler_b200 import _lib as L
    so = _build_fake(tmp_path)
    rc, aborts, queries, secs = _watch_in_child(so, 20000, 5)
    assert rc == L.ERR_NCCL and aborts == 1 and queries == 5
    assert secs < 5.0                                   # long before the 20 s limit


@pytest.mark.gpu
def test_device_side_wait_runs_out_and_the_context_survives():
    import numpy as np
    import torch

    import swcompiler_b200 as swc
    from swcompiler_b200 import _lib as L
    be = swc.Backend(0, swc.TC_BF16)
    be.set_wait_limit(1_000_000)                        # about half a millisecond
    t0 = time.perf_counter()
    be.selftest_wait_timeout()
    with pytest.raises(L.SwcError) as e:
        be.sync()
    assert e.value.status == L.ERR_TIMEOUT and "gave up waiting" in str(e.value)
    assert time.perf_counter() - t0 < 5.0
    be.sync()                                           # the status was cleared: clean again
    # the context and the GPU are fine: a tensor-core layer right after it gives the right numbers
    be.set_wait_limit(4_000_000_000)
    g = torch.Generator(device="cuda").manual_seed(3)
    a = torch.randn((256, 512), generator=g, device="cuda").to(torch.bfloat16)
    w = (torch.randn((512, 384), generator=g, device="cuda") / 22.6)
    out = be.fc_bf16(a, be.pack_weight_bf16(w), None, swc.ACT_NONE, torch.float32)
    be.sync()
    ref = a.float() @ w.to(torch.bfloat16).float()
    assert float((out - ref).abs().max()) <= 2e-3
