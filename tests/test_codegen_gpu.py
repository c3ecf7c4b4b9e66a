"""GPU: the emitted programs, compiled with g++ on the spot and run as separate processes, against the CPU oracle.
This is the drop-in path end to end: reference graph API -> reference passes -> B200Codegen -> C-ABI kernel table."""
import os
import shutil
import subprocess

import numpy as np
import pytest

from codegen_util import compile_emitted, convnet_inputs, convnet_oracle, parse_printed
from conftest import GOLDEN

pytestmark = pytest.mark.gpu


def test_emitted_mlp8_reproduces_the_known_answer(tmp_path, oracle, mnist8, golden):
    exe = compile_emitted("mlp8", str(tmp_path))
    for f in os.listdir(os.path.join(GOLDEN, "mnist8")):
        shutil.copyfile(os.path.join(GOLDEN, "mnist8", f), os.path.join(tmp_path, f))
    r = subprocess.run([exe], capture_output=True, text=True, cwd=str(tmp_path), timeout=120)
    assert r.returncode == 0, r.stderr
    got = parse_printed(r.stdout)
    assert got["top3"].astype(int).tolist() == golden["mnist8/top3"].tolist()
    assert got["top3"][:, 0].astype(int).tolist() == [5, 0, 4, 1, 9, 2, 1, 3]
    assert np.allclose(got["data4"], golden["mnist8/probs"], atol=5.1e-4)   # printed with three decimals


def test_emitted_convnet_matches_oracle(tmp_path, oracle):
    exe = compile_emitted("convnet", str(tmp_path))
    t = convnet_inputs()
    for name, arr in t.items():
        arr.tofile(os.path.join(tmp_path, name))
    r = subprocess.run([exe], capture_output=True, text=True, cwd=str(tmp_path), timeout=120)
    assert r.returncode == 0, r.stderr
    got = parse_printed(r.stdout)
    want = convnet_oracle(oracle, t)
    assert np.allclose(got["probs"], want, atol=5.1e-4)
    assert got["top1"][:, 0].astype(int).tolist() == oracle.argMax_i(want, 1)[:, 0].tolist()
