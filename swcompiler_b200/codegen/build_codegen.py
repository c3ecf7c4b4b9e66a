"""Builds the B200Codegen generator against a reference checkout and emits the sample programs.

    python -m swcompiler_b200.codegen.build_codegen [reference_root]

The reference's own build system (cmake + protobuf) is not used: its library sources under src/ (all but
the importer, which needs protobuf, and the emitted-program utilities) are compiled in place with g++,
together with B200Codegen.cpp and gen_driver.cpp.  Objects and the binary go to codegen/build/ (not
tracked); the emitted sample programs are written to tests/golden/emitted/ (tracked test fixtures: they are
what the GPU tests compile and run, since the GPU machine has no reference checkout).

The reference checkout is looked for at $REFERENCE_ROOT, else in a folder `reference` beside the repository.
"""
from __future__ import annotations

import concurrent.futures as cf
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
BUILD = os.path.join(HERE, "build")
EMITTED = os.path.join(ROOT, "tests", "golden", "emitted")


def reference_root() -> str:
    return os.environ.get("REFERENCE_ROOT") or os.path.join(os.path.dirname(ROOT), "reference")


# the sample programs: <graph>[_dp<N> | _mp<N>][_fused], see gen_driver.cpp
PROGRAMS = ("mlp8", "convnet", "resblock", "mlp8_fused", "convnet_fused", "resblock_fused",
            "resproj", "resproj_fused", "convact", "convact_fused", "c2lenet", "c2resnet", "c2resnet_fused",
            "mlp8_dp2", "mlp8_dp2_fused", "fcpair_mp2", "fcpair_mp2_fused", "mlp8_mp2", "resblock_dp2", "mlp_eval", "mlp_eval_fused",
            "mlp8_graph", "resblock_fused_graph")


def reference_sources(ref: str):
    srcs = []
    for path in glob.glob(os.path.join(ref, "src", "**", "*.cpp"), recursive=True):
        rel = os.path.relpath(path, os.path.join(ref, "src"))
        if rel.startswith("importer") or rel.startswith(os.path.join("codegen", "utils")):
            continue
        srcs.append(path)
    return sorted(srcs)


def build(ref: str = None, quiet: bool = True) -> str:
    ref = ref or reference_root()
    if not os.path.exists(os.path.join(ref, "include", "SWC.h")):
        raise FileNotFoundError(f"no reference checkout at {ref}")
    os.makedirs(BUILD, exist_ok=True)
    os.makedirs(EMITTED, exist_ok=True)
    flags = ["-std=c++11", "-O1", "-w", "-I" + os.path.join(ref, "src"), "-I" + os.path.join(ref, "include"), "-I" + HERE]
    jobs, objs = [], []
    ours = [os.path.join(HERE, f) for f in ("B200Codegen.cpp", "Caffe2Import.cpp", "gen_driver.cpp")]
    for s in reference_sources(ref) + ours:
        o = os.path.join(BUILD, os.path.relpath(s, "/").replace(os.sep, "_")[:-4] + ".o")
        objs.append(o)
        hdr = max(os.path.getmtime(os.path.join(HERE, h)) for h in ("B200Codegen.h", "Caffe2Import.h"))
        if not os.path.exists(o) or os.path.getmtime(o) < max(os.path.getmtime(s), hdr):
            jobs.append(["g++", *flags, "-c", s, "-o", o])

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode:
            raise RuntimeError(" ".join(cmd) + "\n" + r.stdout + r.stderr)

    with cf.ThreadPoolExecutor(max_workers=8) as ex:
        list(ex.map(run, jobs))
    exe = os.path.join(BUILD, "gen_driver")
    run(["g++", "-o", exe, *objs])
    return exe


def write_caffe2_models(where: str):
    """The serialized nets of the two synthetic Caffe2 models (tests/golden/caffe2_models.py), for gen_driver's import."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("caffe2_models", os.path.join(ROOT, "tests", "golden", "caffe2_models.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    for name in ("c2lenet", "c2resnet"):
        predict, init, _, _ = mod.model(name)
        open(os.path.join(where, name + "_predict.pb"), "wb").write(predict)
        open(os.path.join(where, name + "_init.pb"), "wb").write(init)


def emit(exe: str, out_dir: str = EMITTED):
    os.makedirs(out_dir, exist_ok=True)
    write_caffe2_models(BUILD)
    for which in PROGRAMS:
        # the generator also drops Graph.cpp / G_Makefile / SW_Makefile and *.dot in its working directory
        r = subprocess.run([exe, which, out_dir, "$(abspath ../../..)"], cwd=BUILD, capture_output=True, text=True)
        if r.returncode:
            raise RuntimeError(r.stdout[-2000:] + r.stderr[-2000:])
    return out_dir


if __name__ == "__main__":
    exe = build(sys.argv[1] if len(sys.argv) > 1 else None, quiet=False)
    print(emit(exe))
