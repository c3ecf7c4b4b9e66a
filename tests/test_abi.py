"""CPU: the C-ABI library loads and exports everything the public header declares; without a GPU it
refuses to create a context instead of falling back."""
import ctypes as C
import os

import pytest

import swcompiler_b200 as swc
from swcompiler_b200 import _lib as L


def test_library_is_built_in_tree():
    assert os.path.exists(L.LIB_PATH), "run python -m swcompiler_b200.build"


def test_every_declared_symbol_is_exported():
    lib = L.lib()
    names = L.declared_symbols()
    assert len(names) >= 25
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def test_header_is_plain_c(tmp_path):
    """The boundary is a C ABI: the header compiles as C99 with no C++ in sight, and a C program links against the library."""
    import subprocess
    src = tmp_path / "use.c"
    src.write_text('#include "swc_b200.h"\nint main(void) { swcb200_ctx *c = 0; return swcb200_version() > 0 && swcb200_destroy(c) != 0 ? 0 : 1; }\n')
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    lib = os.path.join(root, "swcompiler_b200")
    exe = tmp_path / "use"
    r = subprocess.run(["gcc", "-std=c99", "-Wall", "-Wextra", "-pedantic", "-Werror", "-I" + os.path.join(root, "include"), str(src),
                        "-o", str(exe), "-L" + lib, "-lswc_b200", "-Wl,-rpath," + lib], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    assert subprocess.run([str(exe)]).returncode == 0    # version > 0; a null context is refused, not dereferenced


def test_status_strings():
    assert L.status_string(L.OK) == "ok"
    assert "sm_100" in L.status_string(L.ERR_NO_DEVICE)
    assert L.lib().swcb200_version() >= 100


def test_no_cpu_fallback():
    import torch
    if torch.cuda.is_available():
        pytest.skip("GPU present")
    ctx = C.c_void_p()
    rc = L.lib().swcb200_init(C.c_int(0), C.c_int(L.STRICT_F32), C.byref(ctx))
    assert rc in (L.ERR_NO_DEVICE, L.ERR_CUDA) and not ctx.value
    with pytest.raises(RuntimeError):
        swc.Backend(0)


def test_null_context_is_rejected_not_dereferenced():
    lib = L.lib()
    assert lib.swcb200_sync(C.c_void_p()) == L.ERR_BAD_ARG
    assert lib.swcb200_relu_f(C.c_void_p(), C.c_void_p(), C.c_void_p(), C.c_size_t(4)) == L.ERR_BAD_ARG


def test_product_does_not_import_the_oracle():
    pkg = os.path.dirname(swc.__file__)
    for root, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".cpp")):
                text = open(os.path.join(root, f)).read()
                assert "oracle" not in text.lower(), f
