"""The C ABI from plain C: the header compiles as C99 on its own, and a C program that links libdcb200.so runs a query on
the GPU without any Python in the way."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_header_is_self_contained_c99(tmp_path):
    src = tmp_path / "h.c"
    src.write_text('#include "dcb200.h"\nint main(void) { return DCB_ABI_VERSION - 1; }\n')
    subprocess.run(["gcc", "-std=c99", "-pedantic", "-Wall", "-Werror", "-fsyntax-only", "-I", os.path.join(ROOT, "include"), str(src)], check=True)


def _build_client(built_library, tmp_path):
    exe = tmp_path / "c_client"
    libdir = os.path.dirname(built_library)
    subprocess.run(["gcc", "-std=c99", "-O1", "-Wall", "-I", os.path.join(ROOT, "include"), os.path.join(ROOT, "tests", "c_abi", "c_client.c"),
                    "-L", libdir, "-ldcb200", "-lm", f"-Wl,-rpath,{libdir}", "-o", str(exe)], check=True)
    return exe


def test_c_client_builds_and_links(built_library, tmp_path):
    assert os.path.exists(_build_client(built_library, tmp_path))


@pytest.mark.gpu
def test_c_client_runs_on_gpu(built_library, tmp_path):
    exe = _build_client(built_library, tmp_path)
    out = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stderr
    assert "c_client ok" in out.stdout


def test_pinvoke_stub_is_complete_and_current():
    """include/Dcb200.PInvoke.cs (the LibraryImport class for the managed side) has one line per prototype of the header
    and is what include/make_pinvoke.py generates from the header as it is now."""
    import importlib.util
    inc = os.path.join(ROOT, "include")
    spec = importlib.util.spec_from_file_location("make_pinvoke", os.path.join(inc, "make_pinvoke.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    with open(os.path.join(inc, "dcb200.h")) as f:
        want = mod.generate(f.read())
    with open(os.path.join(inc, "Dcb200.PInvoke.cs")) as f:
        have = f.read()
    assert have == want, "run python include/make_pinvoke.py"
    from dotcompute_b200 import native
    for name in native.declared_symbols():
        assert f" {name}(" in have, name
