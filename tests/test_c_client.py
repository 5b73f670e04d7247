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
