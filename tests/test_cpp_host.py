"""The C++ host mirror (include/leviathan_cuda.hpp): the header compiles and links against the
shared library on any machine; on a GPU the C++ parity program (tests/cpp/host_parity.cpp, the
reference's known-answer cases written against the mirror) runs green."""
import os
import shutil
import subprocess

import pytest

from leviathan_b200 import _lib as L

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _build(tmp_path):
    if not os.path.exists(L.LIB_PATH):
        from leviathan_b200.build import build_library

        build_library()
    exe = os.path.join(str(tmp_path), "host_parity")
    libdir = os.path.dirname(L.LIB_PATH)
    cmd = ["g++", "-std=c++17", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"),
           os.path.join(ROOT, "tests", "cpp", "host_parity.cpp"), "-o", exe, "-L", libdir, "-lleviathan_cuda",
           f"-Wl,-rpath,{libdir}"]
    subprocess.run(cmd, check=True, capture_output=True, text=True)
    return exe


@pytest.mark.skipif(shutil.which("g++") is None, reason="no C++ compiler")
def test_cpp_host_mirror_compiles_and_links(tmp_path):
    assert os.path.exists(_build(tmp_path))


@pytest.mark.gpu
@pytest.mark.skipif(shutil.which("g++") is None, reason="no C++ compiler")
def test_cpp_host_parity_program(tmp_path):
    out = subprocess.run([_build(tmp_path), str(tmp_path / "known.gguf")], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stdout + out.stderr
    assert out.stdout.strip().startswith("ok ")
