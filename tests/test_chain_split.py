"""The work split of the persistent matvec kernel, walked on the CPU: tests/cpp/chain_split_check.cpp
includes the kernel's own split functions (leviathan_b200/csrc/lev_chain_split.h) and checks, over
many tile counts, K-steps per tile, grid sizes and warp counts, that every tile is finished exactly
once and that every awaited arrival count is the number of arrivals that happen."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(shutil.which("g++") is None, reason="no C++ compiler")
def test_chain_split_walk(tmp_path):
    exe = os.path.join(str(tmp_path), "chain_split_check")
    subprocess.run(["g++", "-O2", "-std=c++17", "-Wall", "-I", os.path.join(ROOT, "leviathan_b200", "csrc"),
                    os.path.join(ROOT, "tests", "cpp", "chain_split_check.cpp"), "-o", exe], check=True)
    out = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stdout[-2000:]
    assert out.stdout.strip().endswith("ok")
