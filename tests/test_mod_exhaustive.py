"""The kernels' modular reductions over every reachable input, on the host: the header that the
CUDA kernels include (immerdink_b200/csrc/common/modred.hpp) is compiled with g++ into a small
program that compares each function with plain integer arithmetic (tests/mod_exhaustive.cpp)."""
import os
import subprocess

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_modular_reductions_exhaustively(tmp_path):
    exe = tmp_path / "mod_exhaustive"
    subprocess.run(["g++", "-std=c++17", "-O2", "-ffp-contract=off",
                    "-I" + os.path.join(ROOT, "immerdink_b200", "csrc"),
                    os.path.join(ROOT, "tests", "mod_exhaustive.cpp"), "-o", str(exe)], check=True)
    out = subprocess.run([str(exe)], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0 and out.stdout.startswith("ok "), out.stdout + out.stderr
    assert int(out.stdout.split()[1]) > 300_000_000
