"""The kernels' Float64 exp (knet.jl_b200/csrc/exp64.cuh) as a host program: the header uses IEEE
adds, multiplies and fused multiply-adds only, so its host build computes what the kernel
computes.  tests/exp64_check.cpp compares it with the 113-bit libquadmath value rounded once on
pseudo-random arguments (whole range, sigm's range, tiny values, near-multiples of ln2/64)."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_exp64_is_correctly_rounded_on_a_sample(tmp_path):
    cxx = shutil.which("g++")
    if cxx is None:
        pytest.skip("no g++")
    exe = str(tmp_path / "exp64_check")
    subprocess.check_call([cxx, "-O2", "-std=c++17", "-ffp-contract=off", "-march=x86-64-v3",
                           "-I", os.path.join(ROOT, "knet.jl_b200", "csrc"),
                           os.path.join(ROOT, "tests", "exp64_check.cpp"), "-o", exe, "-l:libquadmath.so.0"])
    n = int(os.environ.get("KNET_EXP64_CHECK_N", "1500000"))
    out = subprocess.run([exe, str(n), "7"], capture_output=True, text=True)
    assert out.returncode == 0, out.stdout[-2000:]
    words = out.stdout.split()
    assert int(words[words.index("mismatches") + 1]) == 0
    slow = int(words[words.index("slow") + 1])
    assert 0 < slow < n // 200          # the second evaluation is taken, and rarely
