"""Index arithmetic of the lane-group kernels and the tiling rules of the rows kernels, checked on the
CPU: tests/geometry_check.cu includes the kernels' own header (knet.jl_b200/csrc/reduce.cuh) and walks
kn::group_geometry / kn::rows_geometry over run lengths, alignments and matrix shapes."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_group_walk_covers_every_run_once_and_row_tiles_cover_the_rows(tmp_path):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("no nvcc")
    exe = str(tmp_path / "geometry_check")
    subprocess.check_call([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-O1",
                           "-I", os.path.join(ROOT, "include"), "-I", os.path.join(ROOT, "knet.jl_b200", "csrc"),
                           os.path.join(ROOT, "tests", "geometry_check.cu"), "-o", exe])
    out = subprocess.run([exe], capture_output=True, text=True)
    assert out.returncode == 0, out.stdout[-2000:]
    words = out.stdout.split()
    assert int(words[words.index("cases") + 1]) > 30000 and int(words[words.index("bad") + 1]) == 0
