"""knet_gemm_S_S (the cuBLAS call behind `*`, A_mul_Bt and At_mul_B, src/knetarrays/linalg.jl:
11-55) against Float64 products, in plain FP32 and, where the process can load a cuBLAS that
offers it, in the FP32 emulation on the BF16 tensor cores.

Tolerances, stated per entry against sum_k |a_ik| |b_kj|: plain FP32 within 64 * 2^-24 (it
accumulates in Float32 over k <= 2048 terms; the observed figure is a few 2^-24); the emulation
must not be worse than twice the plain figure on the same inputs, nor than 8 * 2^-24.  The
checks run in child processes (tests/gemm_check.py) because the cuBLAS copy is chosen when the
process starts."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EPS = 2.0 ** -24
# a CUDA toolkit's own cuBLAS, when the image has one (PyTorch's bundled copy may be older)
TOOLKIT_CUBLAS = os.environ.get("KNET_SM100_TEST_CUBLAS_DIR", "/usr/local/cuda/lib64")


def run_check(extra_env, *args):
    env = dict(os.environ, **extra_env)
    r = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "gemm_check.py"), *args],
                       capture_output=True, text=True, timeout=900, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    return json.loads([l for l in r.stdout.splitlines() if l.startswith("{")][-1])


def emulation_env():
    if not os.path.exists(os.path.join(TOOLKIT_CUBLAS, "libcublas.so.12")):
        pytest.skip("no toolkit cuBLAS to load")
    return {"KNET_SM100_CUBLAS_DIR": TOOLKIT_CUBLAS, "KNET_SM100_GEMM": "emulated"}


def test_plain_fp32_and_fp64_products(K):
    rep = run_check({"KNET_SM100_GEMM": "native"})
    assert rep["gemm_mode"] == "native" and rep["version"] >= 120000
    for case in rep["cases"]:
        assert case["mode0"] <= 64 * EPS, case
        assert case["mode0"] <= 4 * case["torch"] + 2 * EPS, case      # the same library call as torch.mm makes
    assert rep["f64"] <= 1e-14
    assert rep["wrappers"] <= 64 * EPS
    assert rep["argument_errors"] == [-1, -1, -1, -1]


def test_emulated_fp32_products_are_no_less_accurate(K):
    rep = run_check(emulation_env())
    if not rep["emulation"]:
        pytest.skip(f"cuBLAS {rep['version']} in the process does not offer the emulation")
    assert rep["gemm_mode"] == "emulated"
    for case in rep["cases"]:
        for mode in ("mode1", "mode2"):
            assert case[mode] <= max(2 * case["mode0"], 2 * EPS), case
            assert case[mode] <= 8 * EPS, case
    assert rep["wrappers"] <= 64 * EPS
    assert rep["argument_errors"] == [-1, -1, -1, -1]


def test_older_cublas_refuses_the_emulation(K):
    # in this process PyTorch's own cuBLAS is loaded; when it predates 12.9 the emulated modes
    # must answer "not offered" (-8) and leave the handle usable
    import torch
    from knet_sm100 import ops
    g = ops.gemm_handle()
    if g.emulation:
        pytest.skip("this cuBLAS offers the emulation")
    a = torch.ones(16, device="cuda")
    z = torch.zeros(16, device="cuda")
    with pytest.raises(K.KnetError, match="status -8"):
        ops.gemm_(0, 0, 4, 4, 4, a, 4, a, 4, z, 4, mode=1)
    ops.gemm_(0, 0, 4, 4, 4, a, 4, a, 4, z, 4, mode=0)
    assert torch.equal(z, torch.full((16,), 4.0, device="cuda"))


@pytest.mark.parametrize("mode", ["native", "emulated"])
def test_loss_curve_with_library_products(K, mode):
    env = {"KNET_SM100_GEMM": "native"} if mode == "native" else emulation_env()
    rep = run_check(env, "--curve")
    if mode == "emulated" and not rep["emulation"]:
        pytest.skip(f"cuBLAS {rep['version']} in the process does not offer the emulation")
    assert rep["gemm_mode"] == mode
    assert rep["worst"] <= 1e-4 and rep["last"] < 2.0, rep
