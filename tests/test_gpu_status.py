"""The bounded waits of the staged kernels and the status path that reports one that gave up.

No kernel is made to hang or fault: the probe kernel announces more bytes on an mbarrier than it
copies, its wait runs out after a few thousand polls, it balances the barrier itself and returns."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_a_wait_that_runs_out_is_reported_once_and_the_context_stays_usable(K):
    lib = K.lib.libknet
    assert lib.knet_device_status() == 0
    out = torch.zeros(6, dtype=torch.int32, device="cuda")
    K.knet("knet_debug_wait_probe", 4000, K.lib.ptr(out))
    torch.cuda.synchronize()
    assert out.tolist() == [1, 1, 11, 22, 33, 44]      # first wait gave up, second completed, the copy landed
    assert lib.knet_device_status() == 1               # reported ...
    assert lib.knet_device_status() == 0               # ... once
    # the context is intact: staged kernels of both translation units still run and report nothing
    x = K.KnetArray(torch.randn(50257 * 8, device="cuda"), (50257, 8))
    y = K.softmax(x, 1)
    assert abs(float(K.ops.sum(y)) - 8.0) < 1e-3
    rows = torch.randint(1, 1025, (512,), device="cuda", dtype=torch.int32)
    xm = torch.randn(1024 * 600, device="cuda")
    ym = torch.empty(512 * 600, device="cuda")
    K.knet8("getrows_32", 1024, 600, 512, K.lib.ptr(rows), K.lib.ptr(xm), K.lib.ptr(ym))
    want = xm.view(600, 1024)[:, (rows - 1).long()]
    assert torch.equal(ym.view(600, 512), want)
    assert lib.knet_device_status() == 0
    assert lib.knet_debug_wait_probe(0, K.lib.ptr(out), None) == -1
    assert lib.knet_debug_wait_probe(4000, None, None) == -1
