"""The reduction entry point for hosts that may not allocate device memory.

Some users of the library sit inside a runtime that already owns all GPU memory through its
own pool, or run a loop that must not touch the allocator once it has started; they can pass
inputs and outputs but no workspace, and the library must not ask the driver for one.
knet_reduce_noalloc_32 keeps its partial results in an array inside the library image
instead.  It has to give exactly what knet_reduce_32 gives with a caller-supplied workspace
(same kernels, same merge order: bit-identical), on repeated calls, whether this file runs
alone in a fresh process or after every other test."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_noalloc_reduction_matches_the_workspace_form_twice(K):
    lib, ptr = K.libknet, K.lib.ptr
    ws = torch.empty(lib.knet_reduce_workspace_bytes(), dtype=torch.uint8, device="cuda")
    want = torch.empty(1, dtype=torch.float32, device="cuda")
    got = torch.full((1,), float("nan"), dtype=torch.float32, device="cuda")
    rng = np.random.default_rng(21)
    stream = K.lib.stream_ptr()
    for call, n in enumerate((3_000_001, 70_003)):          # two calls in a row, different sizes
        x = torch.from_numpy(rng.standard_normal(n + 1).astype(np.float32)).cuda()
        for op in (0, 2, 5):                                 # sum, maximum, sumabs2
            xs = x[1:]                                       # element-offset pointer, like a view
            assert lib.knet_reduce_32(op, n, ptr(xs), ptr(want), ptr(ws), ws.numel(), stream) == 0
            got.fill_(float("nan"))
            assert lib.knet_reduce_noalloc_32(op, n, ptr(xs), ptr(got), stream) == 0
            torch.cuda.synchronize()
            assert got.item() == want.item(), (call, op, got.item(), want.item())
        ref = float(x[1:].double().sum())
        lib.knet_reduce_noalloc_32(0, n, ptr(x[1:]), ptr(got), stream)
        assert abs(got.item() - ref) <= 1e-5 * float(x[1:].abs().double().sum())


def test_noalloc_reduction_rejects_bad_arguments(K):
    lib, ptr = K.libknet, K.lib.ptr
    x = torch.ones(16, device="cuda")
    out = torch.zeros(1, device="cuda")
    assert lib.knet_reduce_noalloc_32(0, 2**31, ptr(x), ptr(out), None) == -2      # beyond the stated maximum
    assert lib.knet_reduce_noalloc_32(0, -1, ptr(x), ptr(out), None) == -1
    assert lib.knet_reduce_noalloc_32(99, 16, ptr(x), ptr(out), None) == -1
    assert lib.knet_reduce_noalloc_32(0, 16, ptr(x), None, None) == -1
    assert lib.knet_reduce_noalloc_32(0, 16, ptr(x), ptr(out), None) == 0
    torch.cuda.synchronize()
    assert out.item() == 16.0
