"""The 64-bit index paths, which only sizes beyond 2^31 elements (or 16-byte vectors) reach:
the Philox kernels and the column gather.  Checked through properties that do not need a
second array of that size: a small call placed at the same counters, sampled columns."""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_gb():
    free, _ = torch.cuda.mem_get_info()
    return free / 2**30


def test_philox_beyond_2_31_elements_matches_small_calls_at_the_same_counters(K):
    if _free_gb() < 24:
        pytest.skip("needs 24 GB of free device memory")
    knet, ptr = K.lib.knet, K.lib.ptr
    n = (1 << 31) + 4096 + 3                       # ragged end, 64-bit index path
    seed, offset = 77, 5
    u = torch.empty(n, dtype=torch.float32, device="cuda")
    knet("knet_dropout_uniform_32", n, seed, offset, ptr(u))
    for start in (0, (1 << 31) - 8, (1 << 31), n - 4099):
        start -= start % 8                          # one counter per 8 elements
        m = min(4096, n - start)
        small = torch.empty(m, dtype=torch.float32, device="cuda")
        knet("knet_dropout_uniform_32", m, seed, offset + start // 8, ptr(small))
        assert torch.equal(u[start:start + m], small)
    assert float(u.min()) >= 0.0 and float(u.max()) < 1.0
    x = torch.ones(n, dtype=torch.float32, device="cuda")
    knet("knet_dropout_philox_32", n, C.c_float(0.25), seed, offset, ptr(x), ptr(x))       # in place
    kept = u > 0.25
    assert torch.equal(x != 0, kept)
    assert float(x.max()) == np.float32(1.0) / np.float32(0.75)
    del u, x, kept


def test_getcols_beyond_2_31_vectors(K):
    if _free_gb() < 44:
        pytest.skip("needs 44 GB of free device memory")
    knet8, ptr = K.lib.knet8, K.lib.ptr
    E, V, n = 4096, 64, (1 << 21) + 1               # E/4 * n = 2^31 + 1024 vectors of 16 bytes
    x = torch.randn(E * V, device="cuda")
    idx = torch.randint(1, V + 1, (n,), device="cuda", dtype=torch.int32)
    y = torch.empty(E * n, device="cuda")
    knet8("getcols_32", E, V, n, ptr(idx), ptr(x), ptr(y))
    X, Y = x.view(V, E), y.view(n, E)
    pick = torch.cat([torch.arange(0, 64, device="cuda"), torch.randint(0, n, (4096,), device="cuda"),
                      torch.arange(n - 64, n, device="cuda")])
    assert torch.equal(Y[pick], X[(idx[pick] - 1).long()])
    # every column: its sum equals the sum of the column it was copied from
    sums = X.double().sum(dim=1)
    for c0 in range(0, n, 1 << 18):
        c1 = min(n, c0 + (1 << 18))
        assert torch.equal(Y[c0:c1].double().sum(dim=1), sums[(idx[c0:c1] - 1).long()])
    del x, y, idx
