"""The benchmark configurations' own shapes against the oracle (not only by properties).

Broadcast `.+ .* ./` on (N,1) (+) (N,M) and (1,M) (+) (N,M) for N in {64,1024,8192}, M in
{128,4096,65536} (both operand orders): bit-identical to the same IEEE operation on the host.
Reductions (sum, maximum, logsumexp over dims 1 and 2), softmax / logsoftmax forward and
backward and nll on C x B logits for C in {10,1000,50257}, B in {64,512,4096}, Float32: the
bars of test_gpu_softmax_nll.py and test_gpu_broadcast_reduce.py (1e-5 relative; sums relative
to the sum of magnitudes; maxima, label gathers and counts exact).  The four activations
forward and backward at 2^28 elements in both precisions: relu and all backward forms
bit-identical, Float32 sigm/tanh/elu within 1 ulp, Float64 sigm/elu bit-identical, tanh 1 ulp.

The oracle's loops run on all host cores here (its OpenMP build: every output is still computed
by one thread in the same order, so the values are those of the serial build)."""
import numpy as np
import pytest
import torch

from test_gpu_broadcast_reduce import _check_reduce
from test_gpu_softmax_nll import _fwd_bwd, close, f64, tol
from ulps import ulp_diff

pytestmark = pytest.mark.gpu


@pytest.fixture
def komp(ko):
    ko.use_openmp(ko.have_openmp())
    yield ko
    ko.use_openmp(False)


def _host(t, shape):
    return t.cpu().numpy().reshape(shape, order="F")


@pytest.mark.parametrize("N", [64, 1024, 8192])
@pytest.mark.parametrize("M", [128, 4096, 65536])
def test_broadcast_config_shapes_are_bit_exact(K, N, M):
    g = torch.Generator(device="cuda").manual_seed(N + M)
    big = K.KnetArray(torch.randn(N * M, device="cuda", generator=g) + 3.0, (N, M))      # divisors away from 0
    col = K.KnetArray(torch.randn(N, device="cuda", generator=g) + 3.0, (N, 1))
    row = K.KnetArray(torch.randn(M, device="cuda", generator=g) + 3.0, (1, M))
    hb = _host(big.data, (N, M))
    fn = {"add": np.add, "mul": np.multiply, "div": np.divide}
    for v in (col, row):
        hv = _host(v.data, v.shape)
        for op in ("add", "mul", "div"):
            for a, b, ha, hbb in ((v, big, hv, hb), (big, v, hb, hv)):
                z = K.ops.broadcast(op, a, b)
                assert z.shape == (N, M)
                got = _host(z.data, (N, M))
                del z
                want = fn[op](ha, hbb)
                assert np.array_equal(got, want), (op, a.shape, b.shape)
                del got, want


@pytest.mark.parametrize("C_", [10, 1000, 50257])
@pytest.mark.parametrize("B_", [64, 512, 4096])
def test_softmax_family_config_shapes(K, komp, C_, B_):
    _fwd_bwd(K, komp, torch.float32, (C_, B_), 1)


@pytest.mark.parametrize("C_", [10, 1000, 50257])
@pytest.mark.parametrize("B_", [64, 512, 4096])
def test_reductions_and_nll_config_shapes(K, komp, C_, B_):
    ko = komp
    rng = np.random.default_rng(C_ + B_)
    x = np.asfortranarray((rng.standard_normal((C_, B_), dtype=np.float32) * 3))
    kx = K.KnetArray(x)
    for dims in (1, 2):
        _check_reduce(K, ko, x, dims, torch.float32, ops=("sum", "maximum") if x.size > (1 << 24) else None)
        lse = K.logsumexp(kx, dims)
        close(lse.numpy(), ko.logsumexp(f64(x), dims), torch.float32, log_domain=True)
        close(lse.numpy(), ko.logsumexp(x, dims), torch.float32, log_domain=True, n=x.shape[dims - 1])
    labels = rng.integers(1, C_ + 1, B_)
    labels[rng.random(B_) < 0.1] = 0
    tot, cnt = K.nll(kx, labels, dims=1, average=False)
    w_tot, w_cnt = ko.nll(x, labels, dims=1, average=False)
    assert cnt == w_cnt == int((labels != 0).sum())
    t64 = float(ko.nll(f64(x), labels, dims=1, average=False)[0])
    assert abs(tot - t64) <= tol(torch.float32) * max(abs(t64), 1e-30)
    assert abs(tot - float(w_tot)) <= tol(torch.float32, B_) * max(abs(t64), 1e-30)
    g = K.ops.nll_back(kx, labels, dims=1).numpy()
    w = ko.nll_bwd(x, labels, dims=1)
    scale = (np.abs(w) + 1.0 / max(cnt, 1))
    assert np.all(np.abs(g - w) <= tol(torch.float32, C_) * scale)
    np.testing.assert_array_equal(g[:, labels == 0], 0)
    assert K.accuracy(kx, labels, dims=1, average=False) == ko.accuracy(x, labels, dims=1, average=False)
    np.testing.assert_array_equal(K.ops.argmax(kx, 1).cpu().numpy().reshape(-1), ko.argmax(x, 1).reshape(-1))


@pytest.mark.parametrize("S", ["32", "64"])
def test_activations_at_2_28_elements(K, komp, S):
    ko = komp
    n = 1 << 28
    dt, tdt = (np.float32, torch.float32) if S == "32" else (np.float64, torch.float64)
    g = torch.Generator(device="cuda").manual_seed(28)
    xd = torch.randn(n, device="cuda", dtype=tdt, generator=g)
    dyd = torch.randn(n, device="cuda", dtype=tdt, generator=g)
    yd = torch.empty_like(xd)
    dxd = torch.empty_like(xd)
    x, dy = xd.cpu().numpy(), dyd.cpu().numpy()
    for op in ("relu", "sigm", "tanh", "elu"):
        K.knet8(f"{op}_{S}", n, K.lib.ptr(xd), K.lib.ptr(yd))
        got, want = yd.cpu().numpy(), ko.unary(op, x)
        if op == "relu" or (S == "64" and op in ("sigm", "elu")):
            assert np.array_equal(got, want), op
        elif op == "elu":
            bad = got != want                      # 1 ulp of exp(x), the number rounded before the subtraction
            assert bad.sum() <= 64 and np.all(np.abs(got[bad] - want[bad]) <= np.spacing(np.exp(x[bad])))
        else:
            bad = got != want
            assert ulp_diff(got[bad], want[bad]).max(initial=0) <= 1, op
        # backward from the oracle's forward value, so that only the backward kernel differs
        yd.copy_(torch.from_numpy(want))
        K.knet8(f"{op}back_{S}_11", n, K.lib.ptr(dyd), K.lib.ptr(yd), K.lib.ptr(dxd))
        assert np.array_equal(dxd.cpu().numpy(), ko.actback(f"{op}back", dy, want)), op + "back"
        del got, want
