"""Parity of softmax / logsoftmax / logsumexp / nll / argmax / accuracy with the oracle.

Tolerance: relative 1e-5 for Float32 (1e-12 for Float64) on probabilities, sums and losses;
log-domain outputs are compared with the same figure as an absolute error scaled by
max(1, |value|).  Label gathers, skipped instances, argmax positions and accuracy counts are
integer work and must be exact.  The shapes walk every kernel path: one thread, one warp,
one CTA with the run staged in shared memory, a cluster of CTAs exchanging through
distributed shared memory, the streamed fallback for runs beyond 8 slices, and the
rows layout (dims=2) with and without a cluster split."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

NPDT = {torch.float32: np.float32, torch.float64: np.float64}


def tol(dtype, n=1):
    """1e-5 (Float32) plus the error bound of the oracle's own sequential sum of n terms in
    the array's precision (n*eps/2); n = 1 when the reference value was computed in Float64."""
    if dtype == torch.float32:
        return 1e-5 + 0.5 * n * np.finfo(np.float32).eps * (n > 1)
    return 1e-12 + 0.5 * n * np.finfo(np.float64).eps * (n > 1)


def close(got, want, dtype, log_domain=False, n=1):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    scale = np.maximum(1.0, np.abs(want)) if log_domain else np.abs(want)
    bad = np.abs(got - want) > tol(dtype, n) * scale + (0 if log_domain else 1e-30)
    assert not bad.any(), (np.abs(got - want).max(), int(bad.sum()))


def f64(a):
    return np.asfortranarray(np.asarray(a, dtype=np.float64))


def logits(shape, dt, seed):
    return np.asfortranarray((np.random.default_rng(seed).standard_normal(shape) * 3).astype(dt))


# (C, B): classes along dim 1
SHAPES1 = [(1, 5), (3, 4), (10, 64), (10, 4096), (33, 100), (1000, 64), (1000, 512), (2048, 300), (2049, 5),
           (5000, 7), (16384, 3), (16385, 3), (50257, 8), (50257, 70), (140001, 2), (5, 1),
           # staged kernels with 13 and 16 register-resident packs per thread (clusters of 4 and of 8)
           (50257, 80), (120000, 3), (60000, 4),
           # one CTA per run with 32 KB slices: the 512-thread backward kernel with 4 packs per thread
           (8192, 300),
           # Float32 runs held in registers by 8, 16 or 32 lanes (2 to 16 packs per lane); odd lengths
           # make the runs start at every offset inside a 16-byte line, and the instance counts leave
           # groups without an instance in the last CTA
           (37, 300), (64, 301), (100, 300), (129, 150), (256, 150), (515, 300), (1001, 200), (1021, 150),
           (1024, 150), (2047, 160)]
# dims = 2 on (R, K): rows layout
SHAPES2 = [(4, 3), (64, 10), (100, 33), (4096, 10), (512, 1000), (31, 5000), (7, 50257), (1, 9),
           # row vectors of 16 bytes (one round in registers; a cluster of 2; several rounds), of 8 bytes
           # (rows not a multiple of 4), single elements (odd row count)
           (8192, 40), (6000, 300), (4800, 3000), (4098, 600), (5001, 64)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("shape", SHAPES1, ids=str)
def test_dims1_forward_backward(K, ko, dtype, shape):
    _fwd_bwd(K, ko, dtype, shape, 1)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("shape", SHAPES2, ids=str)
def test_dims2_forward_backward(K, ko, dtype, shape):
    _fwd_bwd(K, ko, dtype, shape, 2)


def _fwd_bwd(K, ko, dtype, shape, dims):
    dt = NPDT[dtype]
    x = logits(shape, dt, 1)
    dy = np.asfortranarray(np.random.default_rng(2).standard_normal(shape).astype(dt))
    kx, kdy = K.KnetArray(x), K.KnetArray(dy)
    D = shape[dims - 1]
    sm, lsm = K.softmax(kx, dims), K.logsoftmax(kx, dims)
    w_sm, w_lsm = ko.softmax(x, dims), ko.logsoftmax(x, dims)
    x64 = f64(x)
    close(sm.numpy(), ko.softmax(x64, dims), dtype)                      # against the Float64 evaluation
    close(lsm.numpy(), ko.logsoftmax(x64, dims), dtype, log_domain=True)
    close(sm.numpy(), w_sm, dtype, n=D)                                  # against the Float32 oracle
    close(lsm.numpy(), w_lsm, dtype, log_domain=True, n=D)
    close(K.ops.sum(sm, dims).numpy(), 1.0, dtype)                       # test/loss.jl:50
    lse = K.logsumexp(kx, dims)
    w_lse = ko.logsumexp(x, dims)
    assert lse.shape == w_lse.shape
    close(lse.numpy(), ko.logsumexp(x64, dims), dtype, log_domain=True)
    del x64
    close(lse.numpy(), w_lse, dtype, log_domain=True, n=D)
    # backward from the oracle's forward values, so that only the backward kernels differ
    ky, kly = K.KnetArray(w_sm), K.KnetArray(w_lsm)
    g1, w1 = K.ops.softmax_back(ky, kdy, dims).numpy(), ko.softmax_bwd(w_sm, dy, dims)
    scale1 = np.abs(w_sm * dy) + np.abs(w_sm) * np.abs(ko.reduce_dim("sum", np.abs(w_sm * dy), dims))
    assert np.all(np.abs(g1 - w1) <= tol(dtype, D) * scale1 + 1e-30)
    g2, w2 = K.ops.logsoftmax_back(kly, kdy, dims).numpy(), ko.logsoftmax_bwd(w_lsm, dy, dims)
    scale2 = np.abs(dy) + np.exp(w_lsm) * ko.reduce_dim("sum", np.abs(dy), dims)
    assert np.all(np.abs(g2 - w2) <= tol(dtype, D) * scale2)
    red = list(shape)
    red[dims - 1] = 1
    dyr = np.asfortranarray(np.random.default_rng(3).standard_normal(red).astype(dt))
    g3 = K.ops.logsumexp_back(kx, K.KnetArray(w_lse), K.KnetArray(dyr), dims).numpy()
    close(g3, ko.logsumexp_bwd(x, w_lse, dyr, dims), dtype, n=2)
    # in place: y may be x, dx may be dy
    y_inplace = kx.copy()
    K.knet(f"knet_softmax_fwd_{K.lib.sfx(dtype)}", K.lib.ptr(y_inplace.data), K.lib.ptr(y_inplace.data),
           *K.ops._geometry(shape, dims))
    np.testing.assert_array_equal(y_inplace.numpy(), sm.numpy())


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("shape,dims", [((10, 100), 1), ((3, 2), 1), ((1000, 64), 1), ((5000, 9), 1), ((50257, 6), 1),
                                        ((1000, 300), 1), ((1001, 200), 1), ((2047, 160), 1), ((130, 400), 1),
                                        ((100, 10), 2), ((9, 5000), 2), ((4096, 1000), 2), ((8192, 40), 2), ((4800, 3000), 2),
                                        ((5001, 64), 2)], ids=str)
def test_nll_forward_backward_accuracy(K, ko, dtype, shape, dims):
    dt = NPDT[dtype]
    x = logits(shape, dt, 4)
    ninst, ncls = (shape[1], shape[0]) if dims == 1 else (shape[0], shape[1])
    rng = np.random.default_rng(5)
    labels = rng.integers(1, ncls + 1, ninst)
    labels[rng.random(ninst) < 0.2] = 0                                   # skipped instances
    if ninst > 1:
        labels[0], labels[1] = 0, ncls
    kx = K.KnetArray(x)
    tot, cnt = K.nll(kx, labels, dims=dims, average=False)
    w_tot, w_cnt = ko.nll(x, labels, dims=dims, average=False)
    assert cnt == w_cnt == int((labels != 0).sum())
    t64 = float(ko.nll(f64(x), labels, dims=dims, average=False)[0])
    assert abs(tot - t64) <= tol(dtype) * max(abs(t64), 1e-30)
    assert abs(tot - float(w_tot)) <= tol(dtype, ncls) * max(abs(float(w_tot)), 1e-30)
    if cnt:
        assert K.nll(kx, labels, dims=dims) == pytest.approx(t64 / cnt, rel=tol(dtype))
    # per-instance values: the label gather is exact index work
    res = K.ops.nll_device(kx, labels, dims)
    lsm = ko.logsoftmax(x, dims)
    per = res.per_instance.cpu().numpy()[:ninst]
    for j in range(min(ninst, 50)):
        want = 0.0 if labels[j] == 0 else -(lsm[labels[j] - 1, j] if dims == 1 else lsm[j, labels[j] - 1])
        assert abs(per[j] - want) <= tol(dtype, ncls) * max(1.0, abs(want)), j
    if cnt:
        for average in (True, False):
            g = K.ops.nll_back(kx, labels, dims=dims, average=average, dy=1.5).numpy()
            w = ko.nll_bwd(x, labels, dims=dims, average=average, dy=1.5)
            p = ko.softmax(x, dims) * (1.5 / (w_cnt if average else 1))
            assert np.all(np.abs(g - w) <= tol(dtype, ncls) * (np.abs(p) + np.abs(w)) + 1e-30)
            skipped = labels == 0
            sel = g[:, skipped] if dims == 1 else g[skipped, :]
            assert not sel.any()                                          # exact zeros on skipped instances
    # argmax / accuracy: exact integers, first maximum wins
    x2 = x.copy(order="F")
    if dims == 1:
        x2[:, ::3] = np.round(x2[:, ::3])                                 # many ties
    else:
        x2[::3, :] = np.round(x2[::3, :])
    k2 = K.KnetArray(x2)
    np.testing.assert_array_equal(K.argmax(k2, dims).cpu().numpy(), ko.argmax(x2, dims).reshape(-1))
    assert K.accuracy(k2, labels, dims=dims, average=False) == ko.accuracy(x2, labels, dims=dims, average=False)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("shape,dims", [((10, 100000), 1), ((40, 40000), 1), ((20000, 12), 2), ((64, 16385), 1)], ids=str)
def test_nll_total_over_many_instances(K, ko, dtype, shape, dims):
    """Beyond 16384 instances the final sum of the per-instance losses is split over the CTAs of a
    cluster (2, 4 or 8): total and count against the Float64 oracle, and the same bits on a second call."""
    dt = NPDT[dtype]
    x = logits(shape, dt, 14)
    ninst, ncls = (shape[1], shape[0]) if dims == 1 else (shape[0], shape[1])
    rng = np.random.default_rng(15)
    labels = rng.integers(1, ncls + 1, ninst)
    labels[rng.random(ninst) < 0.3] = 0
    labels[-1] = ncls                                                       # the last slice's last instance counts
    kx = K.KnetArray(x)
    tot, cnt = K.nll(kx, labels, dims=dims, average=False)
    t64, c64 = ko.nll(f64(x), labels, dims=dims, average=False)
    assert cnt == c64 == int((labels != 0).sum())
    assert abs(tot - float(t64)) <= tol(dtype) * abs(float(t64))
    again = K.nll(kx, labels, dims=dims, average=False)
    assert again == (tot, cnt)


def test_accuracy_identity_of_the_reference_test(K):
    # test/ops20.jl:120-123
    rng = np.random.default_rng(0)
    scores = np.asfortranarray(rng.standard_normal((10, 100)).astype(np.float32))
    labels1, labels2 = rng.integers(1, 11, 100), rng.integers(1, 101, 10)
    scores[0, :] += 1000
    assert K.accuracy(K.KnetArray(scores), labels1, dims=1) == np.sum(labels1 == 1) / 100
    scores[:, 0] += 10000
    assert K.accuracy(K.KnetArray(scores), labels2, dims=2) == np.sum(labels2 == 1) / 10


def test_three_dimensional_dims_and_generic_fallback(K, ko):
    # test/loss.jl:47-56: dims = 1, 2, 3, (1,2), (1,3), [2,3], [1,2,3]
    a = np.asfortranarray(np.random.default_rng(1).random((10, 10, 10)).astype(np.float32))
    ka = K.KnetArray(a)
    for d in (1, 2, 3):
        close(K.softmax(ka, d).numpy(), ko.softmax(a, d), torch.float32)
        close(K.logsumexp(ka, d).numpy(), ko.logsumexp(a, d), torch.float32, log_domain=True)
    for d in ((1, 2), (2, 3), (1, 3), (1, 2, 3), None):
        sm, lsm = K.softmax(ka, d).numpy(), K.logsoftmax(ka, d).numpy()
        np.testing.assert_allclose(sm, np.exp(lsm), rtol=1e-5)
        axes = tuple(range(3)) if d is None else tuple(i - 1 for i in d)
        np.testing.assert_allclose(sm.sum(axis=axes), 1.0, rtol=1e-5)
        np.testing.assert_allclose(K.logsumexp(ka, d).numpy().reshape(-1),
                                   np.log(np.exp(a.astype(np.float64)).sum(axis=axes)).reshape(-1), rtol=1e-5)


def test_full_size_softmax_properties(K):
    # logits 50257 x 4096 Float32 (823 MB): probabilities sum to 1 per instance, softmax equals
    # exp(logsoftmax), logsumexp is shift-invariant; fused nll equals the gather of logsoftmax
    C_, B_ = 50257, 4096
    g = torch.Generator(device="cuda").manual_seed(3)
    x = K.KnetArray(torch.randn(C_ * B_, device="cuda", generator=g) * 3, (C_, B_))
    sm = K.softmax(x, 1)
    s = K.ops.sum(sm, 1).data
    assert float((s - 1).abs().max()) <= 1e-5
    lsm = K.logsoftmax(x, 1)
    assert float((sm.data - torch.exp(lsm.data)).abs().max()) <= 1e-6
    lse = K.logsumexp(x, 1).data
    ref = torch.logsumexp(x.data.view(B_, C_), dim=1)
    assert float((lse - ref).abs().max()) <= 1e-5 * float(ref.abs().max())
    labels = torch.randint(1, C_ + 1, (B_,), device="cuda", dtype=torch.int32)
    tot, cnt = K.nll(x, labels, dims=1, average=False)
    picked = lsm.data.view(B_, C_).gather(1, (labels.long() - 1).view(-1, 1)).double().sum()
    assert cnt == B_ and abs(tot + float(picked)) <= 1e-5 * abs(float(picked))
    del sm
    dx = K.ops.nll_back(x, labels, dims=1)
    colsum = K.ops.sum(dx, 1).data
    assert float(colsum.abs().max()) <= 1e-5 / B_ * 4                      # (softmax - onehot) sums to 0
    assert K.libknet.knet_device_status() == 0                             # no bounded wait gave up


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("shape", [(10, 64), (1000, 64), (61, 333), (1000, 200), (1001, 200), (5000, 7), (50257, 8), (50257, 80),
                                   (140001, 2)], ids=str)
@pytest.mark.parametrize("offs", [(1, 1, 1), (1, 2, 3), (0, 1, 0)], ids=str)
def test_pointers_off_the_16_byte_grid(K, ko, dtype, shape, offs):
    """KnetArray views hand the kernels pointers aligned to the element size only.  Inputs and
    outputs shifted by different element counts (so that they do not share an offset inside a
    16-byte line) walk the scalar-store and shared-memory fallback paths of the staged
    kernels; the neighbours of every output range must stay untouched."""
    dt, S = NPDT[dtype], K.lib.sfx(dtype)
    knet, ptr = K.knet, K.lib.ptr
    C_, B_ = shape
    n = C_ * B_
    x = logits(shape, dt, 5)
    dy = np.asfortranarray(np.random.default_rng(6).standard_normal(shape).astype(dt))

    def shifted(a, k):
        t = torch.full((a.size + k + 8,), 777.0, dtype=dtype, device="cuda")
        t[k:k + a.size].copy_(torch.from_numpy(np.ascontiguousarray(a.reshape(-1, order="F"))))
        return t, t[k:k + a.size]

    ox, oy, oz = offs
    xb, xv = shifted(x, ox)
    for f, want, log_domain in (("softmax", ko.softmax(f64(x), 1), False), ("logsoftmax", ko.logsoftmax(f64(x), 1), True)):
        yb, yv = shifted(np.zeros(shape, dt), oy)
        knet(f"knet_{f}_fwd_{S}", ptr(xv), ptr(yv), 1, C_, B_)
        close(yv.cpu().numpy().reshape(shape, order="F"), want, dtype, log_domain=log_domain)
        assert float(yb[:oy].sum()) == 777.0 * oy and bool((yb[oy + n:] == 777.0).all())
        # backward from the oracle's forward values
        w = np.asfortranarray(want.astype(dt))
        wb, wv = shifted(w, ox)
        gb, gv = shifted(dy, oy)
        db, dv = shifted(np.zeros(shape, dt), oz)
        knet(f"knet_{f}_bwd_{S}", ptr(wv), ptr(gv), ptr(dv), 1, C_, B_)
        ref = (ko.softmax_bwd if f == "softmax" else ko.logsoftmax_bwd)(f64(w), f64(dy), 1)
        scale = np.abs(dy) * (np.abs(w) if f == "softmax" else 1.0) + \
            (np.abs(w) if f == "softmax" else np.exp(w)) * ko.reduce_dim("sum", np.abs(f64(w) * f64(dy)) if f == "softmax" else np.abs(f64(dy)), 1)
        got = dv.cpu().numpy().reshape(shape, order="F").astype(np.float64)
        assert np.all(np.abs(got - ref) <= tol(dtype, C_) * scale + 1e-30)
        assert float(db[:oz].sum()) == 777.0 * oz and bool((db[oz + n:] == 777.0).all())


@pytest.mark.parametrize("shape,reps", [((50257, 80), 200), ((16384, 3), 300), ((8192, 300), 200)], ids=str)
def test_staged_kernels_repeat_bit_for_bit(K, shape, reps):
    """The staged kernels exchange partial results between the CTAs of a cluster through
    shared-memory barriers; their merge order is fixed, so repeated launches on the same data
    must agree bit for bit, and no bounded wait may have given up."""
    knet, ptr = K.knet, K.lib.ptr
    C_, B_ = shape
    x = torch.randn(C_ * B_, device="cuda") * 3
    dy = torch.randn(C_ * B_, device="cuda")
    y0, d0 = torch.empty_like(x), torch.empty_like(x)
    knet("knet_logsoftmax_fwd_32", ptr(x), ptr(y0), 1, C_, B_)
    knet("knet_logsoftmax_bwd_32", ptr(y0), ptr(dy), ptr(d0), 1, C_, B_)
    y, d = torch.empty_like(x), torch.empty_like(x)
    for _ in range(reps):
        y.fill_(7.0)
        d.fill_(7.0)
        knet("knet_logsoftmax_fwd_32", ptr(x), ptr(y), 1, C_, B_)
        knet("knet_logsoftmax_bwd_32", ptr(y), ptr(dy), ptr(d), 1, C_, B_)
        assert torch.equal(y, y0) and torch.equal(d, d0)
    assert K.libknet.knet_device_status() == 0
