"""Index kernels and KnetArray indexing against the NumPy index oracle: bit-exact, since the
kernels only move values (the scatter-adds are compared on integer-valued data, where every
summation order gives the same bits, and on random data within the order-dependent bound).

The index list is the reference's (test/karray.jl:24-41, 141-148): every supported kind is
read, zeroed, restored and differentiated."""
import ctypes as C

import numpy as np
import pytest
import torch

import index_oracle as io

pytestmark = pytest.mark.gpu

NPDT = {torch.float32: np.float32, torch.float64: np.float64}


def F(a):
    return np.asarray(a).reshape(-1, order="F")


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _cases_2d(X):
    C_, UR, SR, CI = X.COLON, X.UnitRange, X.StepRange, X.CartesianIndex
    return [
        (C_,), (C_, C_), (3,), (2, 3), (UR(3, 5),), (UR(1, 2), UR(3, 4)), (2, C_), (C_, 2), (UR(1, 2), C_),
        (C_, UR(1, 2)), (UR(1, 2), 2), (2, UR(1, 2)), (SR(1, 2, 3),), (SR(1, 2, 3), C_), (C_, SR(1, 2, 3)),
        ([1, 3],), ([2, 2],), ([1, 3], C_), (C_, [1, 3]), ([2, 2], C_), (C_, [2, 2]),
        (np.ones((3, 4), bool),), (np.array([[1, 3], [2, 4]]),), (CI(3),), (CI(2, 3),),
        (C_, np.ones(4, bool)), (np.ones(3, bool), C_), ([CI(2, 2), CI(2, 1)],),
        (C_, np.array([True, False, True, False])), (np.array([False, True, True]), C_),
        (np.asfortranarray(np.random.default_rng(0).random((3, 4)) > 0.5),),
    ]


def _repeats(I):
    for i in I:
        if isinstance(i, (list, np.ndarray)) and np.asarray(i).dtype.kind in "iu":
            a = np.asarray(i).reshape(-1)
            if len(np.unique(a)) != len(a):
                return True
    return False


@pytest.mark.parametrize("dtype", [torch.float64, torch.float32])
@pytest.mark.parametrize("k", range(31))
def test_reference_index_list_2d(K, dtype, k):
    X = K.indexing
    a = np.asfortranarray(np.random.default_rng(7).random((3, 4)).astype(NPDT[dtype]))
    I = _cases_2d(X)[k]
    kk = K.KnetArray(a)
    got, want = kk[I], io.getindex(a, *I)
    if isinstance(want, float):
        assert got == want
        kk[I] = 0
        assert np.array_equal(kk.numpy(), io.setindex(a, 0, *I))
        kk[I] = want
        assert np.array_equal(kk.numpy(), a)
        return
    assert got.shape == want.shape
    assert np.array_equal(got.numpy(), want)
    got = got.copy()                                   # contiguous ranges are views of kk
    kk[I] = 0
    assert np.array_equal(kk.numpy(), io.setindex(a, 0, *I))
    if not _repeats(I):
        kk[I] = got
        assert np.array_equal(kk.numpy(), a)
        kk[I] = 0
        kk[I] = want                                   # host array on the right-hand side
        assert np.array_equal(kk.numpy(), a)


def test_reference_index_list_3d(K):
    X = K.indexing
    C_, UR = X.COLON, X.UnitRange
    a = np.asfortranarray(np.random.default_rng(8).random((3, 4, 5)))
    for I in [(C_,), (C_, C_, C_), (3,), (2, 3, 4), (UR(3, 5),), (C_, C_, 2), (C_, C_, UR(1, 2)),
              (np.ones((3, 4, 5), bool),), (UR(2, 60),), (C_, C_, UR(2, 5))]:
        kk = K.KnetArray(a)
        got, want = kk[I], io.getindex(a, *I)
        if isinstance(want, float):
            assert got == want
            kk[I] = 0
        else:
            assert got.shape == want.shape and np.array_equal(got.numpy(), want)
            kk[I] = 0
        assert np.array_equal(kk.numpy(), io.setindex(a, 0, *I))
        kk[I] = want
        assert np.array_equal(kk.numpy(), a)


def test_errors_follow_the_reference(K):
    X = K.indexing
    kk = K.KnetArray(np.zeros((3, 4)))
    with pytest.raises(IndexError):
        kk[X.COLON, [5]]
    with pytest.raises(IndexError):
        kk[[0]]
    with pytest.raises(IndexError):
        kk[13]
    with pytest.raises(IndexError):
        kk[X.UnitRange(3, 13)]
    with pytest.raises(ValueError):
        kk[X.UnitRange(1, 4), X.COLON]
    with pytest.raises(ValueError):
        kk[X.COLON, [1, 2]] = np.zeros((3, 3))
    with pytest.raises(TypeError):
        kk[[1, 2], [1, 2]]
    assert kk[X.COLON, []].shape == (3, 0)


# (xrows, xcols, n).  getrows stages whole columns in shared memory when the picks are dense
# (n >= xrows/8), the column fits 48 KB and there are at least 16 columns; the last shapes sit on
# both sides of each of those limits
SHAPES = [(1, 5, 3), (3, 4, 2), (4, 9, 6), (6, 130, 77), (128, 300, 513), (513, 64, 200), (1024, 50, 4096),
          (8192, 40, 4096), (12288, 20, 2048), (12292, 20, 2048), (4096, 64, 100), (4096, 64, 512), (640, 15, 640),
          (2048, 700, 1000), (1024, 601, 515)]     # many columns: the double-buffered bulk-copy form


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("xrows,xcols,n", SHAPES)
@pytest.mark.parametrize("offset", [0, 1])
def test_cols_and_rows_kernels(K, dtype, xrows, xcols, n, offset):
    """Raw entry points, with base pointers off the 16-byte grid when offset=1."""
    dt, S = NPDT[dtype], K.lib.sfx(dtype)
    rng = np.random.default_rng(xrows * 31 + n)
    x = rng.integers(-64, 64, xrows * xcols).astype(dt)
    ct = C.c_float if dt == np.float32 else C.c_double
    k8, p = K.lib.knet8, K.lib.ptr

    def buf(a):
        t = torch.zeros(a.size + offset, dtype=dtype, device="cuda")
        t[offset:].copy_(dev(a))
        return t[offset:]

    for kind, count in (("col", xcols), ("row", xrows)):
        idx = rng.integers(1, count + 1, n).astype(np.int32)
        uniq = (rng.permutation(count)[:min(n, count)] + 1).astype(np.int32)
        idx_d, uniq_d = dev(idx), dev(uniq)             # named: they must outlive the launches
        ylen = lambda m: (xrows * m) if kind == "col" else (m * xcols)  # noqa: E731
        o = {f: getattr(io, f"{f}{kind}s") for f in ("get", "set", "add")}
        # get
        xd, yd = buf(x), buf(np.zeros(ylen(n), dt))
        k8(f"get{kind}s_{S}", xrows, xcols, n, p(idx_d), p(xd), p(yd))
        assert np.array_equal(yd.cpu().numpy(), o["get"](xrows, xcols, idx, x))
        # set (distinct indices)
        y = rng.integers(-64, 64, ylen(len(uniq))).astype(dt)
        xd, yd = buf(x), buf(y)
        k8(f"set{kind}s_{S}", xrows, xcols, len(uniq), p(uniq_d), p(xd), p(yd))
        assert np.array_equal(xd.cpu().numpy(), o["set"](xrows, xcols, uniq, x, y))
        # add (repeats; integer-valued data make the sums exact in any order)
        y = rng.integers(-64, 64, ylen(n)).astype(dt)
        xd, yd = buf(x), buf(y)
        k8(f"add{kind}s_{S}", xrows, xcols, n, p(idx_d), p(xd), p(yd))
        assert np.array_equal(xd.cpu().numpy(), o["add"](xrows, xcols, idx, x, y))
        # one scalar
        xd = buf(x)
        k8(f"set{kind}1_{S}", xrows, xcols, n, p(idx_d), p(xd), ct(2.5))
        assert np.array_equal(xd.cpu().numpy(), getattr(io, f"set{kind}1")(xrows, xcols, idx, x, 2.5))
    # nothing to do: no launch, no error
    xd = buf(x)
    k8(f"getcols_{S}", xrows, xcols, 0, None, p(xd), None)
    torch.cuda.synchronize()


def test_addcols_random_values_within_order_bound(K):
    """Float32 scatter-add of random values: the result depends on the order of the atomic
    adds, so compare with a Float64 accumulation within n_repeats * eps * sum|terms|."""
    rng = np.random.default_rng(11)
    xrows, xcols, n = 256, 1000, 20000
    x = rng.standard_normal((xrows, xcols)).astype(np.float32)
    y = rng.standard_normal((xrows, n)).astype(np.float32)
    idx = rng.integers(1, xcols + 1, n).astype(np.int32)
    xd, yd, idx_d = dev(F(x)), dev(F(y)), dev(idx)
    K.lib.knet8("addcols_32", xrows, xcols, n, K.lib.ptr(idx_d), K.lib.ptr(xd), K.lib.ptr(yd))
    want = x.astype(np.float64)
    mag = np.abs(want)
    np.add.at(want.T, idx - 1, y.T.astype(np.float64))
    np.add.at(mag.T, idx - 1, np.abs(y.T).astype(np.float64))
    got = xd.cpu().numpy().reshape(xrows, xcols, order="F")
    reps = np.bincount(idx - 1, minlength=xcols).max() + 1
    assert np.all(np.abs(got - want) <= reps * np.finfo(np.float32).eps * mag)


@pytest.mark.parametrize("nrows,ncols,incx,incy,xoff,yoff", [
    (16, 5, 64, 32, 0, 0), (8, 7, 24, 8, 8, 0), (12, 3, 20, 12, 4, 4), (6, 9, 10, 6, 2, 0),
    (7, 11, 13, 9, 1, 3), (4096, 300, 8192, 4096, 0, 0), (4000, 33, 4100, 4000, 4, 0), (1, 1, 1, 1, 3, 5),
    (100, 1, 100, 100, 0, 16),
])
def test_xcopy_bytes(K, nrows, ncols, incx, incy, xoff, yoff):
    rng = np.random.default_rng(nrows + ncols)
    xb = rng.integers(0, 256, xoff + incx * ncols + nrows, dtype=np.uint8)
    yb = rng.integers(0, 256, yoff + incy * ncols + nrows, dtype=np.uint8)
    xd, yd = dev(xb), dev(yb)
    K.lib.knet8("xcopy", nrows, ncols, C.c_void_p(xd.data_ptr() + xoff), incx, C.c_void_p(yd.data_ptr() + yoff), incy)
    want = yb.copy()
    want[yoff:] = io.xcopy(nrows, ncols, xb[xoff:], incx, yb[yoff:], incy)
    assert np.array_equal(yd.cpu().numpy(), want)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("nrows,ncols,incy,off", [(4, 3, 8, 0), (3, 5, 7, 0), (8, 2, 10, 1), (1024, 100, 2048, 0),
                                                  (5, 1, 5, 2)])
def test_xfill(K, dtype, nrows, ncols, incy, off):
    dt = NPDT[dtype]
    y = np.random.default_rng(1).random(off + incy * ncols + nrows).astype(dt)
    yd = dev(y)
    ct = C.c_float if dt == np.float32 else C.c_double
    K.lib.knet8(f"xfill_{K.lib.sfx(dtype)}", nrows, ncols, ct(-1.5),
                C.c_void_p(yd.data_ptr() + off * y.itemsize), incy)
    want = y.copy()
    want[off:] = io.xfill(nrows, ncols, -1.5, y[off:], incy)
    assert np.array_equal(yd.cpu().numpy(), want)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("n,k", [(5, 3), (1000, 64), (37, 150)])
def test_icat(K, dtype, n, k):
    rng = np.random.default_rng(n)
    vs = [rng.random(n).astype(NPDT[dtype]) for _ in range(k)]
    got = K.indexing.icat([K.KnetArray(v) for v in vs])
    assert got.shape == (n, k) and np.array_equal(F(got.numpy()), io.icat(vs))


def test_embedding_lookup_and_gradient(K):
    """w[:, tokens] for a (T, B) token matrix and its scatter-add gradient through the tape."""
    A = K.autograd
    rng = np.random.default_rng(5)
    V, E, T, B = 1000, 64, 12, 9
    w = np.asfortranarray(rng.integers(-4, 5, (E, V)).astype(np.float32))
    tok = rng.integers(1, V + 1, (T, B))
    tok[0, :] = 7                                            # a hot column: repeats must add up
    pw = A.Param(K.KnetArray(w))
    coef = np.asfortranarray(rng.integers(-3, 4, (E, T, B)).astype(np.float32))
    tape = A.diff(lambda: A.sum(pw[K.indexing.COLON, tok] * K.KnetArray(coef)))
    emb = K.indexing.getindex(pw.value, K.indexing.COLON, tok)
    assert emb.shape == (E, T, B)
    assert np.array_equal(emb.numpy(), w[:, tok - 1])
    want = io.addtoindex(np.zeros_like(w), coef.reshape(E, T * B, order="F"), _Colon(), F(tok))
    assert np.array_equal(A.grad(tape, pw).numpy(), want)


class _Colon:
    def __repr__(self):
        return ":"


@pytest.mark.parametrize("k", [4, 5, 8, 12, 15, 17, 18, 19, 20, 22, 27])
def test_getindex_gradcheck(K, k):
    """gradcheck(getindex, a, i...) as in test/karray.jl:60-61 for the array-valued kinds."""
    A, X = K.autograd, K.indexing
    I = _cases_2d(X)[k]
    a = np.asfortranarray(np.random.default_rng(9).random((3, 4)))
    assert A.gradcheck(lambda x: A.getindex(x, *I) if isinstance(x, A.Value) else X.getindex(x, *I), a)
