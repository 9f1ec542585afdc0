"""The index oracle against hand-written NumPy expressions for the reference's own index list
(test/karray.jl:24-41, 141-148), and its kernel-level loops against its array level."""
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "..", "oracle"))
import index_oracle as io  # noqa: E402


class Colon:
    def __repr__(self):
        return ":"


class UR:
    def __init__(self, a, b):
        self.first, self.last = a, b


class SR:
    def __init__(self, a, s, b):
        self.first, self.step, self.last = a, s, b


class CI:
    def __init__(self, *I):
        self.I = I


C = Colon()
T34 = np.ones((3, 4), bool)

# (Julia index tuple, the same selection written directly in NumPy on the column-major array)
CASES_2D = [
    ((C,), lambda a: a.reshape(-1, order="F")),
    ((C, C), lambda a: a),
    ((3,), lambda a: a.reshape(-1, order="F")[2]),
    ((2, 3), lambda a: a[1, 2]),
    ((UR(3, 5),), lambda a: a.reshape(-1, order="F")[2:5]),
    ((UR(1, 2), UR(3, 4)), lambda a: a[0:2, 2:4]),
    ((2, C), lambda a: a[1, :]),
    ((C, 2), lambda a: a[:, 1]),
    ((UR(1, 2), C), lambda a: a[0:2, :]),
    ((C, UR(1, 2)), lambda a: a[:, 0:2]),
    ((UR(1, 2), 2), lambda a: a[0:2, 1]),
    ((2, UR(1, 2)), lambda a: a[1, 0:2]),
    ((SR(1, 2, 3),), lambda a: a.reshape(-1, order="F")[[0, 2]]),
    ((SR(1, 2, 3), C), lambda a: a[[0, 2], :]),
    ((C, SR(1, 2, 3)), lambda a: a[:, [0, 2]]),
    (([1, 3],), lambda a: a.reshape(-1, order="F")[[0, 2]]),
    (([2, 2],), lambda a: a.reshape(-1, order="F")[[1, 1]]),
    (([1, 3], C), lambda a: a[[0, 2], :]),
    ((C, [1, 3]), lambda a: a[:, [0, 2]]),
    (([2, 2], C), lambda a: a[[1, 1], :]),
    ((C, [2, 2]), lambda a: a[:, [1, 1]]),
    ((T34,), lambda a: a.reshape(-1, order="F")),
    ((np.array([[1, 3], [2, 4]]),), lambda a: a.reshape(-1, order="F")[np.array([[0, 2], [1, 3]])]),
    ((CI(3),), lambda a: a.reshape(-1, order="F")[2]),
    ((CI(2, 3),), lambda a: a[1, 2]),
    ((C, np.ones(4, bool)), lambda a: a),
    ((np.ones(3, bool), C), lambda a: a),
    (([CI(2, 2), CI(2, 1)],), lambda a: np.array([a[1, 1], a[1, 0]])),
]


@pytest.mark.parametrize("k", range(len(CASES_2D)))
def test_getindex_matches_numpy_2d(k):
    a = np.asfortranarray(np.random.default_rng(3).random((3, 4)))
    I, f = CASES_2D[k]
    got, want = io.getindex(a, *I), f(a)
    assert np.shape(got) == np.shape(want)
    assert np.array_equal(np.asarray(got), np.asarray(want))


def test_getindex_3d():
    a = np.asfortranarray(np.random.default_rng(4).random((3, 4, 5)))
    assert io.getindex(a, 2, 3, 4) == a[1, 2, 3]
    assert np.array_equal(io.getindex(a, C, C, 2), a[:, :, 1])
    assert np.array_equal(io.getindex(a, C, C, UR(1, 2)), a[:, :, 0:2])
    assert np.array_equal(io.getindex(a, UR(3, 5)), a.reshape(-1, order="F")[2:5])
    assert np.array_equal(io.getindex(a, C, C, C), a)


def test_setindex_and_addtoindex():
    a = np.asfortranarray(np.arange(12, dtype=np.float64).reshape(3, 4, order="F"))
    b = io.setindex(a, 0, C, [1, 3])
    assert np.array_equal(b[:, [0, 2]], np.zeros((3, 2))) and np.array_equal(b[:, [1, 3]], a[:, [1, 3]])
    b = io.setindex(a, np.array([[100., 200.], [300., 400.]]), UR(2, 3), UR(1, 2))
    assert b[1, 0] == 100 and b[2, 0] == 300 and b[1, 1] == 200 and b[2, 1] == 400
    c = io.addtoindex(np.zeros((3, 4)), np.ones((3, 2)), C, [2, 2])
    assert np.array_equal(c[:, 1], 2 * np.ones(3)) and c.sum() == 6
    d = io.addtoindex(np.zeros(5), np.array([1., 2., 4.]), [2, 2, 5])
    assert np.array_equal(d, [0, 3, 0, 0, 4])
    with pytest.raises(IndexError):
        io.getindex(a, C, [5])
    with pytest.raises(IndexError):
        io.getindex(a, [0])


def test_kernel_level_agrees_with_array_level():
    rng = np.random.default_rng(5)
    x = np.asfortranarray(rng.integers(-8, 8, (6, 7)).astype(np.float32))
    cols, rows = np.array([7, 1, 1, 4], np.int32), np.array([6, 6, 2], np.int32)
    yc = np.asfortranarray(rng.integers(-8, 8, (6, 4)).astype(np.float32))
    yr = np.asfortranarray(rng.integers(-8, 8, (3, 7)).astype(np.float32))
    F = lambda m: m.reshape(-1, order="F")  # noqa: E731
    assert np.array_equal(io.getcols(6, 7, cols, x), F(io.getindex(x, C, cols)))
    assert np.array_equal(io.getrows(6, 7, rows, x), F(io.getindex(x, rows, C)))
    assert np.array_equal(io.addcols(6, 7, cols, x, yc), F(io.addtoindex(x, yc, C, cols)))
    assert np.array_equal(io.addrows(6, 7, rows, x, yr), F(io.addtoindex(x, yr, rows, C)))
    assert np.array_equal(io.setcol1(6, 7, cols, x, 3.0), F(io.setindex(x, 3.0, C, cols)))
    assert np.array_equal(io.setrow1(6, 7, rows, x, 3.0), F(io.setindex(x, 3.0, rows, C)))
    u = np.array([2, 5, 7], np.int32)
    assert np.array_equal(io.setcols(6, 7, u, x, yc[:, :3]), F(io.setindex(x, yc[:, :3], C, u)))
    ents = np.array([1, 42, 42, 7], np.int32)
    assert np.array_equal(io.getents(x, ents), F(x)[[0, 41, 41, 6]])
    assert np.array_equal(io.addents(x, ents, np.ones(4, np.float32)) - F(x),
                          np.bincount(ents - 1, minlength=42).astype(np.float32))
    # pitched copy: a 2x3 block of Float32 out of a 6-row matrix is 3 runs of 8 bytes, pitch 24
    xb = F(x).view(np.uint8)
    blk = io.xcopy(8, 3, xb[(1 + 2 * 6) * 4:], 24, np.zeros(24, np.uint8), 8).view(np.float32)
    assert np.array_equal(blk, F(x[1:3, 2:5]))
    assert np.array_equal(io.xfill(2, 3, 9.0, F(x)[13:], 6)[:14].reshape(-1)[[0, 1, 6, 7, 12, 13]], [9.0] * 6)
    assert np.array_equal(io.icat([x[:, 0], x[:, 3]]), F(x[:, [0, 3]]))
