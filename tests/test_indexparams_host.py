"""indexparams (the host logic behind A[i1:i2, j1:j2], src/knetarrays/getindex.jl:705-737): the
(nelts, nrows, ncols, firstindex, astep) it returns must describe exactly the elements that
the index pair selects, in column-major order.  Runs without a GPU: the array is a stand-in that
only knows its shape."""
import itertools
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "knet.jl_b200"))


class ShapeOnly:
    def __init__(self, shape):
        self.shape = tuple(shape)
        self.ndim = len(shape)

    def __len__(self):
        return int(np.prod(self.shape))

    def size(self, d):
        return self.shape[d - 1] if d <= len(self.shape) else 1

    def stride(self, d):
        return int(np.prod(self.shape[:d - 1]))


@pytest.fixture(scope="module")
def X():
    try:
        from knet_sm100 import indexing
    except ImportError as e:                      # the package needs its built library to import
        pytest.skip(str(e))
    return indexing


def _choices(X, n):
    out = [X.COLON] + list(range(1, n + 1))
    out += [X.UnitRange(a, b) for a in range(1, n + 1) for b in range(a, n + 1)]
    return out


def _np_index(X, i, n):
    if i is X.COLON:
        return np.arange(n)
    if isinstance(i, X.UnitRange):
        return np.arange(i.first - 1, i.last)
    return np.array([i - 1])


@pytest.mark.parametrize("shape", [(3, 4), (1, 5), (4, 1), (5,), (2, 2)])
def test_indexparams_describes_the_selected_block(X, shape):
    A = ShapeOnly(shape)
    rows, cols = shape[0], (shape[1] if len(shape) > 1 else 1)
    lin = np.arange(rows * cols).reshape(rows, cols, order="F")
    for i1, i2 in itertools.product(_choices(X, rows), _choices(X, cols)):
        nelts, nrows, ncols, first, astep = X.indexparams(A, (i1, i2))
        want = lin[np.ix_(_np_index(X, i1, rows), _np_index(X, i2, cols))].reshape(-1, order="F")
        got = np.concatenate([np.arange(nrows) + (first - 1) + c * astep for c in range(ncols)]) if ncols else np.array([], int)
        assert nelts == want.size and nrows * ncols == nelts
        assert np.array_equal(got, want), (i1, i2)


def test_indexparams_rejects_what_the_reference_rejects(X):
    A = ShapeOnly((3, 4))
    with pytest.raises(ValueError):
        X.indexparams(A, (X.UnitRange(2, 1), X.COLON))       # empty range: DimensionMismatch in the reference
    with pytest.raises(ValueError):
        X.indexparams(A, (4, X.COLON))
    with pytest.raises(ValueError):
        X.indexparams(A, (X.COLON, X.UnitRange(3, 5)))
    with pytest.raises(TypeError):
        X.indexparams(ShapeOnly((2, 2, 2)), (X.COLON, X.COLON))
