"""NumPy restatement of Knet's index kernels and of Julia's indexing on column-major arrays.

TEST INFRASTRUCTURE ONLY.  Only the tests may import this module; the shipped package never
does, and this module imports nothing from it.

Two layers:

* kernel level - the loops of src/libknet8/cuda1.jl:108-449 written with NumPy index
  arithmetic (`getcols`, `addrows`, `xcopy`, ...), 1-based Int32 indices, flat column-major
  buffers;
* array level - `getindex(a, *I)`, `setindex(a, v, *I)`, `addtoindex(a, v, *I)`: what Julia
  computes for `a[I...]`, `a[I...] = v` / `a[I...] .= v` and AutoGrad's `addtoindex!` on a
  host `Array`, which is what test/karray.jl:22-63 compares the device arrays with.

Index objects are duck-typed so that the tests can hand the same tuple to both sides: `:` is
any object whose repr is ":", a unit range has `first`/`last`, a step range `first`/`step`/
`last`, a Cartesian index has `.I`; integers, integer arrays and Bool arrays are themselves.
"""
import numpy as np


# ---- kernel level (flat buffers, 1-based indices) ---------------------------------------------------
def _flat(a):
    return np.asarray(a).reshape(-1, order="F")


def getents(x, ents):                      # cuda1.jl:342-348
    return _flat(x)[np.asarray(ents, np.int64) - 1].copy()


def setents(x, ents, y):                   # cuda1.jl:349-355 (distinct indices)
    x = _flat(x).copy()
    x[np.asarray(ents, np.int64) - 1] = _flat(y)
    return x


def addents(x, ents, y):                   # cuda1.jl:356-362
    x = _flat(x).copy()
    np.add.at(x, np.asarray(ents, np.int64) - 1, _flat(y))
    return x


def getcols(xrows, xcols, cols, x):        # cuda1.jl:246-257: y[row + j*xrows] = x[row + (cols[j]-1)*xrows]
    X = _flat(x).reshape(xrows, xcols, order="F")
    return X[:, np.asarray(cols, np.int64) - 1].reshape(-1, order="F")


def setcols(xrows, xcols, cols, x, y):     # cuda1.jl:258-269
    X = _flat(x).reshape(xrows, xcols, order="F").copy(order="F")
    X[:, np.asarray(cols, np.int64) - 1] = _flat(y).reshape(xrows, len(cols), order="F")
    return X.reshape(-1, order="F")


def addcols(xrows, xcols, cols, x, y):     # cuda1.jl:270-281
    X = _flat(x).reshape(xrows, xcols, order="F").copy(order="F")
    Y = _flat(y).reshape(xrows, len(cols), order="F")
    for j, c in enumerate(np.asarray(cols, np.int64) - 1):       # columns in order: one fixed sum order
        X[:, c] += Y[:, j]
    return X.reshape(-1, order="F")


def setcol1(xrows, xcols, cols, x, v):     # cuda1.jl:282-293
    X = _flat(x).reshape(xrows, xcols, order="F").copy(order="F")
    X[:, np.asarray(cols, np.int64) - 1] = v
    return X.reshape(-1, order="F")


def getrows(xrows, xcols, rows, x):        # cuda1.jl:294-305: y[i + c*nrows] = x[rows[i]-1 + c*xrows]
    X = _flat(x).reshape(xrows, xcols, order="F")
    return X[np.asarray(rows, np.int64) - 1, :].reshape(-1, order="F")


def setrows(xrows, xcols, rows, x, y):     # cuda1.jl:306-317
    X = _flat(x).reshape(xrows, xcols, order="F").copy(order="F")
    X[np.asarray(rows, np.int64) - 1, :] = _flat(y).reshape(len(rows), xcols, order="F")
    return X.reshape(-1, order="F")


def addrows(xrows, xcols, rows, x, y):     # cuda1.jl:318-329
    X = _flat(x).reshape(xrows, xcols, order="F").copy(order="F")
    Y = _flat(y).reshape(len(rows), xcols, order="F")
    for i, r in enumerate(np.asarray(rows, np.int64) - 1):
        X[r, :] += Y[i, :]
    return X.reshape(-1, order="F")


def setrow1(xrows, xcols, rows, x, v):     # cuda1.jl:330-341
    X = _flat(x).reshape(xrows, xcols, order="F").copy(order="F")
    X[np.asarray(rows, np.int64) - 1, :] = v
    return X.reshape(-1, order="F")


def xcopy(nrows, ncols, xbytes, incx, ybytes, incy):   # cuda1.jl:134-165, all counts in bytes
    y = np.array(ybytes, dtype=np.uint8, copy=True)
    x = np.asarray(xbytes, dtype=np.uint8)
    for c in range(ncols):
        y[c * incy:c * incy + nrows] = x[c * incx:c * incx + nrows]
    return y


def xfill(nrows, ncols, v, y, incy):       # cuda1.jl:108-131, counts in elements
    y = _flat(y).copy()
    for c in range(ncols):
        y[c * incy:c * incy + nrows] = v
    return y


def icat(vectors):                         # cuda1.jl:168-181: y[row + col*nrows] = x[col][row]
    return np.stack([_flat(v) for v in vectors], axis=1).reshape(-1, order="F")


# ---- array level: Julia's a[I...] on a host Array -------------------------------------------------------
def _is_colon(i):
    return repr(i) == ":"


def _is_real(i):
    return isinstance(i, (int, float, np.integer, np.floating)) and not isinstance(i, (bool, np.bool_))


def _to_numpy_axis(i, n):
    """One Julia index for an axis of length n as a NumPy index (0-based), plus whether the
    axis survives (a Real drops it)."""
    if _is_colon(i):
        return np.arange(n), True
    if _is_real(i):
        if not 1 <= int(i) <= n:
            raise IndexError("BoundsError")
        return int(i) - 1, False
    if hasattr(i, "step"):
        stop = i.last + (1 if i.step > 0 else -1)
        idx = np.arange(i.first, stop, i.step)
    elif hasattr(i, "first"):
        idx = np.arange(i.first, i.last + 1)
    else:
        idx = np.asarray(i)
        if idx.dtype == np.bool_:
            if idx.size != n:
                raise IndexError("BoundsError")
            idx = np.flatnonzero(idx.reshape(-1, order="F")) + 1
    if idx.size and (idx.min() < 1 or idx.max() > n):
        raise IndexError("BoundsError")
    return idx.astype(np.int64) - 1, True


def _linear_of_cartesian(shape, c):
    lin, stride = 0, 1
    for d, j in enumerate(c.I):
        lin += (j - 1) * stride
        stride *= shape[d] if d < len(shape) else 1
    return lin


def _resolve(a, I):
    """(flat 0-based positions in column-major order, result shape or None for a scalar)."""
    a = np.asarray(a)
    n = a.size
    if len(I) == 1:
        i = I[0]
        if hasattr(i, "I"):
            return np.array([_linear_of_cartesian(a.shape, i)]), None
        if isinstance(i, (list, tuple)) and len(i) and hasattr(i[0], "I"):
            pos = np.array([_linear_of_cartesian(a.shape, c) for c in i])
            return pos, (len(i),)
        idx, keep = _to_numpy_axis(i, n)
        if not keep:
            return np.array([idx]), None
        shape = np.asarray(i).shape if not (_is_colon(i) or hasattr(i, "first")) and \
            np.asarray(i).dtype != np.bool_ else (idx.size,)
        return idx.reshape(-1, order="F"), shape
    # several indices: outer product of per-axis positions, missing trailing axes are 1
    dims = list(a.shape) + [1] * (len(I) - a.ndim)
    axes, shape = [], []
    for d, i in enumerate(I):
        idx, keep = _to_numpy_axis(i, dims[d])
        axes.append(np.atleast_1d(idx))
        if keep:
            shape.append(np.atleast_1d(idx).size)
    pos, stride = np.zeros((1,), np.int64), 1
    for d, ax in enumerate(axes):                # column-major: first axis fastest
        pos = (pos[:, None] + (ax * stride)[None, :]).reshape(-1, order="F")
        stride *= dims[d]
    return pos, (tuple(shape) if shape else None)


def getindex(a, *I):
    pos, shape = _resolve(a, I)
    flat = _flat(a)
    if shape is None:
        return flat[pos[0]].item()
    return np.asfortranarray(flat[pos].reshape(shape, order="F"))


def setindex(a, v, *I):
    """Returns the updated copy of a (`a[I...] = v` for a number, `a[I...] .= v` for an array)."""
    pos, _ = _resolve(a, I)
    out = _flat(a).copy()
    out[pos] = v if _is_real(v) else _flat(v)
    return np.asfortranarray(out.reshape(np.asarray(a).shape, order="F"))


def addtoindex(a, v, *I):
    """AutoGrad's addtoindex!: repeated positions accumulate, in index order."""
    pos, _ = _resolve(a, I)
    out = _flat(a).copy()
    np.add.at(out, pos, v if _is_real(v) else _flat(v))
    return np.asfortranarray(out.reshape(np.asarray(a).shape, order="F"))
