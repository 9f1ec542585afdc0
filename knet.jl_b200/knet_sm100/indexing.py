"""getindex / setindex! / addtoindex! for KnetArray with Julia's index kinds, dispatched to the
library's index kernels the way src/knetarrays/getindex.jl and src/autograd_gpu/addto.jl do.

Indices are 1-based, as in Julia:

    COLON                      `:`
    3                          a Real
    UnitRange(2, 5)            `2:5`        (contiguous: a view when the memory is one run)
    StepRange(1, 2, 5)         `1:2:5`      (collected to an index vector, getindex.jl:412-470)
    [1, 3], np.array([[1,3],[2,4]])         integer arrays of any shape (linear indices)
    np.array([True, False, ...])            Bool masks (findall, getindex.jl:482-603)
    CartesianIndex(2, 3), [CartesianIndex(2,2), ...]

Supported forms are the reference's: one index of any kind; (`:`, vector) and (vector, `:`) on
matrices (getcols / getrows); any pair of Real / UnitRange / Colon on matrices (a view or
xcopy / xfill through `indexparams`); (`:`, `:`, Real-or-range) on 3-d arrays.  Other
combinations raise TypeError like Julia's MethodError.  BoundsError -> IndexError,
DimensionMismatch -> ValueError.
"""
import ctypes as C

import numpy as np
import torch

from . import ops
from .karray import KnetArray, _prod
from .lib import knet8, ptr, sfx

_CT = {torch.float32: C.c_float, torch.float64: C.c_double}


class _Colon:
    def __repr__(self):
        return ":"


COLON = _Colon()


class UnitRange:
    def __init__(self, first, last):
        self.first, self.last = int(first), int(last)

    def __len__(self):
        return max(0, self.last - self.first + 1)

    def collect(self):
        return np.arange(self.first, self.last + 1, dtype=np.int64)


class StepRange:
    def __init__(self, first, step, last):
        self.first, self.step, self.last = int(first), int(step), int(last)

    def collect(self):
        stop = self.last + (1 if self.step > 0 else -1)
        return np.arange(self.first, stop, self.step, dtype=np.int64)


class CartesianIndex:
    def __init__(self, *I):
        self.I = tuple(int(i) for i in I)


def _is_real(i):
    return isinstance(i, (int, float, np.integer, np.floating)) and not isinstance(i, (bool, np.bool_))


def _is_index3(i):
    return i is COLON or _is_real(i) or isinstance(i, UnitRange)


def _is_cartesian_list(i):
    return isinstance(i, (list, tuple)) and len(i) > 0 and all(isinstance(c, CartesianIndex) for c in i)


def _as_array(i):
    """An index array (ints or Bools) from a list / NumPy array / StepRange, else None."""
    if isinstance(i, StepRange):
        return i.collect()
    if isinstance(i, np.ndarray):
        return i
    if isinstance(i, (list, tuple)) and not _is_cartesian_list(i):
        return np.asarray(i) if len(i) else np.zeros((0,), np.int64)
    return None


def _linear(shape, J):
    """LinearIndices(shape)[J...] with Julia's rule that trailing missing indices are 1."""
    lin, stride = 1, 1
    for d, j in enumerate(J):
        lin += (j - 1) * stride
        stride *= shape[d] if d < len(shape) else 1
    return lin


def _c2i(shape, cs):
    """c2i (getindex.jl:405): Cartesian indices to Int32 linear indices."""
    return np.array([_linear(shape, c.I) for c in cs], dtype=np.int32)


def _real_tuple(A, I):
    """Linear index of A[i, j, ...] after Julia's per-dimension bounds check (getindex.jl:117-134)."""
    J = tuple(int(i) for i in I)
    for d, j in enumerate(J):
        if not 1 <= j <= A.size(d + 1):
            raise IndexError(f"BoundsError: index {J} of size {A.shape}")
    return _linear(A.shape, J)


def checkbetween(i, lo, hi):
    """Host bounds check before the unchecked kernels (getindex.jl:277-287)."""
    i = np.asarray(i)
    if i.size and (i.min() < lo or i.max() > hi):
        bad = i.reshape(-1)[np.argmax((i.reshape(-1) < lo) | (i.reshape(-1) > hi))]
        raise IndexError(f"BoundsError: attempt to access {lo}:{hi} at index [{int(bad)}]")


def _dev_index(i, device):
    """KnetArray{Int32}(i): the index vector on the device, column-major order."""
    flat = np.ascontiguousarray(np.asarray(i, dtype=np.int32).reshape(-1, order="F"))
    return torch.from_numpy(flat).to(device)


def _value_array(v, like, shape=None):
    """KnetArray{T}(y): the right-hand side of a setindex! as a device array of x's type."""
    if isinstance(v, KnetArray):
        return v if v.dtype == like.dtype else KnetArray(v.data.to(like.dtype), v.shape)
    a = np.asarray(v, dtype=np.float32 if like.dtype == torch.float32 else np.float64)
    return KnetArray(a if a.ndim else a.reshape(1))


# ---- unsafe_* : the kernel calls (getindex.jl:217-271) -------------------------------------------
def _ents(kind, x, idx, y=None, scalar=None):
    n = idx.numel()
    if n == 0:
        return
    S = sfx(x.dtype)
    if kind == "setent1":
        knet8(f"setent1_{S}", n, ptr(idx), ptr(x.data), _CT[x.dtype](scalar))
    else:
        knet8(f"{kind}_{S}", n, ptr(idx), ptr(x.data), ptr(y.data))


def _colsrows(kind, x, idx, y=None, scalar=None):
    S = sfx(x.dtype)
    xr, xc = x.shape
    if kind in ("setcol1", "setrow1"):
        knet8(f"{kind}_{S}", xr, xc, idx.numel(), ptr(idx), ptr(x.data), _CT[x.dtype](scalar))
    else:
        knet8(f"{kind}_{S}", xr, xc, idx.numel(), ptr(idx), ptr(x.data), ptr(y.data))


# ---- indexparams (getindex.jl:705-737) ----------------------------------------------------------------
def indexparams(A, I):
    """(nelts, nrows, ncols, firstindex, astep) of the block A[I...] for Real/UnitRange/Colon
    indices: `ncols` runs of `nrows` contiguous elements, `astep` elements apart."""
    if A.ndim > 2:
        raise TypeError("setindex for ndims > 2 not implemented yet")
    skipped, nrows, nelts, subs1, astep = False, 1, 1, [1, 1], len(A)
    for d, Ii in enumerate(I):
        Ai = A.size(d + 1)
        if Ii is COLON:
            Li, subs1[d] = Ai, 1
        elif _is_real(Ii):
            if not 1 <= int(Ii) <= Ai:
                raise ValueError("DimensionMismatch")
            Li, subs1[d] = 1, int(Ii)
        else:
            if not 1 <= Ii.first <= Ii.last <= Ai:
                raise ValueError("DimensionMismatch")
            Li, subs1[d] = len(Ii), Ii.first
        nelts *= Li
        if not skipped:
            nrows *= Li
            if Li < Ai:
                skipped, astep = True, A.stride(d + 2)
    ncols = nelts // nrows
    return nelts, nrows, ncols, _linear(A.shape, subs1), astep


def _esize(A):
    return A.data.element_size()


def _getindex2(A, I1, I2):
    """getindex2 (getindex.jl:645-664): a view when the block is one run, else xcopy."""
    nelts, nrows, ncols, first, astep = indexparams(A, (I1, I2))
    B1 = A.size(1) if I1 is COLON else (1 if _is_real(I1) else len(I1))
    B2 = A.size(2) if I2 is COLON else (1 if _is_real(I2) else len(I2))
    bsize = (B2,) if _is_real(I1) else (B1,) if _is_real(I2) else (B1, B2)
    if ncols == 1:
        return KnetArray(A.data[first - 1:first - 1 + nrows], bsize)
    B = A.similar(bsize)
    if len(B) == 0:
        return B
    s = _esize(A)
    knet8("xcopy", nrows * s, ncols, C.c_void_p(A.data.data_ptr() + (first - 1) * s), astep * s,
          ptr(B.data), nrows * s)
    return B


def _setindex2(A, B, I1, I2):
    """setindex2! (getindex.jl:666-703): fill / xfill for a number, copy / xcopy for an array."""
    nelts, nrows, ncols, first, astep = indexparams(A, (I1, I2))
    s, S = _esize(A), sfx(A.dtype)
    aptr0 = C.c_void_p(A.data.data_ptr() + (first - 1) * s)
    if _is_real(B):
        v = _CT[A.dtype](B)
        if ncols == 1:
            if nelts > 0:
                knet8(f"fill_{S}", nelts, v, aptr0)
        elif nrows > 0 and ncols > 0:
            knet8(f"xfill_{S}", nrows, ncols, v, aptr0, astep)
        return A
    B = _value_array(B, A)
    if len(B) != nelts:
        raise ValueError("DimensionMismatch")
    if ncols == 1:
        if nelts > 0:
            A.data[first - 1:first - 1 + nelts].copy_(B.data)      # cuMemcpyDtoD in the reference
    elif nrows > 0 and ncols > 0:
        knet8("xcopy", nrows * s, ncols, ptr(B.data), nrows * s, aptr0, astep * s)
    return A


# ---- getindex ------------------------------------------------------------------------------------------
def _mask(i, n, err):
    if i.size != n:
        raise err
    return np.flatnonzero(i.reshape(-1, order="F")) + 1


def getindex(A, *I):
    """A[I...] (src/knetarrays/getindex.jl)."""
    if len(I) == 1:
        i = I[0]
        if i is COLON:
            return A.vec()                                               # :195-197
        if isinstance(i, CartesianIndex):
            return getindex(A, *i.I)                                     # :138-140
        if _is_real(i):
            j = int(i)
            if not 1 <= j <= len(A):
                raise IndexError(f"BoundsError: index {j} of {len(A)} elements")
            return A.data[j - 1].item()                                  # :99-103
        if isinstance(i, UnitRange):                                     # :153-159, a view
            if not 1 <= i.first <= i.last <= len(A):
                raise IndexError(f"BoundsError: range {i.first}:{i.last} of {len(A)} elements")
            return A.view(i.first - 1, len(i))
        if isinstance(i, KnetArray):                                     # :574-580, a 0/1 array as mask
            return getindex(A, i.numpy() != 0)
        if _is_cartesian_list(i):
            return getindex(A, _c2i(A.shape, i))                         # :406
        arr = _as_array(i)
        if arr is None:
            raise TypeError(f"MethodError: getindex(KnetArray, {type(i).__name__})")
        if arr.dtype == np.bool_:                                        # :482-488
            j = _mask(arr, len(A), IndexError("BoundsError: mask length"))
            y = A.similar((len(j),))
            _ents("getents", A, _dev_index(j, A.data.device), y)
            return y
        y = A.similar(arr.shape)                                         # :291-298
        if len(y) == 0:
            return y
        checkbetween(arr, 1, len(A))
        _ents("getents", A, _dev_index(arr, A.data.device), y)
        return y
    if all(_is_real(i) for i in I):                                      # :117-124
        return A.data[_real_tuple(A, I) - 1].item()
    if len(I) == 2:
        i1, i2 = I
        if _is_index3(i1) and _is_index3(i2):
            return _getindex2(A, i1, i2)
        if A.ndim != 2:
            raise TypeError("MethodError: vector indices need a matrix")
        xrows, xcols = A.shape
        if i1 is COLON:                                                  # :319-327, :507-514
            arr = _as_array(i2)
            if arr is not None and arr.ndim == 2 and arr.dtype != np.bool_:      # :798-800
                sub = getindex(A, COLON, arr.reshape(-1, order="F"))
                return sub.reshape(xrows, arr.shape[0], arr.shape[1])
            if arr is None or arr.ndim != 1:
                raise TypeError("MethodError: getindex(KnetMatrix, :, ?)")
            if arr.dtype == np.bool_:
                arr = _mask(arr, xcols, IndexError("BoundsError: mask length"))
            y = A.similar((xrows, len(arr)))
            if len(y) == 0:
                return y
            checkbetween(arr, 1, xcols)
            _colsrows("getcols", A, _dev_index(arr, A.data.device), y)
            return y
        if i2 is COLON:                                                  # :360-368, :535-542
            arr = _as_array(i1)
            if arr is None or arr.ndim != 1:
                raise TypeError("MethodError: getindex(KnetMatrix, ?, :)")
            if arr.dtype == np.bool_:
                arr = _mask(arr, xrows, IndexError("BoundsError: mask length"))
            y = A.similar((len(arr), xcols))
            if len(y) == 0:
                return y
            checkbetween(arr, 1, xrows)
            _colsrows("getrows", A, _dev_index(arr, A.data.device), y)
            return y
        raise TypeError("MethodError: getindex(KnetMatrix, ?, ?)")
    if len(I) == 3 and I[0] is COLON and I[1] is COLON:                  # :746-757
        if I[2] is COLON:
            return A
        B = A.reshape(A.stride(3), A.size(3))
        sub = getindex(B, COLON, I[2])
        if _is_real(I[2]):
            return sub.reshape(A.size(1), A.size(2))
        return sub.reshape(A.size(1), A.size(2), len(I[2]))
    raise TypeError(f"MethodError: getindex with {len(I)} indices of these kinds")


# ---- setindex! -----------------------------------------------------------------------------------------
def setindex_(A, v, *I):
    """A[I...] = v (a number, or an array with the block's element count)."""
    if len(I) == 1:
        i = I[0]
        if i is COLON:                                                   # :199-211
            if _is_real(v):
                return ops.fill_(A, v)
            B = _value_array(v, A)
            if len(B) != len(A):
                raise ValueError("DimensionMismatch")
            A.data.copy_(B.data)
            return A
        if isinstance(i, CartesianIndex):
            return setindex_(A, v, *i.I)
        if _is_real(i):                                                  # :105-110
            j = int(i)
            if not 1 <= j <= len(A):
                raise IndexError(f"BoundsError: index {j} of {len(A)} elements")
            A.data[j - 1] = float(v)
            return A
        if isinstance(i, UnitRange):                                     # :169-190
            if len(i) == 0:
                return A
            if not 1 <= i.first <= i.last <= len(A):
                raise IndexError("BoundsError")
            dst = A.view(i.first - 1, len(i))
            if _is_real(v):
                ops.fill_(dst, v)
            else:
                B = _value_array(v, A)
                if len(B) != len(i):
                    raise ValueError("DimensionMismatch")
                dst.data.copy_(B.data)
            return A
        if isinstance(i, KnetArray):
            return setindex_(A, v, i.numpy() != 0)
        if _is_cartesian_list(i):
            return setindex_(A, v, _c2i(A.shape, i))
        arr = _as_array(i)
        if arr is None:
            raise TypeError(f"MethodError: setindex!(KnetArray, v, {type(i).__name__})")
        if arr.dtype == np.bool_:                                        # :490-503
            arr = _mask(arr, len(A), ValueError("DimensionMismatch"))
            if not _is_real(v) and len(_value_array(v, A)) != len(arr):
                raise IndexError("BoundsError: value count differs from the mask's")
        elif not _is_real(v) and len(_value_array(v, A)) != arr.size:    # :308-315
            raise ValueError("DimensionMismatch")
        if arr.size == 0:
            return A
        checkbetween(arr, 1, len(A))
        idx = _dev_index(arr, A.data.device)
        if _is_real(v):
            _ents("setent1", A, idx, scalar=v)
        else:
            _ents("setents", A, idx, _value_array(v, A))
        return A
    if all(_is_real(i) for i in I):                                      # :126-134
        A.data[_real_tuple(A, I) - 1] = float(v)
        return A
    if len(I) == 3 and I[0] is COLON and I[1] is COLON:                  # :769-777
        if I[2] is COLON:
            return setindex_(A, v, COLON)
        setindex_(A.reshape(A.stride(3), A.size(3)), v, COLON, I[2])
        return A
    if len(I) == 2:
        i1, i2 = I
        if _is_index3(i1) and _is_index3(i2):
            return _setindex2(A, v, i1, i2)
        if A.ndim != 2:
            raise TypeError("MethodError: vector indices need a matrix")
        xrows, xcols = A.shape
        cols = i1 is COLON
        if not (cols or i2 is COLON):
            raise TypeError("MethodError: setindex!(KnetMatrix, v, ?, ?)")
        arr = _as_array(i2 if cols else i1)
        if arr is None or arr.ndim != 1:
            raise TypeError("MethodError: setindex!(KnetMatrix, v, ...)")
        if arr.dtype == np.bool_:
            arr = _mask(arr, xcols if cols else xrows, IndexError("BoundsError: mask length"))
        if _is_real(v):                                                  # :329-336, :370-377
            if arr.size == 0:
                return A
            checkbetween(arr, 1, xcols if cols else xrows)
            _colsrows("setcol1" if cols else "setrow1", A, _dev_index(arr, A.data.device), scalar=v)
            return A
        B = _value_array(v, A)                                           # :338-348, :379-389
        want = (xrows, len(arr)) if cols else (len(arr), xcols)
        if B.ndim != 2 or tuple(B.shape) != want:
            raise ValueError("DimensionMismatch")
        if len(B) == 0:
            return A
        checkbetween(arr, 1, xcols if cols else xrows)
        _colsrows("setcols" if cols else "setrows", A, _dev_index(arr, A.data.device), B)
        return A
    raise TypeError(f"MethodError: setindex! with {len(I)} indices of these kinds")


# ---- addtoindex! (src/autograd_gpu/addto.jl:24-82) --------------------------------------------------------
def addtoindex_(A, X, *I):
    """A[I...] += X where repeated indices accumulate (the backward of getindex)."""
    if len(I) == 1 and _is_cartesian_list(I[0]):
        return addtoindex_(A, X, _c2i(A.shape, I[0]))
    arrs = [_as_array(i) for i in I]
    int_array = [a is not None and a.dtype != np.bool_ for a in arrs]
    if len(I) == 1 and int_array[0]:
        checkbetween(arrs[0], 1, len(A))
        _ents("addents", A, _dev_index(arrs[0], A.data.device), _value_array(X, A))
        return A
    if len(I) == 2 and A.ndim == 2 and I[0] is COLON and int_array[1]:
        checkbetween(arrs[1], 1, A.size(2))
        _colsrows("addcols", A, _dev_index(arrs[1], A.data.device), _value_array(X, A))
        return A
    if len(I) == 2 and A.ndim == 2 and I[1] is COLON and int_array[0]:
        checkbetween(arrs[0], 1, A.size(1))
        _colsrows("addrows", A, _dev_index(arrs[0], A.data.device), _value_array(X, A))
        return A
    if any(int_array):
        raise TypeError("MethodError: addtoindex! for this index combination")
    cur = getindex(A, *I)                     # no repeats possible: get, add, set (addto.jl:40,54-55)
    if _is_real(cur):
        return setindex_(A, cur + float(X if _is_real(X) else _value_array(X, A).data.item()), *I)
    Xa = X if _is_real(X) else _value_array(X, A).reshape(cur.shape)
    return setindex_(A, ops.broadcast("add", cur, Xa), *I)


def icat(vectors):
    """Columns of equal-length device vectors side by side (icat_S, src/libknet8/cuda1.jl:168-214)."""
    n, k = len(vectors[0]), len(vectors)
    y = vectors[0].similar((n, k))
    table = (C.c_void_p * k)(*[v.data.data_ptr() for v in vectors])
    knet8(f"icat_{sfx(y.dtype)}", n, k, C.cast(table, C.c_void_p), ptr(y.data))
    return y
