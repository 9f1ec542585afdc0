"""ctypes/NumPy front end of the CPU checker (oracle/knet_oracle.c).

TEST INFRASTRUCTURE ONLY.  Only the tests, the smoke check and the CPU-baseline leg of the
benchmark may import this module; the shipped package never does.

Arrays are NumPy arrays in Fortran (column-major) order carrying Julia shapes, so that a
`(C,B)` score matrix here is the same memory image as Knet's.  `dims` arguments are 1-based
like Julia's.  The functions restate Knet's CPU definitions:
src/ops20/activation.jl, softmax.jl, loss.jl, dropout.jl, src/train20/update.jl,
distributions.jl, train.jl (one `@diff` plus one `update!` per parameter).
"""
import ctypes as C
import os
import subprocess
import time

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libknet_oracle.so")

RED_OPS = {"sum": 0, "prod": 1, "maximum": 2, "minimum": 3, "sumabs": 4, "sumabs2": 5,
           "maxabs": 6, "minabs": 7, "countnz": 8}


_SO_OMP = os.path.join(_HERE, "libknet_oracle_omp.so")


def build(force=False):
    """Compile the C restatement (and its OpenMP copy for the timing legs) with the committed Makefile."""
    src = os.path.join(_HERE, "knet_oracle.c")
    for so in (_SO, _SO_OMP):
        if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
            try:
                subprocess.check_call(["make", "-C", _HERE, "-B", os.path.basename(so)],
                                      stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)
            except subprocess.CalledProcessError:
                if so == _SO:
                    raise                      # the checker itself must build; the OpenMP copy is optional
    return _SO


def have_openmp():
    return os.path.exists(_SO_OMP)


_lib = None
_libs = {}


def lib():
    global _lib
    if _lib is None:
        use_openmp(False)
    return _lib


def use_openmp(flag):
    """Switch between the serial checker (the default, and the only one the tests use) and the
    OpenMP copy whose loops over independent outputs run on all host cores (same results)."""
    global _lib
    so = _SO_OMP if flag else _SO
    if so not in _libs:
        if not os.path.exists(so):
            build()
        _libs[so] = C.CDLL(so)
    _lib = _libs[so]
    return _lib


def _sfx(dt):
    dt = np.dtype(dt)
    if dt == np.float32:
        return "f32", C.c_float
    if dt == np.float64:
        return "f64", C.c_double
    raise TypeError(dt)


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def _f(a, dt=None):
    """Fortran-contiguous copy/view with the array's (or the given) dtype."""
    return np.asfortranarray(a, dtype=dt)


def _call(name, dt, *args, restype=None):
    s, _ = _sfx(dt)
    fn = getattr(lib(), f"{name}_{s}")
    fn.restype = restype
    return fn(*args)


# ---- elementwise -------------------------------------------------------------------------
def unary(name, x):
    x = _f(x)
    y = np.empty_like(x, order="F")
    _call(f"ko_{name}", x.dtype, C.c_int64(x.size), _p(x), _p(y))
    return y


def unary_truth(name, x):
    """The same expression evaluated in Float64 and rounded once to x's type."""
    return unary(name, _f(x, np.float64)).astype(x.dtype)


def actback(name, dy, y):
    dy, y = _f(dy), _f(y)
    dx = np.empty_like(y, order="F")
    _call(f"ko_{name}", y.dtype, C.c_int64(y.size), _p(dy), _p(y), _p(dx))
    return dx


_BIN = {
    "add": np.add, "sub": np.subtract, "mul": np.multiply, "div": np.divide,
    "max": lambda a, b: np.where(a > b, a, b), "min": lambda a, b: np.where(a < b, a, b),
    "eq": np.equal, "ne": np.not_equal, "gt": np.greater, "ge": np.greater_equal,
    "lt": np.less, "le": np.less_equal,
}


def binary(name, x, y):
    """Julia broadcast of a scalar op in the arrays' precision; comparisons give 0/1 in T
    (src/libknet8/ops.jl:87-100; trailing singleton dims are implied as in Julia)."""
    x, y = np.asarray(x), np.asarray(y)
    dt = x.dtype if x.dtype.kind == "f" else y.dtype
    nd = max(x.ndim, y.ndim)
    xs = x.reshape(x.shape + (1,) * (nd - x.ndim), order="F")
    ys = y.reshape(y.shape + (1,) * (nd - y.ndim), order="F")
    with np.errstate(all="ignore"):
        z = _BIN[name](xs.astype(dt, copy=False), ys.astype(dt, copy=False))
    return np.asfortranarray(z.astype(dt, copy=False))


# ---- reductions ----------------------------------------------------------------------------
def _geom(shape, d):
    """(inner, D, outer) for 1-based dim d of a column-major array."""
    shape = tuple(shape) + (1,) * max(0, d - len(shape))
    inner = int(np.prod(shape[:d - 1], dtype=np.int64))
    outer = int(np.prod(shape[d:], dtype=np.int64))
    return inner, int(shape[d - 1]), outer


def reduce_dim(op, x, dims):
    """`op(x, dims=dims)`; several dims are reduced one after the other."""
    x = _f(x)
    if isinstance(dims, int):
        dims = (dims,)
    first = True
    for d in dims:
        inner, D, outer = _geom(x.shape, d)
        shp = list(x.shape)
        shp[d - 1] = 1
        y = np.empty(shp, dtype=x.dtype, order="F")
        # after the first pass the items are already |x|, x^2 ...: merge only
        code = RED_OPS[op] if first else {4: 0, 5: 0, 6: 2, 7: 3, 8: 0}.get(RED_OPS[op], RED_OPS[op])
        _call("ko_reduce_dim", x.dtype, C.c_int(code), C.c_int64(inner), C.c_int64(D),
              C.c_int64(outer), _p(x), _p(y))
        x, first = y, False
    return x


def reduce_all(op, x):
    x = _f(x)
    _, ct = _sfx(x.dtype)
    return x.dtype.type(_call("ko_reduce_all", x.dtype, C.c_int(RED_OPS[op]),
                              C.c_int64(x.size), _p(x), restype=ct))


# ---- softmax family ------------------------------------------------------------------------
def _soft(name, mode, x, dims, *more):
    x = _f(x)
    inner, D, outer = _geom(x.shape, dims)
    out = np.empty_like(x, order="F")
    args = [C.c_int64(inner), C.c_int64(D), C.c_int64(outer), _p(x)] + [_p(_f(m, x.dtype)) for m in more]
    if mode is not None:
        args = [C.c_int(mode)] + args
    _call(name, x.dtype, *args, _p(out))
    return out


def softmax(x, dims=1):
    return _soft("ko_softmax_fwd", 0, x, dims)


def logsoftmax(x, dims=1):
    return _soft("ko_softmax_fwd", 1, x, dims)


def softmax_bwd(y, dy, dims=1):
    return _soft("ko_softmax_bwd", 0, y, dims, dy)


def logsoftmax_bwd(y, dy, dims=1):
    return _soft("ko_softmax_bwd", 1, y, dims, dy)


def logsumexp(x, dims=1):
    x = _f(x)
    inner, D, outer = _geom(x.shape, dims)
    shp = list(x.shape)
    shp[dims - 1] = 1
    y = np.empty(shp, dtype=x.dtype, order="F")
    _call("ko_logsumexp_fwd", x.dtype, C.c_int64(inner), C.c_int64(D), C.c_int64(outer), _p(x), _p(y))
    return y


def logsumexp_bwd(x, y, dy, dims=1):
    x = _f(x)
    inner, D, outer = _geom(x.shape, dims)
    dx = np.empty_like(x, order="F")
    _call("ko_logsumexp_bwd", x.dtype, C.c_int64(inner), C.c_int64(D), C.c_int64(outer),
          _p(x), _p(_f(y, x.dtype)), _p(_f(dy, x.dtype)), _p(dx))
    return dx


# ---- nll / accuracy ------------------------------------------------------------------------
def _rk(scores):
    s = _f(scores)
    R = s.shape[0]
    return s, R, s.size // R


def nll(scores, labels, dims=1, average=True):
    s, R, K = _rk(scores)
    lab = np.ascontiguousarray(labels, dtype=np.int32)
    _, ct = _sfx(s.dtype)
    tot = ct(0)
    cnt = _call("ko_nll", s.dtype, C.c_int64(R), C.c_int64(K), C.c_int(dims), _p(s), _p(lab),
                C.byref(tot), restype=C.c_int64)
    total = s.dtype.type(tot.value)
    return (total / s.dtype.type(cnt)) if average else (total, cnt)


def nll_bwd(scores, labels, dims=1, average=True, dy=1.0):
    s, R, K = _rk(scores)
    lab = np.ascontiguousarray(labels, dtype=np.int32)
    _, ct = _sfx(s.dtype)
    dx = np.empty_like(s, order="F")
    _call("ko_nll_bwd", s.dtype, C.c_int64(R), C.c_int64(K), C.c_int(dims), C.c_int(int(average)),
          _p(s), _p(lab), ct(dy), _p(dx))
    return dx


def argmax(x, dims=1):
    x = _f(x)
    inner, D, outer = _geom(x.shape, dims)
    shp = list(x.shape)
    shp[dims - 1] = 1
    idx = np.empty(shp, dtype=np.int32, order="F")
    _call("ko_argmax", x.dtype, C.c_int64(inner), C.c_int64(D), C.c_int64(outer), _p(x), _p(idx))
    return idx


def accuracy(scores, labels, dims=1, average=True):
    s, R, K = _rk(scores)
    lab = np.ascontiguousarray(labels, dtype=np.int32)
    cnt = C.c_int64(0)
    ok = _call("ko_accuracy", s.dtype, C.c_int64(R), C.c_int64(K), C.c_int(dims), _p(s), _p(lab),
               C.byref(cnt), restype=C.c_int64)
    return (ok / cnt.value) if average else (ok, cnt.value)


# ---- dropout -------------------------------------------------------------------------------
def dropout(x, p, u):
    """`u` holds the uniforms that Knet's rand!(y) would have drawn."""
    x = _f(x)
    y = np.array(u, dtype=x.dtype, order="F", copy=True)
    _call("ko_dropout", x.dtype, C.c_int64(x.size), C.c_double(p), _p(x), _p(y))
    return y


def dropback(p, y, dy):
    y = _f(y)
    dx = np.empty_like(y, order="F")
    _call("ko_dropback", y.dtype, C.c_int64(y.size), C.c_double(p), _p(y), _p(_f(dy, y.dtype)), _p(dx))
    return dx


# ---- optimizers (in place on w and the state arrays) ----------------------------------------
def _inplace(a):
    assert a.flags.f_contiguous or a.flags.c_contiguous
    return _p(a)


def sgd(w, g, lr=0.1):
    _call("ko_sgd", w.dtype, C.c_int64(w.size), _inplace(w), _p(_f(g)), C.c_double(lr))


def momentum(w, g, v, lr=0.05, gamma=0.95):
    _call("ko_momentum", w.dtype, C.c_int64(w.size), _inplace(w), _p(_f(g)), _inplace(v),
          C.c_double(lr), C.c_double(gamma))


def nesterov(w, g, v, lr=0.05, gamma=0.95):
    _call("ko_nesterov", w.dtype, C.c_int64(w.size), _inplace(w), _p(_f(g)), _inplace(v),
          C.c_double(lr), C.c_double(gamma))


def adagrad(w, g, G, lr=0.05, eps=1e-6):
    _call("ko_adagrad", w.dtype, C.c_int64(w.size), _inplace(w), _p(_f(g)), _inplace(G),
          C.c_double(lr), C.c_double(eps))


def rmsprop(w, g, G, lr=0.01, rho=0.9, eps=1e-6):
    _call("ko_rmsprop", w.dtype, C.c_int64(w.size), _inplace(w), _p(_f(g)), _inplace(G),
          C.c_double(lr), C.c_double(rho), C.c_double(eps))


def adadelta(w, g, G, delta, lr=1.0, rho=0.9, eps=1e-6):
    _call("ko_adadelta", w.dtype, C.c_int64(w.size), _inplace(w), _p(_f(g)), _inplace(G),
          _inplace(delta), C.c_double(lr), C.c_double(rho), C.c_double(eps))


def adam(w, g, m, v, t, lr=0.001, beta1=0.9, beta2=0.999, eps=1e-8):
    """`t` is the step number after Adam's increment (1 on the first call)."""
    _call("ko_adam", w.dtype, C.c_int64(w.size), _inplace(w), _p(_f(g)), _inplace(m), _inplace(v),
          C.c_double(lr), C.c_double(beta1), C.c_double(beta2), C.c_double(eps), C.c_int(t))


def gemm(A, B, ta=False, tb=False):
    """op(A)*op(B) with plain loops in the arrays' precision (for tiny cases)."""
    A, B = _f(A), _f(B)
    m = A.shape[1] if ta else A.shape[0]
    k = A.shape[0] if ta else A.shape[1]
    n = B.shape[0] if tb else B.shape[1]
    Cm = np.empty((m, n), dtype=A.dtype, order="F")
    _call("ko_gemm", A.dtype, C.c_int(ta), C.c_int(tb), C.c_int64(m), C.c_int64(n), C.c_int64(k),
          _p(A), _p(B), _p(Cm))
    return Cm


def matmul(A, B):
    """A*B for column-major operands with a column-major result, as Knet's CPU path gets it from
    BLAS gemm (src/knetarrays/linalg.jl:27-55 is the GPU twin): NumPy's product of the transposed
    views is row-major, so its transpose is the column-major A*B without a copy."""
    return (B.T @ A.T).T


def xavier_uniform(rows, cols, rng, dtype=np.float32):
    """param(rows, cols): Float64 draw, Float64 arithmetic, then conversion to `dtype`."""
    u = np.asfortranarray(rng.random((rows, cols)))
    w = np.empty_like(u, order="F")
    fn = lib().ko_xavier_uniform
    fn.restype = None
    fn(C.c_int64(rows), C.c_int64(cols), _p(u), _p(w))
    return np.asfortranarray(w.astype(dtype))


# ---- the MLP of README.md:55-62 / tutorial/40.mlp.ipynb trained as train.jl:22-36 does ------
class MLP:
    """chain of relu.(w*x .+ b) [+ dropout], last layer linear, loss nll(scores, labels).

    One step = forward, backward by AutoGrad's rules for these primitives, then
    update!(param, grad) with a per-parameter Adam (or SGD / Momentum) in params() order.
    `matmul` is NumPy's (BLAS) by default, the way Knet's CPU path calls BLAS gemm."""

    def __init__(self, sizes, rng, dtype=np.float32, pdrop=0.0, optimizer="adam", **hyper):
        self.dtype = np.dtype(dtype)
        self.w = [xavier_uniform(sizes[i + 1], sizes[i], rng, dtype) for i in range(len(sizes) - 1)]
        self.b = [np.zeros(sizes[i + 1], dtype=dtype) for i in range(len(sizes) - 1)]
        self.pdrop = pdrop
        self.optimizer = optimizer
        self.hyper = hyper
        self.state = [dict(t=0) for _ in range(2 * len(self.w))]
        self.timers = None         # set to {} to collect seconds spent in "gemm" and "update"

    def _mm(self, A, B):
        if self.timers is None:
            return matmul(A, B)
        t0 = time.perf_counter()
        r = matmul(A, B)
        self.timers["gemm"] = self.timers.get("gemm", 0.0) + time.perf_counter() - t0
        return r

    def params(self):
        out = []
        for w, b in zip(self.w, self.b):
            out += [w, b]
        return out

    def forward(self, x, uniforms=None):
        self.cache = []
        h = _f(x, self.dtype)
        L = len(self.w)
        for i, (w, b) in enumerate(zip(self.w, self.b)):
            z = binary("add", self._mm(w, h), b.reshape(-1, 1))
            if i < L - 1:
                y = unary("relu", z)
                if self.pdrop > 0 and uniforms is not None:
                    d = dropout(y, self.pdrop, uniforms[i])
                else:
                    d = None
                self.cache.append((h, y, d))
                h = d if d is not None else y
            else:
                self.cache.append((h, None, None))
                h = z
        return h

    def loss_and_grads(self, x, labels, uniforms=None):
        scores = self.forward(x, uniforms)
        loss = nll(scores, labels, dims=1)
        dz = nll_bwd(scores, labels, dims=1)
        grads = [None] * (2 * len(self.w))
        for i in reversed(range(len(self.w))):
            h, y, d = self.cache[i]
            if y is not None:
                if d is not None:
                    dz = dropback(self.pdrop, d, dz)
                dz = actback("reluback", dz, y)
            grads[2 * i + 1] = reduce_dim("sum", dz, 2).reshape(-1)
            grads[2 * i] = self._mm(dz, h.T)
            if i > 0:
                dz = self._mm(self.w[i].T, dz)
        return loss, grads

    def update(self, grads):
        for p, g, st in zip(self.params(), grads, self.state):
            if self.optimizer == "sgd":
                sgd(p, g, **self.hyper)
            elif self.optimizer == "momentum":
                if "v" not in st:
                    st["v"] = np.zeros_like(p, order="F")
                momentum(p, g, st["v"], **self.hyper)
            else:
                if "m" not in st:
                    st["m"] = np.zeros_like(p, order="F")
                    st["v"] = np.zeros_like(p, order="F")
                st["t"] += 1
                adam(p, g, st["m"], st["v"], st["t"], **self.hyper)

    def step(self, x, labels, uniforms=None):
        loss, grads = self.loss_and_grads(x, labels, uniforms)
        t0 = time.perf_counter()
        self.update(grads)
        if self.timers is not None:
            self.timers["update"] = self.timers.get("update", 0.0) + time.perf_counter() - t0
        return loss
