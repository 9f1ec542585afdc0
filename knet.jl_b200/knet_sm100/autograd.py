"""A small reverse-mode tape with Knet's backward rules, so that models written as plain
functions of `Param`s run through the library's forward and backward kernels the way
AutoGrad-recorded Knet models do.

AutoGrad.jl itself is an external Julia package; what is mirrored here is the part of its
contract that Knet relies on (src/train20/train.jl:4,26-31): `diff(f)` records a call and
returns a tape whose value is the loss, `grad(tape, param)` returns the gradient, `params(tape)`
lists the parameters met.  The backward rule of each primitive is the one Knet declares:
activations `@primitive relu(x),dy,y reluback.(dy,y)` (src/ops20/activation.jl:13-56),
dropout (src/ops20/dropout.jl:42), softmax family (src/ops20/softmax.jl:76-78), broadcasting
arithmetic with AutoGrad's unbroadcast (a sum over the broadcast dims), `w*x` with
A_mul_Bt / At_mul_B (src/knetarrays/linalg.jl:12-18), `sum`, and nll as one fused primitive.
"""
import numpy as np
import torch

from . import ops
from .karray import KnetArray, _prod

_tape = None


class Value:
    """A tracked array: `.value` is the KnetArray, `.grad` is filled by backward."""

    def __init__(self, value):
        self.value, self.grad = value, None

    shape = property(lambda self: self.value.shape)
    dtype = property(lambda self: self.value.dtype)

    def __add__(self, o): return add(self, o)
    def __radd__(self, o): return add(o, self)
    def __sub__(self, o): return sub(self, o)
    def __rsub__(self, o): return sub(o, self)
    def __mul__(self, o): return mul(self, o)
    def __rmul__(self, o): return mul(o, self)
    def __truediv__(self, o): return div(self, o)
    def __rtruediv__(self, o): return div(o, self)
    def __matmul__(self, o): return matmul(self, o)
    def __rmatmul__(self, o): return matmul(o, self)
    def __neg__(self): return mul(self, -1.0)
    def __getitem__(self, I): return getindex(self, *(I if isinstance(I, tuple) else (I,)))


class Param(Value):
    """A parameter (src/train20/param.jl:22-24): a tracked leaf with an optimizer slot."""

    def __init__(self, value, opt=None):
        super().__init__(value)
        self.opt = opt


class Tape:
    def __init__(self):
        self.nodes, self.leaves, self.result = [], [], None

    def value(self):
        r = self.result
        return r if not isinstance(r, Value) else r.value


def _val(x):
    return x.value if isinstance(x, Value) else x


def _tracked(*xs):
    return _tape is not None and any(isinstance(x, Value) for x in xs)


def _record(out, parents, back):
    """out: KnetArray result; parents: inputs (Value or not); back(dy) -> grads per parent."""
    if not _tracked(*parents):
        return out
    node = Value(out)
    for p in parents:
        if isinstance(p, Param) and p not in _tape.leaves:
            _tape.leaves.append(p)
    _tape.nodes.append((node, parents, back))
    return node


def recording():
    """AutoGrad.recording(): True inside diff()."""
    return _tape is not None


def diff(f, *args, **kw):
    """`@diff f(args...)`: run f with recording on and back-propagate from its result, which
    must be a tracked scalar-like array (one element) or a Python float built from one."""
    global _tape
    tape, prev = Tape(), _tape
    _tape = tape
    try:
        tape.result = f(*args, **kw)
    finally:
        _tape = prev
    res = tape.result
    if isinstance(res, Value):
        for node, _, _ in tape.nodes:
            node.grad = None
        for leaf in tape.leaves:
            leaf.grad = None
        res.grad = ops.fill_(res.value.similar(), 1.0)
        for node, parents, back in reversed(tape.nodes):
            if node.grad is None:
                continue
            grads = back(node.grad)
            for p, g in zip(parents, grads):
                if isinstance(p, Value) and g is not None:
                    p.grad = g if p.grad is None else ops.broadcast("add", p.grad, g)   # addto!
            if node is not res:
                node.grad = None                                                         # free early
    return tape


def grad(tape, p):
    return p.grad


def params(tape):
    return list(tape.leaves)


# ---- unbroadcast: sum the incoming gradient over the dims that were broadcast -------------------------
def _unbroadcast(g, shape):
    gs = g.shape
    if tuple(gs) == tuple(shape):
        return g
    if _prod(shape) == 1:
        s = ops.reduce("sum", g, None)
        return KnetArray(torch.full((1,), s, dtype=g.dtype, device=g.data.device), shape if shape else (1,))
    nd = len(gs)
    full = tuple(shape) + (1,) * (nd - len(shape))
    dims = tuple(i + 1 for i in range(nd) if full[i] == 1 and gs[i] > 1)
    out = ops.reduce("sum", g, dims) if dims else g
    return out.reshape(shape)


def _binary(op, x, y, dfx, dfy):
    xv, yv = _val(x), _val(y)
    z = ops.broadcast(op, xv, yv)

    def back(dz):
        gx = _unbroadcast(dfx(dz, xv, yv, z), xv.shape) if isinstance(x, Value) else None
        gy = _unbroadcast(dfy(dz, xv, yv, z), yv.shape) if isinstance(y, Value) else None
        return gx, gy

    return _record(z, (x, y), back)


def add(x, y): return _binary("add", x, y, lambda dz, a, b, z: dz, lambda dz, a, b, z: dz)
def sub(x, y): return _binary("sub", x, y, lambda dz, a, b, z: dz, lambda dz, a, b, z: ops.unary("neg", dz))
def mul(x, y): return _binary("mul", x, y, lambda dz, a, b, z: dz * b, lambda dz, a, b, z: dz * a)
def div(x, y): return _binary("div", x, y, lambda dz, a, b, z: dz / b, lambda dz, a, b, z: ops.unary("neg", dz * z / b))


def matmul(w, x):
    wv, xv = _val(w), _val(x)
    z = ops.matmul(wv, xv)
    return _record(z, (w, x), lambda dz: (ops.A_mul_Bt(dz, xv) if isinstance(w, Value) else None,
                                          ops.At_mul_B(wv, dz) if isinstance(x, Value) else None))


def getindex(x, *I):
    """x[I...] with Julia's index kinds; the backward is AutoGrad's ungetindex: a zero array of
    x's shape that receives dy through addtoindex!, repeated indices accumulating
    (src/autograd_gpu/getindex.jl:5-18, addto.jl:24-82)."""
    from . import indexing
    xv = _val(x)
    y = indexing.getindex(xv, *I)
    if not isinstance(y, KnetArray):
        return y

    def back(dy):
        dx = ops.fill_(xv.similar(), 0.0)
        return (indexing.addtoindex_(dx, dy, *I),)

    return _record(y, (x,), back)


def _activation(name):
    def f(x):
        y = ops.unary(name, _val(x))
        return _record(y, (x,), lambda dy: (ops.actback(name + "back", dy, y),))
    f.__name__ = name
    return f


relu, sigm, tanh, elu, selu = (_activation(n) for n in ("relu", "sigm", "tanh", "elu", "selu"))


def dropout(x, p, seed=0, drop=None, uniforms=None):
    """dropout(x, p; seed, drop=recording()) (src/ops20/dropout.jl:15-42)."""
    drop = recording() if drop is None else drop
    xv = _val(x)
    y = ops.dropout(xv, p, seed=seed, drop=drop, uniforms=uniforms)
    if y is xv:
        return x
    return _record(y, (x,), lambda dy: (ops.dropback(dy, y, xv, p),))


def _soft(fwd, bwd):
    def f(x, dims=None):
        y = fwd(_val(x), dims)
        return _record(y, (x,), lambda dy: (bwd(y, dy, dims),))
    return f


softmax = _soft(ops.softmax, ops.softmax_back)
logsoftmax = _soft(ops.logsoftmax, ops.logsoftmax_back)
logp = logsoftmax


def logsumexp(x, dims=None):
    xv = _val(x)
    y = ops.logsumexp(xv, dims)
    return _record(y, (x,), lambda dy: (ops.logsumexp_back(xv, y, dy, dims),))


def sum(x, dims=None):  # noqa: A001
    """sum(x; dims); with dims=None the result is a one-element tracked array."""
    xv = _val(x)
    if dims is None:
        s = ops.reduce("sum", xv, None)
        y = KnetArray(torch.full((1,), s, dtype=xv.dtype, device=xv.data.device), (1,))
    else:
        y = ops.reduce("sum", xv, dims)

    def back(dy):
        ones = ops.fill_(xv.similar(), 1.0)
        return (ops.broadcast("mul", ones, dy.reshape(y.shape) if dims is not None else dy),)

    return _record(y, (x,), back)


def nll(scores, labels, dims=1, average=True):
    """nll(scores, labels; dims, average) (src/ops20/loss.jl:37-41) as one fused primitive: the
    forward keeps total and count on the device, the backward is (softmax - onehot) * dy/count."""
    sv = _val(scores)
    res = ops.nll_device(sv, labels, dims)
    if not _tracked(scores):
        return res.value(average)
    y = KnetArray((res.total / res.count.to(res.total.dtype)) if average else res.total.clone(), (1,))

    def back(dy):
        return (ops.nll_back(sv, res.labels, dims=dims, average=average, dy=float(dy.data.item()), count=res.count),)

    return _record(y, (scores,), back)


def minimize_step(f, args, algo, parameters=None):
    """One iteration of `minimize(f, data, algo)` (src/train20/train.jl:22-36): differentiate
    f(args...), give every parameter a clone of `algo` on first sight, update!, return the loss."""
    from .train import update_
    tape = diff(f, *args)
    for p in (parameters if parameters is not None else params(tape)):
        if p.opt is None:
            p.opt = algo.clone()
        if p.grad is not None:
            update_(p.value, p.grad, p.opt)
    return float(tape.value().data.item())


def _total(r):
    """sum of an untracked result: an array, or the float/tuple an untracked nll returns."""
    if isinstance(r, tuple):
        r = r[0]
    return float(r) if not isinstance(r, (Value, KnetArray)) else float(ops.reduce("sum", _val(r), None))


def gradcheck(f, x, delta=None, rtol=1e-4, atol=1e-6, nsample=12, seed=0):
    """Numerical check in the spirit of AutoGrad.gradcheck: compares the tape's gradient of
    sum(f(x)) with central differences on a sample of entries.  x is a host NumPy array."""
    rng = np.random.default_rng(seed)
    p = Param(KnetArray(np.asfortranarray(x)))
    diff(lambda: sum(f(p)))
    g = p.grad.numpy()
    delta = delta or (1e-6 if x.dtype == np.float64 else 1e-2)
    flat = np.asfortranarray(x).reshape(-1, order="F")
    ok = True
    for i in rng.choice(flat.size, size=min(nsample, flat.size), replace=False):
        xp, xm = flat.copy(), flat.copy()
        xp[i] += delta
        xm[i] -= delta
        fp, fm = (_total(f(KnetArray(v.reshape(x.shape, order="F")))) for v in (xp, xm))
        num = (fp - fm) / (2 * delta)
        ana = g.reshape(-1, order="F")[i]
        if abs(num - ana) > atol + rtol * max(abs(num), abs(ana)):
            ok = False
    return ok
