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
The backward functions (reluback, sigmback, tanhback, eluback, seluback, the softmax family's)
are recorded primitives themselves with the second-order rules Knet declares
(src/ops20/activation.jl:15,29,42,58, src/ops20_gpu/activation.jl:13, src/ops20_gpu/softmax.jl:61-83),
so `gradfun(gradfun(f))` works as AutoGrad's `grad(grad(f))` does.
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
    """out: KnetArray result; parents: inputs (Value or not); back(dy, node) -> grads per parent,
    where `node` is the tracked result.  The rules are written with the tracked primitives of this
    module and refer to their tracked operands, so that a backward pass run while recording is
    itself recorded (gradients of gradients)."""
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


def _backprop(nodes, result, seed):
    """Reverse sweep over `nodes` (forward order) from `result` with incoming gradient `seed`;
    returns {id(value): gradient}.  Gradients are accumulated with this module's `add`
    (AutoGrad's addto!), which records when a tape is active."""
    grads = {id(result): seed}
    for node, parents, back in reversed(nodes):
        g = grads.get(id(node))
        if g is None:
            continue
        for p, gp in zip(parents, back(g, node)):
            if isinstance(p, Value) and gp is not None:
                grads[id(p)] = gp if id(p) not in grads else add(grads[id(p)], gp)
        if node is not result:
            del grads[id(node)]                                                      # free early
    return grads


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
        for leaf in tape.leaves:
            leaf.grad = None
        grads = _backprop(tape.nodes, res, ops.fill_(res.value.similar(), 1.0))
        for leaf in tape.leaves:
            leaf.grad = grads.get(id(leaf))
        res.grad = grads.get(id(res))
    return tape


def grad(tape, p):
    return p.grad


def params(tape):
    return list(tape.leaves)


def gradfun(f):
    """AutoGrad's `grad(f)`: the function x -> d sum(f(x)) / dx.  Called on a tracked value while
    a tape is recording, its backward sweep is recorded too, so gradfun(f) can be differentiated
    again (test/unary.jl:67-71 checks `grad(grad(f))` this way)."""
    def g(x):
        if _tape is not None and isinstance(x, Value):
            start = len(_tape.nodes)
            y = f(x)
            if not isinstance(y, Value):
                return None
            nodes = _tape.nodes[start:]
            return _backprop(nodes, y, ops.fill_(y.value.similar(), 1.0)).get(id(x))
        p = Param(_val(x))
        diff(lambda: sum(f(p)))
        return p.grad
    return g


# ---- shape helpers as primitives ------------------------------------------------------------------------
def reshape(x, shape):
    xv = _val(x)
    return _record(xv.reshape(shape), (x,), lambda dy, y: (reshape(dy, xv.shape),))


def _unbroadcast(g, shape):
    """AutoGrad's unbroadcast: sum the incoming gradient over the dims that were broadcast."""
    gs = _val(g).shape
    if tuple(gs) == tuple(shape):
        return g
    if _prod(shape) == 1:
        return reshape(sum(g), shape if shape else (1,))
    nd = len(gs)
    full = tuple(shape) + (1,) * (nd - len(shape))
    dims = tuple(i + 1 for i in range(nd) if full[i] == 1 and gs[i] > 1)
    return reshape(sum(g, dims) if dims else g, shape)


def _binary(op, x, y, dfx, dfy):
    xv, yv = _val(x), _val(y)
    z = ops.broadcast(op, xv, yv)

    def back(dz, znode):
        gx = _unbroadcast(dfx(dz, x, y, znode), xv.shape) if isinstance(x, Value) else None
        gy = _unbroadcast(dfy(dz, x, y, znode), yv.shape) if isinstance(y, Value) else None
        return gx, gy

    return _record(z, (x, y), back)


def add(x, y): return _binary("add", x, y, lambda dz, a, b, z: dz, lambda dz, a, b, z: dz)
def sub(x, y): return _binary("sub", x, y, lambda dz, a, b, z: dz, lambda dz, a, b, z: neg(dz))
def mul(x, y): return _binary("mul", x, y, lambda dz, a, b, z: mul(dz, b), lambda dz, a, b, z: mul(dz, a))
def div(x, y): return _binary("div", x, y, lambda dz, a, b, z: div(dz, b), lambda dz, a, b, z: neg(div(mul(dz, z), b)))
def neg(x): return mul(x, -1.0)


def exp(x):
    return _record(ops.exp(_val(x)), (x,), lambda dy, y: (mul(dy, y),))


def _mask(op, y, s):
    """(y op s) as a constant 0/1 array (no gradient flows through a comparison)."""
    return ops.broadcast(op, _val(y), s)


# ---- matrix products: w*x, a*b' and a'*b, each the backward of the others (linalg.jl:11-18) ---------------
def matmul(w, x):
    z = ops.matmul(_val(w), _val(x))
    return _record(z, (w, x), lambda dz, _: (A_mul_Bt(dz, x) if isinstance(w, Value) else None,
                                             At_mul_B(w, dz) if isinstance(x, Value) else None))


def A_mul_Bt(a, b):
    z = ops.A_mul_Bt(_val(a), _val(b))
    return _record(z, (a, b), lambda dz, _: (matmul(dz, b) if isinstance(a, Value) else None,
                                             At_mul_B(dz, a) if isinstance(b, Value) else None))


def At_mul_B(a, b):
    z = ops.At_mul_B(_val(a), _val(b))
    return _record(z, (a, b), lambda dz, _: (A_mul_Bt(b, dz) if isinstance(a, Value) else None,
                                             matmul(a, dz) if isinstance(b, Value) else None))


# ---- indexing ----------------------------------------------------------------------------------------------
def getindex(x, *I):
    """x[I...] with Julia's index kinds; the backward is AutoGrad's ungetindex: a zero array of
    x's shape that receives dy through addtoindex!, repeated indices accumulating
    (src/autograd_gpu/getindex.jl:5-18, addto.jl:24-82)."""
    from . import indexing
    xv = _val(x)
    y = indexing.getindex(xv, *I)
    if not isinstance(y, KnetArray):
        return y
    return _record(y, (x,), lambda dy, _: (_ungetindex(dy, xv, I),))


def _ungetindex(dy, like, I):
    """zeros(like) with dy added at I; linear in dy, so its own backward is getindex."""
    from . import indexing
    dx = indexing.addtoindex_(ops.fill_(like.similar(), 0.0), _val(dy), *I)
    return _record(dx, (dy,), lambda ddx, _: (getindex(ddx, *I),))


# ---- activations and their backward forms, both as primitives ------------------------------------------------
_LAMBDA01, _LAMBDA_ALPHA01 = 1.0507009873554805, 1.7580993408473773


def _second(name, ddx, dy, y):
    """Gradient of <name>back.(dy, y) wrt y for an incoming ddx (src/ops20/activation.jl:15,29,42,58;
    tanh: src/ops20_gpu/activation.jl:13)."""
    if name == "relu":
        return None
    if name in ("elu", "selu"):
        return mul(mul(ddx, dy), _mask("lt", y, 0.0))                      # ddx.*dy.*(y.<0)
    if name == "sigm":
        return mul(mul(ddx, dy), sub(1.0, mul(2.0, y)))                    # ddx.*dy.*(1 .- 2 .* y)
    if name == "tanh":
        return mul(ddx, mul(-2.0, mul(dy, y)))                             # ddx.*(-2 .* dy.*y)
    raise KeyError(name)


def _actback_primitive(name):
    def fb(dy, y):
        """<name>back.(dy, y); every one of them is linear in dy, so the gradient wrt dy of an
        incoming ddx is <name>back.(ddx, y) (e.g. reluback: ddx.*(y.>0))."""
        dx = ops.actback(name + "back", _val(dy), _val(y))
        return _record(dx, (dy, y), lambda ddx, _: (fb(ddx, y) if isinstance(dy, Value) else None,
                                                    _second(name, ddx, dy, y) if isinstance(y, Value) else None))
    fb.__name__ = name + "back"
    return fb


reluback, sigmback, tanhback, eluback, seluback = (_actback_primitive(n) for n in ("relu", "sigm", "tanh", "elu", "selu"))
_ACTBACK = {"relu": reluback, "sigm": sigmback, "tanh": tanhback, "elu": eluback, "selu": seluback}


def _activation(name):
    def f(x):
        y = ops.unary(name, _val(x))
        return _record(y, (x,), lambda dy, ynode: (_ACTBACK[name](dy, ynode),))
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
    return _record(y, (x,), lambda dy, _: (_dropback(dy, y, xv, p),))


def _dropback(dy, y, x, p):
    """dropback(dy, y, x, p): a fixed mask and scale applied to dy, so linear in dy."""
    return _record(ops.dropback(_val(dy), y, x, p), (dy,), lambda ddx, _: (_dropback(ddx, y, x, p),))


# ---- softmax family; the backward forms are primitives with the rules of src/ops20_gpu/softmax.jl:61-83 -----
def softmax_back(y, dy, dims=None):
    """∇softmax = y.*dy .- y.*sum(y.*dy).  wrt y: ddx.*dy - dy.*sum(y.*ddx) - ddx.*sum(y.*dy);
    wrt dy: y.*(ddx .- sum(y.*ddx)) (csb1 / csb2 of the reference)."""
    dx = ops.softmax_back(_val(y), _val(dy), dims)

    def back(ddx, _):
        gy = gdy = None
        if isinstance(y, Value):
            gy = sub(sub(mul(ddx, dy), mul(dy, sum(mul(y, ddx), dims))), mul(ddx, sum(mul(y, dy), dims)))
        if isinstance(dy, Value):
            gdy = softmax_back(y, ddx, dims)
        return gy, gdy

    return _record(dx, (y, dy), back)


def logsoftmax_back(y, dy, dims=None):
    """∇logsoftmax = dy - exp.(y).*sum(dy).  wrt y: -ddx.*exp.(y).*sum(dy); wrt dy:
    ddx .- sum(ddx.*exp.(y))."""
    dx = ops.logsoftmax_back(_val(y), _val(dy), dims)

    def back(ddx, _):
        gy = gdy = None
        if isinstance(y, Value):
            gy = neg(mul(mul(ddx, exp(y)), sum(dy, dims)))
        if isinstance(dy, Value):
            gdy = sub(ddx, sum(mul(ddx, exp(y)), dims))
        return gy, gdy

    return _record(dx, (y, dy), back)


def softmax(x, dims=None):
    return _record(ops.softmax(_val(x), dims), (x,), lambda dy, y: (softmax_back(y, dy, dims),))


def logsoftmax(x, dims=None):
    return _record(ops.logsoftmax(_val(x), dims), (x,), lambda dy, y: (logsoftmax_back(y, dy, dims),))


logp = logsoftmax


def logsumexp_back(x, y, dy, dims=None):
    """∇logsumexp = dy .* exp.(x .- y) (src/ops20/softmax.jl:72-74), fused; its own gradients are
    spelled with the generic primitives: with e = exp.(x .- y), wrt x: ddx.*dy.*e, wrt y:
    -sum(ddx.*dy.*e), wrt dy: sum(ddx.*e)."""
    dx = ops.logsumexp_back(_val(x), _val(y), _val(dy), dims)

    def back(ddx, dxnode):
        e = exp(sub(x, y))
        t = mul(ddx, dxnode)
        return (t if isinstance(x, Value) else None,
                neg(sum(t, dims)) if isinstance(y, Value) else None,
                sum(mul(ddx, e), dims) if isinstance(dy, Value) else None)

    return _record(dx, (x, y, dy), back)


def logsumexp(x, dims=None):
    return _record(ops.logsumexp(_val(x), dims), (x,), lambda dy, y: (logsumexp_back(x, y, dy, dims),))


def sum(x, dims=None):  # noqa: A001
    """sum(x; dims); with dims=None the result is a one-element tracked array."""
    xv = _val(x)
    if dims is None:
        s = ops.reduce("sum", xv, None)
        y = KnetArray(torch.full((1,), s, dtype=xv.dtype, device=xv.data.device), (1,))
    else:
        y = ops.reduce("sum", xv, dims)

    def back(dy, _):
        ones = ops.fill_(xv.similar(), 1.0)
        return (mul(ones, reshape(dy, y.shape) if dims is not None else dy),)

    return _record(y, (x,), back)


def _reduction(op, rule):
    """A reduction with `dims` as a primitive; `rule(dyb, x, yb)` gives the gradient from the
    incoming gradient and the result, both broadcast back to x's shape by the arithmetic itself.
    The rules are AutoGrad's for Base reductions (gradcheck'ed on KnetArrays in test/reduction.jl:40-70)."""
    def f(x, dims=None):
        xv = _val(x)
        if dims is None:
            v = ops.reduce(op, xv, None)
            y = KnetArray(torch.full((1,), v, dtype=xv.dtype, device=xv.data.device), (1,) * max(xv.ndim, 1))
        else:
            y = ops.reduce(op, xv, dims)
        return _record(y, (x,), lambda dy, ynode: (rule(reshape(dy, y.shape), x, ynode),))
    f.__name__ = op
    return f


def _ones_like(x):
    return ops.fill_(_val(x).similar(), 1.0)


def _sign(x):
    return ops.unary("sign", _val(x))


maximum = _reduction("maximum", lambda dy, x, y: mul(mul(_ones_like(x), dy), _mask("eq", ops.broadcast("sub", _val(x), _val(y)), 0.0)))
minimum = _reduction("minimum", lambda dy, x, y: mul(mul(_ones_like(x), dy), _mask("eq", ops.broadcast("sub", _val(x), _val(y)), 0.0)))
prod = _reduction("prod", lambda dy, x, y: div(mul(dy, y), x))
sumabs = _reduction("sumabs", lambda dy, x, y: mul(dy, _sign(x)))
sumabs2 = _reduction("sumabs2", lambda dy, x, y: mul(mul(dy, 2.0), x))
maxabs = _reduction("maxabs", lambda dy, x, y: mul(mul(dy, _sign(x)), _mask("eq", ops.broadcast("sub", ops.unary("abs", _val(x)), _val(y)), 0.0)))
minabs = _reduction("minabs", lambda dy, x, y: mul(mul(dy, _sign(x)), _mask("eq", ops.broadcast("sub", ops.unary("abs", _val(x)), _val(y)), 0.0)))


def _nll_back(scores, res, dims, average, dy):
    """Gradient of the fused nll wrt scores, (softmax(scores) - onehot) * dy / count on the used
    instances, as a primitive of (scores, dy).  Its own backward for an incoming ddx: wrt scores
    dy/count * mask .* (p .* ddx .- p .* sum(p .* ddx)) with p = softmax(scores), i.e. the softmax
    backward rule applied to ddx; wrt dy sum(ddx .* dx) / dy.  That is what differentiating
    -sum(logsoftmax(scores)[labels]) / count twice gives (src/ops20/loss.jl:37-41 composes nll that way)."""
    sv, dyv = _val(scores), _val(dy)
    dyf = float(dyv.data.item())
    dx = ops.nll_back(sv, res.labels, dims=dims, average=average, dy=dyf, count=res.count)

    def back(ddx, _):
        R = sv.shape[0]
        K = len(sv) // R
        used = (res.labels != 0).to(sv.dtype)
        mask = KnetArray(used, (1, K) if dims == 1 else (R, 1))
        scale = (1.0 / max(int(res.count.item()), 1)) if average else 1.0
        v = mul(ddx, mask.reshape(mask.shape + (1,) * (sv.ndim - 2)) if sv.ndim > 2 else mask)
        gs = gdy = None
        if isinstance(scores, Value):
            gs = mul(softmax_back(ops.softmax(sv, dims), v, dims), mul(dy, scale))
        if isinstance(dy, Value):
            unit = ops.nll_back(sv, res.labels, dims=dims, average=average, dy=1.0, count=res.count)
            gdy = reshape(sum(mul(ddx, unit)), dyv.shape)
        return gs, gdy

    return _record(dx, (scores, dy), back)


def nll(scores, labels, dims=1, average=True):
    """nll(scores, labels; dims, average) (src/ops20/loss.jl:37-41) as one fused primitive: the
    forward keeps total and count on the device, the backward is (softmax - onehot) * dy/count,
    itself a primitive, so the loss can be differentiated twice."""
    sv = _val(scores)
    res = ops.nll_device(sv, labels, dims)
    if not _tracked(scores):
        return res.value(average)
    y = KnetArray((res.total / res.count.to(res.total.dtype)) if average else res.total.clone(), (1,))
    return _record(y, (scores,), lambda dy, _: (_nll_back(scores, res, dims, average, dy),))


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
    g = p.grad.numpy() if p.grad is not None else np.zeros(x.shape)      # `nothing` is a zero gradient
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
