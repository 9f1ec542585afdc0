"""Gradient checks in the manner of the reference's own tests (AutoGrad gradcheck on every
primitive: test/unary.jl:48-79, test/binary.jl:50-127, test/reduction.jl:46-53,
test/loss.jl:12-19,63-72, test/dropout.jl:9-13) and a model written as a plain function of
Params trained with minimize's loop (src/train20/train.jl:22-36).  Float64, central
differences against the tape's gradient."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def rnd(shape, seed, shift=0.0):
    return np.asfortranarray(np.random.default_rng(seed).standard_normal(shape) + shift)


@pytest.mark.parametrize("name", ["relu", "sigm", "tanh", "elu", "selu"])
def test_activation_gradients(K, name):
    ag = K.autograd
    x = rnd((7, 5), 1)
    x[np.abs(x) < 0.05] += 0.2                      # keep away from the kink of relu/elu
    assert ag.gradcheck(getattr(ag, name), x)


@pytest.mark.parametrize("name", ["relu", "sigm", "tanh", "elu", "selu"])
def test_backward_functions_are_primitives_with_second_order_rules(K, name):
    """test/unary.jl:60-79: `@gcheck reluback.(dy,y)` etc. (gradients of the backward function wrt both
    of its arguments) and `grad(grad(f))` checked numerically."""
    ag = K.autograd
    fb = getattr(ag, name + "back")
    y = rnd((6, 4), 21)
    y[np.abs(y) < 0.05] += 0.2
    if name in ("sigm",):
        y = 1 / (1 + np.exp(-y))                      # values an output of sigm can take
    if name == "tanh":
        y = np.tanh(y)
    dy = rnd((6, 4), 22)
    ky, kdy = K.KnetArray(y), K.KnetArray(dy)
    assert ag.gradcheck(lambda v: fb(v, ky), dy), "wrt dy"
    assert ag.gradcheck(lambda v: fb(kdy, v), y), "wrt y"
    # second derivative of sum(c .* f(x)) through the recorded backward sweep
    x = rnd((5, 3), 23)
    x[np.abs(x) < 0.05] += 0.2
    c = K.KnetArray(rnd((5, 3), 24))
    f = getattr(ag, name)
    g = ag.gradfun(lambda v: ag.mul(f(v), c))
    assert ag.gradcheck(g, x), "grad(grad(f))"
    if name in ("sigm", "tanh"):                      # and the value of the first derivative itself
        got = g(K.KnetArray(x)).numpy()
        s = 1 / (1 + np.exp(-x))
        want = c.numpy() * (s * (1 - s) if name == "sigm" else 1 - np.tanh(x) ** 2)
        np.testing.assert_allclose(got, want, rtol=1e-12)


@pytest.mark.parametrize("dims", [1, 2, None])
def test_softmax_family_second_order(K, dims):
    """test/loss.jl:80-98: gradients of the softmax / logsoftmax backward functions wrt y and dy
    (the csb1 / csb2 rules), and grad(grad) of the forward functions."""
    ag = K.autograd
    x, dy = rnd((3, 4), 31), rnd((3, 4), 32)
    kx, kdy = K.KnetArray(x), K.KnetArray(dy)
    y1, y2 = K.softmax(kx, dims).numpy(), K.logsoftmax(kx, dims).numpy()
    c = K.KnetArray(rnd((3, 4), 33))
    for fb, y in ((ag.softmax_back, y1), (ag.logsoftmax_back, y2)):
        ky = K.KnetArray(y)
        assert ag.gradcheck(lambda v: ag.mul(fb(v, kdy, dims), c), y), (fb.__name__, "wrt y")
        assert ag.gradcheck(lambda v: ag.mul(fb(ky, v, dims), c), dy), (fb.__name__, "wrt dy")
    for f in (ag.softmax, ag.logsoftmax, ag.logsumexp):
        g = ag.gradfun(lambda v: ag.mul(f(v, dims), c) if f is not ag.logsumexp else f(v, dims))
        assert ag.gradcheck(g, x), (f.__name__, "grad(grad)")


def test_second_order_through_arithmetic_matmul_and_indexing(K):
    ag = K.autograd
    w = K.KnetArray(rnd((4, 5), 41))
    x = rnd((5, 3), 42)
    # f(x) = sum(tanh(w*x) .* (w*x)) ; its gradient function differentiated again
    g = ag.gradfun(lambda v: ag.mul(ag.tanh(ag.matmul(w, v)), ag.matmul(w, v)))
    assert ag.gradcheck(g, x)
    a = rnd((6, 4), 43, shift=3.0)
    b = K.KnetArray(rnd((6, 1), 44, shift=3.0))
    g2 = ag.gradfun(lambda v: ag.div(ag.mul(v, v), ag.add(v, b)))
    assert ag.gradcheck(g2, a)
    col = K.indexing.COLON
    g3 = ag.gradfun(lambda v: ag.mul(ag.getindex(v, col, [1, 3, 3]), ag.getindex(v, col, [2, 2, 4])))
    assert ag.gradcheck(g3, a)


@pytest.mark.parametrize("shapes", [((6, 5), (6, 5)), ((6, 5), (6, 1)), ((6, 5), (1, 5)), ((6,), (6, 5)),
                                    ((3, 4, 5), (3, 1, 5)), ((1,), (4, 3))], ids=str)
def test_broadcast_arithmetic_gradients(K, shapes):
    ag = K.autograd
    a, b = rnd(shapes[0], 2, shift=3.0), rnd(shapes[1], 3, shift=3.0)
    kb, ka = K.KnetArray(b), K.KnetArray(a)
    for op in (ag.add, ag.sub, ag.mul, ag.div):
        assert ag.gradcheck(lambda v: op(v, kb), a), (op.__name__, "lhs")
        assert ag.gradcheck(lambda v: op(ka, v), b), (op.__name__, "rhs")


def test_matmul_and_sum_gradients(K):
    ag = K.autograd
    w, x = rnd((4, 6), 4), rnd((6, 3), 5)
    assert ag.gradcheck(lambda v: ag.matmul(v, K.KnetArray(x)), w)
    assert ag.gradcheck(lambda v: ag.matmul(K.KnetArray(w), v), x)
    a = rnd((5, 4, 3), 6)
    c = K.KnetArray(rnd((5, 4, 3), 7))
    for dims in (1, 2, 3, (1, 2), (1, 3)):
        assert ag.gradcheck(lambda v: ag.mul(ag.sum(ag.mul(v, c), dims), 1.5), a), dims


@pytest.mark.parametrize("name", ["maximum", "minimum", "prod", "sumabs", "sumabs2", "maxabs", "minabs"])
def test_reduction_gradients(K, name):
    """test/reduction.jl:40-58: gradcheck of every reduction with dims = :, 1, 2 on small shapes."""
    ag = K.autograd
    f = getattr(ag, name)
    for shape in ((1,), (2,), (2, 1), (1, 2), (2, 2), (5, 4)):
        n = int(np.prod(shape))
        rng = np.random.default_rng(n + len(shape))
        if name == "prod":
            x = np.exp(0.01 * rng.standard_normal(shape))
        else:                       # distinct magnitudes, so that the extremum is unique
            x = (0.01 * rng.permutation(np.arange(1, n + 1)) * rng.choice([-1.0, 1.0], n)).reshape(shape)
        x = np.asfortranarray(x)
        c = K.KnetArray(rnd(shape, 7))
        assert ag.gradcheck(lambda v: f(v), x, delta=1e-7), (name, shape, "all")
        for d in range(1, len(shape) + 1):
            assert ag.gradcheck(lambda v: ag.mul(f(v, d), 1.5), x, delta=1e-7), (name, shape, d)
    # the gradient itself: maximum picks the position of the maximum
    p = ag.Param(K.KnetArray(np.asfortranarray(np.array([[1.0, 5.0], [3.0, 2.0]]))))
    ag.diff(lambda: ag.sum(ag.maximum(p, 1)))
    np.testing.assert_array_equal(p.grad.numpy(), [[0.0, 1.0], [1.0, 0.0]])


@pytest.mark.parametrize("dims", [1, 2, None])
def test_softmax_family_gradients(K, dims):
    ag = K.autograd
    a = rnd((10, 10), 8)
    c = K.KnetArray(rnd((10, 10), 9))
    for f in (ag.softmax, ag.logsoftmax):
        assert ag.gradcheck(lambda v: ag.mul(f(v, dims), c), a), f
    assert ag.gradcheck(lambda v: ag.logsumexp(v, dims), a)
    a3 = rnd((6, 5, 4), 10)
    for d in (1, 2, 3, (1, 2), (2, 3)):
        assert ag.gradcheck(lambda v: ag.logsumexp(v, d), a3), d


@pytest.mark.parametrize("dims", [1, 2])
def test_nll_gradient(K, dims):
    ag = K.autograd
    a = rnd((10, 10), 11)
    labels = np.random.default_rng(12).integers(0, 11, 10)
    labels[0] = 3
    assert ag.gradcheck(lambda v: ag.nll(v, labels, dims=dims), a)
    tot = lambda v: ag.nll(v, labels, dims=dims, average=False)     # noqa: E731
    assert ag.gradcheck(tot, a)


@pytest.mark.parametrize("dims", [1, 2])
@pytest.mark.parametrize("average", [True, False])
def test_nll_second_order(K, dims, average):
    """grad(grad) through the fused nll: the gradient function of v -> nll(c .* v) differentiated again,
    and the same for a loss built on top of the first gradient."""
    ag = K.autograd
    a = rnd((6, 6), 51)
    labels = np.array([1, 3, 0, 6, 2, 2])
    c = K.KnetArray(rnd((6, 6), 52))
    g = ag.gradfun(lambda v: ag.nll(ag.mul(v, c), labels, dims=dims, average=average))
    assert ag.gradcheck(g, a)
    g2 = ag.gradfun(lambda v: ag.mul(ag.nll(v, labels, dims=dims, average=average), ag.sum(ag.mul(v, v))))
    assert ag.gradcheck(g2, a)


def test_dropout_gradient_and_modes(K):
    ag = K.autograd
    a = rnd((20, 10), 13)
    assert ag.gradcheck(lambda v: ag.dropout(v, 0.5, seed=1, drop=True), a)
    x = K.KnetArray(a)
    assert ag.dropout(x, 0.5) is x                                   # not recording: identity
    p = ag.Param(x)
    t = ag.diff(lambda: ag.sum(ag.dropout(p, 0.5, seed=2)))          # recording: active
    y_zero = (p.grad.numpy() == 0).mean()
    assert 0.3 < y_zero < 0.7 and t.value().data.item() != a.sum()


def test_model_as_a_plain_function_trains_like_the_oracle(K, ko):
    # tutorial/40.mlp.ipynb style: params, a chain, nll; minimize's loop with Adam
    ag = K.autograd
    rng = np.random.default_rng(1)
    sizes, B = [784, 64, 10], 100
    ws = [ko.xavier_uniform(sizes[i + 1], sizes[i], rng) for i in range(2)]
    ref = ko.MLP(sizes, np.random.default_rng(0), lr=1e-3)
    ref.w = [np.asfortranarray(w.copy()) for w in ws]
    w1, w2 = (ag.Param(K.KnetArray(w)) for w in ws)
    b1, b2 = (ag.Param(K.KnetArray.zeros((n,))) for n in (64, 10))

    def model(x, y):
        h = ag.relu(w1 @ x + b1)
        return ag.nll(w2 @ h + b2, y)

    x = rng.random((784, B)).astype(np.float32)
    y = rng.integers(1, 11, B)
    kx = K.KnetArray(x)
    for step in range(25):
        l_ref = float(ref.step(x, y))
        l_gpu = ag.minimize_step(model, (kx, y), K.Adam(lr=1e-3))
        assert abs(l_gpu - l_ref) <= 1e-4, (step, l_gpu, l_ref)
    assert l_gpu < 2.2 and w1.opt.t == 25 and b2.opt.t == 25
    assert model(kx, y) == pytest.approx(float(ref.loss_and_grads(x, y)[0]), abs=1e-4)   # untracked call: a float
