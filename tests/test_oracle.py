"""Pins of the CPU checker against the known answers Knet's own sources and tests hold for
this path.  These run without a GPU."""
import json
import os

import numpy as np
import pytest

with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "knet_known_answers.json")) as _f:
    GOLDEN = json.load(_f)


def test_nll_docstring_example(ko):
    # src/ops20/loss.jl:22-34: the docstring prints 2.1657e-5 for this example; evaluating its
    # own formula -(log p[1,1] + log p[2,2])/2 in Float64 gives 2.1100e-5, so the printed
    # digits are matched to two figures and the formula exactly.
    ex = GOLDEN["nll_docstring_example"]
    scores, labels = np.array(ex["scores"]), ex["labels"]
    got = ko.nll(scores, labels)
    p = np.exp(scores) / np.exp(scores).sum(axis=0)
    want = -(np.log(p[0, 0]) + np.log(p[1, 1])) / 2
    assert got == pytest.approx(want, rel=1e-12)
    assert got == pytest.approx(ex["printed_value"], rel=3e-2)
    tot, cnt = ko.nll(scores, labels, average=False)
    assert cnt == 2 and tot == pytest.approx(2 * want, rel=1e-12)
    # Float32 follows the same path
    assert ko.nll(scores.astype(np.float32), labels) == pytest.approx(want, rel=2e-3)


def test_nll_skips_zero_labels_and_dims2(ko):
    rng = np.random.default_rng(3)
    s = np.asfortranarray(rng.standard_normal((10, 7)))
    lab = rng.integers(1, 11, 7)
    full = ko.nll(s, lab, dims=1, average=False)
    lab0 = lab.copy()
    lab0[2] = 0
    part = ko.nll(s, lab0, dims=1, average=False)
    lsm = ko.logsoftmax(s, 1)
    assert part[1] == 6 and full[1] == 7
    assert full[0] - part[0] == pytest.approx(-lsm[lab[2] - 1, 2], rel=1e-12)
    # dims=2: instances in rows (findindices, loss.jl:129-137)
    assert ko.nll(np.asfortranarray(s.T), lab, dims=2) == pytest.approx(ko.nll(s, lab, dims=1), rel=1e-12)


def test_accuracy_identities(ko):
    # test/ops20.jl:120-123: after adding 1000 to row 1, argmax is class 1 everywhere
    rng = np.random.default_rng(0)
    scores = np.asfortranarray(rng.standard_normal((10, 100)))
    labels1 = rng.integers(1, 11, 100)
    labels2 = rng.integers(1, 101, 10)
    scores[0, :] += 1000
    assert ko.accuracy(scores, labels1, dims=1) == np.sum(labels1 == 1) / len(labels1)
    scores[:, 0] += 10000
    assert ko.accuracy(scores, labels2, dims=2) == np.sum(labels2 == 1) / len(labels2)


def test_argmax_first_maximum_wins(ko):
    x = np.asfortranarray(np.array([[1.0, 5.0, 5.0], [7.0, 7.0, 2.0]]).T)  # (3,2)
    assert ko.argmax(x, 1).reshape(-1).tolist() == [2, 1]
    assert ko.argmax(x, 2).reshape(-1).tolist() == [2, 2, 1]


@pytest.mark.parametrize("dims", [1, 2, 3])
def test_softmax_is_exp_logsoftmax_and_sums_to_one(ko, dims):
    # test/loss.jl:47-56
    a = np.random.default_rng(1).random((10, 10, 10))
    sm, ls = ko.softmax(a, dims), ko.logsoftmax(a, dims)
    np.testing.assert_allclose(sm, np.exp(ls), rtol=1e-12)
    np.testing.assert_allclose(ko.reduce_dim("sum", sm, dims), 1.0, rtol=1e-12)
    np.testing.assert_allclose(ko.logsumexp(a, dims), np.log(np.exp(a).sum(axis=dims - 1, keepdims=True)), rtol=1e-12)


def _numgrad(f, x, eps=1e-6):
    g = np.zeros_like(x)
    it = np.nditer(x, flags=["multi_index"])
    for _ in it:
        i = it.multi_index
        xp, xm = x.copy(order="F"), x.copy(order="F")
        xp[i] += eps
        xm[i] -= eps
        g[i] = (f(xp) - f(xm)) / (2 * eps)
    return g


@pytest.mark.parametrize("dims", [1, 2])
def test_backward_rules_against_numerical_gradients(ko, dims):
    # the reference checks these rules with gradcheck (test/loss.jl:12-19,63-66)
    rng = np.random.default_rng(5)
    x = np.asfortranarray(rng.standard_normal((6, 5)))
    dy = np.asfortranarray(rng.standard_normal((6, 5)))
    for fwd, bwd in ((ko.softmax, ko.softmax_bwd), (ko.logsoftmax, ko.logsoftmax_bwd)):
        ana = bwd(fwd(x, dims), dy, dims)
        num = _numgrad(lambda v: float((fwd(v, dims) * dy).sum()), x)
        np.testing.assert_allclose(ana, num, atol=1e-7)
    shp = [6, 5]
    shp[dims - 1] = 1
    dyr = np.asfortranarray(rng.standard_normal(shp))
    ana = ko.logsumexp_bwd(x, ko.logsumexp(x, dims), dyr, dims)
    num = _numgrad(lambda v: float((ko.logsumexp(v, dims) * dyr).sum()), x)
    np.testing.assert_allclose(ana, num, atol=1e-7)
    n_inst = x.shape[1] if dims == 1 else x.shape[0]
    n_cls = x.shape[0] if dims == 1 else x.shape[1]
    lab = rng.integers(0, n_cls + 1, n_inst)
    lab[0] = 0
    ana = ko.nll_bwd(x, lab, dims)
    num = _numgrad(lambda v: float(ko.nll(v, lab, dims)), x)
    np.testing.assert_allclose(ana, num, atol=1e-7)


def test_activation_definitions(ko):
    # src/ops20/activation.jl:12-13,26-27,55-56; ops20_gpu/activation.jl:11
    x = np.array([-2.0, -0.0, 0.0, 0.5, 3.0])
    np.testing.assert_array_equal(ko.unary("relu", x), [0, 0, 0, 0.5, 3])
    assert not np.signbit(ko.unary("relu", x)[1])
    np.testing.assert_allclose(ko.unary("sigm", x), 1 / (1 + np.exp(-x)), rtol=1e-15)
    np.testing.assert_allclose(ko.unary("elu", x), np.where(x >= 0, x, np.exp(x) - 1), rtol=1e-15)
    np.testing.assert_allclose(ko.unary("tanh", x), np.tanh(x), rtol=1e-15)
    y, dy = np.array([-0.5, 0.0, 0.25, 2.0]), np.array([1.0, 2.0, 3.0, 4.0])
    np.testing.assert_array_equal(ko.actback("reluback", dy, y), [0, 0, 3, 4])
    np.testing.assert_array_equal(ko.actback("eluback", dy, y), [0.5, 2, 3, 4])
    np.testing.assert_array_equal(ko.actback("sigmback", dy, y), dy * y * (1 - y))
    np.testing.assert_array_equal(ko.actback("tanhback", dy, y), dy * (1 - y * y))
    assert np.isnan(ko.unary("relu", np.array([np.nan]))[0])


def test_float32_exp_is_correctly_rounded(ko):
    x = np.random.default_rng(7).standard_normal(20000).astype(np.float32) * 5
    np.testing.assert_array_equal(ko.unary("exp", x), np.exp(x.astype(np.float64)).astype(np.float32))


def test_float64_exp_tanh_log_are_correctly_rounded(ko):
    """The oracle's Float64 exp / tanh / log against 200-bit mpmath values rounded once to double
    (the long double value decides unless it is too close to a rounding boundary, then libquadmath)."""
    import mpmath as mp
    rng = np.random.default_rng(3)
    x = np.concatenate([rng.standard_normal(6000) * 4, rng.uniform(-700, 700, 2000), [0.0, -0.0, 1e-300, -745.0, 709.7]])
    with mp.workprec(200):
        for name, f, arg in (("exp", mp.exp, x), ("tanh", mp.tanh, x), ("log", mp.log, np.abs(x[np.abs(x) > 0]))):
            got = ko.unary(name, arg.astype(np.float64))
            want = np.array([float(f(mp.mpf(float(v)))) for v in arg])
            np.testing.assert_array_equal(got, want, err_msg=name)


def test_dropout_matches_cpu_loop_and_second_moment(ko):
    # src/ops20/dropout.jl:45-71; statistical check of test/dropout.jl:14-16
    G = GOLDEN["dropout_second_moment"]
    rng = np.random.default_rng(2)
    x = rng.random(tuple(G["shape"]))
    u = rng.random(tuple(G["shape"]))
    y = ko.dropout(x, G["p"], u)
    np.testing.assert_array_equal(y, np.where(u > 0.5, x / 0.5, 0))
    assert (y ** 2).sum() == pytest.approx(2 * (x ** 2).sum(), rel=G["rtol"])
    dy = rng.standard_normal((100, 100))
    np.testing.assert_array_equal(ko.dropback(0.5, y, dy), np.where(y == 0, 0, dy / 0.5))


def test_reductions_regression_shapes(ko):
    # test/reduction.jl:59-70 shapes; Julia keeps reduced dims as size 1
    rng = np.random.default_rng(4)
    for shape in ((10, 1000), (1000, 10)):
        x = np.asfortranarray(rng.standard_normal(shape))
        for op, ref in (("sum", np.sum), ("maximum", np.max), ("minimum", np.min)):
            for d in (1, 2):
                np.testing.assert_allclose(ko.reduce_dim(op, x, d), ref(x, axis=d - 1, keepdims=True), rtol=1e-12)
            assert ko.reduce_all(op, x) == pytest.approx(ref(x), rel=1e-12)
        np.testing.assert_allclose(ko.reduce_dim("sumabs2", x, 1), (x * x).sum(0, keepdims=True), rtol=1e-12)
        assert ko.reduce_all("countnz", x) == x.size


def rosenbrock_grad(x):
    f = np.sum((1 - x[:-1]) ** 2 + 100 * (x[1:] - x[:-1] ** 2) ** 2)
    g = np.zeros_like(x)
    g[:-1] += -2 * (1 - x[:-1]) - 400 * x[:-1] * (x[1:] - x[:-1] ** 2)
    g[1:] += 200 * (x[1:] - x[:-1] ** 2)
    return f, g


@pytest.mark.parametrize("name,hyper", sorted(GOLDEN["rosenbrock"]["optimizers"].items()))
def test_rosenbrock_convergence(ko, name, hyper):
    # test/update.jl:26-62: 6-d Rosenbrock must reach f <= 0.1 within 10000 steps.  The start is
    # a normal draw; Julia's stream for seed 123456789 cannot be reproduced here and the
    # reference notes that the test is sensitive to it (update.jl test, line 24): the 6-d
    # function has a second minimum at f = 3.97 that some starts fall into.
    R = GOLDEN["rosenbrock"]
    w = np.random.default_rng(0).standard_normal(R["dims"])
    st = [np.zeros(R["dims"]), np.zeros(R["dims"])]
    f, t = 1.0, 0
    for t in range(1, R["maxiter"] + 1):
        f, g = rosenbrock_grad(w)
        if f <= R["ftol"]:
            break
        if name == "sgd":
            ko.sgd(w, g, **hyper)
        elif name == "adam":
            ko.adam(w, g, st[0], st[1], t, **hyper)
        elif name == "adadelta":
            ko.adadelta(w, g, st[0], st[1], **hyper)
        else:
            getattr(ko, name)(w, g, st[0], **hyper)
    assert f <= R["ftol"], (name, f, t)


def test_adam_operation_order(ko):
    # update.jl:559-570 written out in NumPy with the same roundings
    rng = np.random.default_rng(9)
    w = rng.standard_normal(1000).astype(np.float32)
    g = (rng.standard_normal(1000) * 1e-3).astype(np.float32)
    m, v = np.zeros_like(w), np.zeros_like(w)
    w0 = w.copy()
    ko.adam(w, g, m, v, 1)
    f32 = np.float32
    m_ref = (f32(1 - 0.9) * g.astype(np.float64)).astype(f32)          # fma onto 0 is one rounding
    v_ref = (f32(1 - 0.999) * (g * g).astype(np.float64)).astype(f32)
    np.testing.assert_array_equal(m, m_ref)
    np.testing.assert_array_equal(v, v_ref)
    u = (m_ref / f32(1 - 0.9)) / (np.sqrt(v_ref / f32(1 - 0.999)) + f32(1e-8))
    w_ref = (w0.astype(np.float64) + np.float64(f32(-0.001)) * u.astype(np.float64)).astype(f32)
    np.testing.assert_array_equal(w, w_ref)


def test_xavier_uniform_range_and_conversion(ko):
    rng = np.random.default_rng(1)
    w = ko.xavier_uniform(64, 784, rng)
    s = np.sqrt(6 / (64 + 784))
    assert w.dtype == np.float32 and w.shape == (64, 784)
    assert np.abs(w).max() <= np.float32(s) and np.abs(w).max() > 0.99 * s


def test_mlp_loss_decreases(ko):
    rng = np.random.default_rng(1)
    m = ko.MLP([784, 64, 10], rng, lr=1e-3)
    x = rng.random((784, 100)).astype(np.float32)
    y = rng.integers(1, 11, 100)
    losses = [m.step(x, y) for _ in range(30)]
    assert losses[0] == pytest.approx(np.log(10), rel=0.2)
    assert losses[-1] < 0.7 * losses[0]
