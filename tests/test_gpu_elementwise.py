"""Parity of the pointwise kernels with Knet's CPU definitions (the oracle), through the C ABI.

Tolerances (stated per case below): ops made of IEEE-exact steps only (relu, the backward
forms, + - * /, comparisons, max/min, fill, dropout arithmetic) must be bit-identical.
Float32 sigm/tanh/elu/exp: at most 1 ulp from the oracle, whose exp/tanh are the correctly
rounded values.  Float64 exp, sigm and elu: bit-identical (the kernels' exp is correctly rounded
too and the remaining steps are IEEE operations in Knet's order); Float64 tanh: at most 1 ulp."""
import ctypes as C

import numpy as np
import pytest
import torch

from ulps import ulp_diff

pytestmark = pytest.mark.gpu

SIZES = [0, 1, 3, 4, 5, 31, 32, 33, 1000, 4099, (1 << 16) + 3, 1 << 20]
DT = {"32": (np.float32, torch.float32, C.c_float), "64": (np.float64, torch.float64, C.c_double)}


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def inputs(n, npdt, seed, scale=3.0):
    rng = np.random.default_rng(seed)
    x = (rng.standard_normal(n) * scale).astype(npdt)
    special = np.array([0.0, -0.0, 1.0, -1.0, 0.5, -0.5, 20.0, -20.0, 88.0, -88.0, 100.0, -104.0, 1e-8, -1e-8,
                        0.55, -0.55, 0.5499999, 9.0, -9.5], dtype=npdt)
    k = min(n, len(special))
    x[:k] = special[:k]
    return x


@pytest.mark.parametrize("S", ["32", "64"])
@pytest.mark.parametrize("op", ["relu", "sigm", "tanh", "elu"])
def test_activation_forward(K, ko, S, op):
    npdt, _, _ = DT[S]
    worst = 0
    for n in SIZES:
        x = inputs(n, npdt, n + 1)
        xd = dev(x)
        yd = torch.empty_like(xd)
        K.knet8(f"{op}_{S}", n, K.lib.ptr(xd), K.lib.ptr(yd))
        got, want = yd.cpu().numpy(), ko.unary(op, x)
        if op == "relu":
            np.testing.assert_array_equal(got, want)
            assert not np.signbit(got[x == 0]).any()
            continue
        d = ulp_diff(got, want)
        if op == "elu":
            # exp(x)-1 cancels for small |x|: a 1-ulp difference in exp(x), the number that was
            # rounded before the subtraction, is allowed; beyond that the result's own ulp rules
            neg = x < 0
            np.testing.assert_array_equal(got[~neg], want[~neg])
            ok = np.abs(got.astype(np.float64) - want) <= np.spacing(np.exp(x.astype(np.float64)).astype(npdt))
            d = np.where(ok, np.minimum(d, 1), d)
        if S == "64" and op in ("sigm", "elu"):
            # a correctly rounded exp on both sides, then the same IEEE operations
            np.testing.assert_array_equal(got, want)
        assert d.max(initial=0) <= 1, (op, S, n, int(d.max()), x[np.argmax(d)])
        worst = max(worst, int(d.max(initial=0)))
    if S == "32":
        print(f"{op}_{S}: worst {worst} ulp")


@pytest.mark.parametrize("S", ["32", "64"])
@pytest.mark.parametrize("op", ["relu", "sigm", "tanh", "elu", "exp"])
def test_special_values(K, ko, S, op):
    """NaN propagates, infinities and huge magnitudes give the limits, signed zeros and tiny values
    behave as on the CPU."""
    npdt, _, _ = DT[S]
    x = np.array([np.nan, np.inf, -np.inf, 0.0, -0.0, 1e-30, -1e-30, 104.0, -104.0, 200.0, -200.0, 88.7, -87.4,
                  -103.97, 1e-38, -1e-38, 3e38, -3e38], dtype=npdt)
    xd = dev(x)
    yd = torch.empty_like(xd)
    K.knet8(f"{op}_{S}", x.size, K.lib.ptr(xd), K.lib.ptr(yd))
    got = yd.cpu().numpy()
    with np.errstate(all="ignore"):
        want = ko.unary(op, x)
    np.testing.assert_array_equal(np.isnan(got), np.isnan(want))
    np.testing.assert_array_equal(np.isinf(got), np.isinf(want))
    fin = np.isfinite(want)
    assert ulp_diff(got[fin], want[fin]).max(initial=0) <= 1, (op, got, want)
    if op in ("relu", "sigm", "tanh"):
        np.testing.assert_array_equal(np.signbit(got[fin]), np.signbit(want[fin]))


@pytest.mark.parametrize("S", ["32", "64"])
def test_float32_exp_matches_correct_rounding(K, ko, S):
    npdt, _, _ = DT[S]
    x = (np.random.default_rng(5).standard_normal(1 << 22) * 8).astype(npdt)
    xd = dev(x)
    yd = torch.empty_like(xd)
    K.knet8(f"exp_{S}", x.size, K.lib.ptr(xd), K.lib.ptr(yd))
    d = ulp_diff(yd.cpu().numpy(), ko.unary("exp", x))
    if S == "32":
        # evaluated in Float64 and rounded once: differences from the correctly rounded value
        # need a Float64 result within 1e-16 relative of a rounding boundary
        assert d.max() <= 1 and (d > 0).sum() <= 2
    else:
        assert d.max() == 0          # correctly rounded on both sides


def test_float64_exp_sigm_elu_tanh_on_a_large_sample(K, ko):
    """2^23 draws over sigm's working range plus the ends of the exp range: exp, sigm and elu must
    reproduce the oracle bit for bit, tanh within 1 ulp."""
    rng = np.random.default_rng(13)
    x = rng.standard_normal(1 << 23) * 4
    x[:4096] = rng.uniform(-745.2, 709.8, 4096)              # subnormal results, overflow threshold
    x[4096:4112] = [0.0, -0.0, 709.0, -708.0, 709.78, -708.4, -745.13, -745.14, -750.0, 710.0, np.inf, -np.inf,
                    np.nan, 1e-300, -1e-300, 2.0 ** -60]
    xd = dev(x)
    yd = torch.empty_like(xd)
    for op in ("exp", "sigm", "elu", "tanh"):
        K.knet8(f"{op}_64", x.size, K.lib.ptr(xd), K.lib.ptr(yd))
        got, want = yd.cpu().numpy(), ko.unary(op, x)
        inner = (x >= -708) & (x <= 709)                         # outside: CUDA's exp, 1 ulp
        if op == "tanh":
            assert ulp_diff(got, want).max() <= 1
            continue
        np.testing.assert_array_equal(got[inner], want[inner])
        fin = ~inner & np.isfinite(want)
        assert ulp_diff(got[fin], want[fin]).max(initial=0) <= 1
        np.testing.assert_array_equal(np.isnan(got), np.isnan(want))
        np.testing.assert_array_equal(np.isinf(got), np.isinf(want))


def test_float32_sigm_tanh_elu_on_a_large_sample(K, ko):
    # 2^24 normal draws: sigm and elu follow Knet's float operations on a correctly rounded exp,
    # so they must reproduce the oracle bit for bit (a handful of 1-ulp cases are possible where
    # the Float64 evaluation of exp lands within 1e-16 of a rounding boundary); tanh is a
    # Float64 evaluation rounded once and must match the correctly rounded value likewise.
    x = (np.random.default_rng(12).standard_normal(1 << 24) * 4).astype(np.float32)
    xd = dev(x)
    yd = torch.empty_like(xd)
    for op in ("sigm", "tanh", "elu"):
        K.knet8(f"{op}_32", x.size, K.lib.ptr(xd), K.lib.ptr(yd))
        got, want = yd.cpu().numpy(), ko.unary(op, x)
        if op == "elu":
            bad = got != want
            assert bad.sum() <= 4 and np.all(np.abs(got[bad] - want[bad]) <= np.spacing(np.exp(x[bad])))
        else:
            d = ulp_diff(got, want)
            # tanh loses a few bits to the subtraction exp(-2|x|) - 1 for small |x|: still within
            # 1 ulp everywhere, a few elements per million off by that one ulp
            allowed = 4 if op == "sigm" else x.size // 100000
            assert d.max() <= 1 and (d > 0).sum() <= allowed, (op, int(d.max()), int((d > 0).sum()))


@pytest.mark.parametrize("S", ["32", "64"])
@pytest.mark.parametrize("op", ["reluback", "sigmback", "tanhback", "eluback"])
def test_activation_backward_is_bit_exact(K, ko, S, op):
    npdt, _, _ = DT[S]
    for n in SIZES:
        rng = np.random.default_rng(n + 7)
        y = inputs(n, npdt, n + 3, scale=1.0)
        dy = rng.standard_normal(n).astype(npdt)
        yd, dyd = dev(y), dev(dy)
        dxd = torch.empty_like(yd)
        K.knet8(f"{op}_{S}_11", n, K.lib.ptr(dyd), K.lib.ptr(yd), K.lib.ptr(dxd))
        np.testing.assert_array_equal(dxd.cpu().numpy(), ko.actback(op, dy, y))


@pytest.mark.parametrize("S", ["32", "64"])
def test_three_argument_backward_forms(K, ko, S):
    npdt, _, _ = DT[S]
    n = 5000
    rng = np.random.default_rng(1)
    x, y, dy = (rng.standard_normal(n).astype(npdt) for _ in range(3))
    xd, yd, dyd = dev(x), dev(y), dev(dy)
    out = torch.empty_like(xd)
    for name, ref in (("sigmback", "sigmback"), ("tanh_back", "tanhback"), ("eluback", "eluback")):
        K.knet8(f"{name}_{S}_111", n, K.lib.ptr(xd), K.lib.ptr(yd), K.lib.ptr(dyd), K.lib.ptr(out))
        np.testing.assert_array_equal(out.cpu().numpy(), ko.actback(ref, dy, y))


@pytest.mark.parametrize("S", ["32", "64"])
def test_relu_with_keyword_arguments(K, S):
    npdt, _, ct = DT[S]
    n = 3001
    x = inputs(n, npdt, 2)
    dy = np.random.default_rng(3).standard_normal(n).astype(npdt)
    xd, dyd = dev(x), dev(dy)
    out = torch.empty_like(xd)
    for maxv, slope, thr in ((np.inf, 0.0, 0.0), (6.0, 0.0, 0.0), (np.inf, 0.1, 0.0), (4.0, 0.2, 1.0)):
        K.knet8(f"relu_{S}_1", n, ct(maxv), ct(slope), ct(thr), K.lib.ptr(xd), K.lib.ptr(out))
        m, s, t = npdt(maxv), npdt(slope), npdt(thr)
        want = np.where(x >= m, m, np.where(x >= t, x, npdt(0) if s == 0 else s * (x - t))).astype(npdt)
        np.testing.assert_array_equal(out.cpu().numpy(), want)
        K.knet8(f"reluback_{S}_1", n, ct(maxv), ct(slope), ct(thr), K.lib.ptr(xd), K.lib.ptr(out),
                K.lib.ptr(dyd), K.lib.ptr(out))
        want = (dy * np.where(x >= m, npdt(0), np.where(x >= t, npdt(1), s))).astype(npdt)
        np.testing.assert_array_equal(out.cpu().numpy(), want)


BIN = ["add", "sub", "mul", "div", "max", "min", "eq", "ne", "gt", "ge", "lt", "le"]


@pytest.mark.parametrize("S", ["32", "64"])
def test_same_size_and_scalar_binary_ops_are_bit_exact(K, ko, S):
    npdt, _, ct = DT[S]
    for n in [0, 1, 7, 1024, 100003]:
        rng = np.random.default_rng(n)
        x = rng.standard_normal(n).astype(npdt)
        y = (rng.standard_normal(n) + 3).astype(npdt)
        if n > 4:
            y[:3] = x[:3]                      # equal pairs for the comparisons
        xd, yd = dev(x), dev(y)
        zd = torch.empty_like(xd)
        for op in BIN:
            K.knet8(f"{op}_{S}_11", n, K.lib.ptr(xd), K.lib.ptr(yd), K.lib.ptr(zd))
            np.testing.assert_array_equal(zd.cpu().numpy(), ko.binary(op, x, y).reshape(-1), err_msg=op)
            K.knet8(f"{op}_{S}_01", n, ct(1.25), K.lib.ptr(yd), K.lib.ptr(zd))
            np.testing.assert_array_equal(zd.cpu().numpy(), ko.binary(op, np.full(n, 1.25, npdt), y).reshape(-1),
                                          err_msg=op)
        if n:
            K.knet8(f"pow_{S}_11", n, K.lib.ptr(yd), K.lib.ptr(xd), K.lib.ptr(zd))
            np.testing.assert_allclose(zd.cpu().numpy(), np.power(y.astype(np.float64), x), rtol=2e-6 if S == "32" else 1e-14)


@pytest.mark.parametrize("S", ["32", "64"])
def test_unaligned_views_and_in_place(K, ko, S):
    # KnetArray views hand over pointers aligned only to the element size
    # (src/knetarrays/getindex.jl:153-159): same offset on all, different offsets, in place
    npdt, _, _ = DT[S]
    n = 10007
    x = inputs(n + 8, npdt, 4)
    dy = np.random.default_rng(6).standard_normal(n + 8).astype(npdt)
    xd, dyd = dev(x), dev(dy)
    out = torch.zeros(n + 16, dtype=xd.dtype, device="cuda")
    for ox, oo in ((1, 1), (1, 2), (3, 0), (0, 3), (2, 2)):
        K.knet8(f"sigm_{S}", n, K.lib.ptr(xd[ox:]), K.lib.ptr(out[oo:]))
        d = ulp_diff(out[oo:oo + n].cpu().numpy(), ko.unary("sigm", x[ox:ox + n]))
        assert d.max() <= (1 if S == "32" else 2)
        K.knet8(f"reluback_{S}_11", n, K.lib.ptr(dyd[oo:]), K.lib.ptr(xd[ox:]), K.lib.ptr(out[ox:]))
        np.testing.assert_array_equal(out[ox:ox + n].cpu().numpy(), ko.actback("reluback", dy[oo:oo + n], x[ox:ox + n]))
    guard = out[n + 3:].clone()
    y = xd.clone()
    K.knet8(f"relu_{S}", n, K.lib.ptr(y[1:]), K.lib.ptr(y[1:]))            # in place on a view
    np.testing.assert_array_equal(y[1:n + 1].cpu().numpy(), ko.unary("relu", x[1:n + 1]))
    assert y[0].item() == x[0] and y[n + 1].item() == x[n + 1]              # neighbours untouched
    assert torch.equal(guard, out[n + 3:])


@pytest.mark.parametrize("S", ["32", "64"])
def test_other_unary_ops_follow_their_definitions(K, S):
    npdt, _, _ = DT[S]
    n = 20011
    x = (np.random.default_rng(8).random(n) * 2 + 0.25).astype(npdt)     # positive, away from 0
    xd = dev(x)
    yd = torch.empty_like(xd)
    x64 = x.astype(np.float64)
    cases = {"abs2": x64 * x64, "abs": np.abs(x64), "neg": -x64, "one": np.ones(n), "zero": np.zeros(n),
             "sign": np.sign(x64), "sqrt": np.sqrt(x64), "log": np.log(x64), "exp": np.exp(x64),
             "invx": 1 / x64, "floor": np.floor(x64), "ceil": np.ceil(x64), "round": np.rint(x64),
             "trunc": np.trunc(x64), "log2": np.log2(x64), "log10": np.log10(x64), "log1p": np.log1p(x64),
             "expm1": np.expm1(x64), "exp2": np.exp2(x64), "sin": np.sin(x64), "cos": np.cos(x64),
             "tan": np.tan(x64), "sinh": np.sinh(x64), "cosh": np.cosh(x64), "atan": np.arctan(x64),
             "asinh": np.arcsinh(x64), "cbrt": np.cbrt(x64), "tanh_": np.tanh(x64),
             "selu": 1.0507009873554805 * x64, "hardsigmoid": np.clip((x64 + 3) / 6, 0, 1),
             "swish": x64 / (1 + np.exp(-x64))}
    tol = 4 if S == "32" else 4      # CUDA's documented bounds for these functions are 1-4 ulp
    for name, want in cases.items():
        K.knet8(f"{name}_{S}", n, K.lib.ptr(xd), K.lib.ptr(yd))
        d = ulp_diff(yd.cpu().numpy(), want.astype(npdt))
        assert d.max() <= tol, (name, int(d.max()))


@pytest.mark.parametrize("S", ["32", "64"])
def test_digamma_and_trigamma(K, S):
    """digamma_impl / trigamma_impl (src/libknet8/ops.jl:37-38) against SciPy's psi and polygamma(1, .)
    (Cephes), an independent implementation: 4e-6 (Float32) / 2e-13 (Float64) of max(1, |value|) on
    positive and negative arguments, plus the poles."""
    from scipy import special
    npdt, _, _ = DT[S]
    rng = np.random.default_rng(15)
    x = np.concatenate([rng.random(5000) * 30 + 1e-3, -rng.random(5000) * 12, [1.0, 2.0, 10.0, 0.5, 1.4616321449683622,
                                                                                  100.0, 1e4, -0.5, -1.5, -2.25]]).astype(npdt)
    frac = np.abs(x - np.rint(x))
    x = x[(x > 0) | (frac > 1e-2)]                                     # negative arguments: stay off the poles
    xd = dev(x)
    yd = torch.empty_like(xd)
    x64 = x.astype(np.float64)
    tol = 4e-6 if S == "32" else 2e-13
    for name, want in (("digamma_impl", special.digamma(x64)), ("trigamma_impl", special.polygamma(1, x64))):
        K.knet8(f"{name}_{S}", x.size, K.lib.ptr(xd), K.lib.ptr(yd))
        got = yd.cpu().numpy().astype(np.float64)
        # near a pole the function's own conditioning amplifies the rounding of the argument
        cond = 1 + np.abs(special.polygamma(1 if name == "digamma_impl" else 2, x64) * x64)
        assert np.all(np.abs(got - want) <= tol * np.maximum(1, np.abs(want)) * cond), (name, np.abs(got - want).max())
    poles = dev(np.array([0.0, -1.0, -2.0, -7.0], dtype=npdt))
    out = torch.empty_like(poles)
    K.knet8(f"digamma_impl_{S}", 4, K.lib.ptr(poles), K.lib.ptr(out))
    o = out.cpu().numpy()
    assert o[0] == -np.inf and np.isnan(o[1:]).all()
    K.knet8(f"trigamma_impl_{S}", 4, K.lib.ptr(poles), K.lib.ptr(out))
    assert np.isinf(out.cpu().numpy()).all()


@pytest.mark.parametrize("S", ["32", "64"])
def test_fill_and_entry_gather_scatter(K, S):
    npdt, tdt, ct = DT[S]
    n = 5003
    y = torch.zeros(n + 2, dtype=tdt, device="cuda")
    K.knet8(f"fill_{S}", n, ct(2.5), K.lib.ptr(y[1:]))
    assert y[0] == 0 and y[n + 1] == 0 and bool((y[1:n + 1] == 2.5).all())
    rng = np.random.default_rng(0)
    x = rng.standard_normal(n).astype(npdt)
    idx = rng.integers(1, n + 1, 777).astype(np.int32)                   # 1-based, with repeats
    xd, idd = dev(x), dev(idx)
    g = torch.empty(777, dtype=tdt, device="cuda")
    K.knet8(f"getents_{S}", 777, K.lib.ptr(idd), K.lib.ptr(xd), K.lib.ptr(g))
    np.testing.assert_array_equal(g.cpu().numpy(), x[idx - 1])
    acc = torch.zeros(n, dtype=tdt, device="cuda")
    K.knet8(f"addents_{S}", 777, K.lib.ptr(idd), K.lib.ptr(acc), K.lib.ptr(g))
    want = np.zeros(n, dtype=np.float64)
    np.add.at(want, idx - 1, x[idx - 1].astype(np.float64))
    np.testing.assert_allclose(acc.cpu().numpy(), want, rtol=1e-6 if S == "32" else 1e-14)


def test_full_size_properties_float32(K):
    # 2^28 elements, the largest size of the elementwise sweep: relu is idempotent and
    # equals max(x,0); reluback(dy, relu(x)) passes dy exactly where x > 0
    n = 1 << 28
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn(n, device="cuda", generator=g)
    y = torch.empty_like(x)
    K.knet8("relu_32", n, K.lib.ptr(x), K.lib.ptr(y))
    assert torch.equal(y, torch.clamp_min(x, 0))
    z = torch.empty_like(x)
    K.knet8("relu_32", n, K.lib.ptr(y), K.lib.ptr(z))
    assert torch.equal(z, y)
    K.knet8("reluback_32_11", n, K.lib.ptr(x), K.lib.ptr(y), K.lib.ptr(z))    # dy := x
    assert torch.equal(z, y)                                                # x where x>0 else 0
    K.knet8("tanh_32", n, K.lib.ptr(x), K.lib.ptr(y))
    assert float((y - torch.tanh(x)).abs().max()) <= 1.2e-7
    K.knet8("sigm_32", n, K.lib.ptr(x), K.lib.ptr(y))
    K.knet8("neg_32", n, K.lib.ptr(x), K.lib.ptr(z))
    K.knet8("sigm_32", n, K.lib.ptr(z), K.lib.ptr(z))
    assert float((y + z - 1).abs().max()) <= 1.2e-7                         # sigm(x)+sigm(-x) = 1
