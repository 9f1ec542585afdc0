"""Parity of the broadcasting and reduction kernels with Julia's semantics (NumPy on
column-major arrays for the exact ops, the oracle's sequential sums for the others).

Broadcast results are single IEEE operations, so they must be bit-identical.  maximum,
minimum, maxabs, minabs and countnz are order-independent and must be exact; sums and
products are compared at a relative 1e-5 (Float32) / 1e-12 (Float64) of the sum of
magnitudes, since the summation order differs from Julia's."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

NPDT = {torch.float32: np.float32, torch.float64: np.float64}


def rnd(shape, dt, seed, shift=0.0):
    rng = np.random.default_rng(seed)
    return np.asfortranarray((rng.standard_normal(shape) + shift).astype(dt))


# the shape pairs of Knet's own test (test/binary.jl:18-21, kept in tests/golden/; the >5-d pairs
# belong to the _17 kernels, which are not provided) plus the benchmark's families
import json
import os
with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "knet_known_answers.json")) as _f:
    _SIZE12 = [(tuple(a), tuple(b)) for a, b in json.load(_f)["broadcast_shape_pairs"]["size12"] if len(a) <= 5]
PAIRS = _SIZE12 + [
         ((8, 8, 16, 4), (8, 1, 16, 1)), ((3, 5, 7), (3, 1, 7)),
         ((2, 3, 4, 5, 6), (2, 1, 4, 1, 6)),
         ((64, 1), (64, 128)), ((1, 128), (64, 128)), ((1, 4096), (64, 4096)), ((64, 4096), (1, 4096)),
         ((1024, 1), (1024, 128)), ((1, 128), (1024, 128)), ((1023, 1), (1023, 77)), ((1, 77), (1023, 77)),
         ((64,), (64, 100)), ((64, 100), (64,)), ((7, 1), (1, 9)), ((1,), (5, 6)), ((5, 6), (1, 1)),
         ((6, 5), (6, 5))]


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("shapes", PAIRS, ids=lambda p: f"{p[0]}x{p[1]}")
def test_broadcast_is_bit_exact(K, ko, dtype, shapes):
    dt = NPDT[dtype]
    x, y = rnd(shapes[0], dt, 1), rnd(shapes[1], dt, 2, shift=3.0)   # divisor kept away from 0
    kx, ky = K.KnetArray(x), K.KnetArray(y)
    for op in ("add", "sub", "mul", "div", "max", "min", "lt", "ge", "eq"):
        z = K.ops.broadcast(op, kx, ky)
        want = ko.binary(op, x, y)
        assert z.shape == want.shape, (op, z.shape, want.shape)
        np.testing.assert_array_equal(z.numpy(), want, err_msg=op)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_array_scalar_forms(K, ko, dtype):
    dt = NPDT[dtype]
    x = rnd((37, 11), dt, 3, shift=2.0)
    kx = K.KnetArray(x)
    s = 1.7
    np.testing.assert_array_equal((kx + s).numpy(), x + dt(s))
    np.testing.assert_array_equal((s + kx).numpy(), dt(s) + x)
    np.testing.assert_array_equal((kx - s).numpy(), x - dt(s))
    np.testing.assert_array_equal((s - kx).numpy(), dt(s) - x)
    np.testing.assert_array_equal((kx * s).numpy(), x * dt(s))
    np.testing.assert_array_equal((kx / s).numpy(), x / dt(s))        # a true division, as on the CPU
    np.testing.assert_array_equal((s / kx).numpy(), dt(s) / x)
    np.testing.assert_array_equal(K.ops.broadcast("gt", kx, 2.0).numpy(), (x > 2).astype(dt))
    np.testing.assert_array_equal(K.ops.broadcast("le", 2.0, kx).numpy(), (2 <= x).astype(dt))


def _f32_from_bits(sign, exp, mant):
    return ((sign.astype(np.uint32) << 31) | (exp.astype(np.uint32) << 23) | mant.astype(np.uint32)).view(np.float32)


def test_float32_broadcast_division_is_the_ieee_quotient(K):
    """x ./ y of the _12 kernel against NumPy's division, bit for bit, on operands that cover the
    kernel's two routes (a Newton sequence for groups of ordinary magnitudes, the compiler's
    division otherwise): random signs, exponents over the whole range, random and extreme
    significands (all ones, all zeros, one bit), zeros, subnormals, infinities and NaN."""
    rng = np.random.default_rng(11)
    n = 1 << 22
    specials = np.array([0, 1, 0x7FFFFF, 0x7FFFFE, 0x400000, 0x3FFFFF, 0x400001, 0x555555, 0x2AAAAA], np.uint32)

    def draw(lo, hi, special_mant):
        e = rng.integers(lo, hi + 1, n)
        m = rng.integers(0, 1 << 23, n)
        if special_mant:
            pick = rng.random(n) < 0.5
            m = np.where(pick, specials[rng.integers(0, len(specials), n)], m)
        return _f32_from_bits(rng.integers(0, 2, n), e, m)

    cases = [(draw(127 - 40, 127 + 40, False), draw(127 - 40, 127 + 40, False)),     # every group on the Newton route
             (draw(127 - 59, 127 + 59, True), draw(127 - 59, 127 + 59, True)),        # extreme significands, route's edges
             (draw(0, 255, True), draw(0, 255, True)),                                # everything: zeros, subnormals, inf, NaN
             (draw(127 - 70, 127 + 70, False), draw(127 - 70, 127 + 70, False))]      # groups that mix both routes
    # consecutive significands around a power of two, divided by all-ones significands
    a = _f32_from_bits(np.zeros(n), np.full(n, 127), np.arange(n) % (1 << 23))
    b = _f32_from_bits(np.zeros(n), rng.integers(100, 150, n), np.full(n, 0x7FFFFF))
    cases.append((a, b))
    for ci, (x, y) in enumerate(cases):
        xd, yd = torch.from_numpy(x).cuda(), torch.from_numpy(y).cuda()
        zd = torch.empty_like(xd)
        K.knet8("div_32_12", n, K.lib.ptr(xd), 1, n, K.lib.ptr(yd), 1, n, K.lib.ptr(zd))
        with np.errstate(all="ignore"):
            want = x / y
        got = zd.cpu().numpy()
        nan = np.isnan(want)
        assert np.array_equal(np.isnan(got), nan), ci
        bad = np.flatnonzero((got.view(np.uint32) != want.view(np.uint32)) & ~nan)
        assert bad.size == 0, (ci, bad[:5], x[bad[:5]], y[bad[:5]], got[bad[:5]], want[bad[:5]])
        # the same-shape (compiler's division) and scalar ./ array (group form) entry points
        import ctypes
        K.knet8("div_32_11", n, K.lib.ptr(xd), K.lib.ptr(yd), K.lib.ptr(zd))
        got = zd.cpu().numpy()
        assert np.array_equal(got.view(np.uint32)[~nan], want.view(np.uint32)[~nan]) and np.array_equal(np.isnan(got), nan), ci
        for s in (1.0, -3.7, 1e-30, 6.5e37):
            K.knet8("div_32_01", n, ctypes.c_float(s), K.lib.ptr(yd), K.lib.ptr(zd))
            with np.errstate(all="ignore"):
                w1 = np.float32(s) / y
            got = zd.cpu().numpy()
            ok = ~np.isnan(w1)
            assert np.array_equal(got.view(np.uint32)[ok], w1.view(np.uint32)[ok]) and np.array_equal(np.isnan(got), ~ok), (ci, s)
        # a vector operand along each dim takes the same arithmetic (and the multiply-high index math)
        rows = 1 << 10
        vd = yd[:rows].contiguous()
        K.knet8("div_32_12", n, K.lib.ptr(xd), 1, n, K.lib.ptr(vd), 1, rows, K.lib.ptr(zd))
        with np.errstate(all="ignore"):
            want = (x.reshape(-1, rows) / y[:rows]).reshape(-1)
        got = zd.cpu().numpy()
        assert np.array_equal(got.view(np.uint32)[~np.isnan(want)], want.view(np.uint32)[~np.isnan(want)]), ci
        cols = n // rows
        wd = yd[:cols].contiguous()
        K.knet8("div_32_12", n, K.lib.ptr(wd), rows, cols, K.lib.ptr(xd), 1, n, K.lib.ptr(zd))
        with np.errstate(all="ignore"):
            want = (y[:cols, None] / x.reshape(cols, rows)).reshape(-1)
        got = zd.cpu().numpy()
        assert np.array_equal(got.view(np.uint32)[~np.isnan(want)], want.view(np.uint32)[~np.isnan(want)]), ci


def test_broadcast_on_unaligned_views(K, ko):
    x = rnd((1001,), np.float32, 5)
    b = rnd((13,), np.float32, 6)
    big = K.KnetArray(np.concatenate([np.zeros(3, np.float32), x]))
    kb = K.KnetArray(np.concatenate([np.zeros(1, np.float32), b]))
    xv = big.view(3, 1001).reshape(13, 77)                          # element-offset pointers
    bv = kb.view(1, 13)
    z = xv + bv
    np.testing.assert_array_equal(z.numpy(), x.reshape(13, 77, order="F") + b.reshape(13, 1))
    z = xv.reshape(77, 13) * bv.reshape(1, 13)
    np.testing.assert_array_equal(z.numpy(), x.reshape(77, 13, order="F") * b.reshape(1, 13))


def _check_reduce(K, ko, x, dims, dtype, ops=None):
    """Order-independent ops exact.  Sums: within 1e-5 (Float32) of the Float64 evaluation of
    the same reduction, relative to the sum of magnitudes; and within that plus the error
    bound of the oracle's own sequential sum (n*eps/2) of the oracle in the array's precision."""
    kx = K.KnetArray(x)
    rt = 1e-5 if dtype == torch.float32 else 1e-12
    eps = np.finfo(x.dtype).eps
    x64 = np.asfortranarray(x.astype(np.float64))

    def ref(op, a):
        return ko.reduce_all(op, a) if dims is None else ko.reduce_dim(op, a, dims)

    for op in (ops or K.ops.REDUCTIONS):
        if op == "prod":
            if x.size >= 4000:
                continue
            xs = (np.abs(x) * 0.2 + 0.9).astype(x.dtype)
            got = K.ops.reduce(op, K.KnetArray(xs), dims)
            g = np.asarray(got) if dims is None else got.numpy()
            np.testing.assert_allclose(g, ref(op, xs.astype(np.float64)), rtol=1e-4 if dtype == torch.float32 else 1e-11)
            continue
        got = K.ops.reduce(op, kx, dims)
        want = ref(op, x)
        g = np.asarray(got) if dims is None else got.numpy()
        if dims is not None:
            assert g.shape == want.shape, (op, dims, g.shape, want.shape)
        if op in ("maximum", "minimum", "maxabs", "minabs", "countnz"):
            np.testing.assert_array_equal(g, want, err_msg=f"{op} dims={dims}")
            continue
        truth = ref(op, x64)
        mag = ref("sumabs2" if op == "sumabs2" else "sumabs", x64)
        nred = max(x.size // max(np.size(want), 1), 1)
        assert np.all(np.abs(g - truth) <= rt * np.maximum(mag, 1e-300)), (op, dims, "vs Float64")
        assert np.all(np.abs(g - want) <= (rt + 0.5 * nred * eps) * np.maximum(mag, 1e-300)), (op, dims)


SHAPES = [(1,), (2,), (1, 1), (2, 1), (1, 2), (2, 2), (10, 1000), (1000, 10), (10, 100000), (100000, 10),
          (1000, 64), (64, 1000), (5021, 67), (67, 5021), (3, 4, 5), (7, 33, 9), (2, 3, 4, 5), (4, 3, 2, 3, 4),
          # dims=1: runs held by a group of 8, 16 or 32 lanes (odd lengths: every start offset);
          # dims=2: few rows, 32 (Float32) or 16 (Float64) columns in flight per thread, plus the tail
          (129, 400), (515, 301), (1000, 300), (2047, 300), (2048, 297), (250, 2500)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("shape", SHAPES, ids=str)
def test_reductions_over_every_single_dim_and_all(K, ko, dtype, shape):
    # test/reduction.jl:40-70,115-141: every dims choice, including the >64K regression shapes
    x = rnd(shape, NPDT[dtype], 7)
    x.reshape(-1, order="F")[::7] = 0                                     # something for countnz
    _check_reduce(K, ko, x, None, dtype)
    for d in range(1, len(shape) + 1):
        _check_reduce(K, ko, x, d, dtype)


def test_two_stage_reduction_in_a_graph_and_on_two_streams(K, ko):
    """A matrix with few rows and more than 8 MiB is reduced over dims=2 in two stages whose scratch
    is a stream-ordered allocation: the call must be capturable into a graph, repeat bit for bit, and
    calls on two streams at once must not disturb each other."""
    from knet_sm100.lib import knet8, ptr
    rows, cols = 64, 40000
    xs = [rnd((rows, cols), np.float32, 30 + i) for i in range(2)]
    want = [ko.reduce_dim("sum", x.astype(np.float64), 2).reshape(-1) for x in xs]
    mag = [ko.reduce_dim("sumabs", x.astype(np.float64), 2).reshape(-1) for x in xs]
    kx = [K.KnetArray(x) for x in xs]
    eager = K.ops.reduce("sum", kx[0], 2).data.reshape(-1).clone()           # also creates the pool
    assert np.all(np.abs(eager.cpu().numpy() - want[0]) <= 1e-5 * mag[0])
    y = torch.zeros(rows, device="cuda")
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        knet8("sum_32_21", rows * cols, ptr(kx[0].data), 1, rows, ptr(y))
    for _ in range(3):
        y.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(y, eager)
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    outs = [torch.zeros(rows, device="cuda") for _ in range(2)]
    torch.cuda.synchronize()
    for rep in range(20):
        for i, st in enumerate(streams):
            with torch.cuda.stream(st):
                knet8("sum_32_21", rows * cols, ptr(kx[i].data), 1, rows, ptr(outs[i]))
    torch.cuda.synchronize()
    assert torch.equal(outs[0], eager)
    assert np.all(np.abs(outs[1].cpu().numpy() - want[1]) <= 1e-5 * mag[1])


@pytest.mark.parametrize("dims", [(1, 2), (2, 3), (1, 3), (1, 2, 3), (3, 1)])
def test_reductions_over_several_dims(K, ko, dims):
    x = rnd((6, 7, 8), np.float32, 9)
    _check_reduce(K, ko, x, dims, torch.float32)


def test_scalar_reduction_entry_points(K, ko):
    import ctypes as C
    n = 1_000_003
    x = rnd((n,), np.float32, 11)
    xd = torch.from_numpy(x).cuda()
    ws = torch.empty(K.libknet.knet_reduce_workspace_bytes(), dtype=torch.uint8, device="cuda")
    out = torch.empty(1, dtype=torch.float32, device="cuda")
    for op, name in enumerate(K.ops.REDUCTIONS):
        if name == "prod":
            continue
        K.knet("knet_reduce_32", op, n - 1, K.lib.ptr(xd[1:]), K.lib.ptr(out), K.lib.ptr(ws), ws.numel())
        want = ko.reduce_all(name, x[1:])
        legacy = K.knet8r(f"{name}_32_20", n - 1, K.lib.ptr(xd[1:]))
        assert out.item() == legacy                                         # same kernels, same order
        assert abs(out.item() - want) <= 1e-5 * max(ko.reduce_all("sumabs", x[1:]), 1)
    assert K.libknet.knet_reduce_32(0, n, K.lib.ptr(xd), K.lib.ptr(out), None, 0, None) == -3
    assert K.libknet.knet_reduce_32(99, n, K.lib.ptr(xd), K.lib.ptr(out), K.lib.ptr(ws), ws.numel(), None) == -1
    assert K.knet8r("sum_32_20", 0, K.lib.ptr(xd)) == 0.0                    # n <= 0 is a no-op


def test_full_size_reductions_by_properties(K):
    # 50257 x 4096 Float32 (823 MB), the largest reduction shape: column and row sums of the
    # same matrix must agree on the grand total, maxima must agree with the global maximum
    C_, B_ = 50257, 4096
    g = torch.Generator(device="cuda").manual_seed(2)
    x = K.KnetArray(torch.randn(C_ * B_, device="cuda", generator=g), (C_, B_))
    s1, s2 = K.ops.sum(x, 1), K.ops.sum(x, 2)
    assert s1.shape == (1, B_) and s2.shape == (C_, 1)
    t1, t2, t = K.ops.sum(s1), K.ops.sum(s2), K.ops.sum(x)
    ref = float(x.data.double().sum())
    mag = float(x.data.abs().double().sum())
    for v in (t1, t2, t):
        assert abs(v - ref) <= 1e-5 * mag
    m = K.ops.maximum(x)
    assert m == float(x.data.max())
    assert K.ops.maximum(K.ops.maximum(x, 1)) == m and K.ops.maximum(K.ops.maximum(x, 2)) == m
    ref1 = x.data.view(B_, C_).sum(dim=1)
    assert float((s1.data - ref1).abs().max()) <= 1e-5 * float(x.data.view(B_, C_).abs().sum(dim=1).max())
