"""update! kernels and dropout against the oracle.

The optimizer kernels perform the same IEEE operations in the same order as Knet's CPU
`_update!` (src/train20/update.jl:513-570), so weights and state must be bit-identical to the
oracle after every step.  Dropout masks are integer decisions on supplied uniforms and must
be exact; the scaling is one IEEE division and is exact too."""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

NPDT = {torch.float32: np.float32, torch.float64: np.float64}


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def make(n, dt, seed):
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal(n) * 0.02).astype(dt)
    gs = [(rng.standard_normal(n) * 1e-3).astype(dt) for _ in range(4)]
    return w, gs


OPTS = [
    ("sgd", dict(lr=0.1), 0), ("momentum", dict(lr=0.05, gamma=0.9), 1), ("nesterov", dict(lr=0.05, gamma=0.95), 1),
    ("adagrad", dict(lr=0.05, eps=1e-6), 1), ("rmsprop", dict(lr=0.01, rho=0.9, eps=1e-6), 1),
    ("adadelta", dict(lr=1.0, rho=0.9, eps=1e-6), 2), ("adam", dict(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8), 2),
]


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("name,hyper,nstate", OPTS, ids=[o[0] for o in OPTS])
def test_single_tensor_update_is_bit_exact(K, ko, dtype, name, hyper, nstate):
    dt = NPDT[dtype]
    cls = {"sgd": K.SGD, "momentum": K.Momentum, "nesterov": K.Nesterov, "adagrad": K.Adagrad,
           "rmsprop": K.Rmsprop, "adadelta": K.Adadelta, "adam": K.Adam}[name]
    for n, off in ((1, 0), (5, 0), (1000, 0), (8192, 0), (8193, 1), (100003, 3), (300000, 0)):
        w, gs = make(n, dt, n)
        st = [np.zeros(n, dt) for _ in range(nstate)]
        base = torch.zeros(n + 8, dtype=dtype, device="cuda")
        kw = K.KnetArray(base[off:off + n])                       # unaligned view when off > 0
        kw.data.copy_(dev(w))
        opt = cls(**hyper)
        for t, g in enumerate(gs, 1):
            K.update_(kw, K.KnetArray(dev(g)), opt)
            if name == "sgd":
                ko.sgd(w, g, **hyper)
            elif name == "adam":
                ko.adam(w, g, st[0], st[1], t, **hyper)
            elif name == "adadelta":
                ko.adadelta(w, g, st[0], st[1], **hyper)
            else:
                getattr(ko, name)(w, g, st[0], **hyper)
            np.testing.assert_array_equal(kw.data.cpu().numpy(), w, err_msg=f"{name} n={n} step {t}")
        if name == "adam":
            np.testing.assert_array_equal(opt.fstm.data.cpu().numpy(), st[0])
            np.testing.assert_array_equal(opt.scndm.data.cpu().numpy(), st[1])
            assert opt.t == 4
        assert float(base[:off].abs().sum()) == 0 and float(base[off + n:].abs().sum()) == 0


def test_update_containers_param_and_clone(K, ko):
    # update! on tuples / dicts of arrays and on Param (update.jl:470-501)
    rng = np.random.default_rng(0)
    ws = [rng.standard_normal(50).astype(np.float32), rng.standard_normal((7, 3)).astype(np.float32)]
    gs = [rng.standard_normal(50).astype(np.float32), rng.standard_normal((7, 3)).astype(np.float32)]
    kws, kgs = [K.KnetArray(w) for w in ws], [K.KnetArray(g) for g in gs]
    proto = K.Adam(lr=0.005, beta1=0.9, beta2=0.95)
    opts = [proto.clone(), proto.clone()]
    K.update_(kws, kgs, opts)
    K.update_({"a": kws[0]}, {"a": kgs[0]}, {"a": opts[0]})
    for w, g, n in zip(ws, gs, (2, 1)):
        wf, gf = np.asfortranarray(w), np.asfortranarray(g)
        m, v = np.zeros_like(wf), np.zeros_like(wf)
        for t in range(1, n + 1):
            ko.adam(wf, gf, m, v, t, lr=0.005, beta1=0.9, beta2=0.95)
        w[...] = wf
    np.testing.assert_array_equal(kws[0].numpy(), ws[0])
    np.testing.assert_array_equal(kws[1].numpy(), ws[1])
    assert opts[0].t == 2 and opts[1].t == 1 and proto.t == 0 and proto.fstm is None
    p = K.Param(K.KnetArray(ws[0].copy()), K.SGD(lr=0.5))
    K.update_(p, kgs[0])
    w = ws[0].copy()
    ko.sgd(w, gs[0], lr=0.5)
    np.testing.assert_array_equal(p.value.numpy(), w)
    assert K.update_(p, None) is p                                # a `nothing` gradient is skipped


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_multi_tensor_update_matches_per_array_oracle(K, ko, dtype):
    dt = NPDT[dtype]
    sizes = [4096 * 3, 4096, 17, 8192, 1, 20001, 8193]
    rng = np.random.default_rng(1)
    total = sum(sizes) + 3
    flat_w = torch.zeros(total, dtype=dtype, device="cuda")
    flat_g, flat_m, flat_v = (torch.zeros_like(flat_w) for _ in range(3))
    host = []
    arrays, o = [], 3                                            # the whole set starts unaligned
    for n in sizes:
        w = (rng.standard_normal(n) * 0.02).astype(dt)
        flat_w[o:o + n].copy_(dev(w))
        host.append([w, np.zeros(n, dt), np.zeros(n, dt)])
        arrays.append((flat_w[o:o + n], flat_g[o:o + n], flat_m[o:o + n], flat_v[o:o + n]))
        o += n
    plan = K.MultiTensorPlan(arrays)
    opt = K.Adam()
    for t in range(1, 4):
        o = 3
        for i, n in enumerate(sizes):
            g = (rng.standard_normal(n) * 1e-3).astype(dt)
            flat_g[o:o + n].copy_(dev(g))
            ko.adam(host[i][0], g, host[i][1], host[i][2], t)
            o += n
        K.update_multi_(plan, opt)
        o = 3
        for i, n in enumerate(sizes):
            np.testing.assert_array_equal(flat_w[o:o + n].cpu().numpy(), host[i][0], err_msg=f"tensor {i} step {t}")
            np.testing.assert_array_equal(flat_v[o:o + n].cpu().numpy(), host[i][2])
            o += n
    assert float(flat_w[:3].abs().sum()) == 0
    # SGD and Momentum through the same table
    for opt2, ref in ((K.SGD(lr=0.1), lambda w, g, s: ko.sgd(w, g, lr=0.1)),
                      (K.Momentum(lr=0.05, gamma=0.9), lambda w, g, s: ko.momentum(w, g, s, lr=0.05, gamma=0.9))):
        flat_m.zero_()
        o = 3
        for i, n in enumerate(sizes):
            host[i][1][:] = 0
            ref(host[i][0], flat_g[o:o + n].cpu().numpy(), host[i][1])
            o += n
        K.update_multi_(plan, opt2)
        o = 3
        for i, n in enumerate(sizes):
            np.testing.assert_array_equal(flat_w[o:o + n].cpu().numpy(), host[i][0])
            o += n


def test_gradient_scale_and_argument_errors(K, ko):
    n = 5000
    w, gs = make(n, np.float32, 3)
    kw, kg = K.KnetArray(w.copy()), K.KnetArray(gs[0] * 4)
    K.update_(kw, kg, K.SGD(lr=0.1), gscale=0.25)                # 0.25 * (4 g) == g exactly
    ko.sgd(w, gs[0], lr=0.1)
    np.testing.assert_array_equal(kw.numpy(), w)
    lib = K.libknet
    assert lib.knet_adam_32(n, K.lib.ptr(kw.data), None, None, None, 1e-3, 0.9, 0.999, 1e-8, 1, 1.0, None) == -1
    assert lib.knet_adam_32(n, K.lib.ptr(kw.data), K.lib.ptr(kg.data), K.lib.ptr(kg.data), K.lib.ptr(kg.data),
                            1e-3, 0.9, 0.999, 1e-8, 0, 1.0, None) == -1          # t starts at 1
    assert lib.knet_sgd_32(-1, K.lib.ptr(kw.data), K.lib.ptr(kg.data), 0.1, 1.0, None) == -1
    assert lib.knet_sgd_32(0, None, None, 0.1, 1.0, None) == 0


def test_gradient_clipping(K):
    g = K.KnetArray(np.full(100, 3.0, np.float32))               # norm 30
    K.train.gclip_(g, 100.0)
    assert float(g.data[0]) == 3.0
    K.train.gclip_(g, 3.0)
    assert abs(float(K.ops.sumabs2(g)) ** 0.5 - 3.0) < 1e-5


# ---- dropout -------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("p", [0.5, 0.2, 0.9])
def test_dropout_with_supplied_uniforms_is_exact(K, ko, dtype, p):
    dt = NPDT[dtype]
    rng = np.random.default_rng(1)
    for n in (1, 7, 10000, 100003):
        x = rng.standard_normal(n).astype(dt)
        u = rng.random(n).astype(dt)
        u[:1] = dt(p)                                            # u == p is dropped (strict >)
        y = K.dropout(K.KnetArray(x), p, uniforms=K.KnetArray(u))
        want = ko.dropout(x, p, u)
        np.testing.assert_array_equal(y.numpy(), want)
        dy = rng.standard_normal(n).astype(dt)
        dx = K.ops.dropback(K.KnetArray(dy), y, K.KnetArray(x), p)
        np.testing.assert_array_equal(dx.numpy(), ko.dropback(p, want, dy))


def test_dropout_switches(K):
    x = K.KnetArray(np.arange(10, dtype=np.float32))
    assert K.dropout(x, 0.5, drop=False) is x and K.dropout(x, 0) is x
    assert not K.dropout(x, 1).data.any()
    with pytest.raises(ValueError):
        K.dropout(x, 1.5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_in_kernel_generator(K, ko, dtype):
    S, dt = K.lib.sfx(dtype), NPDT[dtype]
    ct = C.c_float if dtype == torch.float32 else C.c_double
    n = 1_000_003
    u = torch.empty(n, dtype=dtype, device="cuda")
    K.knet(f"knet_dropout_uniform_{S}", n, 1234, 0, K.lib.ptr(u))
    uh = u.cpu().numpy()
    assert uh.min() >= 0 and uh.max() < 1
    assert abs(uh.mean() - 0.5) < 2e-3 and abs(uh.var() - 1 / 12) < 2e-3
    assert abs(np.corrcoef(uh[:-1], uh[1:])[0, 1]) < 5e-3
    u2 = torch.empty_like(u)
    K.knet(f"knet_dropout_uniform_{S}", n, 1234, 0, K.lib.ptr(u2))
    assert torch.equal(u, u2)                                     # counter-based: reproducible
    K.knet(f"knet_dropout_uniform_{S}", n, 1235, 0, K.lib.ptr(u2))
    assert not torch.equal(u, u2)
    # dropout_philox(x) == dropout with those uniforms, exactly, also through an unaligned view
    x = torch.from_numpy(np.random.default_rng(2).standard_normal(n + 1).astype(dt)).cuda()
    for off in (0, 1):
        y = torch.empty(n + 1, dtype=dtype, device="cuda")
        K.knet(f"knet_dropout_philox_{S}", n, ct(0.5), 1234, 0, K.lib.ptr(x[off:]), K.lib.ptr(y[off:]))
        want = ko.dropout(x[off:off + n].cpu().numpy(), 0.5, uh)
        np.testing.assert_array_equal(y[off:off + n].cpu().numpy(), want)
    # offset shifts the counter: group k of a call at offset o equals group k+o at offset 0
    G = 8 if dtype == torch.float32 else 4
    K.knet(f"knet_dropout_uniform_{S}", n - 5 * G, 1234, 5, K.lib.ptr(u2))
    assert torch.equal(u2[:n - 5 * G], u[5 * G:])


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("p", [0.0, 0.5])
def test_fused_layer_pieces_equal_the_unfused_chain(K, ko, dtype, p):
    S, dt = K.lib.sfx(dtype), NPDT[dtype]
    ct = C.c_float if dtype == torch.float32 else C.c_double
    rng = np.random.default_rng(4)
    for N, B in ((64, 100), (1000, 37), (13, 11)):
        z = np.asfortranarray(rng.standard_normal((N, B)).astype(dt))
        b = rng.standard_normal(N).astype(dt)
        zd, bd = dev(z.reshape(-1, order="F")), dev(b)
        y = torch.empty_like(zd)
        K.knet(f"knet_bias_relu_dropout_fwd_{S}", K.lib.ptr(zd), K.lib.ptr(bd), K.lib.ptr(y), N, B, ct(p), 77, 3)
        r = ko.unary("relu", ko.binary("add", z, b.reshape(-1, 1)))
        if p > 0:
            u = torch.empty_like(zd)
            K.knet(f"knet_dropout_uniform_{S}", N * B, 77, 3, K.lib.ptr(u))
            r = ko.dropout(r, p, u.cpu().numpy().reshape(N, B, order="F"))
        np.testing.assert_array_equal(y.cpu().numpy().reshape(N, B, order="F"), r)
        dy = np.asfortranarray(rng.standard_normal((N, B)).astype(dt))
        dz = torch.empty_like(zd)
        K.knet(f"knet_relu_dropout_bwd_{S}", K.lib.ptr(y), K.lib.ptr(dev(dy.reshape(-1, order="F"))), K.lib.ptr(dz),
               N * B, ct(p))
        d1 = ko.dropback(p, r, dy) if p > 0 else dy
        relu_out = r if p == 0 else ko.unary("relu", ko.binary("add", z, b.reshape(-1, 1)))
        want = ko.actback("reluback", d1, relu_out)
        np.testing.assert_array_equal(dz.cpu().numpy().reshape(N, B, order="F"), want)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("p", [0.0, 0.5, 0.3])
def test_fused_backward_with_bias_gradient(K, ko, dtype, p):
    """knet_relu_dropout_bias_bwd: dz bit-identical to dropback + reluback of the oracle, db = the
    oracle's sum(dz, dims=2) within 1e-5 of sum|dz| (Float32; the summation order differs), also in
    place, on shapes that take the 16-byte path, the scalar path and the cluster split."""
    S, dt = K.lib.sfx(dtype), NPDT[dtype]
    ct = C.c_float if dtype == torch.float32 else C.c_double
    rng = np.random.default_rng(8)
    for N, B, shift in ((64, 100, 0), (1000, 37, 0), (13, 11, 0), (4096, 1030, 0), (256, 8192, 0), (8192, 640, 0),
                        (1024, 515, 1), (130, 1, 0), (128, 0, 0)):
        r = np.asfortranarray(np.maximum(rng.standard_normal((N, B)), 0).astype(dt))     # relu output
        u = np.asfortranarray(rng.random((N, B)).astype(dt))
        y = ko.dropout(r, p, u) if p > 0 else r
        dy = np.asfortranarray(rng.standard_normal((N, B)).astype(dt))
        d1 = ko.dropback(p, y, dy) if p > 0 else dy
        want = ko.actback("reluback", d1, r) if B > 0 else np.zeros((N, 0), dt)
        yd = dev(np.concatenate([np.zeros(shift, dt), y.reshape(-1, order="F")]))[shift:]
        dyd = dev(np.concatenate([np.zeros(shift, dt), dy.reshape(-1, order="F")]))[shift:]
        dz = torch.full((N * B + 2 + shift,), 7.0, dtype=dtype, device="cuda")
        db = torch.full((N + 2,), 7.0, dtype=dtype, device="cuda")
        K.knet(f"knet_relu_dropout_bias_bwd_{S}", K.lib.ptr(yd), K.lib.ptr(dyd), K.lib.ptr(dz[1 + shift:]), K.lib.ptr(db[1:]),
               N, B, ct(p))
        got = dz[1 + shift:1 + shift + N * B].cpu().numpy().reshape(N, B, order="F")
        np.testing.assert_array_equal(got, want)
        assert float(dz[shift]) == 7.0 and float(dz[-1]) == 7.0 and float(db[0]) == 7.0 and float(db[-1]) == 7.0
        ref_db = want.astype(np.float64).sum(axis=1)
        bound = (1e-5 if dtype == torch.float32 else 1e-12) * np.abs(want).astype(np.float64).sum(axis=1) + 1e-30
        assert (np.abs(db[1:-1].cpu().numpy() - ref_db) <= bound).all(), (N, B)
        if B > 0:       # in place on dy, as the MLP calls it; the summation order is fixed by the geometry,
            db2, db3 = (torch.empty(N, dtype=dtype, device="cuda") for _ in range(2))   # so two runs agree bit for bit
            save = dyd.clone()
            K.knet(f"knet_relu_dropout_bias_bwd_{S}", K.lib.ptr(yd), K.lib.ptr(dyd), K.lib.ptr(dyd), K.lib.ptr(db2), N, B, ct(p))
            np.testing.assert_array_equal(dyd.cpu().numpy().reshape(N, B, order="F"), want)
            assert (np.abs(db2.cpu().numpy() - ref_db) <= bound).all(), (N, B, "in place")
            dyd.copy_(save)
            K.knet(f"knet_relu_dropout_bias_bwd_{S}", K.lib.ptr(yd), K.lib.ptr(dyd), K.lib.ptr(dyd), K.lib.ptr(db3), N, B, ct(p))
            assert torch.equal(db2, db3)
    lib = K.lib.libknet
    assert getattr(lib, f"knet_relu_dropout_bias_bwd_{S}")(None, None, None, None, 4, -1, ct(0.5), None) == -1
    assert getattr(lib, f"knet_relu_dropout_bias_bwd_{S}")(None, None, None, None, 4, 4, ct(0.5), None) == -1
    assert getattr(lib, f"knet_relu_dropout_bias_bwd_{S}")(None, None, None, K.lib.ptr(db), 4, 4, ct(1.0), None) == -1
    assert getattr(lib, f"knet_relu_dropout_bias_bwd_{S}")(None, None, None, None, 0, 4, ct(0.5), None) == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_consecutive_generator_calls_use_disjoint_counters(K, dtype):
    """Two dropout calls in a row under the default seed, and the hidden layers of the MLP within a
    step and across steps, must draw from counter ranges that do not overlap: one counter serves 4
    Float32 but only 2 Float64 elements."""
    S = K.lib.sfx(dtype)
    n = 10001
    G = 8 if dtype == torch.float32 else 4
    assert K.ops.philox_groups(n, dtype) == (n + G - 1) // G
    x = K.KnetArray(torch.ones(n, dtype=dtype, device="cuda"))
    off0 = K.ops._philox_offset[0]
    y1, y2 = K.dropout(x, 0.5), K.dropout(x, 0.5)
    u = torch.empty(n, dtype=dtype, device="cuda")
    for y, off in ((y1, off0), (y2, off0 + K.ops.philox_groups(n, dtype))):
        K.knet(f"knet_dropout_uniform_{S}", n, 0x5EED, off, K.lib.ptr(u))
        assert torch.equal(y.data != 0, u > 0.5)
    assert K.ops._philox_offset[0] == off0 + 2 * K.ops.philox_groups(n, dtype)
    m = K.MLP([16, 40, 24, 8], 10, pdrop=0.5, dtype=dtype)
    spans = []
    for step in range(3):
        for i in range(2):
            lo = step * m._drop_per_step + m._drop_base[i]
            spans.append((lo, lo + K.ops.philox_groups(m.sizes[i + 1] * 10, dtype)))
    spans.sort()
    assert all(a[1] <= b[0] for a, b in zip(spans, spans[1:]))
    # and the layers really use them
    xin = K.KnetArray(torch.randn(16 * 10, dtype=dtype, device="cuda").abs() + 1, (16, 10))
    m.step_no = 2
    m.forward(xin)
    for i in range(2):
        nn = m.sizes[i + 1] * 10
        uu = torch.empty(nn, dtype=dtype, device="cuda")
        K.knet(f"knet_dropout_uniform_{S}", nn, m.seed, 2 * m._drop_per_step + m._drop_base[i], K.lib.ptr(uu))
        kept = m.h[i].data != 0
        assert not (kept & ~(uu > 0.5)).any()          # nothing kept that the counters say is dropped


def test_dropout_second_moment_like_the_reference_test(K):
    # test/dropout.jl:14-16: sum(abs2, dropout(x, 0.5)) within 10% of the CPU figure, whose
    # expectation is 2*sum(abs2, x)
    x = np.random.default_rng(2).random((100, 100)).astype(np.float32)
    y = K.dropout(K.KnetArray(x), 0.5, seed=1)
    assert float((y.numpy() ** 2).sum()) == pytest.approx(2 * float((x ** 2).sum()), rel=0.1)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("optname", ["sgd", "momentum", "adam"])
def test_fused_gradient_clipping_matches_per_array_gclip(K, dtype, optname):
    """The multi-tensor update with clipping factors computed on the device against update! on
    every array with gclip! (norm on the host): the norms are summed in a different order, so
    weights agree to a few ulps, not bit for bit; without clipping in effect they are identical."""
    dt = NPDT[dtype]
    rng = np.random.default_rng(12)
    sizes = [20000, 7, 8192 * 3 + 5, 1]
    mk = {"sgd": lambda c: K.SGD(lr=0.1, gclip=c), "momentum": lambda c: K.Momentum(lr=0.05, gamma=0.9, gclip=c),
          "adam": lambda c: K.Adam(lr=1e-3, gclip=c)}[optname]
    nstate = {"sgd": 0, "momentum": 1, "adam": 2}[optname]
    for clip in (0.5, 1e9):                      # 0.5 clips the large arrays, 1e9 clips nothing
        w0 = [rng.standard_normal(n).astype(dt) for n in sizes]
        g0 = [(rng.standard_normal(n) * (0.01 if n > 10 else 0.001)).astype(dt) for n in sizes]
        # eager: one optimizer per array
        we = [K.KnetArray(w.copy()) for w in w0]
        ge = [K.KnetArray(g.copy()) for g in g0]
        opts = [mk(clip) for _ in sizes]
        # fused: one plan
        wf = [dev(w.copy()) for w in w0]
        gf = [dev(g.copy()) for g in g0]
        st = [[torch.zeros_like(w) for w in wf] for _ in range(nstate)]
        plan = K.MultiTensorPlan([(wf[i], gf[i]) + tuple(s[i] for s in st) for i in range(len(sizes))])
        popt = mk(clip)
        for step in range(3):
            for w, g, o in zip(we, ge, opts):
                g.data.copy_(dev(g0[sizes.index(len(g))]))          # gclip! scales g in place: restore it
                K.update_(w, g, o)
            K.update_multi_(plan, popt)
        norms = np.array([np.sqrt((g.astype(np.float64) ** 2).sum()) for g in g0])
        want = np.where(norms > clip, clip / norms, 1.0)
        np.testing.assert_allclose(plan.clip_factors.cpu().numpy(), want, rtol=1e-6 if dtype == torch.float32 else 1e-13)
        for a, b in zip(we, wf):
            if clip > 1e6:
                assert np.array_equal(a.numpy(), b.cpu().numpy())
            else:
                np.testing.assert_allclose(a.numpy(), b.cpu().numpy(), rtol=0, atol=4 * np.finfo(dt).eps * 3)
