"""Checks of the knet_gemm_* entry points in a process of their own, so that the environment
(KNET_SM100_GEMM, KNET_SM100_CUBLAS_DIR) is in place before PyTorch loads its cuBLAS.
Prints one JSON line; run by tests/test_gpu_gemm.py.

  python tests/gemm_check.py            products against Float64, every mode the process offers
  python tests/gemm_check.py --curve    the 784-64-10 loss curve against the oracle's
"""
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (os.path.join(ROOT, "knet.jl_b200"), os.path.join(ROOT, "oracle"), os.path.join(ROOT, "tests")):
    sys.path.insert(0, p)

import knet_sm100 as K          # noqa: E402  (before torch: see knet_sm100/__init__.py)
import numpy as np              # noqa: E402
import torch                    # noqa: E402
from knet_sm100 import ops      # noqa: E402


def rel_err(got, want, scale=None):
    """Largest error of an entry relative to `scale` (entry by entry: sum_k |a_ik| |b_kj|, the
    size rounding errors of a product are measured against), else to the largest entry."""
    d = np.abs(got.astype(np.float64) - want)
    return float((d / scale).max()) if scale is not None else float(d.max() / np.abs(want).max())


def products():
    rng = np.random.default_rng(7)
    g = ops.gemm_handle()
    rep = {"version": g.version, "emulation": g.emulation, "gemm_mode": ops.GEMM_MODE, "cases": []}
    modes = [0] + ([1, 2] if g.emulation else [])
    for (m, n, k) in ((1024, 768, 2048), (257, 130, 515), (8, 4096, 64), (4096, 8, 1000), (1, 1, 1)):
        a = rng.standard_normal((m, k)).astype(np.float32)
        b = rng.standard_normal((k, n)).astype(np.float32)
        # wide dynamic range: rows of a and columns of b scaled over 2^-20 .. 2^20
        a2 = a * np.exp2(rng.integers(-20, 21, (m, 1))).astype(np.float32)
        b2 = b * np.exp2(rng.integers(-20, 21, (1, n))).astype(np.float32)
        for tag, (aa, bb) in (("normal", (a, b)), ("scaled", (a2, b2))):
            want = aa.astype(np.float64) @ bb.astype(np.float64)
            sc = np.abs(aa).astype(np.float64) @ np.abs(bb).astype(np.float64)
            A, B = K.KnetArray(np.asfortranarray(aa)), K.KnetArray(np.asfortranarray(bb))
            At, Bt = K.KnetArray(np.asfortranarray(aa.T)), K.KnetArray(np.asfortranarray(bb.T))
            case = {"shape": [m, n, k], "data": tag}
            for mode in modes:
                z = A.similar((m, n))
                ops.gemm_(0, 0, m, n, k, A.data, m, B.data, k, z.data, m, mode=mode)
                e_nn = rel_err(z.numpy(), want, sc)
                ops.gemm_(0, 1, m, n, k, A.data, m, Bt.data, n, z.data, m, mode=mode)
                e_nt = rel_err(z.numpy(), want, sc)
                ops.gemm_(1, 0, m, n, k, At.data, k, B.data, k, z.data, m, mode=mode)
                e_tn = rel_err(z.numpy(), want, sc)
                # alpha and beta: z <- 0.5*A*B - 2*z  (z holds A*B) = -1.5*A*B
                ops.gemm_(0, 0, m, n, k, A.data, m, B.data, k, z.data, m, alpha=0.5, beta=-2.0, mode=mode)
                e_ab = rel_err(z.numpy(), -1.5 * want, 2.5 * sc)
                case[f"mode{mode}"] = max(e_nn, e_nt, e_tn, e_ab)
            t = torch.mm(torch.from_numpy(aa).cuda(), torch.from_numpy(bb).cuda()).cpu().numpy()
            case["torch"] = rel_err(t, want, sc)
            rep["cases"].append(case)
    # Float64 and the argument checks
    a = rng.standard_normal((300, 200))
    b = rng.standard_normal((200, 100))
    A, B = K.KnetArray(np.asfortranarray(a)), K.KnetArray(np.asfortranarray(b))
    z = A.similar((300, 100))
    ops.gemm_(0, 0, 300, 100, 200, A.data, 300, B.data, 200, z.data, 300, mode=0)
    rep["f64"] = rel_err(z.numpy(), a @ b)
    bad = []
    for args in ((0, 0, 300, 100, 200, A.data, 299, B.data, 200, z.data, 300),      # lda < m
                 (0, 2, 300, 100, 200, A.data, 300, B.data, 200, z.data, 300),      # unknown op
                 (0, 0, -1, 100, 200, A.data, 300, B.data, 200, z.data, 300)):
        try:
            ops.gemm_(*args, mode=0)
            bad.append(0)
        except K.KnetError as e:
            bad.append(-1 if "status -1" in str(e) else 1)
    try:
        ops.gemm_(0, 0, 300, 100, 200, A.data, 300, B.data, 200, z.data, 300, mode=1)   # Float64 emulation: refused
        bad.append(0)
    except K.KnetError as e:
        bad.append(-1 if "status -1" in str(e) else 1)
    rep["argument_errors"] = bad
    # products through the package's own wrappers in the mode the environment chose
    w = K.KnetArray(np.asfortranarray(rng.standard_normal((64, 96)).astype(np.float32)))
    x = K.KnetArray(np.asfortranarray(rng.standard_normal((96, 32)).astype(np.float32)))
    dz = K.KnetArray(np.asfortranarray(rng.standard_normal((64, 32)).astype(np.float32)))
    wn, xn, dn = (t.numpy().astype(np.float64) for t in (w, x, dz))
    if ops.GEMM_MODE == "emulated" and not g.emulation:       # nothing more to check in this process
        return rep
    rep["wrappers"] = max(rel_err(ops.matmul(w, x).numpy(), wn @ xn), rel_err(ops.A_mul_Bt(dz, x).numpy(), dn @ xn.T),
                          rel_err(ops.At_mul_B(w, dz).numpy(), wn.T @ dn))
    return rep


def curve():
    if ops.GEMM_MODE == "emulated" and not ops.gemm_handle().emulation:
        return {"gemm_mode": ops.GEMM_MODE, "emulation": False, "version": ops.gemm_handle().version}
    import knet_oracle as ko
    ko.build()
    sizes, B = [784, 64, 10], 100
    rng = np.random.default_rng(1)
    ws = [ko.xavier_uniform(sizes[i + 1], sizes[i], rng) for i in range(len(sizes) - 1)]
    weights = [(w, np.zeros(w.shape[0], np.float32)) for w in ws]
    ref = ko.MLP(sizes, np.random.default_rng(0), lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8)
    ref.w = [np.asfortranarray(w.copy()) for w, _ in weights]
    ref.b = [b.copy() for _, b in weights]
    gpu = K.MLP(sizes, B, weights=weights, optimizer=K.Adam(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8))
    rng = np.random.default_rng(1)
    x = rng.random((784, B)).astype(np.float32)
    y = rng.integers(1, 11, B)
    worst = 0.0
    for _ in range(100):
        l_ref = float(ref.step(x, y))
        tot, cnt = gpu.step(K.KnetArray(x), torch.from_numpy(y.astype(np.int32)).cuda())
        worst = max(worst, abs(float(tot.item()) / int(cnt.item()) - l_ref))
    g = ops.gemm_handle() if ops.GEMM_MODE != "torch" else None
    return {"gemm_mode": ops.GEMM_MODE, "worst": worst, "last": l_ref,
            "emulation": bool(g and g.emulation), "version": g.version if g else 0}


if __name__ == "__main__":
    torch.cuda.set_device(0)
    out = curve() if "--curve" in sys.argv else products()
    torch.cuda.synchronize()
    print(json.dumps(out))
