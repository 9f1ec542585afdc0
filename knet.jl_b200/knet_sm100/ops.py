"""Knet's array operations on KnetArray, dispatched to libknet_sm100 the way Knet's Julia
wrappers dispatch to libknet8.

Mirrors: unary ops src/knetarrays/unary.jl:11-32 and src/ops20_gpu/activation.jl:16-46;
binary broadcast src/knetarrays/binary.jl:13-282; reductions src/knetarrays/reduction.jl:
21-77; softmax family src/ops20/softmax.jl:36-78 and src/ops20_gpu/softmax.jl:10-59; nll and
accuracy src/ops20/loss.jl:37-62; dropout src/ops20/dropout.jl:15-42; matrix products
src/knetarrays/linalg.jl:11-55 (cuBLAS, through torch.mm or knet_gemm_S_S).  `dims` is 1-based.
"""
import ctypes as C

import numpy as np
import torch

from .karray import KnetArray, _prod
from .lib import knet, knet8, knet8r, ptr, sfx

_CT = {torch.float32: C.c_float, torch.float64: C.c_double}


# ---- unary ---------------------------------------------------------------------------------
def unary(name, x, out=None):
    y = x.similar() if out is None else out
    knet8(f"{name}_{sfx(x.dtype)}", len(x), ptr(x.data), ptr(y.data))
    return y


def relu(x): return unary("relu", x)
def sigm(x): return unary("sigm", x)
def tanh(x): return unary("tanh", x)
def elu(x): return unary("elu", x)
def selu(x): return unary("selu", x)
def exp(x): return unary("exp", x)
def log(x): return unary("log", x)
def sqrt(x): return unary("sqrt", x)
def abs2(x): return unary("abs2", x)


def actback(name, dy, y, out=None):
    """reluback/sigmback/tanhback/eluback.(dy, y) (src/ops20_gpu/activation.jl:30-46)."""
    dx = y.similar() if out is None else out
    knet8(f"{name}_{sfx(y.dtype)}_11", len(y), ptr(dy.data), ptr(y.data), ptr(dx.data))
    return dx


def reluback(dy, y): return actback("reluback", dy, y)
def sigmback(dy, y): return actback("sigmback", dy, y)
def tanhback(dy, y): return actback("tanhback", dy, y)
def eluback(dy, y): return actback("eluback", dy, y)


def fill_(x, v):
    knet8(f"fill_{sfx(x.dtype)}", len(x), _CT[x.dtype](v), ptr(x.data))
    return x


# ---- binary broadcast --------------------------------------------------------------------------
def vbroadcast_shape(xshape, yshape):
    """Index/offset arguments of the vector-broadcast kernels (binary.jl:152-212):
    returns (dz, sx, nx, sy, ny, xlast, ylast, xdims, ydims, multi)."""
    nz = max(len(xshape), len(yshape))
    xs = tuple(xshape) + (1,) * (nz - len(xshape))
    ys = tuple(yshape) + (1,) * (nz - len(yshape))
    dz = [1] * nz
    xdims = ydims = xsame = ysame = xlast = ylast = 0
    for i in range(nz):
        if xs[i] > 1:
            xdims += 1
            xlast = i + 1
            dz[i] = xs[i]
        if ys[i] > 1:
            ydims += 1
            ylast = i + 1
            if dz[i] == 1:
                dz[i] = ys[i]
            elif dz[i] != ys[i]:
                raise ValueError("arrays could not be broadcast to a common size")
        xsame += dz[i] == xs[i]
        ysame += dz[i] == ys[i]
    zlen = _prod(dz)
    multi = (xsame != nz and xdims > 1) or (ysame != nz and ydims > 1)

    def sn(dims, last, same):
        if dims == 0:
            return zlen, 1
        if dims == 1:
            return _prod(dz[:last - 1]), dz[last - 1]
        if same == nz:
            return 1, zlen
        if not multi:
            raise ValueError("Broadcasting error")
        return -1, -1

    sx, nx = sn(xdims, xlast, xsame)
    sy, ny = sn(ydims, ylast, ysame)
    return tuple(dz), sx, nx, sy, ny, xlast, ylast, xdims, ydims, multi


def _strides(shape, n):
    shape = tuple(shape) + (1,) * (n - len(shape))
    return [_prod(shape[:i]) for i in range(n)], shape


def get_strides(xshape, yshape, zshape):
    """Per-dim strides with 0 on broadcast dims (binary.jl:214-231)."""
    n = max(len(xshape), len(yshape), len(zshape))
    sx, dx = _strides(xshape, n)
    sy, dy = _strides(yshape, n)
    sz, _ = _strides(zshape, n)
    for i in range(n):
        if dx[i] == dy[i]:
            continue
        if dx[i] == 1:
            sx[i] = 0
        else:
            sy[i] = 0
    return sx, sy, sz


_COMMUTE = {"add": "add", "mul": "mul", "max": "max", "min": "min", "eq": "eq", "ne": "ne",
            "gt": "lt", "ge": "le", "lt": "gt", "le": "ge"}


def _scalar_first(op, s, y):
    z = y.similar()
    knet8(f"{op}_{sfx(y.dtype)}_01", len(z), _CT[y.dtype](s), ptr(y.data), ptr(z.data))
    return z


def broadcast(op, x, y):
    """`x .op y` for KnetArrays and scalars; comparisons give 0/1 in the array type."""
    xa, ya = isinstance(x, KnetArray), isinstance(y, KnetArray)
    if not xa and not ya:
        raise TypeError("broadcast needs at least one KnetArray")
    if not xa:
        return _scalar_first(op, float(x), y)
    if not ya:
        s = float(y)
        if op in _COMMUTE:                       # f(x, s) == f'(s, x)
            return _scalar_first(_COMMUTE[op], s, x)
        if op == "sub":                          # x - s == (-s) + x exactly (binary.jl:346)
            return _scalar_first("add", -s, x)
        # div, pow: a true x/s as on the CPU, through the scalar-operand case of the _12 kernel
        sd = torch.tensor([s], dtype=x.dtype, device=x.data.device)
        z = x.similar()
        n = len(z)
        knet8(f"{op}_{sfx(x.dtype)}_12", n, ptr(x.data), 1, n, ptr(sd), n, 1, ptr(z.data))
        return z
    if x.dtype != y.dtype:
        raise TypeError("element types differ")
    S = sfx(x.dtype)
    if x.shape == y.shape:
        z = x.similar()
        knet8(f"{op}_{S}_11", len(z), ptr(x.data), ptr(y.data), ptr(z.data))
        return z
    dz, sx, nx, sy, ny, xlast, ylast, xdims, ydims, multi = vbroadcast_shape(x.shape, y.shape)
    z = x.similar(dz)
    n = len(z)
    if n >= 2 ** 31:
        raise ValueError("libknet sizes are 32-bit")
    if n == 0:
        return z
    if len(dz) <= 2:
        if len(x) == 1 or len(y) == 1 or not multi and (
                nx == 1 or ny == 1
                or (xdims == 1 and (xlast == 1 or 512 < sx)) or (ydims == 1 and (ylast == 1 or sy < 512))
                or (xdims == 1 and nx < 704) or (ydims == 1 and ny < 704)):
            knet8(f"{op}_{S}_12", n, ptr(x.data), sx, nx, ptr(y.data), sy, ny, ptr(z.data))
        elif xdims == 1:
            ds = y.stride(xlast)
            ns = 0 if xlast + 1 > y.ndim else y.stride(xlast + 1)
            md = _prod(y.shape[xlast:])
            knet8(f"{op}_{S}_13_y_x", ptr(y.data), ptr(x.data), ptr(z.data), ds, ns, md, len(y), len(x))
        elif ydims == 1:
            ds = x.stride(ylast)
            ns = 0 if ylast + 1 > x.ndim else x.stride(ylast + 1)
            md = _prod(x.shape[ylast:])
            knet8(f"{op}_{S}_13_x_y", ptr(x.data), ptr(y.data), ptr(z.data), ds, ns, md, len(x), len(y))
        else:
            raise ValueError(f"cannot broadcast {x.shape} with {y.shape}")
        return z
    if len(dz) <= 5:
        sxs, sys_, szs = get_strides(x.shape, y.shape, dz)
        knet8(f"{op}_{S}_16_{len(dz)}", ptr(x.data), ptr(y.data), ptr(z.data), *sxs, *sys_, *szs, n)
        return z
    raise NotImplementedError("broadcast over more than 5 dims (libknet8's _17 kernel) is not provided")


# ---- reductions --------------------------------------------------------------------------------
REDUCTIONS = ("sum", "prod", "maximum", "minimum", "sumabs", "sumabs2", "maxabs", "minabs", "countnz")


def reduce(op, x, dims=None):
    """`op(x; dims)`; dims=None is Julia's `:` and returns a Python float after a sync."""
    S = sfx(x.dtype)
    if dims is None:
        return knet8r(f"{op}_{S}_20", len(x), ptr(x.data))
    dims = (dims,) if isinstance(dims, int) else tuple(dims)
    nd = x.ndim
    rdims = tuple(1 if (i + 1) in dims else x.shape[i] for i in range(nd))
    vdims = nd - len(dims)
    if len(dims) != 1 or nd == 1:
        vdims = len([r for r in rdims if r > 1])
    if vdims == 0:
        return fill_(x.similar(rdims), reduce(op, x))
    if vdims == 1:
        kept = [i + 1 for i in range(nd) if (i + 1) not in dims]
        if len(kept) != 1:
            # several kept dims of which only one is larger than 1: fold the others away
            kept = [k for k in kept if x.shape[k - 1] > 1]
        i0 = kept[0]
        y = x.similar(rdims)
        knet8(f"{op}_{S}_21", len(x), ptr(x.data), x.stride(i0), len(y), ptr(y.data))
        return y
    if vdims == nd - 1:
        d = dims[0]
        y = x.similar(rdims)
        knet8(f"{op}_{S}_22", len(x), x.shape[d - 1] - 1, ptr(x.data), x.stride(d), x.stride(d + 1),
              len(y), ptr(y.data))
        return y
    y = reduce(op, x, dims[0])
    f = "sum" if op in ("sumabs2", "sumabs", "countnz") else {"maxabs": "maximum", "minabs": "minimum"}.get(op, op)
    for k in dims[1:]:
        y = reduce(f, y, k)
    return y


def sum(x, dims=None): return reduce("sum", x, dims)          # noqa: A001
def maximum(x, dims=None): return reduce("maximum", x, dims)
def minimum(x, dims=None): return reduce("minimum", x, dims)
def sumabs2(x, dims=None): return reduce("sumabs2", x, dims)


# ---- softmax family ------------------------------------------------------------------------------
def _geometry(shape, dims):
    """(inner, D, outer) when `dims` (None = all) is a run of adjacent dims, else None."""
    nd = len(shape)
    if dims is None:
        return 1, _prod(shape), 1
    dims = sorted({dims} if isinstance(dims, int) else set(dims))
    dims = [d for d in dims if d <= nd]
    if not dims:
        return _prod(shape), 1, 1
    if dims != list(range(dims[0], dims[-1] + 1)):
        return None
    return _prod(shape[:dims[0] - 1]), _prod(shape[dims[0] - 1:dims[-1]]), _prod(shape[dims[-1]:])


def _soft(fn, x, dims, *more):
    g = _geometry(x.shape, dims)
    if g is None:
        raise NotImplementedError("dims must be adjacent for the fused kernels")
    y = x.similar()
    knet(f"{fn}_{sfx(x.dtype)}", ptr(x.data), *[ptr(m.data) for m in more], ptr(y.data), *g)
    return y


def softmax(x, dims=None):
    if _geometry(x.shape, dims) is None:          # generic path of src/ops20/softmax.jl:53-59
        e = exp(x - maximum(x, dims))
        return e / sum(e, dims)
    return _soft("knet_softmax_fwd", x, dims)


def logsoftmax(x, dims=None):
    if _geometry(x.shape, dims) is None:          # src/ops20/softmax.jl:42-47
        x1 = x - maximum(x, dims)
        return x1 - log(sum(exp(x1), dims))
    return _soft("knet_logsoftmax_fwd", x, dims)


logp = logsoftmax


def softmax_back(y, dy, dims=None):
    """∇softmax: y.*dy .- y.*sum(y.*dy, dims) (softmax.jl:61-63)."""
    if _geometry(y.shape, dims) is None:
        return y * dy - y * sum(y * dy, dims)
    return _soft("knet_softmax_bwd", y, dims, dy)


def logsoftmax_back(y, dy, dims=None):
    """∇logsoftmax: dy - exp.(y).*sum(dy, dims) (softmax.jl:49-51)."""
    if _geometry(y.shape, dims) is None:
        return dy - exp(y) * sum(dy, dims)
    return _soft("knet_logsoftmax_bwd", y, dims, dy)


def _reduced_shape(shape, dims):
    if dims is None:
        return (1,) * len(shape)
    dims = {dims} if isinstance(dims, int) else set(dims)
    return tuple(1 if (i + 1) in dims else s for i, s in enumerate(shape))


def logsumexp(x, dims=None):
    g = _geometry(x.shape, dims)
    if g is None:                                   # src/ops20/softmax.jl:65-70
        m = maximum(x, dims)
        return m + log(sum(exp(x - m), dims))
    y = x.similar(_reduced_shape(x.shape, dims))
    knet(f"knet_logsumexp_fwd_{sfx(x.dtype)}", ptr(x.data), ptr(y.data), *g)
    return y


def logsumexp_back(x, y, dy, dims=None):
    """∇logsumexp: dy .* exp.(x .- y) (softmax.jl:72-74)."""
    g = _geometry(x.shape, dims)
    if g is None:
        return dy * exp(x - y)
    dx = x.similar()
    knet(f"knet_logsumexp_bwd_{sfx(x.dtype)}", ptr(x.data), ptr(y.data), ptr(dy.data), ptr(dx.data), *g)
    return dx


# ---- loss ------------------------------------------------------------------------------------------
def _labels(labels, device):
    """Int32 device labels (1-based, 0 = skip); host arrays are uploaded once per call."""
    if isinstance(labels, torch.Tensor):
        return labels.to(device=device, dtype=torch.int32).contiguous().view(-1)
    return torch.from_numpy(np.ascontiguousarray(np.asarray(labels).reshape(-1, order="F"),
                                                 dtype=np.int32)).to(device)


def _rk(scores):
    R = scores.shape[0]
    return R, len(scores) // R if R else 0


class NllResult:
    """Device-side result of the fused nll forward: total = -sum(lp), count, and the
    per-instance buffer the kernel needs as scratch."""

    def __init__(self, total, count, per_instance, labels):
        self.total, self.count, self.per_instance, self.labels = total, count, per_instance, labels

    def value(self, average=True):
        t, c = float(self.total.item()), int(self.count.item())
        return (t / c) if average else (t, c)


def nll_device(scores, labels, dims=1):
    R, K = _rk(scores)
    ninst = K if dims == 1 else R
    lab = _labels(labels, scores.data.device)
    if lab.numel() != ninst:
        raise ValueError("DimensionMismatch: one label per instance is needed")
    total = torch.empty(1, dtype=scores.dtype, device=scores.data.device)
    count = torch.empty(1, dtype=torch.int32, device=scores.data.device)
    per = torch.empty(max(ninst, 1), dtype=scores.dtype, device=scores.data.device)
    knet(f"knet_nll_fwd_{sfx(scores.dtype)}", ptr(scores.data), ptr(lab), R, K, dims, ptr(total),
         ptr(count), ptr(per))
    return NllResult(total, count, per, lab)


def nll(scores, labels, dims=1, average=True):
    """Negative log likelihood (loss.jl:37-41): a float, or (total, count) if not average."""
    return nll_device(scores, labels, dims).value(average)


def nll_back(scores, labels, dims=1, average=True, dy=1.0, count=None):
    """Gradient of nll wrt scores: (softmax - onehot) * dy [/ count]."""
    R, K = _rk(scores)
    lab = _labels(labels, scores.data.device)
    if average and count is None:
        count = (lab != 0).sum().to(torch.int32).view(1)
    dx = scores.similar()
    knet(f"knet_nll_bwd_{sfx(scores.dtype)}", ptr(scores.data), ptr(lab), R, K, dims, int(average),
         _CT[scores.dtype](dy), ptr(count), ptr(dx.data))
    return dx


def argmax(x, dims=1):
    """1-based position of the first maximum along `dims` (Julia argmax, as Int32)."""
    g = _geometry(x.shape, dims)
    idx = torch.empty(max(g[0] * g[2], 1), dtype=torch.int32, device=x.data.device)
    knet(f"knet_argmax_{sfx(x.dtype)}", ptr(x.data), ptr(idx), *g)
    return idx[:g[0] * g[2]]


def accuracy(scores, labels, dims=1, average=True):
    """Share of instances whose first maximal score is at the label (loss.jl:54-62)."""
    R, K = _rk(scores)
    lab = _labels(labels, scores.data.device)
    res = torch.empty(2, dtype=torch.int32, device=scores.data.device)
    knet(f"knet_accuracy_{sfx(scores.dtype)}", ptr(scores.data), ptr(lab), R, K, dims, ptr(res))
    ok, cnt = (int(v) for v in res.tolist())
    return (ok / cnt) if average else (ok, cnt)


# ---- dropout ---------------------------------------------------------------------------------------
_philox_offset = [0]


def philox_groups(n, dtype):
    """Counters one generator call over n elements consumes: the kernels draw one Philox counter
    per 8 Float32 or per 4 Float64 elements (32 bytes), so consecutive calls under one seed must
    advance their offset by this much to use disjoint counter ranges."""
    g = 8 if dtype == torch.float32 else 4
    return (n + g - 1) // g


def dropout(x, p, seed=0, drop=True, uniforms=None):
    """dropout(x, p; seed, drop) (dropout.jl:15-27).  `uniforms` supplies the U[0,1) draws
    that Knet's rand!(y) would make; without it the in-kernel Philox generator is used."""
    if not drop or p == 0:
        return x
    if p == 1:
        return fill_(x.similar(), 0)
    if not 0 < p < 1:
        raise ValueError(f"Dropout probability not in [0:1]: {p}")
    S = sfx(x.dtype)
    if uniforms is not None:
        y = KnetArray(uniforms.data.clone(), x.shape)
        knet8(f"dropout_{S}", len(x), _CT[x.dtype](p), ptr(x.data), ptr(y.data))
        return y
    y = x.similar()
    if seed == 0:
        seed, off = 0x5EED, _philox_offset[0]
        _philox_offset[0] += philox_groups(len(x), x.dtype)
    else:
        off = 0
    knet(f"knet_dropout_philox_{S}", len(x), _CT[x.dtype](p), seed, off, ptr(x.data), ptr(y.data))
    return y


def dropback(dy, y, x, p):
    """dropback(dy, y, x, p) (dropout.jl:29-39)."""
    if p == 0:
        return dy
    if p == 1:
        return fill_(x.similar(), 0)
    dx = y.similar()
    knet8(f"dropback_{sfx(y.dtype)}", len(y), _CT[y.dtype](p), ptr(x.data), ptr(y.data), ptr(dy.data),
          ptr(dx.data))
    return dx


# ---- matrix products (cuBLAS; not part of this library's kernels) ----------------------------------
# KNET_SM100_GEMM chooses who makes the cuBLAS call: "torch" (default) is torch.mm; "native" is
# knet_gemm_S_S in plain FP32/FP64 arithmetic; "emulated" is knet_gemm_32_S with cuBLAS's FP32
# emulation on the BF16 tensor cores (Float64 stays native), which needs cuBLAS 12.9 or later
# in the process.
import os
import threading

GEMM_MODE = os.environ.get("KNET_SM100_GEMM", "torch")
if GEMM_MODE not in ("torch", "native", "emulated"):
    raise ValueError(f"KNET_SM100_GEMM={GEMM_MODE!r}: expected torch, native or emulated")
_gemm_tls = threading.local()


class GemmHandle:
    """One cuBLAS handle of the calling thread and current device (knet_gemm_create), with
    the scratch cuBLAS may use (KNET_SM100_GEMM_WS_MB, default 2048 for the emulation, which
    stores the BF16 terms of both operands there)."""

    def __init__(self, device):
        from .lib import check, libknet
        h = C.c_void_p()
        check(libknet.knet_gemm_create(C.byref(h)), "knet_gemm_create")
        self.h, self.device = h, device
        self.version = libknet.knet_gemm_version(h)
        self.emulation = libknet.knet_gemm_emulation(h) == 1
        mb = int(os.environ.get("KNET_SM100_GEMM_WS_MB", "2048" if GEMM_MODE == "emulated" else "0"))
        self.ws = torch.empty(mb << 20, dtype=torch.uint8, device=device) if mb > 0 else None

    def __del__(self):
        try:
            from .lib import libknet
            libknet.knet_gemm_destroy(self.h)
        except Exception:
            pass


def gemm_handle():
    dev = torch.cuda.current_device()
    tab = _gemm_tls.__dict__.setdefault("handles", {})
    if dev not in tab:
        tab[dev] = GemmHandle(torch.device("cuda", dev))
    return tab[dev]


def gemm_(ta, tb, m, n, k, a, lda, b, ldb, c, ldc, alpha=1.0, beta=0.0, mode=None):
    """gemm!(transA, transB, alpha, A, B, beta, C) on flat column-major storage
    (src/knetarrays/linalg.jl:27-55) through knet_gemm_S_S."""
    g = gemm_handle()
    if mode is None:
        mode = 1 if (GEMM_MODE == "emulated" and c.dtype == torch.float32) else 0
    ct = _CT[c.dtype]
    knet(f"knet_gemm_{sfx(c.dtype)}_S", g.h, int(ta), int(tb), m, n, k, ct(alpha), ptr(a), lda, ptr(b), ldb,
         ct(beta), ptr(c), ldc, mode, ptr(g.ws), 0 if g.ws is None else g.ws.numel())


def matmul(w, x, out=None):
    """w*x for column-major matrices (linalg.jl:11): (m,k)*(k,n) -> (m,n)."""
    m, n = w.shape[0], (x.shape[1] if x.ndim > 1 else 1)
    z = w.similar((m, n)) if out is None else out
    if GEMM_MODE == "torch":
        torch.mm(x.data.view(n, -1), w.as_rowmajor(), out=z.data.view(n, m))
    else:
        k = w.shape[1]
        gemm_(0, 0, m, n, k, w.data, m, x.data, k, z.data, m)
    return z


def A_mul_Bt(a, b, out=None):
    """a*b' (linalg.jl:12): (m,n)*(k,n)' -> (m,k)."""
    m, k, n = a.shape[0], b.shape[0], a.shape[1]
    z = a.similar((m, k)) if out is None else out
    if GEMM_MODE == "torch":
        torch.mm(b.data.view(n, k).t(), a.data.view(n, m), out=z.data.view(k, m))
    else:
        gemm_(0, 1, m, k, n, a.data, m, b.data, k, z.data, m)
    return z


def At_mul_B(a, b, out=None):
    """a'*b (linalg.jl:13): (m,k)'*(m,n) -> (k,n)."""
    m, k, n = a.shape[0], a.shape[1], b.shape[1]
    z = a.similar((k, n)) if out is None else out
    if GEMM_MODE == "torch":
        torch.mm(b.data.view(n, m), a.data.view(k, m).t(), out=z.data.view(n, k))
    else:
        gemm_(1, 0, k, n, m, a.data, m, b.data, m, z.data, k)
    return z
