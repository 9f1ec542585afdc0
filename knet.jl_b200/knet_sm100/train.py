"""Optimizers and update! (src/train20/update.jl) on top of the fused update kernels.

The optimizer classes hold the same hyper-parameters, defaults and lazily created state as
Knet's structs (update.jl:125-141,172-183,210-217,257-264,300-308,348-357,398-413);
`update_` is `update!(w, g, p)` for arrays and for containers of arrays (update.jl:470-511).
`update_multi_` covers a whole parameter set with one launch.
"""
import copy
import ctypes as C

import torch

from .karray import KnetArray
from .lib import knet, knet8, knet8r, libknet, ptr, sfx
from . import ops


class Optimizer:
    gclip = 0

    def clone(self):
        """Same hyper-parameters, fresh state (update.jl `clone`)."""
        c = copy.copy(self)
        c._reset()
        return c

    def _reset(self):
        pass


class SGD(Optimizer):
    def __init__(self, lr=0.1, gclip=0):
        self.lr, self.gclip = lr, gclip


class Momentum(Optimizer):
    def __init__(self, lr=0.05, gclip=0, gamma=0.95):
        self.lr, self.gamma, self.gclip, self.velocity = lr, gamma, gclip, None

    def _reset(self):
        self.velocity = None


class Nesterov(Momentum):
    pass


class Adagrad(Optimizer):
    def __init__(self, lr=0.05, gclip=0, eps=1e-6):
        self.lr, self.eps, self.gclip, self.G = lr, eps, gclip, None

    def _reset(self):
        self.G = None


class Rmsprop(Optimizer):
    def __init__(self, lr=0.01, gclip=0, rho=0.9, eps=1e-6):
        self.lr, self.rho, self.eps, self.gclip, self.G = lr, rho, eps, gclip, None

    def _reset(self):
        self.G = None


class Adadelta(Optimizer):
    def __init__(self, lr=1.0, gclip=0, rho=0.9, eps=1e-6):
        self.lr, self.rho, self.eps, self.gclip, self.G, self.delta = lr, rho, eps, gclip, None, None

    def _reset(self):
        self.G = self.delta = None


class Adam(Optimizer):
    def __init__(self, lr=0.001, gclip=0, beta1=0.9, beta2=0.999, eps=1e-8):
        self.lr, self.beta1, self.beta2, self.eps, self.gclip = lr, beta1, beta2, eps, gclip
        self.t, self.fstm, self.scndm = 0, None, None

    def _reset(self):
        self.t, self.fstm, self.scndm = 0, None, None


def _zero_like(w):
    return KnetArray(torch.zeros_like(w.data), w.shape)


def gclip_(g, gclip):
    """gclip!(g, gclip) (update.jl:572-583): rescale g in place when norm(g) > gclip."""
    if gclip == 0:
        return g
    gnorm = knet8r(f"sumabs2_{sfx(g.dtype)}_20", len(g), ptr(g.data)) ** 0.5
    if gnorm > gclip:
        ct = C.c_float if g.dtype == torch.float32 else C.c_double
        # lmul!(gclip/gnorm, g): the scalar-times-array kernel, in place
        knet8(f"mul_{sfx(g.dtype)}_01", len(g), ct(gclip / gnorm), ptr(g.data), ptr(g.data))
    return g


def update_(w, g, p=None, gscale=1.0):
    """update!(w, g, p): in-place step on w (and p's state) with gradient g."""
    if g is None:
        return w
    if isinstance(w, dict):
        for k in g:
            update_(w[k], g[k], p[k] if isinstance(p, dict) else p, gscale)
        return w
    if isinstance(w, (list, tuple)):
        ps = p if isinstance(p, (list, tuple)) else [p] * len(w)
        if not (len(w) == len(g) == len(ps)):
            raise ValueError("weight, gradient, and optimization parameters not the same length.")
        for wi, gi, pi in zip(w, g, ps):
            update_(wi, gi, pi, gscale)
        return w
    if hasattr(w, "value") and hasattr(w, "opt"):     # Param
        if p is None:
            p = w.opt
        w = w.value
    if p is None:
        p = SGD()
    gclip_(g, p.gclip)
    S = sfx(w.dtype)
    n = len(w)
    if isinstance(p, SGD):
        knet(f"knet_sgd_{S}", n, ptr(w.data), ptr(g.data), p.lr, gscale)
    elif isinstance(p, Nesterov):
        if p.velocity is None:
            p.velocity = _zero_like(w)
        knet(f"knet_nesterov_{S}", n, ptr(w.data), ptr(g.data), ptr(p.velocity.data), p.lr, p.gamma, gscale)
    elif isinstance(p, Momentum):
        if p.velocity is None:
            p.velocity = _zero_like(w)
        knet(f"knet_momentum_{S}", n, ptr(w.data), ptr(g.data), ptr(p.velocity.data), p.lr, p.gamma, gscale)
    elif isinstance(p, Adagrad):
        if p.G is None:
            p.G = _zero_like(w)
        knet(f"knet_adagrad_{S}", n, ptr(w.data), ptr(g.data), ptr(p.G.data), p.lr, p.eps, gscale)
    elif isinstance(p, Rmsprop):
        if p.G is None:
            p.G = _zero_like(w)
        knet(f"knet_rmsprop_{S}", n, ptr(w.data), ptr(g.data), ptr(p.G.data), p.lr, p.rho, p.eps, gscale)
    elif isinstance(p, Adadelta):
        if p.G is None:
            p.G, p.delta = _zero_like(w), _zero_like(w)
        knet(f"knet_adadelta_{S}", n, ptr(w.data), ptr(g.data), ptr(p.G.data), ptr(p.delta.data),
             p.lr, p.rho, p.eps, gscale)
    elif isinstance(p, Adam):
        if p.fstm is None:
            p.fstm, p.scndm = _zero_like(w), _zero_like(w)
        p.t += 1
        knet(f"knet_adam_{S}", n, ptr(w.data), ptr(g.data), ptr(p.fstm.data), ptr(p.scndm.data),
             p.lr, p.beta1, p.beta2, p.eps, p.t, gscale)
    else:
        raise TypeError(f"unknown optimizer {type(p)}")
    return w


# ---- multi-tensor update ---------------------------------------------------------------------------
class TensorDesc(C.Structure):
    _fields_ = [("p", C.c_void_p * 4), ("n", C.c_int64), ("first_chunk", C.c_int64)]


class MultiTensorPlan:
    """Device-resident descriptor table for one parameter set: built once, reused every step.
    `arrays` is a list of (w, g, s1, s2) tuples of 1-D tensors / KnetArrays (None when unused)."""

    def __init__(self, arrays):
        def tptr(a):
            if a is None:
                return None
            return (a.data if isinstance(a, KnetArray) else a).data_ptr()

        n = len(arrays)
        host = (TensorDesc * max(n, 1))()
        for i, tup in enumerate(arrays):
            tup = tuple(tup) + (None,) * (4 - len(tup))
            for k in range(4):
                host[i].p[k] = tptr(tup[k])
            w = tup[0].data if isinstance(tup[0], KnetArray) else tup[0]
            host[i].n = w.numel()
        self.dtype = (arrays[0][0].data if isinstance(arrays[0][0], KnetArray) else arrays[0][0]).dtype
        self.ntensors = n
        self.total_chunks = libknet.knet_multi_plan(C.cast(host, C.c_void_p), n)
        raw = bytes(host)
        self.table = torch.frombuffer(bytearray(raw), dtype=torch.uint8).cuda()
        self._keep = arrays
        self.clip_partials = self.clip_factors = None      # scratch of the fused gradient clipping


def update_multi_(plan, p, gscale=1.0, advance=True):
    """One launch for every array of `plan` with optimizer `p` (state arrays are in the plan;
    Adam's step counter lives in `p`; `advance=False` keeps the counter where it is, for the
    second and later launches of one step whose parameter set was split over several plans).  With `p.gclip > 0` every array's gradient is clipped
    to that norm as `gclip!` does (src/train20/update.jl:572-583), without the host round
    trip of norm(g): two small launches leave the per-array factors on the device and the
    update applies them to the gradient as it loads it."""
    S = sfx(plan.dtype)
    clip = getattr(p, "gclip", 0) or 0
    tail = ()
    sfx_c = ""
    if clip > 0:
        if plan.clip_partials is None:
            plan.clip_partials = torch.empty(max(int(plan.total_chunks), 1), dtype=plan.dtype, device=plan.table.device)
            plan.clip_factors = torch.ones(max(plan.ntensors, 1), dtype=torch.float64, device=plan.table.device)
        knet(f"knet_gclip_factors_{S}", ptr(plan.table), plan.ntensors, plan.total_chunks, float(clip), float(gscale),
             ptr(plan.clip_partials), ptr(plan.clip_factors))
        tail, sfx_c = (ptr(plan.clip_factors),), "_c"
    if isinstance(p, Adam):
        if advance:
            p.t += 1
        knet(f"knet_adam_multi{sfx_c}_{S}", ptr(plan.table), plan.ntensors, plan.total_chunks, p.lr, p.beta1,
             p.beta2, p.eps, p.t, gscale, *tail)
    elif isinstance(p, Momentum) and not isinstance(p, Nesterov):
        knet(f"knet_momentum_multi{sfx_c}_{S}", ptr(plan.table), plan.ntensors, plan.total_chunks, p.lr, p.gamma,
             gscale, *tail)
    elif isinstance(p, SGD):
        knet(f"knet_sgd_multi{sfx_c}_{S}", ptr(plan.table), plan.ntensors, plan.total_chunks, p.lr, gscale, *tail)
    else:
        raise TypeError(f"no multi-tensor kernel for {type(p)}")


# ---- parameters and initialisation (src/train20/param.jl:22-24, distributions.jl:35-52) ------------
class Param:
    def __init__(self, value, opt=None):
        self.value, self.opt = value, opt


def xavier_uniform(rows, cols, rng, dtype=torch.float32, gain=1.0):
    """2s*rand(rows,cols) - s with s = gain*sqrt(6/(fanin+fanout)), drawn and computed in
    Float64 on the host, then converted to the array type as param() does."""
    import numpy as np
    u = rng.random((rows, cols))
    s = gain * np.sqrt(6.0 / (rows + cols))
    w = (2 * s) * u - s
    return KnetArray(np.asfortranarray(w.astype(np.float32 if dtype == torch.float32 else np.float64)))


def param(rows, cols, rng, dtype=torch.float32):
    return Param(xavier_uniform(rows, cols, rng, dtype))


def param0(n, dtype=torch.float32):
    return Param(KnetArray.zeros((n,), dtype))
