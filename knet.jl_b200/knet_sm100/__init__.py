"""Host-side mirror of the Knet interface served by libknet_sm100.so.

Importing this package loads the shared library and fails if it has not been built: there
is no CPU or PyTorch fallback for the kernels.
"""
import ctypes as _C
import os as _os
import sys as _sys


def _preload_cublas():
    """KNET_SM100_CUBLAS_DIR names a directory with libcublas.so.12 and libcublasLt.so.12 to use
    instead of the copies PyTorch would bring (e.g. a cuBLAS recent enough for the FP32
    emulation of knet_gemm_32_S).  The dynamic loader binds one copy per process, the first
    one loaded, so this only takes effect when the package is imported before torch."""
    d = _os.environ.get("KNET_SM100_CUBLAS_DIR")
    if not d or "torch" in _sys.modules:
        return
    for name in ("libcublasLt.so.12", "libcublas.so.12"):
        _C.CDLL(_os.path.join(d, name), mode=_C.RTLD_GLOBAL)


_preload_cublas()

from .lib import KnetError, libknet, knet, knet8, knet8r  # noqa: F401
from .karray import KnetArray  # noqa: F401
from . import autograd, indexing, ops, train  # noqa: F401
from .ops import (relu, sigm, tanh, elu, selu, softmax, logsoftmax, logp, logsumexp, nll, accuracy,  # noqa: F401
                  dropout, argmax)
from .train import (SGD, Momentum, Nesterov, Adagrad, Rmsprop, Adadelta, Adam, Param, update_,  # noqa: F401
                    update_multi_, MultiTensorPlan, param, param0)
from .mlp import MLP  # noqa: F401
