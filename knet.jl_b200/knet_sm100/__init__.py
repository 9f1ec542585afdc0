"""Host-side mirror of the Knet interface served by libknet_sm100.so.

Importing this package loads the shared library and fails if it has not been built: there
is no CPU or PyTorch fallback for the kernels.
"""
from .lib import KnetError, libknet, knet, knet8, knet8r  # noqa: F401
from .karray import KnetArray  # noqa: F401
from . import autograd, indexing, ops, train  # noqa: F401
from .ops import (relu, sigm, tanh, elu, selu, softmax, logsoftmax, logp, logsumexp, nll, accuracy,  # noqa: F401
                  dropout, argmax)
from .train import (SGD, Momentum, Nesterov, Adagrad, Rmsprop, Adadelta, Adam, Param, update_,  # noqa: F401
                    update_multi_, MultiTensorPlan, param, param0)
from .mlp import MLP  # noqa: F401
