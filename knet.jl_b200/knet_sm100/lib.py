"""Loader of libknet_sm100.so and the `@knet8`-style call helper.

Mirrors src/libknet8/LibKnet8.jl:50-62: `knet8(fun, *args)` appends `_stream` to the symbol
name and the current CUDA stream to the arguments; `knet8r` is the value-returning form.
There is no fallback: if the shared library is missing the import of this module fails.
"""
import ctypes as C
import os

import torch

from . import abi

LIBPATH = os.environ.get("KNET_SM100_LIB", os.path.join(abi.ROOT, "libknet_sm100.so"))

if not os.path.exists(LIBPATH):
    raise ImportError(
        f"{LIBPATH} not found: build it with `python knet.jl_b200/build.py` "
        "(there is no CPU or PyTorch fallback for these kernels)")

libknet = abi.bind(C.CDLL(LIBPATH))


class KnetError(RuntimeError):
    pass


_ERR = {-1: "invalid argument", -2: "size not supported", -3: "workspace missing or too small",
        -4: "pointer not aligned to its element size", -5: "NCCL could not be loaded",
        -6: "timed out waiting for the other ranks (communicator aborted)",
        -7: "cuBLAS could not be loaded", -8: "the loaded cuBLAS does not offer the requested mode"}


def check(rc, name):
    if rc != 0:
        msg = _ERR.get(rc, (f"cuBLAS status {rc - 2000}" if rc >= 2000 else f"NCCL error {rc - 1000}" if rc >= 1000 else f"CUDA error {rc}") if rc > 0 else "unknown error")
        raise KnetError(f"{name}: {msg} (status {rc})")


def stream_ptr():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def ptr(t):
    """Device pointer of a tensor (or None)."""
    return None if t is None else C.c_void_p(t.data_ptr())


def knet8(fun, *args):
    """Call the void entry point `fun`_stream on the current stream."""
    getattr(libknet, fun + "_stream")(*args, stream_ptr())


def knet8r(fun, *args):
    """Call the value-returning entry point `fun`_stream (it synchronises the stream)."""
    return getattr(libknet, fun + "_stream")(*args, stream_ptr())


def knet(fun, *args):
    """Call an int-status entry point (stream is its last argument) and raise on error."""
    check(getattr(libknet, fun)(*args, stream_ptr()), fun)


def sfx(dtype):
    if dtype == torch.float32:
        return "32"
    if dtype == torch.float64:
        return "64"
    raise TypeError(f"libknet_sm100 kernels exist for Float32 and Float64, not {dtype}")
