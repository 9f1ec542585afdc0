"""The C-ABI boundary without a GPU: the library loads, exports every symbol the header
declares, and the host-side argument decoding matches Knet's dispatch rules."""
import ctypes
import os

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB = os.path.join(ROOT, "knet.jl_b200", "libknet_sm100.so")


@pytest.fixture(scope="module")
def sigs():
    from knet_sm100 import abi
    return abi.parse_header()


@pytest.fixture(scope="module")
def lib():
    if not os.path.exists(LIB):
        import importlib.util
        spec = importlib.util.spec_from_file_location("knet_build", os.path.join(ROOT, "knet.jl_b200", "build.py"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        mod.build(verbose=False)
    return ctypes.CDLL(LIB)


def test_header_declares_the_libknet8_families(sigs):
    # names Knet's Julia side ccalls (src/libknet8/*.jl launchers, `_stream` forms)
    for name in ["relu_32_stream", "sigm_64_stream", "tanh_32_stream", "elu_32_stream",
                 "add_32_01_stream", "div_64_11_stream", "reluback_32_11_stream", "sigmback_64_11_stream",
                 "tanhback_32_11_stream", "eluback_32_11_stream", "mul_32_12_stream",
                 "add_32_13_x_y_stream", "add_64_13_y_x_stream", "sub_32_16_3_stream", "max_32_16_5_stream",
                 "sum_32_20_stream", "maximum_64_21_stream", "sumabs2_32_22_stream",
                 "dropout_32_stream", "dropback_64_stream", "getents_32_stream", "addents_64_stream",
                 "fill_32_stream", "relu_32_1_stream", "reluback_64_1_stream", "sigmback_32_111_stream",
                 "tanh_back_32_111_stream"]:
        assert name in sigs, name
        assert name.replace("_stream", "") in sigs
    assert len(sigs) > 800


def test_every_declared_symbol_is_exported(sigs, lib):
    missing = [n for n in sigs if not hasattr(lib, n)]
    assert missing == []


def test_argument_lists_match_libknet8(sigs):
    # (Cint,Ptr,Ptr) + stream: src/knetarrays/unary.jl:19-21
    assert sigs["relu_32_stream"] == [None, ["c_int", "c_void_p", "c_void_p", "c_void_p"]]
    # (Cint,T,Ptr,Ptr): src/knetarrays/binary.jl:33-37
    assert sigs["add_32_01_stream"][1] == ["c_int", "c_float", "c_void_p", "c_void_p", "c_void_p"]
    assert sigs["add_64_01_stream"][1][1] == "c_double"
    # (Cint,Ptr,Cint,Cint,Ptr,Cint,Cint,Ptr): binary.jl:69-72
    assert sigs["add_32_12_stream"][1] == ["c_int", "c_void_p", "c_int", "c_int", "c_void_p", "c_int", "c_int",
                                           "c_void_p", "c_void_p"]
    # (Ptr,Ptr,Ptr,Cint x5): binary.jl:78-81
    assert sigs["add_32_13_x_y_stream"][1] == ["c_void_p"] * 3 + ["c_int"] * 5 + ["c_void_p"]
    # value-returning scalar reduction: src/knetarrays/reduction.jl:31-33
    assert sigs["sum_32_20_stream"] == ["c_float", ["c_int", "c_void_p", "c_void_p"]]
    assert sigs["sum_64_20_stream"][0] == "c_double"
    # (Cint,Ptr,Cint,Cint,Ptr) and (Cint,Cint,Ptr,Cint,Cint,Cint,Ptr): reduction.jl:55,63-64
    assert sigs["sum_32_21_stream"][1] == ["c_int", "c_void_p", "c_int", "c_int", "c_void_p", "c_void_p"]
    assert sigs["sum_32_22_stream"][1] == ["c_int", "c_int", "c_void_p", "c_int", "c_int", "c_int", "c_void_p",
                                           "c_void_p"]
    # dropout (Cint,T,Ptr,Ptr), dropback (Cint,T,Ptr,Ptr,Ptr,Ptr): src/ops20_gpu/dropout.jl:14-21
    assert sigs["dropout_32_stream"][1] == ["c_int", "c_float", "c_void_p", "c_void_p", "c_void_p"]
    assert sigs["dropback_32_stream"][1] == ["c_int", "c_float"] + ["c_void_p"] * 5


def test_host_only_entry_points(lib):
    assert lib.knet_sm100_arch() == 100
    lib.knet_reduce_workspace_bytes.restype = ctypes.c_size_t
    assert lib.knet_reduce_workspace_bytes() >= 1024

    class Desc(ctypes.Structure):
        _fields_ = [("p", ctypes.c_void_p * 4), ("n", ctypes.c_int64), ("first_chunk", ctypes.c_int64)]

    t = (Desc * 4)()
    for i, n in enumerate([8192, 1, 0, 8193]):
        t[i].n = n
    lib.knet_multi_plan.restype = ctypes.c_int64
    total = lib.knet_multi_plan(ctypes.cast(t, ctypes.c_void_p), 4)
    assert total == 1 + 1 + 0 + 2
    assert [t[i].first_chunk for i in range(4)] == [0, 1, 2, 2]
    t[1].n = -5
    assert lib.knet_multi_plan(ctypes.cast(t, ctypes.c_void_p), 4) == -1


def test_argument_errors_are_status_codes_without_a_gpu(lib):
    """Bad arguments come back as negative status codes before anything is launched, so these
    calls are safe on a machine without a GPU."""
    import numpy as np
    i64, dbl, vp = ctypes.c_int64, ctypes.c_double, ctypes.c_void_p
    # data-parallel entry points: no communicator, bad ranks
    assert lib.knet_dp_allreduce_sum_32(None, None, i64(16), None) == -1
    assert lib.knet_dp_allgather_64(None, None, None, i64(4), None) == -1
    assert lib.knet_dp_init(None, 0, 2, 1000, None) == -1
    ident, handle = (ctypes.c_ubyte * 128)(), vp()
    assert lib.knet_dp_init(ident, 3, 2, 1000, ctypes.byref(handle)) == -1          # rank outside the world
    assert lib.knet_dp_init(ident, 0, 2, 0, ctypes.byref(handle)) == -1             # no deadline
    assert lib.knet_dp_rank(None) == -1 and lib.knet_dp_destroy(None) == -1
    # graph-friendly Adam needs its device scalars
    assert lib.knet_adam_multi_g_32(vp(8), 1, i64(1), dbl(1e-3), dbl(0.9), dbl(0.999), dbl(1e-8), None, dbl(1.0), None) == -1
    # Adam's bias corrections, computed on the host as the eager entry point computes them
    out = (ctypes.c_float * 2)()
    lib.knet_adam_bias_corr_32(dbl(0.9), dbl(0.999), 3, out)
    assert out[0] == np.float32(1 - 0.9 ** 3) and out[1] == np.float32(1 - 0.999 ** 3)
    outd = (ctypes.c_double * 2)()
    lib.knet_adam_bias_corr_64(dbl(0.9), dbl(0.999), 1, outd)
    assert outd[0] == 1 - 0.9 and outd[1] == 1 - 0.999
    # sizes and probabilities
    assert lib.knet_dropout_philox_32(i64(-1), ctypes.c_float(0.5), 1, 0, None, None, None) == -1
    assert lib.knet_dropout_philox_32(i64(8), ctypes.c_float(1.0), 1, 0, vp(16), vp(16), None) == -1
    assert lib.knet_bias_relu_dropout_fwd_g_32(vp(16), vp(16), vp(16), i64(4), i64(-2), ctypes.c_float(0.5), 1, 0, None, None) == -1
    assert lib.knet_softmax_fwd_32(None, None, i64(-1), i64(4), i64(4), None) == -1
    assert lib.knet_softmax_fwd_32(vp(16), vp(16), i64(0), i64(4), i64(4), None) == 0    # empty: nothing to do


def test_vbroadcast_shape_decoding():
    # the (s,n) pairs of src/knetarrays/binary.jl:152-212 for the shapes Knet's tests and the
    # benchmark configurations use
    from knet_sm100.ops import get_strides, vbroadcast_shape as vb
    dz, sx, nx, sy, ny, xlast, ylast, xdims, ydims, multi = vb((64, 100), (64,))
    assert (dz, sx, nx, sy, ny) == ((64, 100), 1, 6400, 1, 64)          # bias add
    assert vb((8192, 1), (8192, 128))[:5] == ((8192, 128), 1, 8192, 1, 8192 * 128)
    assert vb((1, 4096), (64, 4096))[:5] == ((64, 4096), 64, 4096, 1, 64 * 4096)
    assert vb((513, 1025), (1, 1025))[:5] == ((513, 1025), 1, 513 * 1025, 513, 1025)
    assert vb((5,), (1,))[:5] == ((5,), 1, 5, 5, 1)                     # scalar-like operand
    assert vb((3, 1), (1, 4))[:5] == ((3, 4), 1, 3, 3, 4)               # two vectors
    assert vb((8, 8, 16, 4), (8, 8, 1, 4))[9] is True                   # needs the strided kernel
    with pytest.raises(ValueError):
        vb((3, 4), (5, 4))
    sx, sy, sz = get_strides((8, 8, 16, 4), (8, 8, 1, 4), (8, 8, 16, 4))
    assert sx == [1, 8, 64, 1024] and sy == [1, 8, 0, 64] and sz == [1, 8, 64, 1024]


def test_shard_ranges_cover_the_batch():
    from knet_sm100.dp import bucket_bounds, shard_range
    for n, world in ((8192, 8), (100, 3), (7, 8)):
        spans = [shard_range(n, r, world) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == n
        assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
        assert max(b - a for a, b in spans) - min(b - a for a, b in spans) <= 1
    assert bucket_bounds(np.array([0, 10, 25, 31])) == [(25, 31), (10, 25), (0, 10)]
