"""The data-parallel step rules on two CPU ranks over gloo: batch sharding, per-layer gradient
buckets summed with all-reduce, the 1/world scale, identical updates on every rank.  The
compute is the CPU checker's MLP; the rules under test are knet_sm100.dp's."""
import os
import socket
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SIZES = [20, 16, 12, 5]
BATCH, STEPS = 24, 3


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _data():
    rng = np.random.default_rng(11)
    x = np.asfortranarray(rng.standard_normal((SIZES[0], BATCH)).astype(np.float32))
    y = rng.integers(1, SIZES[-1] + 1, BATCH)
    return x, y


def _flatten(grads):
    return np.concatenate([np.asarray(g).reshape(-1, order="F") for g in grads])


def _worker(rank, world, port, out):
    for p in (os.path.join(ROOT, "knet.jl_b200"), os.path.join(ROOT, "oracle")):
        sys.path.insert(0, p)
    import knet_oracle as ko
    from knet_sm100 import dp
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    x, y = _data()
    model = ko.MLP(SIZES, np.random.default_rng(1), lr=1e-2)       # same weights on every rank
    lo, hi = dp.shard_range(BATCH, rank, world)
    sizes = [p.size for p in model.params()]
    offsets = np.concatenate([[0], np.cumsum(sizes)])[::2]          # one bucket per (W,b) pair
    losses = []
    for _ in range(STEPS):
        loss, grads = model.loss_and_grads(x[:, lo:hi], y[lo:hi])
        flat = torch.from_numpy(_flatten(grads))
        works = [dp.allreduce_bucket(flat, b) for b in dp.bucket_bounds(offsets)]
        for w in works:
            w.wait()
        flat *= dp.gradient_scale(world)
        g, o = [], 0
        for p in model.params():
            g.append(np.asfortranarray(flat.numpy()[o:o + p.size].reshape(p.shape, order="F")))
            o += p.size
        model.update(g)
        tot, cnt = dp.reduce_loss(torch.tensor(float(loss) * (hi - lo)), torch.tensor(hi - lo))
        losses.append(tot / cnt)
    out[rank] = (np.concatenate([p.reshape(-1, order="F") for p in model.params()]), losses)
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_step_equals_single_process_step():
    world = 2
    port = _free_port()
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, port, out), nprocs=world, join=True)
    for p in (os.path.join(ROOT, "oracle"),):
        if p not in sys.path:
            sys.path.insert(0, p)
    import knet_oracle as ko
    x, y = _data()
    ref = ko.MLP(SIZES, np.random.default_rng(1), lr=1e-2)
    ref_losses = [float(ref.step(x, y)) for _ in range(STEPS)]
    ref_w = np.concatenate([p.reshape(-1, order="F") for p in ref.params()])
    w0, l0 = out[0]
    w1, l1 = out[1]
    np.testing.assert_array_equal(w0, w1)                           # replicas stay identical
    np.testing.assert_allclose(w0, ref_w, rtol=0, atol=2e-5)        # summation order differs
    np.testing.assert_allclose(l0, ref_losses, rtol=1e-5)
    np.testing.assert_allclose(l0, l1, rtol=0, atol=0)


# ---- sharded update: reduce-scatter -> own shard -> all-gather ------------------------------------
def _sharded_worker(rank, world, port, out):
    for p in (os.path.join(ROOT, "knet.jl_b200"), os.path.join(ROOT, "oracle")):
        sys.path.insert(0, p)
    from knet_sm100 import dp
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    counts = [37, 8, 101]
    offs = dp.padded_offsets(counts, world)
    rng = np.random.default_rng(100 + rank)
    g = torch.from_numpy(rng.integers(-8, 8, offs[-1]).astype(np.float32))     # integer-valued: exact sums
    w = torch.zeros(offs[-1])
    g_all = sum(np.random.default_rng(100 + r).integers(-8, 8, offs[-1]).astype(np.float32) for r in range(world))
    for i in range(len(counts)):
        b = (offs[i], offs[i + 1])
        wk = dp.reduce_scatter_bucket(g, b, rank, world)
        if wk is not None:
            wk.wait()
        lo, hi = dp.shard_bounds(b, rank, world)
        assert lo % 4 == 0 and (hi - lo) * world == b[1] - b[0]
        np.testing.assert_array_equal(g[lo:hi].numpy(), g_all[lo:hi])
        w[lo:hi] = -0.5 * g[lo:hi]                                              # the "update" of the own shard
        wk = dp.allgather_bucket(w, b, rank, world)
        if wk is not None:
            wk.wait()
    out[rank] = w.numpy().copy()
    np.testing.assert_array_equal(out[rank], -0.5 * g_all)
    dist.barrier()
    dist.destroy_process_group()


def test_sharded_update_helpers_on_two_ranks():
    world = 2
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_sharded_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    np.testing.assert_array_equal(out[0], out[1])


def test_padded_offsets_and_shards():
    sys.path.insert(0, os.path.join(ROOT, "knet.jl_b200"))
    # dp has no device code; importing it through the package would need the built library
    import importlib.util
    spec = importlib.util.spec_from_file_location("dp_only", os.path.join(ROOT, "knet.jl_b200", "knet_sm100", "dp.py"))
    dp = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(dp)
    offs = dp.padded_offsets([1, 31, 32, 33], 8)
    assert offs == [0, 32, 64, 96, 160]
    assert dp.shard_bounds((32, 64), 3, 8) == (44, 48)
    covered = [dp.shard_bounds((96, 160), r, 8) for r in range(8)]
    assert covered[0][0] == 96 and covered[-1][1] == 160 and all(covered[r][1] == covered[r + 1][0] for r in range(7))
    import pytest
    with pytest.raises(ValueError):
        dp.shard_bounds((0, 10), 0, 4)
