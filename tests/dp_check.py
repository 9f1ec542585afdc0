"""Run under torchrun on N >= 2 GPUs: the data-parallel MLP step with all-reduce and with the
sharded update (reduce-scatter -> own shard -> all-gather) against a single-GPU run of the
whole batch on rank 0.  Prints one JSON line on rank 0 and exits non-zero on a mismatch.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        --master-port 29533 tests/dp_check.py
"""
import json
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "knet.jl_b200"))

SIZES, BATCH, STEPS = [96, 130, 64, 10], 64, 4        # 130: buckets that need padding


def weights_of(m):
    m.sync_weights()
    return [np.concatenate([w.numpy().reshape(-1, order="F"), b.numpy()]) for w, b in zip(m.w, m.b)]


def main():
    import knet_sm100 as K
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl")
    rng = np.random.default_rng(3)
    x = np.asfortranarray(rng.standard_normal((SIZES[0], BATCH * world)).astype(np.float32))
    y = rng.integers(1, SIZES[-1] + 1, BATCH * world).astype(np.int32)
    lo, hi = K.dp.shard_range(BATCH * world, rank, world)
    xs, ys = K.KnetArray(np.asfortranarray(x[:, lo:hi])), torch.from_numpy(y[lo:hi]).cuda()
    runs = {}
    comm = K.dp.KnetComm(rank, world, timeout_ms=60000)          # the library's own communicator
    groups = {"allreduce": dist.group.WORLD, "sharded": dist.group.WORLD, "knet_allreduce": comm, "knet_sharded": comm}
    for name, kw in (("allreduce", {}), ("sharded", {"shard_update": True}), ("knet_allreduce", {}),
                     ("knet_sharded", {"shard_update": True})):
        m = K.MLP(SIZES, BATCH, pdrop=0.0, seed=1, optimizer=K.Adam(lr=1e-2), process_group=groups[name], **kw)
        losses = []
        for _ in range(STEPS):
            tot, cnt = m.step(xs, ys)
            losses.append(K.dp.reduce_loss(tot, cnt, groups[name]))
        runs[name] = (weights_of(m), [t / c for t, c in losses])
        if name == "sharded":
            state_elems = sum(s.numel() for s in m.state)
    ok, report = True, {"world": world}
    if rank == 0:
        ref = K.MLP(SIZES, BATCH * world, pdrop=0.0, seed=1, optimizer=K.Adam(lr=1e-2))
        xa, ya = K.KnetArray(x), torch.from_numpy(y).cuda()
        ref_losses = []
        for _ in range(STEPS):
            tot, cnt = ref.step(xa, ya)
            ref_losses.append(float(tot) / int(cnt))
        ref_w = weights_of(ref)
        for name, (w, losses) in runs.items():
            dw = max(float(np.max(np.abs(a - b))) for a, b in zip(w, ref_w))
            dl = float(np.max(np.abs(np.array(losses) - np.array(ref_losses))))
            report[name] = {"max_weight_diff": dw, "max_loss_diff": dl}
            ok &= dw <= 5e-5 and dl <= 1e-4          # summation order differs between the three
        dws = max(float(np.max(np.abs(a - b))) for a, b in zip(runs["allreduce"][0], runs["sharded"][0]))
        report["allreduce_vs_sharded_max_weight_diff"] = dws
        report["sharded_state_elems_per_rank"] = state_elems
        report["replicated_state_elems_per_rank"] = 2 * sum(w.size for w in ref_w)
        ok &= dws <= 5e-5
    # every rank must hold the same weights after either scheme
    for name, (w, _) in runs.items():
        flat = torch.from_numpy(np.concatenate(w)).cuda()
        top = flat.clone()
        dist.broadcast(top, 0)
        same = torch.tensor([float(torch.equal(flat, top))], device="cuda")
        dist.all_reduce(same, op=dist.ReduceOp.MIN)
        if rank == 0:
            report[name]["replicas_identical"] = bool(same.item())
            ok &= bool(same.item())
    # raw collectives of the library's communicator against torch.distributed's on the same data
    g = torch.Generator(device="cpu").manual_seed(50 + rank)
    for dt in (torch.float32, torch.float64):
        n = 4096 * world
        a = torch.randint(-64, 64, (n,), generator=g).to(dt).cuda()          # integer-valued: exact sums
        b, c = a.clone(), a.clone()
        comm.all_reduce(b)
        dist.all_reduce(c)
        same = torch.equal(b, c)
        shard, shard_ref = torch.empty(n // world, dtype=dt, device="cuda"), torch.empty(n // world, dtype=dt, device="cuda")
        comm.reduce_scatter(shard, a)
        dist.reduce_scatter_tensor(shard_ref, a)
        same &= torch.equal(shard, shard_ref) and torch.equal(shard, c[rank * (n // world):(rank + 1) * (n // world)])
        full = torch.empty(n, dtype=dt, device="cuda")
        comm.all_gather(full, shard)
        same &= torch.equal(full, c)
        bc = a.clone()
        comm.broadcast(bc, root=world - 1)
        ref = a.clone()
        dist.broadcast(ref, world - 1)
        same &= torch.equal(bc, ref)
        flag = torch.tensor([float(same)], device="cuda")
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if rank == 0:
            report[f"knet_collectives_{str(dt).split('.')[-1]}_match_torch"] = bool(flag.item())
            ok &= bool(flag.item())
    comm.destroy()
    if rank == 0:
        report["ok"] = bool(ok)
        print(json.dumps(report), flush=True)
    flag = torch.tensor([1.0 if ok else 0.0], device="cuda")
    dist.broadcast(flag, 0)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if flag.item() == 1.0 else 1)


def timeout_check():
    """A peer that never joins: rank 0 asks for a 2-rank communicator that rank 1 never enters and
    must get the timeout status after the deadline, with its CUDA context still usable."""
    import ctypes as C
    import time
    import knet_sm100 as K
    rank = int(os.environ["RANK"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("gloo")
    out = {}
    if rank == 0:
        ident, handle = (C.c_ubyte * 128)(), C.c_void_p()
        K.lib.check(K.libknet.knet_dp_unique_id(ident), "knet_dp_unique_id")
        t0 = time.perf_counter()
        rc = K.libknet.knet_dp_init(ident, 0, 2, 2000, C.byref(handle))
        out = {"status": rc, "seconds": time.perf_counter() - t0,
               "context_alive": bool(torch.ones(4, device="cuda").sum().item() == 4.0)}
        out["ok"] = rc == -6 and out["context_alive"] and out["seconds"] < 30
        print(json.dumps(out), flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if (rank != 0 or out["ok"]) else 1)


if __name__ == "__main__":
    timeout_check() if "--timeout-check" in sys.argv else main()
