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
    for name, kw in (("allreduce", {}), ("sharded", {"shard_update": True})):
        m = K.MLP(SIZES, BATCH, pdrop=0.0, seed=1, optimizer=K.Adam(lr=1e-2), process_group=dist.group.WORLD, **kw)
        losses = []
        for _ in range(STEPS):
            tot, cnt = m.step(xs, ys)
            losses.append(K.dp.reduce_loss(tot, cnt))
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
    if rank == 0:
        report["ok"] = bool(ok)
        print(json.dumps(report), flush=True)
    flag = torch.tensor([1.0 if ok else 0.0], device="cuda")
    dist.broadcast(flag, 0)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if flag.item() == 1.0 else 1)


if __name__ == "__main__":
    main()
