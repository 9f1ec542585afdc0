"""The MLP training step (forward, backward, update!) against the oracle's MLP.

Loss curves must agree within 1e-4 (absolute) over 100 steps: the matrix products are cuBLAS
on one side and BLAS on the other, every other operation follows the same order."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def host_weights(ko, sizes, seed):
    rng = np.random.default_rng(seed)
    ws = [ko.xavier_uniform(sizes[i + 1], sizes[i], rng) for i in range(len(sizes) - 1)]
    return [(w, np.zeros(w.shape[0], np.float32)) for w in ws]


def oracle_model(ko, sizes, weights, **kw):
    m = ko.MLP(sizes, np.random.default_rng(0), **kw)
    m.w = [np.asfortranarray(w.copy()) for w, _ in weights]
    m.b = [b.copy() for _, b in weights]
    return m


def test_mnist_shaped_mlp_loss_curve_100_steps(K, ko):
    # 784-64-10, batch 100, x ~ U[0,1), labels 1..10, Adam(1e-3, 0.9, 0.999, 1e-8), seed 1
    sizes, B = [784, 64, 10], 100
    weights = host_weights(ko, sizes, 1)
    rng = np.random.default_rng(1)
    ref = oracle_model(ko, sizes, weights, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8)
    gpu = K.MLP(sizes, B, weights=weights, optimizer=K.Adam(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8))
    worst = 0.0
    x = rng.random((784, B)).astype(np.float32)                 # one batch, as the configuration says
    y = rng.integers(1, 11, B)
    for step in range(100):
        l_ref = float(ref.step(x, y))
        tot, cnt = gpu.step(K.KnetArray(x), torch.from_numpy(y.astype(np.int32)).cuda())
        l_gpu = float(tot.item()) / int(cnt.item())
        worst = max(worst, abs(l_gpu - l_ref))
        assert abs(l_gpu - l_ref) <= 1e-4, (step, l_gpu, l_ref)
    assert l_ref < 2.0 and worst <= 1e-4
    # Adam's step is lr*m/sqrt(v): where a gradient is near zero, gemm rounding decides its
    # sign, so single weights may drift by a few lr; the bulk must agree closely
    for (w, b), kw_, kb in zip(zip(ref.w, ref.b), gpu.w, gpu.b):
        for got, want in ((kw_.numpy(), w), (kb.numpy(), b)):
            assert np.abs(got - want).mean() <= 2e-4 and np.abs(got - want).max() <= 5e-3
    assert gpu.launches > 0


@pytest.mark.parametrize("optname", ["adam", "momentum", "sgd"])
def test_mlp_with_dropout_on_supplied_uniforms(K, ko, optname):
    sizes, B, p = [32, 24, 16, 5], 40, 0.5
    weights = host_weights(ko, sizes, 2)
    hyper = {"adam": dict(lr=1e-2), "momentum": dict(lr=0.05, gamma=0.9), "sgd": dict(lr=0.1)}[optname]
    opt = {"adam": K.Adam, "momentum": K.Momentum, "sgd": K.SGD}[optname](**hyper)
    ref = oracle_model(ko, sizes, weights, pdrop=p, optimizer=optname, **hyper)
    gpu = K.MLP(sizes, B, pdrop=p, weights=weights, optimizer=opt)
    rng = np.random.default_rng(3)
    x = rng.standard_normal((32, B)).astype(np.float32)
    y = rng.integers(1, 6, B)
    yd = torch.from_numpy(y.astype(np.int32)).cuda()
    for step in range(20):
        us = [np.asfortranarray(rng.random((sizes[i + 1], B)).astype(np.float32)) for i in range(2)]
        l_ref = float(ref.step(x, y, us))
        tot, cnt = gpu.step(K.KnetArray(x), yd, [K.KnetArray(u) for u in us])
        assert abs(float(tot.item()) / int(cnt.item()) - l_ref) <= 1e-4, step


def test_bias_gradient_fused_into_the_backward_kernel_matches_the_separate_sum(K, ko):
    sizes, B = [48, 256, 128, 10], 96
    weights = host_weights(ko, sizes, 5)
    rng = np.random.default_rng(6)
    x = K.KnetArray(rng.standard_normal((48, B)).astype(np.float32))
    y = torch.from_numpy(rng.integers(1, 11, B).astype(np.int32)).cuda()
    a = K.MLP(sizes, B, pdrop=0.5, weights=weights, optimizer=K.Adam(lr=1e-3), dropout_seed=3, fuse_bias_grad=True)
    b = K.MLP(sizes, B, pdrop=0.5, weights=weights, optimizer=K.Adam(lr=1e-3), dropout_seed=3, fuse_bias_grad=False)
    for step in range(5):
        ta, ca = a.step(x, y)
        tb, cb = b.step(x, y)
        assert abs(float(ta) - float(tb)) <= 1e-5 * abs(float(tb))
        for i in range(3):
            ga, gb = a.db[i].numpy(), b.db[i].numpy()
            assert np.abs(ga - gb).max() <= 1e-5 * max(np.abs(gb).max(), 1e-6)
    assert a.launches == b.launches - 5 * 2          # two launches fewer per step


def test_sharded_update_rejects_gradient_clipping(K):
    class FakeGroup(K.dp.KnetComm):
        def __init__(self):
            self.rank, self.world = 0, 2
    with pytest.raises(ValueError, match="clipping"):
        K.MLP([8, 8, 4], 4, optimizer=K.Adam(gclip=1.0), process_group=FakeGroup(), shard_update=True)


def test_resume_from_saved_state_is_bitwise(K, ko):
    # parameters, both Adam moments, the step count and the dropout counter are the whole
    # training state: 50 + 50 steps after a save/load equal 100 steps in one go
    sizes, B = [64, 48, 10], 32
    weights = host_weights(ko, sizes, 5)
    rng = np.random.default_rng(6)
    xs = [K.KnetArray(rng.standard_normal((64, B)).astype(np.float32)) for _ in range(4)]
    ys = [torch.from_numpy(rng.integers(1, 11, B).astype(np.int32)).cuda() for _ in range(4)]

    def run(model, lo, hi):
        for s in range(lo, hi):
            model.step(xs[s % 4], ys[s % 4])

    a = K.MLP(sizes, B, pdrop=0.5, weights=weights, seed=9)
    run(a, 0, 100)
    b = K.MLP(sizes, B, pdrop=0.5, weights=weights, seed=9)
    run(b, 0, 50)
    saved = dict(w=b.flat_w.cpu().numpy().copy(), m=b.state[0].cpu().numpy().copy(),
                 v=b.state[1].cpu().numpy().copy(), t=b.opt.t, step_no=b.step_no)
    c = K.MLP(sizes, B, pdrop=0.5, weights=weights, seed=9)
    c.flat_w.copy_(torch.from_numpy(saved["w"]))
    c.state[0].copy_(torch.from_numpy(saved["m"]))
    c.state[1].copy_(torch.from_numpy(saved["v"]))
    c.opt.t, c.step_no = saved["t"], saved["step_no"]
    run(c, 50, 100)
    assert torch.equal(a.flat_w, c.flat_w) and torch.equal(a.state[1], c.state[1])


def test_data_parallel_schemes_agree_on_two_gpus(K):
    """All-reduce and sharded-update steps on 2 GPUs against the single-GPU step of the whole
    batch (tests/dp_check.py under torchrun); needs two devices."""
    import json
    import os
    import subprocess
    import sys
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", "29533", os.path.join(root, "tests", "dp_check.py")],
                       capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    rep = json.loads([l for l in r.stdout.splitlines() if l.startswith("{")][-1])
    assert rep["ok"] and rep["sharded_state_elems_per_rank"] * 2 <= rep["replicated_state_elems_per_rank"] + 64


def test_communicator_times_out_when_a_rank_never_joins(K):
    """Failure made on the host: rank 1 never enters the communicator; rank 0 must get the
    timeout status after its deadline and keep a working CUDA context."""
    import json
    import os
    import subprocess
    import sys
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", "29534", os.path.join(root, "tests", "dp_check.py"),
                        "--timeout-check"], capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    rep = json.loads([l for l in r.stdout.splitlines() if l.startswith("{")][-1])
    assert rep["status"] == -6 and rep["context_alive"]


@pytest.mark.parametrize("sizes,batch,pdrop", [([784, 64, 10], 100, 0.0), ([96, 128, 64, 10], 64, 0.5)])
def test_captured_graph_step_is_bitwise_the_eager_step(K, sizes, batch, pdrop):
    """The whole step replayed as one CUDA graph (dropout offsets and Adam's bias corrections
    refreshed through device memory) against the eager step: same weights, state and losses."""
    rng = np.random.default_rng(4)
    xs = [np.asfortranarray(rng.random((sizes[0], batch)).astype(np.float32)) for _ in range(3)]
    ys = [rng.integers(1, sizes[-1] + 1, batch).astype(np.int32) for _ in range(3)]
    eager = K.MLP(sizes, batch, pdrop=pdrop, seed=1, optimizer=K.Adam(lr=1e-3))
    graph = K.MLP(sizes, batch, pdrop=pdrop, seed=1, optimizer=K.Adam(lr=1e-3)).capture()
    assert torch.equal(eager.flat_w, graph.flat_w)                   # capture leaves the model untouched
    for step in range(12):
        x, y = K.KnetArray(xs[step % 3]), torch.from_numpy(ys[step % 3]).cuda()
        te, _ = eager.step(x, y)
        tg, _ = graph.step_graph(x, y) if step != 5 else graph.step(x, y)      # an eager step in between is fine
        assert torch.equal(te, tg), step
        assert torch.equal(eager.flat_w, graph.flat_w), step
        for a, b in zip(eager.state, graph.state):
            assert torch.equal(a, b), step
    assert graph.opt.t == eager.opt.t == 12
