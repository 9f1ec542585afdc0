"""Host-side logic of bench.py that needs no GPU: the `config` object shared by the two arms, the
step budget of the CPU reference arm, and the per-launch summary of `kernels_step`."""
import importlib.util
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
bench = importlib.util.module_from_spec(spec)
spec.loader.exec_module(bench)


def test_both_arms_describe_the_same_workload():
    for world in (1, 2, 8):
        c = bench.workload_config(world)
        assert c["global_batch"] == 8192 * world and c["parallelism"] == f"dp{world}"
        assert "per-GPU batch 8192" in c["workload"] and c["params"] == 243106792
    assert bench.workload_config(4, sharded=True)["parallelism"] == "dp4+sharded-update"
    assert bench.NPARAMS == 4096 * 8192 + 3 * 8192 * 8192 + 8192 * 1000 + 4 * 8192 + 1000


def test_reference_arm_keeps_full_steps_within_its_budget():
    fit = bench.fit_steps
    assert fit(20, 5, 240.0, 16.0, 6.0) == (5, 20)          # 24 more steps of 6 s fit into 224 s
    assert fit(20, 5, 120.0, 16.0, 6.0) == (1, 17)          # warm-up steps go first, then timed steps
    assert fit(20, 5, 240.0, 40.0, 30.0) == (1, 6)
    assert fit(3, 1, 10.0, 40.0, 30.0) == (1, 1)            # never fewer than one timed full step
    assert fit(2, 3, 240.0, 10.0, 50.0) == (3, 2)
    w, s = fit(10, 4, 100.0, 10.0, 9.0)                     # 10 steps fit: all timed steps, no extra warm-up
    assert (w - 1) + s <= 10 and s == 10 and w == 1


def test_launch_probe_summary():
    class Ev:
        def __init__(self, t): self.t = t
        def record(self): pass
        def elapsed_time(self, other): return other.t - self.t

    p = bench.LaunchProbe.__new__(bench.LaunchProbe)
    p.recs = [("a", 1000, Ev(0.0), Ev(0.5)), ("a", 1000, Ev(1.0), Ev(1.5)), ("b", 4000, Ev(2.0), Ev(3.0))]
    out = p.summary(steps=2, peak=6452.2, step_ms=10.0)
    assert out["probed_steps"] == 2 and abs(out["ms_per_step"] - 1.0) < 1e-12
    assert out["algorithmic_bytes_per_step"] == 3000
    assert out["per_kernel"]["a"]["launches"] == 1.0 and out["per_kernel"]["b"]["launches"] == 0.5
    assert abs(out["share_of_step"] - 0.1) < 1e-12
    assert abs(out["gbs"] - 6000 / 2e-3 / 1e9) < 1e-9
