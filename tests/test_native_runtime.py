import json

import numpy as np
import pytest

from nexus_b200 import _native as N


def test_host_caching_allocator():
    a = N.HostCachingAllocator()
    assert N.HostCachingAllocator.size_class(1) == 64 and N.HostCachingAllocator.size_class(65) == 128
    p = a.allocate(100)
    assert p % 64 == 0
    a.deallocate(p)
    q = a.allocate(120)                       # same size class: served from the cache
    s = a.stats()
    assert q == p and s["hits"] == 1 and s["system_allocs"] == 1 and 0 < s["fragmentation"] < 0.1
    a.deallocate(q)
    a.release_cached()
    assert a.stats()["reserved_bytes"] == 0
    with pytest.raises(ValueError):
        a.deallocate(12345)


def test_memory_planner_reuses_dead_tensors():
    lifetimes = [(1000, 0, 1), (2000, 1, 2), (1000, 2, 3), (500, 0, 3)]
    offs, arena = N.plan_memory(lifetimes, 64)
    assert arena < sum(b for b, _, _ in lifetimes)
    for i, (bi, fi, li) in enumerate(lifetimes):
        for j, (bj, fj, lj) in enumerate(lifetimes):
            if i < j and not (li < fj or lj < fi):
                assert offs[i] + bi <= offs[j] or offs[j] + bj <= offs[i]


def test_profiler_counters_trace_and_ledger(tmp_path):
    N.prof_clear()
    N.prof_enable(True)
    t = N.prof_now_ns()
    N.prof_record("gemm", "kernel", t, 1500)
    N.prof_record("gemm", "kernel", t + 2000, 500)
    N.prof_count("gemm", 2e9, 1e6)
    tot = N.prof_totals()["gemm"]
    assert tot["calls"] == 2 and tot["total_ns"] == 2000 and tot["min_ns"] == 500 and tot["max_ns"] == 1500
    assert N.prof_counters()["gemm"]["flops"] == 2e9
    p = str(tmp_path / "trace.json")
    assert N.prof_dump_chrome_trace(p) == 2
    ev = json.load(open(p))["traceEvents"]
    assert ev[0]["ph"] == "X" and ev[0]["name"] == "gemm"
    N.prof_enable(False)
    N.prof_record("x", "y", 0, 1)
    assert "x" not in N.prof_totals()
    N.ledger_reset()
    N.ledger_add(0, 2, 100)
    N.ledger_add(0, 2, -40)
    assert N.ledger_current(0, 2) == 60 and N.ledger_peak(0, 2) == 100
    with pytest.raises(IndexError):
        N.ledger_add(9, 0, 1)


def test_native_environments():
    e = N.NativeEnv("LineWorld", 5, 12)
    assert e.reset(0).tolist() == [1, 0, 0, 0, 0]
    total, done = 0.0, False
    while not done:
        o, r, term, trunc = e.step(np.array([1.0], np.float32))
        total += r
        done = term or trunc
    assert total == pytest.approx(4 * 0.1 + 1.0) and o[-1] == 1
    g = N.NativeEnv("GridWorld", 3, 24)
    g.reset(0)
    for a in (0, 0, 2, 2):
        o, r, term, _ = g.step(np.array([a], np.float32))
    assert term and r == 1.0
    pm = N.NativeEnv("PointMass")
    pm.reset(0)
    o, r, _, _ = pm.step(np.array([-1.0], np.float32))
    assert o[0] == pytest.approx(0.5) and r == pytest.approx(-0.25)
    with pytest.raises(ValueError):
        e.step(np.array([7.0], np.float32))
    v = N.NativeVectorEnv("CartPole", 16, workers=4, seed=3)
    obs = v.reset()
    assert obs.shape == (16, 4)
    for _ in range(50):
        obs, rew, term, trunc = v.step(np.ones((16, 1), np.float32))
    assert v.total_steps == 800 and rew.tolist() == [1.0] * 16 and np.isfinite(obs).all()
