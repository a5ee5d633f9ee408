import json

import numpy as np
import pytest
import torch

from nexus_b200 import cpu, memory, prof
from nexus_b200.data.loader import GpuTokenLoader
from nexus_b200.train.lm_trainer import SyntheticTokens


def test_device_caching_allocator_host_backing():
    a = memory.DeviceCachingAllocator("host", 64 << 20)
    p1 = a.alloc(1000, 1)
    p2 = a.alloc(300 << 10, 1)
    s = a.stats()
    assert p1 % 512 == 0 and s["segments"] == 1 and s["reserved_bytes"] == 2 << 20 and s["allocated_bytes"] == 1024 + (300 << 10)
    a.free(p1)
    assert a.alloc(900, 1) == p1 and a.stats()["cache_hits"] >= 1        # same stream: reuse
    q = a.alloc(900, 2)                                                  # another stream: own segment
    assert q != p1 and a.stats()["segments"] == 2
    big = a.alloc(30 << 20, 1)
    assert a.stats()["reserved_bytes"] >= (30 << 20) + (4 << 20)
    a.record_stream(big, 7)
    a.free(big)
    a.free(p2)
    a.free(q)
    before = a.stats()
    assert before["merges"] >= 1 and before["live_blocks"] == 1
    with pytest.raises(ValueError):
        a.free(12345)
    # out of memory -> cache emptied -> retry succeeds
    for _ in range(2):
        x = a.alloc(28 << 20, 3)
        a.free(x)
    y = a.alloc(40 << 20, 4)
    st = a.stats()
    assert st["oom_retries"] >= 1 and st["allocated_bytes"] >= 40 << 20
    with pytest.raises(RuntimeError, match="out of device memory"):
        a.alloc(100 << 20, 4)
    a.free(y)
    a.empty_cache()
    assert a.stats()["fragmentation"] >= 0.0


@pytest.mark.gpu
def test_device_caching_allocator_cuda_backing():
    a = memory.DeviceCachingAllocator("cuda")
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    p = a.alloc(8 << 20, s1.cuda_stream)
    a.record_stream(p, s2.cuda_stream)
    a.free(p)
    assert a.stats()["deferred_frees"] == 1
    torch.cuda.synchronize()
    q = a.alloc(8 << 20, s1.cuda_stream)        # deferred free completed: block is reusable
    assert q == p
    a.free(q)
    a.empty_cache()
    assert a.stats()["reserved_bytes"] == 0


def test_planner_recorder_and_cast_cache():
    r = memory.LifetimeRecorder()
    r.define("a", 1000)
    r.tick()
    r.define("b", 2000)
    r.use("a")
    r.tick()
    r.define("c", 1000)      # a is dead: c may reuse its space
    r.use("b")
    off, arena = r.plan(256)
    assert arena <= 1024 + 2048 and set(off) == {"a", "b", "c"}
    assert off["a"] == off["c"] or arena < 1024 * 2 + 2048
    p = torch.nn.Parameter(torch.randn(8, 8))
    cc = memory.CastCache()
    t1 = cc.get(p)
    assert cc.get(p) is t1 and cc.hits == 1 and t1.dtype == torch.bfloat16
    with torch.no_grad():
        p.add_(1.0)
    t2 = cc.get(p)
    assert cc.misses == 2 and torch.equal(t2, p.detach().bfloat16())
    h = memory.HostCachingAllocator()
    assert h.size_class(100) == 128


def test_profiler_counters_trace_and_ledger(tmp_path):
    prof.clear()
    prof.enable(True)
    with prof.ScopedTimer("step", "train"):
        with prof.ScopedTimer("inner"):
            sum(range(1000))

    @prof.ScopedTimer("decorated")
    def f():
        return 3
    assert f() == 3
    prof.count("gemm", 2e9, 1e6)
    prof.count("gemm", 2e9, 1e6)
    tot, cnt = prof.totals(), prof.counters()
    assert {"step", "inner", "decorated"} <= set(tot) and cnt["gemm"]["calls"] == 2 and cnt["gemm"]["flops"] == 4e9
    n = prof.dump_chrome_trace(str(tmp_path / "t.json"))
    ev = json.load(open(tmp_path / "t.json"))
    events = ev["traceEvents"] if isinstance(ev, dict) else ev
    assert n == 3 and len(events) >= 3 and {e["name"] for e in events} >= {"step", "inner"}
    prof.enable(False)
    L = prof.MemoryLedger
    L.reset()
    with L.track(prof.Label.Activation, prof.Space.Device, 4096):
        assert L.current(prof.Label.Activation, prof.Space.Device) == 4096
    assert L.current(prof.Label.Activation, prof.Space.Device) == 0 and L.peak(prof.Label.Activation, prof.Space.Device) == 4096
    assert L.report()["KvCache"]["Host"]["peak"] == 0


def test_cpu_features_pool_and_quantised_gemm():
    f = cpu.features()
    assert f["logical_cores"] >= 1 and f["physical_cores"] >= 1 and isinstance(f["avx2"], bool) and f["numa_nodes"] >= 1
    p = cpu.ThreadPool(3)
    parts = p.partition(10)
    assert [(b, e) for _, b, e in parts] == [(0, 4), (4, 8), (8, 10)]
    rng = np.random.default_rng(0)
    x, w, b = rng.normal(size=(5, 96)).astype(np.float32), rng.normal(size=(37, 96)).astype(np.float32), rng.normal(size=37).astype(np.float32)
    y1, y4 = cpu.gemm_nt(x, w, b, threads=1), cpu.gemm_nt(x, w, b, threads=4)
    assert np.array_equal(y1, y4) and np.allclose(y1, x @ w.T + b, atol=1e-4)
    for bits, tol in ((8, 0.02), (4, 0.2)):
        pk = cpu.pack_weights(w, bits, 32)
        q1, q3 = cpu.quant_gemm(x, pk, threads=1), cpu.quant_gemm(x, pk, threads=3)
        assert np.array_equal(q1, q3)
        assert np.linalg.norm(q1 - x @ w.T) / np.linalg.norm(x @ w.T) < tol
        assert pk.nbytes < w.nbytes / (3 if bits == 8 else 5)


def test_token_loader_on_cpu_is_ordered():
    src = SyntheticTokens(100, seed=3)
    ref = SyntheticTokens(100, seed=3)
    ld = GpuTokenLoader(src, 2, 8, device="cpu", depth=2)
    for _ in range(5):
        got = ld.next()
        assert np.array_equal(got.numpy(), np.asarray(ref.next_rows(2, 8), dtype=np.int32))
    ld.close()
    assert ld.batches == 5 and ld.h2d_bytes == 5 * 2 * 8 * 4


@pytest.mark.gpu
def test_token_loader_gpu():
    src, ref = SyntheticTokens(100, seed=5), SyntheticTokens(100, seed=5)
    ld = GpuTokenLoader(src, 4, 64, device="cuda", depth=3)
    for _ in range(6):
        got = ld.next()
        assert got.is_cuda and np.array_equal(got.cpu().numpy(), np.asarray(ref.next_rows(4, 64), dtype=np.int32))
    ld.close()


def test_nvme_store_aligned_direct_io_roundtrip(tmp_path):
    """Offload store: one header sector + payload padded to sectors, written and read through page-aligned bounce
    buffers (O_DIRECT where the file system takes it, buffered otherwise); odd sizes, empty payloads, overwrite,
    asynchronous forms, truncated files are refused."""
    import os
    from nexus_b200.parallel.nvme import ALIGN, NvmeStore
    for direct in (True, False):
        st = NvmeStore(str(tmp_path / f"d{int(direct)}"), direct=direct)
        assert isinstance(st.direct, bool) and (st.direct is False or direct)
        blobs = {"a": b"", "b/c": b"x", "odd": os.urandom(ALIGN + 17), "big": os.urandom(3 * ALIGN)}
        for k, v in blobs.items():
            st.write(k, v)
        for k, v in blobs.items():
            assert st.read(k) == v
            assert os.path.getsize(st._path(k)) % ALIGN == 0
        st.write("odd", b"replaced")
        assert st.read("odd") == b"replaced"
        futs = [st.write_async(f"k{i}", bytes([i]) * (100 * i + 1)) for i in range(6)]
        [f.result() for f in futs]
        assert [st.read_async(f"k{i}").result() for i in range(6)] == [bytes([i]) * (100 * i + 1) for i in range(6)]
        assert st.contains("big") and st.bytes_read > 0 and st.bytes_written > 0
        with open(st._path("big"), "r+b") as f:
            f.truncate(ALIGN)
        try:
            st.read("big")
            raise AssertionError("a truncated file was accepted")
        except IOError:
            pass
        st.remove("big")
        assert not st.contains("big")
