import math
import warnings

import numpy as np
import pytest
import torch

from nexus_b200 import backend as B


def _case_tensors(dev):
    g = torch.Generator().manual_seed(0)
    r = lambda *s: torch.randn(*s, generator=g).to(dev)   # noqa: E731
    return r


def _check_driver(d, dev, tol=1e-4):
    ref = B.CpuDriver()
    r = _case_tensors(dev)
    a, b = r(1003), r(1003).abs() + 0.5
    for op in B.ELEMENTWISE:
        x = a.abs() + 0.1 if op in (B.Operation.Log, B.Operation.Sqrt, B.Operation.Rsqrt) else a
        out, want = torch.empty_like(a), torch.empty(1003)
        d.elementwise(op, x, b, out, 0.7)
        ref.elementwise(op, x.cpu(), b.cpu(), want, 0.7)
        assert torch.allclose(out.cpu(), want, atol=tol, rtol=1e-4), op
    for ta, tb in ((False, False), (True, False), (False, True), (True, True)):
        A = r(70, 45) if ta else r(45, 70)
        Bm = r(33, 70) if tb else r(70, 33)
        c = r(45, 33)
        want = c.cpu().clone()
        ref.matmul(A.cpu(), Bm.cpu(), want, a_trans=ta, b_trans=tb, alpha=0.5, beta=2.0)
        d.matmul(A, Bm, c, a_trans=ta, b_trans=tb, alpha=0.5, beta=2.0)
        assert torch.allclose(c.cpu(), want, atol=1e-3)
    x = r(100000)
    out, want = torch.zeros((), device=dev), torch.zeros(())
    d.reduce_sum(x, out)
    ref.reduce_sum(x.cpu(), want)
    assert abs(float(out) - float(want)) < 1e-2
    x, w, bb = r(37, 300), r(300), r(300)
    for fn, args in (("softmax", ()), ("rms_norm", (w,)), ("layer_norm", (w, bb))):
        out, want = torch.empty_like(x), torch.empty(37, 300)
        getattr(d, fn)(x, *args, out)
        getattr(ref, fn)(x.cpu(), *[t.cpu() for t in args], want)
        assert torch.allclose(out.cpu(), want, atol=1e-4), fn
    x = r(6, 20, 32)
    out, want = torch.empty_like(x), torch.empty(6, 20, 32)
    d.rope(x, out, 3, 10000.0)
    ref.rope(x.cpu(), want, 3, 10000.0)
    assert torch.allclose(out.cpu(), want, atol=1e-4)
    x = r(11, 2 * 48)
    out, want = torch.empty(11, 48, device=dev), torch.empty(11, 48)
    d.swiglu(x, out)
    ref.swiglu(x.cpu(), want)
    assert torch.allclose(out.cpu(), want, atol=1e-5)
    q, k, v = r(4, 50, 40), r(4, 50, 40), r(4, 50, 40)
    for causal in (True, False):
        out, want = torch.empty_like(q), torch.empty(4, 50, 40)
        d.attention(q, k, v, out, causal)
        ref.attention(q.cpu(), k.cpu(), v.cpu(), want, causal)
        assert torch.allclose(out.cpu(), want, atol=1e-4)
    a = r(9, 128)
    q8 = torch.randint(-127, 128, (21, 128), dtype=torch.int8).to(dev)
    s8 = (r(21, 4).abs() + 0.01)
    out, want = torch.empty(9, 21, device=dev), torch.empty(9, 21)
    d.quant_matmul_q8(a, q8, s8, out, 32)
    ref.quant_matmul_q8(a.cpu(), q8.cpu(), s8.cpu(), want, 32)
    assert torch.allclose(out.cpu(), want, atol=1e-2, rtol=1e-4)
    q4 = torch.randint(0, 256, (21, 64), dtype=torch.uint8).to(dev)
    d.quant_matmul_q4(a, q4, s8, out, 32)
    ref.quant_matmul_q4(a.cpu(), q4.cpu(), s8.cpu(), want, 32)
    assert torch.allclose(out.cpu(), want, atol=1e-2, rtol=1e-4)
    p, g, m, v = r(500), r(500), r(500) * 0.1, r(500).abs() * 0.1
    pc, mc, vc = p.cpu().clone(), m.cpu().clone(), v.cpu().clone()
    d.adamw_step(p, g, m, v, 1e-2, 0.9, 0.99, 1e-8, 0.1, 3)
    ref.adamw_step(pc, g.cpu(), mc, vc, 1e-2, 0.9, 0.99, 1e-8, 0.1, 3)
    assert torch.allclose(p.cpu(), pc, atol=1e-5) and torch.allclose(v.cpu(), vc, atol=1e-6)
    f = torch.empty(77, device=dev)
    d.fill(f, 2.5)
    assert float(f.min()) == 2.5


def test_cpu_driver_and_registry(monkeypatch):
    reg = B.Registry.instance()
    cpu = reg.require(B.Kind.Cpu)
    _check_driver(cpu, "cpu")
    monkeypatch.setenv("NEXUS_BACKEND", "cpu")
    assert reg.select().kind() == B.Kind.Cpu
    monkeypatch.setenv("NEXUS_BACKEND", "vulkan")
    with pytest.raises(RuntimeError, match="Vulkan"):
        reg.select()
    monkeypatch.delenv("NEXUS_BACKEND")
    assert reg.select().kind() in (B.Kind.Cpu, B.Kind.Cuda)
    for kind in (B.Kind.Hip, B.Kind.Metal, B.Kind.DirectMl, B.Kind.Pjrt):
        d = reg.find(kind)
        assert d is not None and not d.available() and d.unavailable_reason()
    assert B.parse_kind("ROCm") == B.Kind.Hip
    buf = cpu.allocate(0, 256)
    assert cpu.allocator_stats().live_blocks >= 1
    cpu.deallocate(0, buf)


def test_fallback_policy():
    d = B.UnavailableDriver(B.Kind.Vulkan, "vulkan", "x")
    B.reset_fallback_stats()
    B.set_fallback_policy(B.FallbackPolicy.Error)
    with pytest.raises(RuntimeError):
        B.require_cpu_fallback(d, B.Operation.Rope, 10)
    B.set_fallback_policy(B.FallbackPolicy.WarnOnce)
    with warnings.catch_warnings(record=True) as w:
        warnings.simplefilter("always")
        B.require_cpu_fallback(d, B.Operation.Rope, 10)
        B.require_cpu_fallback(d, B.Operation.Rope, 5)
    assert len(w) == 1
    st = B.fallback_stats(B.Kind.Vulkan, B.Operation.Rope)
    assert st.calls == 2 and st.elements == 15
    B.set_fallback_policy(B.FallbackPolicy.Error)


def test_hipify_source():
    src = '#include <cuda_runtime.h>\n#include <nccl.h>\ncudaStream_t s; cudaMallocAsync(&p, n, s); ' \
          'float v = __shfl_xor_sync(0xffffffffu, x, 16); cublasLtMatmul(h); ncclAllReduce(a); nvrtcCompileProgram(p);' \
          ' my_cudaThing(); cudaErrorInvalidValue'
    out = B.hipify_source(src)
    assert "hip/hip_runtime.h" in out and "rccl/rccl.h" in out and "hipStream_t s" in out
    assert "hipMallocAsync" in out and "__shfl_xor(x, 16)" in out and "hipblasLtMatmul" in out
    assert "ncclAllReduce" in out and "hiprtcCompileProgram" in out and "my_cudaThing" in out
    assert "hipErrorInvalidValue" in out


def test_stablehlo_interpreter_and_sharding():
    m = B.StableHloModule("mlp")
    x, w, b = m.arg((4, 8), "{devices=[2,1]0,1}"), m.arg((8, 16)), m.arg((16,))
    h = m.add(m.dot_general(x, w, (1, 0)), m.broadcast_in_dim(b, (4, 16), [1]))
    y = m.multiply(h, m.unary("logistic", h))
    mx = m.reduce(y, [1], "max")
    e = m.unary("exponential", m.subtract(y, m.broadcast_in_dim(mx, (4, 16), [0])))
    sm = m.divide(e, m.broadcast_in_dim(m.reduce(e, [1]), (4, 16), [0]))
    m.ret(sm, m.transpose(m.reshape(h, (4, 4, 4)), [0, 2, 1]))
    rng = np.random.default_rng(0)
    X, W, Bv = rng.normal(size=(4, 8)), rng.normal(size=(8, 16)), rng.normal(size=16)
    out, tr = m.run(X, W, Bv)
    H = torch.tensor(X) @ torch.tensor(W) + torch.tensor(Bv)
    want = torch.softmax(torch.nn.functional.silu(H), -1)
    assert np.allclose(out, want.numpy(), atol=1e-5)
    assert np.allclose(tr, H.float().numpy().reshape(4, 4, 4).transpose(0, 2, 1), atol=1e-5)
    txt = m.text()
    assert "stablehlo.dot_general" in txt and 'mhlo.sharding = "{devices=[2,1]0,1}"' in txt and "func.func public @main" in txt
    assert B.sharding_annotation([2, 4], ["replicate", "replicate"], 2) == "{replicated}"
    assert B.sharding_annotation([2, 4], [("shard", 0), ("shard", 1)], 2) == "{devices=[2,4]0,1,2,3,4,5,6,7}"
    assert B.sharding_annotation([2, 4], [("shard", 1), ("shard", 0)], 2) == "{devices=[4,2]0,4,1,5,2,6,3,7}"
    assert B.sharding_annotation([2, 4], ["replicate", ("shard", 0)], 2) == \
        "{devices=[4,1,2]0,4,1,5,2,6,3,7 last_tile_dim_replicate}"


@pytest.mark.gpu
def test_cuda_driver_matches_cpu_reference():
    d = B.Registry.instance().require(B.Kind.Cuda)
    assert d.devices()[0].subgroup_size == 32
    _check_driver(d, "cuda", tol=2e-4)
    from nexus_b200.ops import _cuda as K
    import ctypes as C
    # dispatcher helpers
    x = torch.randn(1000, device="cuda")
    y = torch.empty(1000, dtype=torch.bfloat16, device="cuda")
    K._check(K.lib().nx_cast(K._p(x), C.c_int(1), K._p(y), C.c_int(0), C.c_int64(1000), K._stream()), "nx_cast")
    assert torch.equal(y, x.bfloat16())
    g = torch.empty_like(x)
    K._check(K.lib().nx_gelu(K._p(x), K._p(None), K._p(g), C.c_int(1), C.c_int64(1000), K._stream()), "nx_gelu")
    assert torch.allclose(g, torch.nn.functional.gelu(x, approximate="tanh"), atol=2e-3)
    T = 40
    s = torch.randn(3 * T, T, device="cuda")
    p = torch.empty_like(s)
    K._check(K.lib().nx_causal_softmax(K._p(s), K._p(None), K._p(p), C.c_int64(3 * T), C.c_int(T), C.c_float(0.5),
                                       K._stream()), "nx_causal_softmax")
    mask = torch.ones(T, T, device="cuda").tril().bool().repeat(3, 1)
    want = torch.softmax((s * 0.5).masked_fill(~mask, float("-inf")), -1)
    assert torch.allclose(p, want, atol=1e-5)
    dy = torch.randn_like(s)
    dx = torch.empty_like(s)
    K._check(K.lib().nx_causal_softmax(K._p(p), K._p(dy), K._p(dx), C.c_int64(3 * T), C.c_int(T), C.c_float(0.5),
                                       K._stream()), "nx_causal_softmax")
    sr = s.clone().requires_grad_(True)
    torch.softmax((sr * 0.5).masked_fill(~mask, float("-inf")), -1).backward(dy)
    assert torch.allclose(dx, sr.grad, atol=1e-5)
    qkv = torch.randn(2, 5, 3, 4, 8, device="cuda").bfloat16()
    q, k, v = (torch.empty(2, 4, 5, 8, device="cuda", dtype=torch.bfloat16) for _ in range(3))
    K._check(K.lib().nx_split_heads(K._p(qkv), K._p(q), K._p(k), K._p(v), C.c_int(2), C.c_int(5), C.c_int(4), C.c_int(8),
                                    C.c_int(0), K._stream()), "nx_split_heads")
    assert torch.equal(k, qkv[:, :, 1].transpose(1, 2))
    back = torch.zeros_like(qkv)
    K._check(K.lib().nx_split_heads(K._p(back), K._p(q), K._p(k), K._p(v), C.c_int(2), C.c_int(5), C.c_int(4), C.c_int(8),
                                    C.c_int(1), K._stream()), "nx_split_heads")
    assert torch.equal(back, qkv)
