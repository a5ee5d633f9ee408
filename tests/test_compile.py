import pytest
import torch

from nexus_b200 import compile as C
from nexus_b200.compile import passes as P
from nexus_b200.lm import LanguageModel
from nexus_b200.lm.config import LmConfig, preset


def llama_cfg():
    return LmConfig(name="tiny-llama", vocab_size=96, d_model=64, n_layer=2, n_head=4, n_kv_head=2, d_ff=128,
                    max_position=64, norm="rmsnorm", mlp="swiglu", pos="rope", bias=False, tie_embeddings=False)


def test_trace_and_patterns_gpt2():
    cfg = preset("nano")
    g = C.trace_lm(cfg)
    L = cfg.n_layer
    assert g.count("Linear") == 4 * L + 1 and g.count("Bias") == 4 * L and g.count("Gelu") == L
    assert g.count("LayerNorm") == 2 * L + 1 and g.count("Attention") == L
    fp = g.fingerprint()
    assert fp == C.trace_lm(cfg).fingerprint() and fp != C.trace_lm(llama_cfg()).fingerprint()
    assert "Embedding" in g.text() and g.dot().startswith("digraph")
    st = P.rewrite_patterns(g)
    assert st["linear_bias_gelu"] == L and st["attention_qkv"] == L and st["linear_ce"] == 1
    assert st["add_norm"] == 2 * L and st["linear_bias"] == 3 * L
    assert g.count("Bias") == 0 and g.count("SplitQKV") == 0 and g.count("FusedLinearCE") == 1
    only = C.trace_lm(cfg)
    st2 = P.rewrite_patterns(only, P.P_LINEAR_CE)
    assert st2["linear_ce"] == 1 and st2["linear_bias_gelu"] == 0 and only.count("Bias") == 4 * L


def test_patterns_llama_and_cleanup_passes():
    g = C.trace_lm(llama_cfg())
    st = P.rewrite_patterns(g)
    assert st["gated"] == 2 and g.count("SwiGlu") == 2 and st["attention_qkv"] == 0   # RoPE sits between split and attention
    g2 = C.Graph("t")
    x = g2.input("x", ["B", 8], "f32")
    (a,) = g2.add("Scale", [x], [x.shape], factor=2.0)
    (b,) = g2.add("Scale", [a], [x.shape], factor=3.0)
    (c1,) = g2.add("Tanh", [b], [x.shape])
    (c2,) = g2.add("Tanh", [b], [x.shape])
    (dead,) = g2.add("Gelu", [x], [x.shape])
    (s,) = g2.add("Add", [c1, c2], [x.shape])
    g2.outputs = [s]
    assert P.constant_fold(g2) == 1 and P.cse(g2) == 1 and g2.count("Gelu") == 0
    assert [n.op for n in g2.nodes] == ["Input", "Scale", "Tanh", "Add"]
    assert float(g2.nodes[1].attrs["factor"]) == 6.0


@pytest.mark.parametrize("make", [lambda: preset("nano"), llama_cfg])
def test_compiled_lm_matches_model(make):
    cfg = make()
    torch.manual_seed(0)
    m = LanguageModel(cfg)
    toks = torch.randint(0, cfg.vocab_size, (2, 16))
    want = m.loss(toks)
    want.backward()
    for opt in (C.CompileOptions(), C.CompileOptions(patterns=0, fuse=False, jit=False)):
        c = C.compile_lm(m, opt)
        assert abs(float(c.loss(toks)) - float(want)) < 1e-5
        loss, grads = c.loss_and_grads(toks)
        assert abs(float(loss) - float(want)) < 1e-5
        named = dict(m.named_parameters())
        assert set(grads) == set(c.graph.params)
        for k, g in grads.items():
            assert torch.allclose(g, named[k].grad, atol=2e-5, rtol=1e-4), k
    c = C.compile_lm(m)
    plan = c.memory_plan(2, 16)
    assert 0 < plan["arena_bytes"] < plan["naive_bytes"]
    rp = c.recompute_plan(2, 16)
    assert rp["saved_bytes"] <= rp["baseline_bytes"] and len(rp["recomputed"]) > 0
    assert "stablehlo.dot_general" in c.export_stablehlo(2, 16) and "HloModule" in c.export_hlo_text(2, 16)


def test_fuse_elementwise_and_cpu_jit():
    g = C.Graph("f")
    x = g.input("x", ["B", 16], "f32")
    y = g.input("y", ["B", 16], "f32")
    (a,) = g.add("Add", [x, y], [x.shape])
    (b,) = g.add("Gelu", [a], [x.shape])
    (c,) = g.add("Scale", [b], [x.shape], factor=0.5)
    (d,) = g.add("Mul", [c, y], [x.shape])
    g.outputs = [d]
    st = P.fuse_elementwise(g)
    assert st["vertical"] == 1 and g.count("Fused") == 1 and len(g.nodes) == 3
    body = g.nodes[-1].attrs["body"]
    k = C.FusedKernel(body, 2, [len(body) - 1])
    assert "__global__" in k.source(True) and "tanhf" in k.source(False)
    xs, ys = torch.randn(5, 16), torch.randn(5, 16)
    (out,) = k(xs, ys)
    want = torch.nn.functional.gelu(xs + ys, approximate="tanh") * 0.5 * ys
    assert torch.allclose(out, want, atol=1e-5)
    h = C.Graph("h")
    z = h.input("z", [4, 4], "f32")
    (p,) = h.add("Tanh", [z], [z.shape])
    (q,) = h.add("Sigmoid", [z], [z.shape])
    (r,) = h.add("Linear", [p, q], [z.shape])
    h.outputs = [r]
    assert P.fuse_elementwise(h)["horizontal"] == 1 and len(h.nodes[1].outputs) == 2


def test_nvrtc_compiles_cluster_for_sm100a(tmp_path, monkeypatch):
    monkeypatch.setenv("NEXUS_JIT_CACHE", str(tmp_path))
    src = C.cluster_source([("Add", {}, [("in", 0), ("in", 1)]), ("Silu", {}, [("tmp", 0)])], 2, 1, True, [1])
    cubin = C.compile_cuda(src)
    assert cubin[:4] == b"\x7fELF" and len(list(tmp_path.iterdir())) == 1
    assert C.compile_cuda(src) == cubin      # second call: disk cache


def test_schedule_communication_hoists_gather():
    g = C.Graph("c")
    w = g.param("w_shard", [8, 8])
    x = g.input("x", ["B", 8], "f32")
    (h,) = g.add("Gelu", [x], [x.shape])
    (full,) = g.add("AllGather", [w], [[16, 8]])
    (y,) = g.add("Linear", [h, full], [["B", 16]])
    g.outputs = [y]
    assert P.schedule_communication(g) == 1
    ops = [n.op for n in g.nodes]
    assert ops.index("AllGather") < ops.index("Gelu")
    ag = g.nodes[ops.index("AllGather")]
    assert ag.attrs["async"] and g.nodes[ag.attrs["wait_before"]].op == "Linear"


@pytest.mark.gpu
def test_compiled_lm_gpu_jit_and_cuda_graph():
    cfg = llama_cfg()
    torch.manual_seed(0)
    m = LanguageModel(cfg).cuda()
    toks = torch.randint(0, cfg.vocab_size, (2, 32), device="cuda")
    want = m.loss(toks)
    want.backward()
    c = C.compile_lm(m)
    assert abs(float(c.loss(toks)) - float(want)) < 1e-4
    replay = c.capture(toks)
    loss, grads = replay(toks)
    torch.cuda.synchronize()
    assert abs(float(loss) - float(want)) < 1e-4
    named = dict(m.named_parameters())
    for k, g in grads.items():
        assert torch.allclose(g, named[k].grad, atol=1e-3, rtol=1e-3), k
    k = C.FusedKernel([("Add", {}, [("in", 0), ("in", 1)]), ("Silu", {}, [("tmp", 0)])], 2, [1])
    a, b = torch.randn(1000, device="cuda"), torch.randn(1000, device="cuda")
    (o,) = k(a, b)
    assert torch.allclose(o, torch.nn.functional.silu(a + b), atol=1e-5)


@pytest.mark.parametrize("kind", ["gpt2", "llama"])
def test_fuse_epilogues_folds_accumulation_into_the_backward_nodes(kind):
    """The joint graph with gradient accumulation folded into the Vjp nodes (beta = 1) and the GELU / bias gradients
    marked as GEMM epilogues: fewer nodes, no Accumulate left where a Vjp result was its only source, and exactly the
    losses and gradients of the unfused joint graph."""
    from nexus_b200.lm.config import preset
    cfg = preset("nano")
    cfg.n_layer, cfg.d_model, cfg.n_head, cfg.d_ff, cfg.vocab_size, cfg.max_position = 2, 32, 2, 64, 61, 16
    if kind == "llama":
        cfg.norm, cfg.mlp, cfg.pos, cfg.bias, cfg.n_kv_head = "rmsnorm", "swiglu", "rope", False, 1
    torch.manual_seed(0)
    m = LanguageModel(cfg)
    toks = torch.randint(0, cfg.vocab_size, (2, 16))
    plain = C.compile_lm(m, C.CompileOptions(epilogues=False))
    fused = C.compile_lm(m, C.CompileOptions())
    st = fused.stats["epilogues"]
    n_acc = lambda c: sum(1 for n in c.graph.nodes if n.op == "Accumulate")      # noqa: E731
    assert st["beta1"] >= 1 and n_acc(fused) == n_acc(plain) - st["beta1"]
    assert len(fused.graph.nodes) == len(plain.graph.nodes) - st["beta1"]
    if kind == "gpt2":
        assert st["dgelu"] == cfg.n_layer and st["bgrad"] >= cfg.n_layer
        assert any(n.attrs.get("epilogue") == "dgelu+bgrad" for n in fused.graph.nodes if n.op == "Vjp")
    assert any("accumulate" in n.attrs for n in fused.graph.nodes if n.op == "Vjp")
    l0, g0 = plain.loss_and_grads(toks)
    l1, g1 = fused.loss_and_grads(toks)
    assert float(l0) == float(l1) and set(g0) == set(g1)
    for k in g0:
        assert torch.allclose(g0[k], g1[k], atol=1e-7, rtol=1e-6), k
    assert float(fused.loss(toks)) == float(l1)
    assert "accumulate=" in fused.graph.text() and fused.graph.fingerprint() != plain.graph.fingerprint()
    # without the rewrite patterns the residual stream leaves many more accumulations: all of them fold away too
    raw0 = C.compile_lm(m, C.CompileOptions(patterns=0, fuse=False, jit=False, epilogues=False))
    raw1 = C.compile_lm(m, C.CompileOptions(patterns=0, fuse=False, jit=False))
    assert raw1.stats["epilogues"]["beta1"] >= 2 * cfg.n_layer and n_acc(raw1) == n_acc(raw0) - raw1.stats["epilogues"]["beta1"]
    (la, ga), (lb, gb) = raw0.loss_and_grads(toks), raw1.loss_and_grads(toks)
    assert float(la) == float(lb) and all(torch.allclose(ga[k], gb[k], atol=1e-7, rtol=1e-6) for k in ga)
