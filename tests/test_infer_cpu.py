"""Host logic of the inference engine and the server on the FP32 reference path (CPU):
paged == contiguous, copy-on-write fork, truncate, speculative == greedy, continuous batching ==
one-by-one generation, preemption by recompute, sampler rules, quantised weights."""
import math

import numpy as np
import pytest
import torch

from nexus_b200.infer import (Chunk, Engine, EngineConfig, Gpt2Weights, QuantOptions, SamplingParams, generate,
                              sample_reference, speculative_generate)
from nexus_b200.serve import Config, Request, Server


def make(layers=2, heads=2, d=32, vocab=97, ctx=64, **kw):
    w = Gpt2Weights.random(layers, heads, d, vocab, ctx, seed=1)
    for lw in w.h:   # larger weights: logits with clear arg-max gaps
        for k in ("attn_w", "fc_w", "proj_w", "fc2_w"):
            lw[k] *= 4.0
    cfg = EngineConfig(precision="fp32", device="cpu", max_seqs=8, max_tokens=256, block_size=4,
                       kv_bytes=kw.pop("kv_bytes", 1 << 20), **kw)
    return w, Engine(w, cfg)


def dense_logits(w: Gpt2Weights, toks):
    """Plain causal transformer over the whole sequence (no cache)."""
    F = torch.nn.functional
    T = len(toks)
    x = w.wte[torch.tensor(toks)] + w.wpe[:T]
    H, D = w.heads, w.d // w.heads
    mask = torch.ones(T, T).tril().bool()
    for lw in w.h:
        h = F.layer_norm(x, (w.d,), lw["ln1_w"], lw["ln1_b"])
        q, k, v = ((h @ lw["attn_w"].t() + lw["attn_b"]).split(w.d, 1))
        q, k, v = (t.view(T, H, D).transpose(0, 1) for t in (q, k, v))
        a = ((q @ k.transpose(1, 2)) / math.sqrt(D)).masked_fill(~mask, float("-inf")).softmax(-1) @ v
        x = x + a.transpose(0, 1).reshape(T, w.d) @ lw["proj_w"].t() + lw["proj_b"]
        h = F.layer_norm(x, (w.d,), lw["ln2_w"], lw["ln2_b"])
        x = x + F.gelu(h @ lw["fc_w"].t() + lw["fc_b"], approximate="tanh") @ lw["fc2_w"].t() + lw["fc2_b"]
    return F.layer_norm(x, (w.d,), w.ln_f_w, w.ln_f_b) @ w.wte.t()


def test_paged_matches_dense_prefill_and_decode():
    w, e = make()
    toks = [5, 17, 3, 88, 41, 2, 9, 30, 11]
    ref = dense_logits(w, toks)
    s = e.add_sequence()
    lg = e.forward([Chunk(s, toks[:6], 6)])
    assert torch.allclose(lg[:, : w.vocab], ref[:6], atol=1e-4)
    for i in range(6, 9):
        lg = e.forward([Chunk(s, [toks[i]], 1, True)])
        assert torch.allclose(lg[0, : w.vocab], ref[i], atol=1e-4)
    assert e.length(s) == 9 and e.tokens(s) == toks
    assert e.last_step().decode_tokens == 1
    e.free_sequence(s)
    assert e.free_blocks() == e.total_blocks()


def test_fork_copy_on_write_and_truncate():
    w, e = make()
    a = e.add_sequence()
    e.forward([Chunk(a, [1, 2, 3, 4, 5, 6], 1)])           # 1.5 blocks
    used = e.total_blocks() - e.free_blocks()
    b = e.fork_sequence(a)
    assert e.total_blocks() - e.free_blocks() == used       # shared
    assert e.blocks_needed(b, 1) == 1                       # shared partial block -> copy
    la = e.forward([Chunk(a, [7], 1)])[0].clone()
    lb = e.forward([Chunk(b, [9], 1)])[0].clone()
    assert torch.allclose(la[: w.vocab], dense_logits(w, [1, 2, 3, 4, 5, 6, 7])[-1], atol=1e-4)
    assert torch.allclose(lb[: w.vocab], dense_logits(w, [1, 2, 3, 4, 5, 6, 9])[-1], atol=1e-4)
    e.truncate(a, 3)
    assert e.length(a) == 3 and e.tokens(a) == [1, 2, 3]
    lt = e.forward([Chunk(a, [50], 1)])[0]
    assert torch.allclose(lt[: w.vocab], dense_logits(w, [1, 2, 3, 50])[-1], atol=1e-4)
    # the fork is untouched by the truncate + rewrite of the other sequence
    lb2 = e.forward([Chunk(b, [10], 1)])[0]
    assert torch.allclose(lb2[: w.vocab], dense_logits(w, [1, 2, 3, 4, 5, 6, 9, 10])[-1], atol=1e-4)
    e.free_sequence(a)
    e.free_sequence(b)
    assert e.free_blocks() == e.total_blocks()
    assert int(e.counts_all.sum()) >= 0


def test_generate_and_speculative_equal_greedy():
    w, e = make(layers=3)
    prompt = [3, 14, 15, 92, 65]
    base = generate(e, prompt, 12)
    spec = speculative_generate(e, prompt, 12, draft_layers=1, gamma=3)
    assert spec == base
    from nexus_b200.infer import SpecStats
    st = SpecStats()
    spec2 = speculative_generate(e, prompt, 12, draft_layers=3, gamma=4, stats=st)   # draft == target: all accepted
    assert spec2 == base and st.accepted == st.drafted and st.tokens_per_step > 2
    assert e.free_blocks() == e.total_blocks()


def test_batch_forward_matches_single():
    w, e = make()
    p1, p2 = [4, 8, 15, 16, 23], [42, 7, 7]
    s1, s2 = e.add_sequence(), e.add_sequence()
    lg = e.forward([Chunk(s1, p1, 1), Chunk(s2, p2, 2)])
    assert e.logit_rows() == 3
    assert torch.allclose(lg[0, : w.vocab], dense_logits(w, p1)[-1], atol=1e-4)
    assert torch.allclose(lg[1:, : w.vocab], dense_logits(w, p2)[-2:], atol=1e-4)
    lg = e.forward([Chunk(s1, [9], 1, True), Chunk(s2, [1, 2], 1, True)])
    assert torch.allclose(lg[0, : w.vocab], dense_logits(w, p1 + [9])[-1], atol=1e-4)
    assert torch.allclose(lg[1, : w.vocab], dense_logits(w, p2 + [1, 2])[-1], atol=1e-4)
    nll = e.nll([5, 6])
    ref = torch.nn.functional.cross_entropy(lg[:, : w.vocab], torch.tensor([5, 6]), reduction="none")
    assert np.allclose(nll, ref.numpy(), atol=1e-4)


def test_server_continuous_batching_matches_one_by_one():
    w, e = make(layers=2)
    prompts = [[1, 2, 3], [9, 8, 7, 6, 5, 4], [11], [20, 21, 22, 23], [30, 31]]
    want = [generate(e, p, 6) for p in prompts]
    srv = Server(e, Config(max_batch_tokens=16, max_running=3))
    seen = {}
    futs = [srv.submit(Request(p, 6, on_token=lambda rid, t: seen.setdefault(rid, []).append(t))) for p in prompts]
    srv.run_until_idle(200)
    got = [f.result(timeout=1) for f in futs]
    assert [g.tokens for g in got] == want
    assert [seen[g.id] for g in got] == want
    m = srv.metrics
    assert m.completed == 5 and m.output_tokens == 30 and m.steps > 6
    assert e.free_blocks() == e.total_blocks()


def test_server_preempts_by_recompute_when_blocks_run_out():
    # 10 blocks of 4 tokens: three requests of 6 + 10 tokens cannot all stay resident
    w, e = make(layers=1, kv_bytes=10 * 4 * (1 * 2 * 2 * 16 * 4))
    assert e.total_blocks() == 10
    prompts = [[1, 2, 3, 4, 5, 6], [7, 8, 9, 10, 11, 12], [13, 14, 15, 16, 17, 18]]
    want = [generate(e, p, 10) for p in prompts]
    srv = Server(e, Config(max_batch_tokens=64, max_running=3))
    futs = [srv.submit(Request(p, 10)) for p in prompts]
    srv.run_until_idle(500)
    got = [f.result(timeout=1) for f in futs]
    assert [g.tokens for g in got] == want
    assert srv.metrics.preemptions > 0 and sum(g.preemptions for g in got) == srv.metrics.preemptions
    assert e.free_blocks() == e.total_blocks()


def test_server_background_thread():
    w, e = make(layers=1)
    srv = Server(e)
    srv.start()
    try:
        f = srv.submit(Request([1, 2, 3], 4))
        assert len(f.result(timeout=30).tokens) == 4
    finally:
        srv.stop()


def test_sampler_reference_rules():
    rng = np.random.default_rng(0)
    logits = rng.normal(size=50).astype(np.float32) * 3
    assert sample_reference(logits, SamplingParams(temperature=0.0)) == int(np.argmax(logits))
    tie = logits.copy()
    tie[7] = tie[31] = tie.max() + 1
    assert sample_reference(tie, SamplingParams(temperature=0.0)) == 7
    top3 = set(np.argsort(logits)[-3:].tolist())
    draws = [sample_reference(logits, SamplingParams(temperature=1.0, top_k=3, seed=5), offset=i) for i in range(200)]
    assert set(draws) <= top3 and len(set(draws)) >= 2
    p = np.exp(logits - logits.max())
    p /= p.sum()
    order = np.argsort(-p)
    nucleus = set(order[: int(np.searchsorted(np.cumsum(p[order]), 0.6)) + 1].tolist())
    draws = [sample_reference(logits, SamplingParams(temperature=1.0, top_p=0.6, seed=9), offset=i) for i in range(200)]
    assert set(draws) <= nucleus
    draws = [sample_reference(logits, SamplingParams(temperature=1.0, min_p=0.5, seed=1), offset=i) for i in range(100)]
    assert all(p[d] >= 0.5 * p.max() - 1e-7 for d in draws)
    # distribution check (chi-square-ish) for plain temperature sampling
    n = 4000
    draws = np.array([sample_reference(logits, SamplingParams(temperature=1.0, seed=3), offset=i) for i in range(n)])
    freq = np.bincount(draws, minlength=50) / n
    assert np.abs(freq - p).max() < 0.03
    # penalties
    counts = np.zeros(50, dtype=np.int32)
    best = int(np.argmax(logits))
    counts[best] = 3
    pen = SamplingParams(temperature=0.0, frequency_penalty=100.0)
    assert sample_reference(logits, pen, counts, counts) != best
    rep = SamplingParams(temperature=0.0, repetition_penalty=1e6)
    assert sample_reference(np.abs(logits) + 1, rep, counts, None) != best or np.argmax(np.abs(logits) + 1) != best
    # same (seed, offset) -> same draw
    sp = SamplingParams(temperature=0.8, seed=77)
    assert sample_reference(logits, sp, offset=5) == sample_reference(logits, sp, offset=5)


@pytest.mark.parametrize("mode,tol", [("w8a8", 0.08), ("w4a16", 0.25)])
def test_quantised_weights_stay_close(mode, tol):
    w = Gpt2Weights.random(2, 2, 128, 97, 32, seed=2)
    toks = [5, 6, 7, 8, 9, 10, 11, 12]
    cfg = dict(precision="fp32", device="cpu", max_seqs=2, max_tokens=64, block_size=4, kv_bytes=1 << 20)
    e0 = Engine(w, EngineConfig(**cfg))
    eq = Engine(w, EngineConfig(quant=QuantOptions(weights=mode, w4_group=32, calibration=toks), **cfg))
    assert eq.weight_bytes() < e0.weight_bytes()
    a = e0.forward([Chunk(e0.add_sequence(), toks, 8)])[:, :97]
    b = eq.forward([Chunk(eq.add_sequence(), toks, 8)])[:, :97]
    rel = (a - b).norm() / a.norm()
    assert rel < tol
    pa = a.log_softmax(-1)
    nll0 = -pa[torch.arange(7), torch.tensor(toks[1:])].mean()
    nllq = -b.log_softmax(-1)[torch.arange(7), torch.tensor(toks[1:])].mean()
    assert abs(float(nll0 - nllq)) < 0.1


def test_int8_kv_close_to_fp():
    w = Gpt2Weights.random(2, 2, 32, 97, 32, seed=3)
    cfg = dict(precision="fp32", device="cpu", max_seqs=2, max_tokens=64, block_size=4, kv_bytes=1 << 20)
    e0 = Engine(w, EngineConfig(**cfg))
    e8 = Engine(w, EngineConfig(quant=QuantOptions(kv="int8"), **cfg))
    assert e8.kv_bytes_per_token() < e0.kv_bytes_per_token()
    toks = list(range(3, 13))
    s0, s8 = e0.add_sequence(), e8.add_sequence()
    e0.forward([Chunk(s0, toks, 0)])
    e8.forward([Chunk(s8, toks, 0)])
    a = e0.forward([Chunk(s0, [40], 1)])[0, :97]
    b = e8.forward([Chunk(s8, [40], 1)])[0, :97]
    assert (a - b).norm() / a.norm() < 0.02


@pytest.mark.parametrize("ranks,heads", [(2, 4), (3, 4), (4, 2)])
def test_tensor_parallel_engine_with_uneven_heads_matches_one_rank(ranks, heads):
    """Heads and MLP columns sharded over a group, also when the heads do not divide evenly (the last ranks hold fewer
    heads or none and only take part in the all-reduce): every rank owns the same number of KV blocks and produces the
    tokens of the single-rank engine."""
    from nexus_b200.parallel.process_group import ThreadWorld
    w = Gpt2Weights.random(2, heads, 48, 97, 64, seed=3)
    for lw in w.h:
        for k in ("attn_w", "fc_w", "proj_w", "fc2_w"):
            lw[k] *= 4.0
    cfg = dict(precision="fp32", device="cpu", max_seqs=4, max_tokens=128, block_size=4, kv_bytes=1 << 20)
    prompt = [5, 17, 3, 44, 9, 60, 2]
    want = generate(Engine(w, EngineConfig(**cfg)), prompt, 12, SamplingParams(temperature=0.0))

    def run(pg):
        eng = Engine(w, EngineConfig(tp_comm="nccl", **cfg), group=pg)
        return eng.n_blocks, generate(eng, prompt, 12, SamplingParams(temperature=0.0))

    out = ThreadWorld(ranks).run(run)
    assert len({nb for nb, _ in out}) == 1
    for _, toks in out:
        assert toks == want


@pytest.mark.parametrize("kv_bytes,max_running", [(1 << 20, 8), (1 << 20, 3), (40 * 1024, 8)])
def test_pipelined_decode_equals_step_by_step(kv_bytes, max_running):
    """Launching decode step n + 1 before the tokens of step n are read (device-fed tokens, tokens consumed one step
    late, zombie steps of requests that hit their stop token) produces exactly the tokens, stop points and engine-side
    token lists of the ordinary loop: with admission in the middle of decoding, with preemption by recompute when
    blocks run out, with stop tokens, seeds and penalties."""
    outs = {}
    for pipe in (False, True):
        w, eng = make(layers=2, heads=2, d=32, vocab=97, ctx=64, kv_bytes=kv_bytes)
        srv = Server(eng, Config(max_batch_tokens=64, max_running=max_running, pipeline_decode=pipe))
        g = torch.Generator().manual_seed(5)
        futs, streamed = [], {}
        for i in range(7):
            prompt = torch.randint(0, 97, (int(torch.randint(3, 14, (1,), generator=g)),), generator=g).tolist()
            sp = SamplingParams(temperature=0.0) if i % 2 == 0 else \
                SamplingParams(temperature=0.9, top_k=20, top_p=0.95, seed=100 + i, repetition_penalty=1.1)
            futs.append(srv.submit(Request(prompt, 5 + 3 * i, sampling=sp, stop_token=11 if i % 3 == 0 else None,
                                           on_token=lambda rid, t, d=streamed: d.setdefault(rid, []).append(t))))
        srv.run_until_idle()
        res = [f.result() for f in futs]
        assert all(streamed[r.id] == r.tokens for r in res)
        assert eng.free_blocks() == eng.total_blocks()            # every sequence (zombies included) was released
        assert (srv.metrics.pipelined_steps > 0) == pipe
        outs[pipe] = [(r.tokens, r.preemptions) for r in res]
    assert outs[True] == outs[False]
