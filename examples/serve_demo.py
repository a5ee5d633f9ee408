"""Continuous batching on the paged-KV engine: 64 concurrent requests against GPT-2 124M (random weights).

    python examples/serve_demo.py [--requests 64] [--max-new 64] [--quant w8a8|w4a16] [--kv int8|fp8]
"""
import argparse
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from nexus_b200.infer import Engine, EngineConfig, Gpt2Weights, QuantOptions, SamplingParams, generate  # noqa: E402
from nexus_b200.serve import Config, Request, Server  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--requests", type=int, default=64)
    ap.add_argument("--max-new", type=int, default=64)
    ap.add_argument("--prompt-len", type=int, default=32)
    ap.add_argument("--quant", default="bf16")
    ap.add_argument("--kv", default="bf16")
    ap.add_argument("--small", action="store_true", help="2-layer model (CPU friendly)")
    a = ap.parse_args()
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    w = Gpt2Weights.random(2, 4, 256, 1000, 256) if a.small else Gpt2Weights.random(12, 12, 768, 50257, 1024)
    eng = Engine(w, EngineConfig(device=dev, precision="bf16" if dev == "cuda" else "fp32", max_seqs=64, max_tokens=4096,
                                 kv_bytes=2 << 30, quant=QuantOptions(weights=a.quant, kv=a.kv)))
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, w.vocab, (a.prompt_len,), generator=g).tolist() for _ in range(a.requests)]
    sp = SamplingParams(temperature=0.8, top_k=50, top_p=0.95, seed=7)
    generate(eng, prompts[0], 8, sp)                # warm-up: scratch buffers and the decode graph of batch size 1
    t0 = time.perf_counter()
    single = generate(eng, prompts[0], a.max_new, sp)
    t_single = time.perf_counter() - t0
    srv = Server(eng, Config(max_batch_tokens=4096, max_running=64))
    futs = [srv.submit(Request(p, a.max_new, sampling=sp)) for p in prompts]
    t0 = time.perf_counter()
    srv.run_until_idle()
    dt = time.perf_counter() - t0
    total = sum(len(f.result().tokens) for f in futs)
    m = srv.metrics
    print(f"single request: {len(single) / t_single:,.0f} tok/s;  {a.requests} concurrent: {total / dt:,.0f} tok/s "
          f"({m.steps} steps, mean TTFT {m.mean_ttft_ms():.1f} ms, mean TPOT {m.mean_tpot_ms():.2f} ms, "
          f"{m.preemptions} preemptions, {eng.graphs_captured()} decode graphs)")


if __name__ == "__main__":
    main()
