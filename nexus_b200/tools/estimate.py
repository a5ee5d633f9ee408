"""`nexus_estimate`: analytic parameter counts, memory, FLOPs and roofline time of an LM training step, and
an `--auto-parallel` search over (dp, tp, pp, cp, zero, micro batch) under a per-GPU memory limit.

Memory model: static = params + grads + optimizer (+ FP32 master), each divided by TP x PP and, per ZeRO
stage, by DP (stage 1: optimizer; 2: + grads; 3: + params); activations per layer =
``s*b*h*(34 + 5*a*s/h)`` bytes (16-bit activations, no flash) or ``34*s*b*h`` with flash attention, divided
by TP (with sequence parallelism) and CP, 2*s*b*h per layer with full recomputation; logits = s*b*V*(2+4).
Time model: compute = 6*N*tokens (+ attention) / (peak * mfu); TP / CP / DP communication from ring
volumes over the intra- or inter-node bandwidth; pipeline bubble (pp-1)/(m+pp-1).
Defaults describe an 8-GPU B200 node (180 GB, measured cuBLAS BF16 rate, NVLink 5 bus bandwidth).

    python -m nexus_b200.tools.estimate --preset gpt2-124m --batch 16 --seq 1024 [--auto-parallel --gpus 8]

Parity: tools/nexus_estimate/{estimate,autoparallel}.{hpp,cpp}, main.cpp of the reference."""
from __future__ import annotations

import argparse
import json
import sys
from dataclasses import asdict, dataclass, field
from typing import List, Optional


@dataclass
class ModelShape:
    n_layer: int = 12
    d_model: int = 768
    n_head: int = 12
    n_kv_head: int = 12
    d_ff: int = 3072
    vocab: int = 50257
    seq_len: int = 1024
    micro_batch: int = 1
    learned_pos: int = 0         # GPT-2: context length; RoPE models: 0
    tie_head: bool = True
    ffn_swiglu: bool = False
    bias: bool = True
    rmsnorm: bool = False
    gradient_accum: int = 1

    @staticmethod
    def from_config(cfg, seq_len: Optional[int] = None, micro_batch: int = 1) -> "ModelShape":
        return ModelShape(cfg.n_layer, cfg.d_model, cfg.n_head, cfg.kv_heads(), cfg.d_ff, cfg.vocab_size,
                          seq_len or cfg.max_position, micro_batch, cfg.max_position if cfg.pos == "learned" else 0,
                          cfg.tie_embeddings, cfg.gated_mlp(), cfg.bias, cfg.norm == "rmsnorm")


@dataclass
class DTypePlan:
    param_bytes: int = 2          # BF16 shadow used by the GEMMs
    grad_bytes: int = 4
    optim_bytes: int = 8          # Adam m + v in FP32
    master_bytes: int = 4         # FP32 master copy
    activation_elem_bytes: int = 2


@dataclass
class Plan:
    dp: int = 1
    tp: int = 1
    pp: int = 1
    cp: int = 1
    zero_stage: int = 0
    full_recompute: bool = False
    flash_attention: bool = True
    sequence_parallel: bool = True


def param_breakdown(m: ModelShape) -> dict:
    d, hd = m.d_model, m.d_model // m.n_head
    qkv = d * (m.n_head + 2 * m.n_kv_head) * hd + (((m.n_head + 2 * m.n_kv_head) * hd) if m.bias else 0)
    proj = d * d + (d if m.bias else 0)
    ffn = (3 if m.ffn_swiglu else 2) * d * m.d_ff + ((m.d_ff + d) if m.bias else 0)
    norms = 2 * d * (1 if m.rmsnorm else 2)
    per_layer = qkv + proj + ffn + norms
    emb = m.vocab * d + m.learned_pos * d
    head = 0 if m.tie_head else m.vocab * d
    final_norm = d * (1 if m.rmsnorm else 2)
    total = m.n_layer * per_layer + emb + head + final_norm
    return {"embedding": emb, "per_layer": per_layer, "attention": qkv + proj, "ffn": ffn, "norms": norms,
            "head": head, "final_norm": final_norm, "total": total}


def flops_per_token(m: ModelShape, causal: bool = True) -> float:
    """Training FLOPs per token: 6 per matrix parameter plus the attention score / value products."""
    p = param_breakdown(m)
    matrix = p["total"] - p["embedding"] + (m.vocab * m.d_model if m.tie_head else 0)
    attn = 12 * m.n_layer * m.d_model * m.seq_len * (0.5 if causal else 1.0)
    return 6.0 * matrix + attn


def memory_bytes(m: ModelShape, dt: DTypePlan, plan: Plan) -> dict:
    n = param_breakdown(m)["total"] / (plan.tp * plan.pp)
    z = plan.zero_stage
    params = n * dt.param_bytes / (plan.dp if z >= 3 else 1)
    grads = n * dt.grad_bytes / (plan.dp if z >= 2 else 1)
    optim = n * (dt.optim_bytes + dt.master_bytes) / (plan.dp if z >= 1 else 1)
    s, b, h, a = m.seq_len / plan.cp, m.micro_batch, m.d_model, m.n_head
    e = dt.activation_elem_bytes / 2.0
    if plan.full_recompute:
        per_layer = 2 * s * b * h * e
    else:
        per_layer = s * b * h * (34 + (0 if plan.flash_attention else 5 * a * s * plan.cp / h)) * e
        if plan.tp > 1:
            per_layer = per_layer / plan.tp if plan.sequence_parallel else (10 + 24 / plan.tp) / 34 * per_layer
    layers = m.n_layer / plan.pp
    in_flight = min(plan.pp, max(1, m.gradient_accum)) if plan.pp > 1 else 1     # 1F1B keeps pp micro-batches alive
    acts = per_layer * layers * in_flight
    logits = s * b * (m.vocab / plan.tp) * (dt.activation_elem_bytes + 4)
    total = params + grads + optim + acts + logits
    return {"params": params, "grads": grads, "optimizer": optim, "activations": acts, "logits": logits,
            "static": params + grads + optim, "total": total}


@dataclass
class Cluster:
    gpus: int = 8
    gpus_per_node: int = 8
    mem_gib: float = 180.0
    peak_tflops: float = 1390.0     # sustained cuBLAS BF16 on a B200 under the power cap
    intra_gbps: float = 725.0       # all-reduce bus bandwidth over NVLink 5 / NVSwitch
    inter_gbps: float = 50.0
    mfu: float = 0.55
    dp_overlap: float = 0.7
    reserve_gib: float = 4.0


def step_time(m: ModelShape, plan: Plan, cl: Cluster, dt: DTypePlan = DTypePlan()) -> dict:
    tokens = m.micro_batch * m.seq_len * m.gradient_accum * plan.dp
    model_flops = flops_per_token(m) * tokens
    gpus = plan.dp * plan.tp * plan.pp * plan.cp
    recompute = 4.0 / 3.0 if plan.full_recompute else 1.0
    compute = model_flops * recompute / (gpus * cl.peak_tflops * 1e12 * cl.mfu)
    def bw(group: int) -> float:
        return (cl.intra_gbps if group <= cl.gpus_per_node else cl.inter_gbps) * 1e9
    per_rank_tokens = m.micro_batch * m.seq_len / plan.cp * m.gradient_accum
    tp_comm = 0.0
    if plan.tp > 1:   # 4 all-reduces (or AG+RS pairs) of [tokens, h] per layer per direction
        vol = 4 * 2 * (m.n_layer / plan.pp) * per_rank_tokens * m.d_model * dt.activation_elem_bytes
        tp_comm = vol * 2 * (plan.tp - 1) / plan.tp / bw(plan.tp)
    cp_comm = 0.0
    if plan.cp > 1:   # K/V blocks travel around the ring once per layer, forward and backward
        kv = 2 * per_rank_tokens * (m.d_model * m.n_kv_head / m.n_head) * dt.activation_elem_bytes
        cp_comm = 0.3 * 3 * (m.n_layer / plan.pp) * kv * (plan.cp - 1) / bw(plan.tp * plan.cp)
    dp_comm = 0.0
    if plan.dp > 1:
        n = param_breakdown(m)["total"] / (plan.tp * plan.pp)
        vol = n * dt.grad_bytes * 2 * (plan.dp - 1) / plan.dp + (n * dt.param_bytes if plan.zero_stage >= 3 else 0)
        dp_comm = (1 - cl.dp_overlap) * vol / bw(gpus)
    bubble = (plan.pp - 1) / (m.gradient_accum + plan.pp - 1) if plan.pp > 1 else 0.0
    step = (compute + tp_comm + cp_comm) / (1 - bubble) + dp_comm
    return {"tokens": tokens, "model_flops": model_flops, "compute_s": compute, "tp_comm_s": tp_comm, "cp_comm_s": cp_comm,
            "dp_comm_s": dp_comm, "bubble": bubble, "step_s": step, "tokens_per_s": tokens / step,
            "mfu": model_flops / (step * gpus * cl.peak_tflops * 1e12)}


@dataclass
class AutoOptions:
    global_batch: int = 512        # sequences per optimizer step
    max_tp: int = 8
    max_pp: int = 8
    max_cp: int = 8
    top: int = 3
    micro_batches: tuple = (1, 2, 4, 8)


@dataclass
class Candidate:
    dp: int = 1
    tp: int = 1
    pp: int = 1
    cp: int = 1
    zero: int = 0
    micro_batch: int = 1
    accum: int = 1
    memory_gib: float = 0.0
    static_gib: float = 0.0
    activation_gib: float = 0.0
    logits_gib: float = 0.0
    compute_s: float = 0.0
    tp_comm_s: float = 0.0
    cp_comm_s: float = 0.0
    dp_comm_s: float = 0.0
    bubble: float = 0.0
    step_s: float = 0.0
    mfu: float = 0.0
    fits: bool = False
    recompute: bool = False


def evaluate(m: ModelShape, cl: Cluster, dp, tp, pp, cp, zero, micro, accum, recompute=False,
             dt: DTypePlan = DTypePlan()) -> Candidate:
    shape = ModelShape(**{**asdict(m), "micro_batch": micro, "gradient_accum": accum})
    plan = Plan(dp, tp, pp, cp, zero, recompute)
    mem = memory_bytes(shape, dt, plan)
    t = step_time(shape, plan, cl, dt)
    gib = 1 << 30
    c = Candidate(dp, tp, pp, cp, zero, micro, accum, mem["total"] / gib, mem["static"] / gib, mem["activations"] / gib,
                  mem["logits"] / gib, t["compute_s"], t["tp_comm_s"], t["cp_comm_s"], t["dp_comm_s"], t["bubble"],
                  t["step_s"], t["mfu"], recompute=recompute)
    c.fits = c.memory_gib + cl.reserve_gib <= cl.mem_gib
    return c


def auto_parallel(m: ModelShape, cl: Cluster, opt: AutoOptions = AutoOptions()) -> dict:
    """Exhaustive search over factorizations of the GPU count; ranks the layouts that fit by step time."""
    def divisors(n):
        return [i for i in range(1, n + 1) if n % i == 0]
    cands: List[Candidate] = []
    tried = 0
    for tp in [t for t in divisors(cl.gpus) if t <= opt.max_tp and m.n_head % t == 0 and t <= cl.gpus_per_node]:
        for pp in [p for p in divisors(cl.gpus // tp) if p <= opt.max_pp and m.n_layer % p == 0]:
            for cp in [c for c in divisors(cl.gpus // (tp * pp)) if c <= opt.max_cp and m.seq_len % (2 * c) == 0]:
                dp = cl.gpus // (tp * pp * cp)
                if opt.global_batch % dp:
                    continue
                per_dp = opt.global_batch // dp
                for micro in opt.micro_batches:
                    if per_dp % micro:
                        continue
                    accum = per_dp // micro
                    for zero in ((0, 1, 2, 3) if dp > 1 else (0,)):
                        for rec in (False, True):
                            tried += 1
                            c = evaluate(m, cl, dp, tp, pp, cp, zero, micro, accum, rec)
                            if c.fits:
                                cands.append(c)
    cands.sort(key=lambda c: (c.step_s, c.tp * c.pp * c.cp, c.zero))
    return {"tried": tried, "feasible": len(cands), "best": [asdict(c) for c in cands[: opt.top]]}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="nexus_estimate")
    ap.add_argument("--preset", default="gpt2-124m")
    ap.add_argument("--config", default="", help="path of an LmConfig JSON (overrides --preset)")
    ap.add_argument("--batch", type=int, default=1, help="micro batch (sequences)")
    ap.add_argument("--seq", type=int, default=0)
    ap.add_argument("--accum", type=int, default=1)
    ap.add_argument("--dp", type=int, default=1)
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--pp", type=int, default=1)
    ap.add_argument("--cp", type=int, default=1)
    ap.add_argument("--zero", type=int, default=0)
    ap.add_argument("--recompute", action="store_true")
    ap.add_argument("--auto-parallel", action="store_true")
    ap.add_argument("--gpus", type=int, default=8)
    ap.add_argument("--gpus-per-node", type=int, default=8)
    ap.add_argument("--mem-gib", type=float, default=180.0)
    ap.add_argument("--global-batch", type=int, default=512)
    ap.add_argument("--json", action="store_true")
    a = ap.parse_args(argv)
    from ..lm import config as C
    cfg = C.load_json(a.config) if a.config and hasattr(C, "load_json") else C.preset(a.preset)
    m = ModelShape.from_config(cfg, a.seq or None, a.batch)
    m.gradient_accum = a.accum
    cl = Cluster(gpus=a.gpus, gpus_per_node=a.gpus_per_node, mem_gib=a.mem_gib)
    out = {"model": cfg.name, "params": param_breakdown(m), "flops_per_token": flops_per_token(m)}
    if a.auto_parallel:
        out["auto_parallel"] = auto_parallel(m, cl, AutoOptions(global_batch=a.global_batch))
    else:
        plan = Plan(a.dp, a.tp, a.pp, a.cp, a.zero, a.recompute)
        out["memory_gib"] = {k: v / (1 << 30) for k, v in memory_bytes(m, DTypePlan(), plan).items()}
        out["time"] = step_time(m, plan, cl)
    if a.json:
        print(json.dumps(out, indent=1))
    else:
        print(f"{out['model']}: {out['params']['total']:,} parameters, {out['flops_per_token'] / 1e9:.3f} GFLOP/token (training)")
        if a.auto_parallel:
            r = out["auto_parallel"]
            print(f"auto-parallel on {a.gpus} GPUs: {r['feasible']} of {r['tried']} layouts fit in {a.mem_gib} GiB")
            for c in r["best"]:
                print(f"  dp{c['dp']} tp{c['tp']} pp{c['pp']} cp{c['cp']} zero{c['zero']} mb{c['micro_batch']}x{c['accum']}"
                      f"{' recompute' if c['recompute'] else ''}: {c['memory_gib']:.1f} GiB, {c['step_s'] * 1e3:.1f} ms/step, MFU {c['mfu']:.2f}")
        else:
            mem, t = out["memory_gib"], out["time"]
            print(f"memory per GPU: {mem['total']:.2f} GiB (static {mem['static']:.2f}, activations {mem['activations']:.2f}, logits {mem['logits']:.2f})")
            print(f"step: {t['step_s'] * 1e3:.2f} ms, {t['tokens_per_s']:,.0f} tokens/s, MFU {t['mfu']:.2f}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
