"""`nexus_estimate`: analytic parameter counts, memory, FLOPs and roofline time of an LM training step, and
an `--auto-parallel` search over (dp, tp, pp, cp, zero, micro batch) under a per-GPU memory limit.

Memory model: static = params + grads + optimizer (+ FP32 master), each divided by TP x PP and, per ZeRO
stage, by DP (stage 1: optimizer; 2: + grads; 3: + params); activations per layer =
``s*b*h*(34 + 5*a*s/h)`` bytes (16-bit activations, no flash) or ``34*s*b*h`` with flash attention, divided
by TP (with sequence parallelism) and CP, 2*s*b*h per layer with full recomputation; logits = s*b*V*(2+4).
Time model: compute = 6*N*tokens (+ attention) / (peak * mfu); TP / CP / DP communication from ring
volumes over the intra- or inter-node bandwidth; pipeline bubble (pp-1)/(m+pp-1).
Defaults describe an 8-GPU B200 node (180 GB, measured cuBLAS BF16 rate, NVLink 5 bus bandwidth).
The arithmetic and the search run in the native host module (`csrc/host/estimate.cpp`); this file holds the
dataclasses and the command line.

    python -m nexus_b200.tools.estimate --preset gpt2-124m --batch 16 --seq 1024 [--auto-parallel --gpus 8]

Parity: tools/nexus_estimate/{estimate,autoparallel}.{hpp,cpp}, main.cpp of the reference."""
from __future__ import annotations

import argparse
import json
import sys
from dataclasses import asdict, dataclass, field
from typing import Optional


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


def _core():
    from .. import _native
    return _native


def param_breakdown(m: ModelShape) -> dict:
    return dict(_core().estimate_params(asdict(m)))


def flops_per_token(m: ModelShape, causal: bool = True) -> float:
    """Training FLOPs per token: 6 per matrix parameter plus the attention score / value products."""
    return float(_core().estimate_flops_per_token(asdict(m), causal))


def memory_bytes(m: ModelShape, dt: DTypePlan, plan: Plan) -> dict:
    return dict(_core().estimate_memory(asdict(m), asdict(dt), asdict(plan)))


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
    return dict(_core().estimate_step_time(asdict(m), asdict(plan), asdict(cl), asdict(dt)))


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
    return Candidate(**_core().estimate_evaluate(asdict(m), asdict(cl), dp, tp, pp, cp, zero, micro, accum, bool(recompute),
                                                 asdict(dt)))


def auto_parallel(m: ModelShape, cl: Cluster, opt: AutoOptions = AutoOptions(), dt: DTypePlan = DTypePlan()) -> dict:
    """Exhaustive search over factorizations of the GPU count; ranks the layouts that fit by step time."""
    r = _core().estimate_auto_parallel(asdict(m), asdict(cl), opt.global_batch, opt.max_tp, opt.max_pp, opt.max_cp, opt.top,
                                       [int(x) for x in opt.micro_batches], asdict(dt))
    return {"tried": int(r["tried"]), "feasible": int(r["feasible"]), "best": [dict(c) for c in r["best"]]}


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
