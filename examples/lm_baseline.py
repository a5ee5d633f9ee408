"""Small language-model baseline with honest measurement.

    python examples/lm_baseline.py [--config cfg.json] [--json out.json] [--trace trace.json]

What it measures and what it does not invent:
* step times are wall-clock `ScopedTimer` records around each optimizer step (CUDA synchronised when on a GPU);
* the parameter count is counted from `model.parameters()`; the closed-form estimate is reported beside it;
* MFU is computed only when the config gives the device peak (`device.peak_tflops`), otherwise it is null;
* process peak memory is VmHWM from /proc (null where that is not available); the ledger counts only what went
  through the framework's memory gate.
Counterpart of apps/lm_baseline of the reference.
"""
import argparse
import json
import os
import statistics
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from nexus_b200 import prof  # noqa: E402
from nexus_b200.lm import LanguageModel, preset  # noqa: E402
from nexus_b200.tools import estimate  # noqa: E402
from nexus_b200.train import AdamW, LanguageTrainerBuilder, SyntheticTokens  # noqa: E402

DEFAULT = {"preset": "nano", "steps": 8, "micro_batch": 4, "seq_len": 64, "lr": 3e-4, "device": {"name": "cpu"}}


def peak_rss_bytes():
    try:
        with open("/proc/self/status") as f:
            for line in f:
                if line.startswith("VmHWM:"):
                    return int(line.split()[1]) * 1024
    except OSError:
        pass
    return None


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--config")
    ap.add_argument("--json")
    ap.add_argument("--trace")
    args = ap.parse_args(argv)
    conf = dict(DEFAULT)
    if args.config:
        with open(args.config) as f:
            conf.update(json.load(f))
    cfg = preset(conf["preset"])
    for k, v in conf.get("model", {}).items():
        setattr(cfg, k, v)
    device = conf["device"].get("name", "cpu")
    model = LanguageModel(cfg)
    prof.enable(True)
    prof.clear()
    trainer = (LanguageTrainerBuilder(model).data(SyntheticTokens(cfg.vocab_size, seed=1))
               .optimizer(AdamW(lr=conf["lr"])).micro_batch(conf["micro_batch"]).seq_len(conf["seq_len"])
               .global_batch_tokens(conf["micro_batch"] * conf["seq_len"])
               .precision("bf16" if device.startswith("cuda") else "f32", "fp32").execution_policy(device)
               .log_every(0).build())
    times = []
    for step in range(conf["steps"]):
        with prof.ScopedTimer("train_step", "step", sync_cuda=device.startswith("cuda")) as t:
            trainer.train(1)
        times.append((prof.now_ns() - t.t0) * 1e-9)
    steady = times[1:] or times
    tokens = conf["micro_batch"] * conf["seq_len"]
    counted = sum(p.numel() for p in model.parameters())
    shape = estimate.ModelShape.from_config(cfg, conf["seq_len"], conf["micro_batch"])
    formula = estimate.param_breakdown(shape)["total"]
    flops_step = 3.0 * estimate.flops_per_token(shape) * tokens          # forward + backward
    peak = conf["device"].get("peak_tflops")
    median = statistics.median(steady)
    report = {
        "preset": conf["preset"], "device": device, "steps": conf["steps"], "tokens_per_step": tokens,
        "params_counted": counted, "params_formula": formula,
        "step_seconds_median": median, "step_seconds_first": times[0], "tokens_per_second": tokens / median,
        "model_flops_per_step": flops_step,
        "mfu": (flops_step / median / (peak * 1e12)) if peak else None,
        "final_loss": trainer.history[-1].loss, "peak_rss_bytes": peak_rss_bytes(),
        "ledger": prof.MemoryLedger.report(), "timers": prof.totals(),
    }
    text = json.dumps(report, indent=1, default=float)
    if args.json:
        with open(args.json, "w") as f:
            f.write(text)
    if args.trace:
        prof.dump_chrome_trace(args.trace)
    print(json.dumps({k: report[k] for k in ("params_counted", "params_formula", "step_seconds_median",
                                             "tokens_per_second", "mfu", "final_loss")}, default=float))
    return 0 if torch.isfinite(torch.tensor(report["final_loss"])) else 1


if __name__ == "__main__":
    sys.exit(main())
