"""Benchmark evidence harness: every case is sampled in several fresh processes (each does its own warm-up
and timed samples), the verdict uses the median over all samples, a case whose coefficient of variation
exceeds 10 % gets no verdict, a median more than 3 % slower than the stored baseline is a regression, and
the record carries SHA-256 digests of the sources and built binaries it was produced from.  Workers are
started in their own process group and the group is terminated when the harness exits.

    python -m nexus_b200.bench --matrix kernels|train|all [--processes 5 --warmup 2 --samples 7] --out evidence.json
    python -m nexus_b200.bench report evidence.json

Parity: python/src/nexus_bench/{cli,evidence,workers,windows_job}.py of the reference."""
from __future__ import annotations

import argparse
import json
import os
import signal
import statistics
import subprocess
import sys
import time
from pathlib import Path
from typing import Dict, List, Optional

ROOT = Path(__file__).resolve().parents[2]
CV_LIMIT, REGRESSION = 0.10, 0.03


def digests() -> Dict[str, str]:
    from .. import _native
    out = {}
    pkg = ROOT / "nexus_b200"
    for pat in ("csrc/cuda/*.cu", "csrc/cuda/*.cuh", "csrc/cuda/*.h", "csrc/host/*.cpp", "lib/*.so", "*.so"):
        for f in sorted(pkg.glob(pat)):
            out[str(f.relative_to(ROOT))] = _native.sha256_file(str(f))
    for f in (ROOT / "bench.py",):
        if f.exists():
            out[f.name] = _native.sha256_file(str(f))
    return out


def run_worker(cmd: List[str], timeout_s: float = 1800.0) -> dict:
    """Runs one worker in its own process group; its last stdout line must be JSON."""
    p = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, start_new_session=True,
                         env=dict(os.environ, PYTHONPATH=str(ROOT)))
    try:
        out, err = p.communicate(timeout=timeout_s)
    except subprocess.TimeoutExpired:
        os.killpg(p.pid, signal.SIGTERM)
        p.wait(10)
        raise
    if p.returncode != 0:
        raise RuntimeError(f"worker {' '.join(cmd)} exited {p.returncode}: {err[-400:]}")
    return json.loads(out.strip().splitlines()[-1])


def summarise(samples: List[float], higher_is_better: bool, baseline: Optional[float]) -> dict:
    med = statistics.median(samples)
    cv = statistics.pstdev(samples) / med if med else float("inf")
    verdict = "ok"
    if cv > CV_LIMIT:
        verdict = "no-verdict (cv > 10 %)"
    elif baseline:
        worse = (baseline - med) / baseline if higher_is_better else (med - baseline) / baseline
        if worse > REGRESSION:
            verdict = f"regression ({worse * 100:.1f} % worse than baseline)"
    return {"median": med, "min": min(samples), "max": max(samples), "cv": cv, "samples": len(samples), "verdict": verdict,
            "baseline": baseline}


def sample_case(name: str, cmd: List[str], key: str, processes: int, higher_is_better: bool,
                baseline: Optional[float]) -> dict:
    vals: List[float] = []
    for _ in range(processes):
        rec = run_worker(cmd)
        got = rec[key] if isinstance(rec, dict) else rec
        vals.extend(got if isinstance(got, list) else [got])
    return {"case": name, "metric": key, "higher_is_better": higher_is_better, **summarise(vals, higher_is_better, baseline)}


def matrix_cases(which: str, warmup: int, samples: int) -> List[dict]:
    py = sys.executable
    cases = []
    if which in ("train", "all"):
        cases.append({"name": "gpt2-124m train step", "key": "value", "hib": True,
                      "cmd": [py, str(ROOT / "bench.py"), "--steps", str(samples), "--warmup", str(max(3, warmup)), "--skip-e2e"]})
    if which in ("kernels", "all"):
        cases.append({"name": "kernels", "key": None, "hib": False,
                      "cmd": [py, "-m", "nexus_b200.bench.kernels", "--iters", str(samples), "--warmup", str(max(1, warmup)),
                              "--json", "/dev/stdout"]})
    return cases


def run_matrix(which: str, processes: int, warmup: int, samples: int, baseline_file: Optional[str]) -> dict:
    base = {}
    if baseline_file and os.path.exists(baseline_file):
        with open(baseline_file) as f:
            base = {r["case"]: r["median"] for r in json.load(f)["results"]}
    results = []
    for c in matrix_cases(which, warmup, samples):
        if c["key"] is not None:
            results.append(sample_case(c["name"], c["cmd"], c["key"], processes, c["hib"], base.get(c["name"])))
            continue
        per_case: Dict[str, List[float]] = {}
        for _ in range(processes):                    # kernel table: one row per kernel case
            p = subprocess.run(c["cmd"][:-2] + ["--json", "/tmp/nexus_kernels.json"], capture_output=True, text=True,
                               env=dict(os.environ, PYTHONPATH=str(ROOT)), start_new_session=True)
            if p.returncode != 0:
                raise RuntimeError(p.stderr[-400:])
            for row in json.load(open("/tmp/nexus_kernels.json")):
                per_case.setdefault(row["case"], []).append(row["ms_median"])
        for k, v in per_case.items():
            results.append({"case": k, "metric": "ms_median", "higher_is_better": False, **summarise(v, False, base.get(k))})
    return {"when": time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime()), "matrix": which, "processes": processes,
            "warmup": warmup, "samples": samples, "digests": digests(), "results": results}


def report(evidence: dict) -> str:
    lines = [f"# benchmark evidence ({evidence['matrix']}, {evidence['when']})", "",
             f"{evidence['processes']} processes x {evidence['warmup']} warm-up x {evidence['samples']} samples; "
             f"{len(evidence['digests'])} files hashed", "", "| case | median | cv | verdict |", "|---|---|---|---|"]
    for r in evidence["results"]:
        lines.append(f"| {r['case']} | {r['median']:.4g} | {r['cv'] * 100:.1f} % | {r['verdict']} |")
    return "\n".join(lines)


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if argv and argv[0] == "report":
        with open(argv[1]) as f:
            print(report(json.load(f)))
        return 0
    ap = argparse.ArgumentParser(prog="nexus bench")
    ap.add_argument("--matrix", default="kernels", choices=["kernels", "train", "all"])
    ap.add_argument("--processes", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--samples", type=int, default=7)
    ap.add_argument("--baseline", default="")
    ap.add_argument("--out", default="evidence.json")
    a = ap.parse_args(argv)
    ev = run_matrix(a.matrix, a.processes, a.warmup, a.samples, a.baseline or None)
    with open(a.out, "w") as f:
        json.dump(ev, f, indent=1)
    print(report(ev))
    return 1 if any(r["verdict"].startswith("regression") for r in ev["results"]) else 0


if __name__ == "__main__":
    sys.exit(main())
