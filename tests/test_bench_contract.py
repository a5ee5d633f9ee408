"""`bench.py` as the outside world calls it, as far as that goes without a GPU: the reference arm answers with one JSON
line and exit code 0 where it cannot run (more than one GPU: the reference's multi-GPU trainer does not build offline;
no CUDA device), and the argument contract (`--gpus --steps --warmup --impl`) parses."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*args):
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True,
                       timeout=300, cwd=ROOT)
    lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
    return r.returncode, (json.loads(lines[-1]) if lines else None), r.stderr


def test_reference_arm_says_unavailable_for_more_than_one_gpu():
    rc, line, err = _run("--impl", "reference", "--gpus", "2", "--steps", "2", "--warmup", "1")
    assert rc == 0, err[-1000:]
    assert line["impl"] == "reference" and "unavailable" in line and "multi-GPU" in line["unavailable"]


def test_reference_arm_without_a_device_answers_in_one_line():
    import torch
    if torch.cuda.is_available():
        import pytest
        pytest.skip("a CUDA device is present: the reference arm would run")
    rc, line, err = _run("--impl", "reference", "--steps", "2", "--warmup", "1")
    assert rc == 0, err[-1000:]
    assert line["impl"] == "reference" and "unavailable" in line


def test_help_names_the_contract_flags():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--help"], capture_output=True, text=True,
                       timeout=120, cwd=ROOT)
    assert r.returncode == 0
    for flag in ("--gpus", "--steps", "--warmup", "--impl"):
        assert flag in r.stdout
