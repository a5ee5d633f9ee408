"""nexus-run launcher: environment, failure handling with a grace period, elastic restart with resharding.
Every failure is made on the host (a rank exits between steps); the ranks are gloo processes on the CPU."""
import json
import os
import subprocess
import sys
import time

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def launcher():
    sys.path.insert(0, ROOT)
    from nexus_b200 import _build
    return str(_build.build_tools()[0])


def test_environment_and_exit_code_table(launcher, tmp_path):
    prog = ("import os, sys; open(os.path.join(%r, 'r' + os.environ['RANK']), 'w').write(' '.join(os.environ[k] for k in "
            "('RANK','LOCAL_RANK','WORLD_SIZE','LOCAL_WORLD_SIZE','GROUP_RANK','MASTER_ADDR','MASTER_PORT','NEXUS_RUN','NEXUS_RESTART_COUNT')))"
            % str(tmp_path))
    r = subprocess.run([launcher, "--nproc-per-node", "3", "--master-port", "29811", "--", sys.executable, "-c", prog],
                       capture_output=True, text=True, timeout=60)
    assert r.returncode == 0, r.stderr
    assert "[rank 0: 0] [rank 1: 0] [rank 2: 0]" in r.stderr
    assert open(tmp_path / "r2").read() == "2 2 3 3 0 127.0.0.1 29811 1 0"
    bad = subprocess.run([launcher, "--nproc-per-node", "0", "--", "true"], capture_output=True, text=True)
    assert bad.returncode == 2 and "usage" in bad.stderr
    missing = subprocess.run([launcher, "--", "/no/such/program"], capture_output=True, text=True, timeout=30)
    assert missing.returncode == 127


def test_failure_ends_the_group_after_the_grace_period(launcher):
    prog = "import os, sys, time; r = int(os.environ['RANK']); sys.exit(3) if r == 1 else time.sleep(60)"
    t0 = time.time()
    r = subprocess.run([launcher, "--nproc-per-node", "3", "--grace-s", "0.5", "--", sys.executable, "-c", prog],
                       capture_output=True, text=True, timeout=60)
    assert r.returncode == 3 and time.time() - t0 < 20
    assert "[rank 1: 3]" in r.stderr and "[rank 0: 143]" in r.stderr       # 128 + SIGTERM


def test_elastic_restart_resumes_with_fewer_ranks(launcher, tmp_path):
    env = dict(os.environ, CKPT_DIR=str(tmp_path), TOTAL_STEPS="8", FAIL_RANK="3", FAIL_STEP="5", PYTHONPATH=ROOT)
    r = subprocess.run([launcher, "--nproc-per-node", "4", "--master-port", "29831", "--max-restarts", "1",
                        "--restart-nproc", "2", "--", sys.executable, os.path.join(ROOT, "tests", "workers", "elastic_worker.py")],
                       capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0, r.stderr[-3000:]
    assert "[rank 3: 9]" in r.stderr and "restarting the group with 2 process(es)" in r.stderr
    res = json.load(open(tmp_path / "result.json"))
    assert res["world"] == 2 and res["attempt"] == 1 and res["resumed"]
    assert res["start_step"] == 4 and res["final_step"] == 8        # newest complete checkpoint before the failure
    assert all(l == l and l < 6.0 for l in res["losses"])
