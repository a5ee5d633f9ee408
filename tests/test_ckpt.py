import json
import os
import subprocess
import sys

import pytest

from nexus_b200 import _native
from nexus_b200.ckpt import CheckpointError, CheckpointManager, CheckpointOptions

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_sha256_known_vectors():
    assert _native.sha256_hex(b"") == "e3b0c44298fc1c149afbf4c8996fb92427ae41e4649b934ca495991b7852b855"
    assert _native.sha256_hex(b"abc") == "ba7816bf8f01cfea414140de5dae2223b00361a396177a9cb410ff61f20015ad"
    assert _native.sha256_hex(b"a" * 1000) == __import__("hashlib").sha256(b"a" * 1000).hexdigest()


def test_nxs3_archive_detects_corruption():
    blob = _native.nxs3_encode([("state", b"123"), ("backend", b"4567")])
    assert blob[:8] == b"NXS3\0\0\0\0" and dict(_native.nxs3_decode(blob))["backend"] == b"4567"
    bad = bytearray(blob)
    bad[20] ^= 1
    with pytest.raises(RuntimeError, match="checksum"):
        _native.nxs3_decode(bytes(bad))


@pytest.mark.parametrize("asynchronous", (False, True))
def test_save_load_prune(tmp_path, asynchronous):
    m = CheckpointManager(CheckpointOptions(str(tmp_path), every=2, keep=2, asynchronous=asynchronous))
    assert m.due(4) and not m.due(3)
    for step in (2, 4, 6, 8):
        m.save(step, {"lr_factor": 1.0, "train_cursor": step * 10}, b"blob%d" % step)
    m.wait()
    assert m.list_steps() == [6, 8]
    assert open(tmp_path / "latest").read() == "step-000000008"
    got = m.load_latest()
    assert got.step == 8 and got.backend_blobs == [b"blob8"] and got.state["train_cursor"] == 80 and not got.resharded
    # damage the newest checkpoint: the loader falls back to the previous one
    f = tmp_path / "step-000000008" / "rank0.nxs3"
    data = bytearray(f.read_bytes())
    data[30] ^= 0xFF
    f.write_bytes(bytes(data))
    assert m.load_latest().step == 6
    with pytest.raises(CheckpointError):
        m.load(8)


def test_world_size_change_is_reported(tmp_path):
    import threading
    ms = [CheckpointManager(CheckpointOptions(str(tmp_path)), rank=r, world=2) for r in range(2)]
    ts = [threading.Thread(target=ms[r].save, args=(5, {"x": r}, b"r%d" % r, "fsdp:3:2")) for r in (1, 0)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    got = CheckpointManager(CheckpointOptions(str(tmp_path)), rank=0, world=1).load_latest()
    assert got.resharded and got.world == 2 and got.backend_blobs == [b"r0", b"r1"] and got.layout == "fsdp:3:2"


@pytest.mark.parametrize("point", ("rank_file", "before_manifest", "before_rename"))
def test_crash_injection_keeps_last_good_checkpoint(tmp_path, point):
    code = ("import sys; sys.path.insert(0, %r)\n"
            "from nexus_b200.ckpt import CheckpointManager, CheckpointOptions\n"
            "m = CheckpointManager(CheckpointOptions(%r))\n"
            "m.save(1, {}, b'good')\nm.save(2, {}, b'new')\n") % (ROOT, str(tmp_path))
    env = dict(os.environ, NEXUS_CKPT_CRASH=point, NEXUS_CKPT_CRASH_STEP="2")
    r = subprocess.run([sys.executable, "-c", code], env=env)
    assert r.returncode == 86
    m = CheckpointManager(CheckpointOptions(str(tmp_path)))
    got = m.load_latest()
    assert got.step == 1 and got.backend_blobs == [b"good"]
    assert not any(n.startswith(".tmp-") for n in os.listdir(tmp_path))
