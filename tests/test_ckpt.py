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
    assert open(tmp_path / "latest").read() == "8"          # the bare step number, as the reference writes it
    got = m.load_latest()
    assert got.step == 8 and got.backend_blobs == [b"blob8"] and got.state["train_cursor"] == 80 and not got.resharded
    # the manifest records the archive's own trailer (digest of everything before the last 32 bytes)
    man = json.load(open(tmp_path / "step-000000008" / "manifest.json"))
    raw = (tmp_path / "step-000000008" / "rank0.nxs3").read_bytes()
    assert man["files"][0]["sha256"] == raw[-32:].hex() == __import__("hashlib").sha256(raw[:-32]).hexdigest()
    assert man["files"][0]["bytes"] == len(raw) and man["state"]["step"] == 8
    # damage the newest checkpoint: the loader warns and falls back to the previous one, or raises when asked to
    f = tmp_path / "step-000000008" / "rank0.nxs3"
    data = bytearray(f.read_bytes())
    data[30] ^= 0xFF
    f.write_bytes(bytes(data))
    with pytest.warns(RuntimeWarning, match="failed verification"):
        assert m.load_latest().step == 6
    with pytest.raises(CheckpointError, match="newest checkpoint"):
        m.load_latest(fallback=False)
    with pytest.raises(CheckpointError):
        m.load(8)


def test_trainer_state_uses_the_reference_byte_layout():
    from nexus_b200.ckpt import TrainerState
    st = TrainerState(step=7, epoch=1, global_sample_index=99, train_cursor="abc", val_cursor="", lr_factor=0.5,
                      schedule_step=7, loss_scale=1024.0, rng_seed=42, rng_offset=3, accum_counter=0, accum_steps=4,
                      micro_batch=8, seq_len=1024, global_batch_tokens=32768, rollbacks=2, world=2, rank=1)
    raw = st.encode()
    # u32 schema | i64 step | i64 epoch | u64 samples | u64 len + bytes (x2) | f64 | i64 | f64 | u64 | u64 | 4 x i32 | i64 | 3 x i32
    assert len(raw) == 4 + 8 + 8 + 8 + (8 + 3) + 8 + 8 + 8 + 8 + 8 + 8 + 16 + 8 + 12
    assert raw[:4] == b"\x01\0\0\0" and raw[4:12] == (7).to_bytes(8, "little") and raw[36:39] == b"abc"
    assert TrainerState.decode(raw) == st
    with pytest.raises(CheckpointError):
        TrainerState.decode(raw[:-5])


def test_world_size_change_is_reported(tmp_path):
    import threading
    ms = [CheckpointManager(CheckpointOptions(str(tmp_path)), rank=r, world=2) for r in range(2)]
    ts = [threading.Thread(target=ms[r].save, args=(5, {"x": r}, b"r%d" % r, "fsdp:3:2")) for r in (1, 0)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    got = CheckpointManager(CheckpointOptions(str(tmp_path)), rank=0, world=1).load_latest()
    assert got.resharded and got.world == 2 and got.backend_blobs == [b"r0", b"r1"] and got.layout == "fsdp:3:2"
    assert got.state["x"] == 0    # keys the fixed record does not know travel in the side entry
    same = CheckpointManager(CheckpointOptions(str(tmp_path)), rank=1, world=2).load_latest()
    assert not same.resharded and same.backend_blobs == [None, b"r1"] and same.state["rank"] == 1


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
