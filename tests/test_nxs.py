import os
import struct

import numpy as np
import pytest
import torch

from nexus_b200 import _native, fnstore, nn, nxs
from nexus_b200.lm import LanguageModel, preset


def test_byte_layout_of_a_small_archive():
    arch = {"layers": [{"type": 1, "name": "fc", "attrs": [("in", 1, 4), ("bias", 3, True)], "children": []}],
            "weights": [("0", [2], np.array([1.5, -2.0], dtype=np.float32))]}
    b = _native.nxs2_encode(arch)
    exp = b"NXS2" + struct.pack("<HH", 1, 0) + struct.pack("<I", 1)
    exp += struct.pack("<H", 1) + struct.pack("<I", 2) + b"fc" + struct.pack("<I", 2)
    exp += bytes([1]) + struct.pack("<I", 2) + b"in" + struct.pack("<i", 4)
    exp += bytes([3]) + struct.pack("<I", 4) + b"bias" + bytes([1])
    exp += struct.pack("<I", 0)
    exp += struct.pack("<I", 1) + struct.pack("<I", 1) + b"0" + struct.pack("<I", 1) + struct.pack("<Q", 2)
    exp += struct.pack("<Q", 2) + struct.pack("<ff", 1.5, -2.0)
    assert b == exp


def test_sections_round_trip():
    arch = {"layers": [], "weights": [],
            "optim": {"algorithm": "adamw", "step": 7, "lr": [1e-3, 2e-3], "blobs": [b"abc", b""], "scalars": [0.9]},
            "trainer": {"epoch": 2, "global_step": 9, "loss": 0.25, "best": 0.2, "stop": True, "metrics": [("acc", 0.5)]},
            "rl": {"kind": "ppo", "config": [("gamma", 2, 0.99), ("name", 4, "x")],
                   "nets": [{"name": "pi", "sizes": [4, 8, 2], "adam_step": 3, "parameters": np.ones(5, np.float32),
                             "moments": np.zeros(10, np.float32)}], "elos": [1000.0], "player_weights": [np.ones(3, np.float32)]},
            "python": b"payload"}
    d = _native.nxs2_decode(_native.nxs2_encode(arch))
    assert d["optim"]["step"] == 7 and d["optim"]["blobs"] == [b"abc", b""]
    assert d["trainer"]["stop"] is True and d["trainer"]["metrics"] == [("acc", 0.5)]
    assert d["rl"]["kind"] == "ppo" and d["rl"]["nets"][0]["sizes"] == [4, 8, 2] and d["python"] == b"payload"
    flags = struct.unpack_from("<H", _native.nxs2_encode(arch), 6)[0]
    assert flags == 1 | 2 | 4 | 8


def test_model_round_trips(tmp_path):
    fnstore.register_python_activation("cube_t", lambda x: x * x * x)
    m = nn.Sequential().add(nn.Linear(4, 8, True)).add(nn.Activation("cube_t")).add(nn.BatchNorm1d(8)) \
        .add(nn.Residual(nn.Linear(8, 8))).add(nn.Linear(8, 2, True))
    m.eval()
    x = torch.randn(5, 4)
    p = str(tmp_path / "m.nxs")
    m.save_nxs(p)
    m2 = nn.Sequential.load_nxs(p)
    m2.eval()
    assert torch.equal(m2(x), m(x))
    g = nn.Graph().add("a", nn.Linear(4, 4)).add("b", nn.Linear(4, 4), ["input"]).add("c", nn.Linear(8, 2), ["a", "b"], True)
    g.save_nxs(p)
    assert torch.equal(nn.Graph.load_nxs(p)(x), g(x))
    lm = LanguageModel(preset("nano"))
    lm.save_nxs(p)
    t = torch.randint(0, 256, (2, 16))
    assert torch.equal(LanguageModel.load_nxs(p).loss(t), lm.loss(t))


def test_python_payload_is_an_nxpy_record_stream_and_survives_a_fresh_process(tmp_path):
    """Byte layout of the python payload (kind / name / marshal code / typed closure cells), closure restrictions,
    and a load in a process that never saw the defining code."""
    import subprocess
    import sys
    scale, shift, flag = 2.5, 3, True

    def squish(x):
        return x * scale + shift if flag else x

    fnstore.register_python_activation("squish_t", squish)
    m = nn.Sequential().add(nn.Linear(3, 3)).add(nn.Activation("squish_t"))
    blob = fnstore.payload_for(m)
    assert blob[:4] == b"NXPY" and struct.unpack_from("<HI", blob, 4) == (1, 1)
    assert blob[10] == 1 and struct.unpack_from("<I", blob, 11)[0] == len("squish_t") and blob[15:23] == b"squish_t"
    (code_len,) = struct.unpack_from("<I", blob, 23)
    cells_at = 27 + code_len
    assert struct.unpack_from("<I", blob, cells_at)[0] == 3
    tags = sorted(blob[cells_at + 4 + 9 * i] for i in range(3))
    assert tags == [1, 2, 3]                         # one float64, one int64, one bool cell
    p = str(tmp_path / "py.nxs")
    m.save_nxs(p)
    x = torch.randn(2, 3)
    torch.save((x, m(x)), str(tmp_path / "io.pt"))
    code = ("import sys, torch; sys.path.insert(0, %r)\nfrom nexus_b200 import nn\n"
            "x, y = torch.load(%r)\nm = nn.Sequential.load_nxs(%r)\nassert torch.equal(m(x), y)\nprint('fresh ok')\n"
            % (os.path.dirname(os.path.dirname(os.path.abspath(__file__))), str(tmp_path / "io.pt"), p))
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True)
    assert "fresh ok" in r.stdout, r.stderr[-2000:]
    table = {"a": 1}
    fnstore.register_python_activation("bad_t", lambda x: x * table["a"])
    with pytest.raises(TypeError, match="float, int or bool"):
        fnstore.payload_for(nn.Sequential().add(nn.Activation("bad_t")))
    with pytest.raises(ValueError, match="NXPY"):
        fnstore.restore_payload(b"\x80\x04junk")       # e.g. a pickle: rejected, never unpickled


def test_rejections(tmp_path):
    p = tmp_path / "t.nxs"
    p.write_bytes(b"NXS1" + b"\0" * 16)
    with pytest.raises(nxs.NxsError, match="trainer state"):
        nxs.load_archive(str(p))
    m = nn.Sequential().add(nn.Linear(4, 8))
    q = str(tmp_path / "m.nxs")
    m.save_nxs(q)
    data = open(q, "rb").read()
    (tmp_path / "cut.nxs").write_bytes(data[: len(data) - 7])
    with pytest.raises(nxs.NxsError, match="truncated"):
        nxs.load_archive(str(tmp_path / "cut.nxs"))
    (tmp_path / "bad.nxs").write_bytes(b"XXXX" + data[4:])
    with pytest.raises(nxs.NxsError, match="magic"):
        nxs.load_archive(str(tmp_path / "bad.nxs"))


def test_graph_errors():
    g = nn.Graph().add("a", nn.Linear(2, 2))
    with pytest.raises(ValueError):
        g.add("b", nn.ReLU(), ["nope"])
    with pytest.raises(ValueError):
        g.add("a", nn.ReLU())
