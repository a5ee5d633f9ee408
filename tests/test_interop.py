import json
import struct

import numpy as np
import pytest
import torch

from nexus_b200.interop import SafetensorsError, SafetensorsFile, dlpack, gguf, hf, load_file, save_file
from nexus_b200.lm import LanguageModel
from nexus_b200.lm.config import LmConfig


def small_llama(tie=False, qkv_bias=False, kv=2):
    cfg = LmConfig(vocab_size=96, d_model=64, n_layer=2, n_head=4, n_kv_head=kv, d_ff=128, max_position=64,
                   norm="rmsnorm", mlp="swiglu", pos="rope", bias=False, qkv_bias=qkv_bias, tie_embeddings=tie)
    return LanguageModel(cfg)


def test_safetensors_round_trip_and_mmap(tmp_path):
    t = {"a": torch.randn(3, 5), "b": torch.arange(7, dtype=torch.int64), "c.h": torch.randn(4).bfloat16(),
         "e": torch.zeros(0, 3), "f8": torch.randn(8).to(torch.float8_e4m3fn)}
    p = str(tmp_path / "x.safetensors")
    save_file(t, p, {"who": "test"})
    f = SafetensorsFile(p)
    assert f.metadata == {"who": "test"} and sorted(f.keys()) == sorted(t)
    for k in t:
        assert torch.equal(f.tensor(k).view(torch.uint8) if k == "f8" else f.tensor(k), t[k].view(torch.uint8) if k == "f8" else t[k])
    back = load_file(p)
    assert torch.equal(back["c.h"], t["c.h"])
    # readable by the same layout rules as the reference implementation of the format
    raw = open(p, "rb").read()
    (hlen,) = struct.unpack("<Q", raw[:8])
    hdr = json.loads(raw[8: 8 + hlen])
    assert hdr["a"]["dtype"] == "F32" and hdr["a"]["shape"] == [3, 5]


def _write(path, header: dict, data: bytes, raw_header: bytes = None):
    hj = raw_header if raw_header is not None else json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)) + hj + data)


def test_safetensors_strict_validation(tmp_path):
    p = str(tmp_path / "bad.safetensors")
    ok = {"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}}
    _write(p, ok, b"\0" * 8)
    SafetensorsFile(p)
    cases = [
        ({"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 12]}}, b"\0" * 12),                      # size mismatch
        ({"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}}, b"\0" * 12),                       # trailing bytes
        ({"a": {"dtype": "F33", "shape": [2], "data_offsets": [0, 8]}}, b"\0" * 8),                        # dtype
        ({"a": {"dtype": "F32", "shape": [-2], "data_offsets": [0, 8]}}, b"\0" * 8),                       # shape
        ({"a": {"dtype": "F32", "shape": [2], "data_offsets": [4, 12]}}, b"\0" * 12),                      # hole
        ({"a": {"dtype": "F32", "shape": [1], "data_offsets": [0, 4]},
          "b": {"dtype": "F32", "shape": [1], "data_offsets": [2, 6]}}, b"\0" * 6),                        # overlap
        ({"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8], "x": 1}}, b"\0" * 8),                # extra key
        ({"a": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}, b"\0" * 8),                       # out of range
    ]
    for hdr, data in cases:
        _write(p, hdr, data)
        with pytest.raises(SafetensorsError):
            SafetensorsFile(p)
    _write(p, None, b"", raw_header=b'{"a": {"dtype":"F32","shape":[0],"data_offsets":[0,0]}, "a": {"dtype":"F32","shape":[0],"data_offsets":[0,0]}}')
    with pytest.raises(SafetensorsError, match="duplicate"):
        SafetensorsFile(p)
    _write(p, None, b"", raw_header=b"{not json")
    with pytest.raises(SafetensorsError):
        SafetensorsFile(p)
    with open(p, "wb") as f:
        f.write(struct.pack("<Q", 1 << 40))
    with pytest.raises(SafetensorsError):
        SafetensorsFile(p)


@pytest.mark.parametrize("mt,tie,bias,kv", [("llama", False, False, 2), ("qwen2", True, True, 4), ("mistral", False, False, 1)])
def test_hf_round_trip_preserves_logits(tmp_path, mt, tie, bias, kv):
    m = small_llama(tie, bias, kv)
    d = str(tmp_path / mt)
    hf.export_hf(m, d, mt)
    cfgj = json.load(open(d + "/config.json"))
    assert cfgj["model_type"] == mt and cfgj["num_key_value_heads"] == kv
    m2 = hf.import_hf(d)
    toks = torch.randint(0, 96, (2, 10))
    assert torch.allclose(m.logits(toks), m2.logits(toks), atol=1e-6)
    names = set(hf.to_hf_state(m))
    assert "model.layers.1.self_attn.k_proj.weight" in names and ("lm_head.weight" in names) == (not tie)
    assert ("model.layers.0.self_attn.q_proj.bias" in names) == bias
    with pytest.raises(ValueError):
        hf.config_from_hf({"model_type": "gpt_neox"})


def test_gguf_quant_blocks_and_llama_round_trip(tmp_path):
    x = np.random.default_rng(0).normal(size=256).astype(np.float32)
    q8 = gguf.dequantize_q8_0(gguf.quantize_q8_0(x), 256)
    assert np.abs(q8 - x).max() < np.abs(x).max() / 127 + 1e-3
    q4 = gguf.dequantize_q4_0(gguf.quantize_q4_0(x), 256)
    assert np.abs(q4 - x).max() < np.abs(x).max() / 7 + 1e-3
    assert len(gguf.quantize_q8_0(x)) == 8 * 34 and len(gguf.quantize_q4_0(x)) == 8 * 18
    w = torch.randn(4 * 16, 32)
    assert torch.equal(gguf.permute_qk(gguf.permute_qk(w, 4), 4, inverse=True), w)
    assert torch.equal(gguf.permute_qk(w, 4)[1], w[8])     # pair (0, D/2) becomes adjacent
    m = small_llama()
    toks = torch.randint(0, 96, (1, 12))
    for ty, tol in ((gguf.T_F32, 1e-6), (gguf.T_F16, 5e-3), (gguf.T_Q8_0, 5e-2)):
        p = str(tmp_path / f"m{ty}.gguf")
        gguf.export_llama(m, p, ty)
        meta, tensors, types = gguf.read_gguf(p)
        assert meta["general.architecture"] == "llama" and meta["llama.block_count"] == 2
        assert types["blk.0.attn_q.weight"] == ty and types["blk.0.attn_norm.weight"] == gguf.T_F32
        m2 = gguf.import_llama(p)
        err = (m.logits(toks) - m2.logits(toks)).abs().max().item()
        assert err < tol * max(1.0, m.logits(toks).abs().max().item()), (ty, err)
    raw = open(p, "rb").read()
    assert raw[:4] == b"GGUF" and struct.unpack("<I", raw[4:8])[0] == 3


def test_dlpack_zero_copy():
    t = torch.randn(4, 4)
    u = dlpack.from_dlpack(dlpack.to_dlpack(t))
    u[0, 0] = 42.0
    assert t[0, 0] == 42.0 and dlpack.device_type(t) == dlpack.K_CPU
    with pytest.raises(TypeError):
        dlpack.to_dlpack(t.half())


def test_dlpack_native_capsules_interoperate_with_torch_and_numpy():
    """Capsules made by the native producer are consumed by torch; capsules made by torch and numpy are consumed by the
    native reader; strided views keep their geometry; a capsule is consumed once; anything but FP32 is refused and
    stays with its producer."""
    import numpy as np
    t = torch.arange(12, dtype=torch.float32).reshape(3, 4)
    cap = dlpack.to_dlpack(t)
    u = torch.from_dlpack(cap)
    u[0, 0] = 42.0
    assert t[0, 0] == 42.0
    with pytest.raises(ValueError, match="already consumed"):
        dlpack.from_dlpack(cap)
    v = dlpack.from_dlpack(torch.utils.dlpack.to_dlpack(t))
    v[1, 1] = 7.0
    assert t[1, 1] == 7.0 and tuple(v.shape) == (3, 4)
    w = dlpack.from_dlpack(dlpack.to_dlpack(t.t()[1:]))
    assert tuple(w.shape) == (3, 3) and w.stride() == (1, 4) and torch.equal(w, t.t()[1:])
    a = np.ones((2, 5), dtype=np.float32)
    x = dlpack.from_dlpack(a)
    x[0, 0] = 3.0
    assert a[0, 0] == 3.0
    with pytest.raises(ValueError, match="FP32"):
        dlpack.from_dlpack(np.ones(3))
    with pytest.raises(ValueError, match="capsule"):
        dlpack.from_dlpack(object())
    assert tuple(dlpack.from_dlpack(dlpack.to_dlpack(torch.empty(0, 3))).shape) == (0, 3)
    from nexus_b200.core.tensor import Tensor
    z = dlpack.from_dlpack(dlpack.to_dlpack(Tensor.from_torch(t)), as_tensor=True)
    assert isinstance(z, Tensor) and z.torch().data_ptr() == t.data_ptr()


def test_dlpack_owner_lives_exactly_as_long_as_the_consumer():
    import gc
    import weakref

    import numpy as np
    from nexus_b200 import _native

    class Owner:
        def __init__(self):
            self.mem = np.full(6, 2.0, dtype=np.float32)

    # consumed capsule: the owner dies when the imported view dies, not when the capsule does
    o = Owner()
    alive = weakref.ref(o)
    cap = _native.dlpack_export(o.mem.ctypes.data, [2, 3], [], 32, dlpack.K_CPU, 0, o)
    del o
    gc.collect()
    assert alive() is not None
    y = dlpack.from_dlpack(cap)
    del cap
    gc.collect()
    assert alive() is not None and float(y.sum()) == 12.0
    del y
    gc.collect()
    assert alive() is None
    # capsule nobody consumed: dropping it releases the owner
    o = Owner()
    alive = weakref.ref(o)
    cap = _native.dlpack_export(o.mem.ctypes.data, [6], [], 32, dlpack.K_CPU, 0, o)
    del o, cap
    gc.collect()
    assert alive() is None
    with pytest.raises(ValueError):
        _native.dlpack_export(0, [4], [], 32, dlpack.K_CPU, 0, None)
    with pytest.raises(ValueError):
        _native.dlpack_export(8, [4], [], 16, dlpack.K_CPU, 0, None)
    with pytest.raises(ValueError):
        _native.dlpack_export(8, [4], [], 32, 7, 0, None)


def test_onnx_export_structure(tmp_path):
    from nexus_b200.interop import onnx as O
    from nexus_b200.lm.config import preset
    m = LanguageModel(preset("nano"))
    p = str(tmp_path / "m.onnx")
    st = O.export_onnx(m, p, opset=17, external_data_threshold=64 * 1024)
    assert st["external_bytes"] > 0 and (tmp_path / "m.onnx.data").exists()
    top = O.parse(open(p, "rb").read())
    fields = {f for f, _, _ in top}
    assert {1, 7, 8} <= fields
    opsets = [O.parse(v) for f, _, v in top if f == 8]
    assert any(dict((a, c) for a, _, c in o).get(2) == 17 for o in opsets)
    graph = O.parse([v for f, _, v in top if f == 7][0])
    ops = [dict((a, c) for a, _, c in O.parse(v))[4].decode() for f, _, v in graph if f == 1]
    assert ops.count("LayerNormalization") == 9 and "Gather" in ops and "MatMul" in ops and "Attention" in ops
    inits = [O.parse(v) for f, _, v in graph if f == 5]
    names = [dict((a, c) for a, _, c in t if a == 8)[8].decode() for t in inits]
    assert "wte" in names and "h.0.attn.qkv.weight" in names
    ext = [t for t in inits if any(a == 14 for a, _, _ in t)]
    small = [t for t in inits if any(a == 9 for a, _, _ in t)]
    assert ext and small
    wte = [t for t in inits if dict((a, c) for a, _, c in t if a == 8)[8] == b"wte"][0]
    kv = dict((O.parse(c)[0][2].decode(), O.parse(c)[1][2].decode()) for a, _, c in wte if a == 13)
    data = open(p + ".data", "rb").read()
    got = np.frombuffer(data[int(kv["offset"]): int(kv["offset"]) + int(kv["length"])], dtype=np.float32)
    assert np.array_equal(got, m.state_dict()["wte"].numpy().reshape(-1))
    ins = [O.parse(v) for f, _, v in graph if f == 11]
    assert [dict((a, c) for a, _, c in i)[1] for i in ins] == [b"tokens", b"positions"]
    with pytest.raises(ValueError):
        O.export_onnx(m, p, opset=11)
