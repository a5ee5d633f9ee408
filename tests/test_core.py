import numpy as np
import pytest
import torch

from nexus_b200 import amp, core
from nexus_b200.core import DType, MemorySpace, Op, Tensor


def test_promote_table():
    assert core.promote(DType.F16, DType.BF16) == DType.F32
    assert core.promote(DType.U8, DType.I8) == DType.I32
    assert core.promote(DType.Bool, DType.I8) == DType.I8
    assert core.promote(DType.I64, DType.F16) == DType.F16
    assert core.promote(DType.F32, DType.F64) == DType.F64
    assert core.promote(DType.I32, DType.I64) == DType.I64
    with pytest.raises(core.TensorError):
        core.promote(DType.F8E4M3, DType.F32)
    assert core.promote(DType.F8E5M2, DType.F8E5M2) == DType.F8E5M2
    assert [core.size_of(d) for d in core.ALL_DTYPES] == [4, 2, 2, 8, 4, 8, 1, 1, 1, 1, 1]
    assert core.parse_dtype("bf16") == DType.BF16 and core.to_string(DType.F8E4M3) == "f8e4m3"


def test_fp8_and_bf16_conversions_match_torch():
    x = np.concatenate([np.random.default_rng(0).normal(size=2000).astype(np.float32) * 50,
                        np.array([0, -0.0, 448, 449, 1e6, -1e6, 2 ** -9, 2 ** -10, 0.0019, 57344, 6e4], np.float32)])
    for fmt, tdt in ((DType.F8E4M3, torch.float8_e4m3fn), (DType.F8E5M2, torch.float8_e5m2)):
        codes = core.fp8_encode(x, fmt)
        sat = np.clip(x, -core.FP8_MAX[fmt], core.FP8_MAX[fmt])
        ref = torch.tensor(sat).to(tdt).view(torch.uint8).numpy()
        assert np.array_equal(codes, ref)
        back = core.fp8_decode(codes, fmt)
        assert np.array_equal(back, torch.tensor(sat).to(tdt).float().numpy())
    bits = core.float_to_bf16_bits(x)
    assert np.array_equal(bits, torch.tensor(x).bfloat16().view(torch.int16).numpy().view(np.uint16))
    assert np.array_equal(core.bf16_bits_to_float(bits), torch.tensor(x).bfloat16().float().numpy())
    assert np.array_equal(core.half_bits_to_float(core.float_to_half_bits(x[:100])), x[:100].astype(np.float16).astype(np.float32))


def test_delayed_scaling():
    s = core.Fp8DelayedScaling(DType.F8E4M3, history=3, margin=1)
    assert s.update(2.0) == 448.0 / 2.0 / 2
    s.update(8.0)
    s.update(1.0)
    assert s.scale == 448.0 / 8.0 / 2
    s.update(1.0)
    s.update(1.0)           # the 8.0 left the window
    assert s.scale == 448.0 / 1.0 / 2 and abs(s.scale_inv() * s.scale - 1) < 1e-12


def test_device_ref_and_shape():
    assert core.DeviceRef.parse("cuda:3") == core.DeviceRef.cuda(3)
    assert core.DeviceRef.parse("CPU").is_cpu() and str(core.DeviceRef.parse("cuda")) == "cuda:0"
    assert core.DeviceRef.parse("hybrid").is_hybrid() and str(core.DeviceRef.hybrid()) == "hybrid"
    for bad in ("hybrid:1", "gpu:0", "cuda:x", "cpu:1"):
        with pytest.raises(core.TensorError):
            core.DeviceRef.parse(bad)
    assert core.Shape([2, 3, 4]).numel() == 24 and core.Shape([2, 3, 4]).contiguous_strides() == (12, 4, 1)
    with pytest.raises(core.TensorError):
        core.Shape([1] * 9)
    with pytest.raises(core.TensorError):
        core.Shape([1 << 40, 1 << 40]).numel()
    assert core.ExecutionPolicy.hybrid_cpu_multi_gpu([0, 1]).gpus == (0, 1)


def test_tensor_views_share_storage_and_copy_is_deep():
    t = Tensor.from_torch(torch.arange(24, dtype=torch.float32).view(2, 3, 4))
    v = t.transpose(0, 2).narrow(1, 1, 2).select(0, 3)
    assert torch.equal(v.torch(), t.torch().transpose(0, 2)[3, 1:3])
    assert v.storage is t.storage
    v.torch().fill_(-1)
    assert t.torch()[0, 1, 3] == -1
    assert torch.equal(t.slice(2, 0, 4, 2).torch(), t.torch()[:, :, 0:4:2])
    assert torch.equal(t.permute([2, 0, 1]).torch(), t.torch().permute(2, 0, 1))
    assert t.unsqueeze(1).shape == (2, 1, 3, 4) and t.unsqueeze(1).squeeze(1).shape == (2, 3, 4)
    assert t.narrow(0, 0, 1).expand([5, 3, 4]).torch().shape == (5, 3, 4)
    with pytest.raises(core.TensorError):
        t.transpose(0, 1).reshape([6, 4])
    assert t.reshape([6, -1]).shape == (6, 4)
    c = t.copy()
    c.torch().zero_()
    assert t.torch().abs().sum() > 0
    v0 = t.version()
    t.fill(2.0)
    assert t.version() == v0 + 1 and float(t.torch().mean()) == 2.0
    assert t.to(DType.BF16).dtype == DType.BF16 and t.to(DType.F32) is t


def test_dispatcher_explicit_errors_and_math():
    a = Tensor.from_torch(torch.randn(4, 5))
    b = Tensor.from_torch(torch.randn(5, 3))
    assert torch.allclose(core.matmul(a, b).torch(), a.torch() @ b.torch())
    h = Tensor.from_torch(torch.randn(4, 5).half())
    assert core.add(a, h).dtype == DType.F32
    assert torch.allclose(core.unary(a, "silu").torch(), torch.nn.functional.silu(a.torch()))
    with pytest.raises(core.TensorError):
        core.dispatch(Op.Matmul, DType.I8, MemorySpace.Host)
    with pytest.raises(core.TensorError):
        core.dispatch(Op.Fill, DType.F8E4M3, MemorySpace.Device)
    g = core.dispatch(Op.UnaryGrad, DType.F32, MemorySpace.Host)(a, Tensor.from_torch(torch.ones(4, 5)), "tanh")
    assert torch.allclose(g.torch(), 1 - torch.tanh(a.torch()) ** 2, atol=1e-6)
    assert abs(core.dispatch(Op.SqNorm, DType.F32, MemorySpace.Host)(a) - float((a.torch().double() ** 2).sum())) < 1e-9


def test_memory_gate_counters_and_alignment():
    g = core.MemoryGate()
    buf = g.alloc(1000, alignment=256)
    assert buf.data_ptr() % 256 == 0 and buf.numel() == 1000
    src = torch.arange(1000, dtype=torch.uint8)
    g.copy_bytes(buf, src)
    assert torch.equal(buf, src) and g.counters.copied_bytes == 1000
    assert g.counters.live_bytes["host"] == 1000 and g.counters.peak_bytes["host"] == 1000
    g.free(buf)
    assert g.counters.live_bytes["host"] == 0
    with pytest.raises(core.TensorError):
        g.free(buf)


def test_mirrored_tensor_state_machine_unified():
    m = core.MirroredTensor([4, 4], core.DeviceRef.cpu())
    assert m.unified and m.state == core.MirrorState.Synced
    m.modify_host()
    m.sync_device()
    assert m.state == core.MirrorState.Synced and m.bytes_to_device == 0
    assert m.device_data() is m.host


@pytest.mark.gpu
def test_mirrored_tensor_gpu_round_trip():
    m = core.MirroredTensor([256, 256], core.DeviceRef.cuda(0))
    m.host.fill_(3.0)
    m.modify_host()
    assert m.needs_sync_device()
    with pytest.raises(RuntimeError):
        m.modify_device()
    m.sync_device(blocking=False)
    assert m.copy_pending()
    m.device_data().mul_(2)
    m.modify_device()
    m.synchronize()
    with pytest.raises(RuntimeError):
        m.modify_host()
    m.sync_host()
    assert float(m.host.mean()) == 6.0 and m.bytes_to_device == m.bytes_to_host == 256 * 256 * 4
    g = core.gate()
    d = core.DeviceBuffer(4096)
    assert d.ptr() % 256 == 0 and g.counters.live_bytes["device"] >= 4096


def test_autocast_table():
    from nexus_b200.amp import AutocastGuard, CastPolicy, OpClass, cast_dtype, policy_for
    assert policy_for(OpClass.Linear) == CastPolicy.Lower and policy_for(OpClass.Softmax) == CastPolicy.Fp32
    assert policy_for(OpClass.Cat) == CastPolicy.Promote and policy_for(OpClass.Dropout) == CastPolicy.Keep
    assert cast_dtype(OpClass.Matmul, [DType.F32, DType.F32]) == DType.F32
    with AutocastGuard(dtype=DType.BF16):
        assert cast_dtype(OpClass.Matmul, [DType.F32, DType.F32]) == DType.BF16
        assert cast_dtype(OpClass.LayerNorm, [DType.BF16]) == DType.F32
        assert cast_dtype(OpClass.Add, [DType.BF16, DType.F32]) == DType.F32
        with AutocastGuard(enabled=False):
            assert cast_dtype(OpClass.Matmul, [DType.F32, DType.F32]) == DType.F32
        assert amp.autocast_state()[0]
    assert not amp.autocast_state()[0]
    with pytest.raises(core.TensorError):
        AutocastGuard(dtype=DType.F32)


def test_native_low_precision_conversions_match_numpy_and_torch():
    """Bit-level float32 -> BF16 / F16 / FP8 conversions of the native host module against numpy (F16), torch (BF16,
    FP8 in range) and exhaustive midpoints (ties go to the even mantissa); FP8 saturates and has one NaN code."""
    import numpy as np
    import torch
    from nexus_b200.core import dtype as D
    rng = np.random.default_rng(0)
    x = rng.integers(0, 2 ** 32, size=200_000, dtype=np.uint64).astype(np.uint32).view(np.float32)
    sp = np.array([0.0, np.inf, np.nan, 1e-45, 1.17549435e-38, 6.1e-5, 5.96e-8, 2.98e-8, 65504, 65519.99, 65520, 70000, 448,
                   449, 464, 465, 480, 1e9, 57344, 61440, 61439, 2.0 ** -9, 2.0 ** -10, 2.0 ** -17, 2.0 ** -16], dtype=np.float32)
    x = np.concatenate([x, sp, -sp])
    nan = np.isnan(x)
    with np.errstate(over="ignore", invalid="ignore"):
        f16 = x.astype(np.float16).view(np.uint16)
    got = D.float_to_half_bits(x)
    assert got.dtype == np.uint16 and np.array_equal(got[~nan], f16[~nan]) and np.isnan(got[nan].view(np.float16)).all()
    codes = np.arange(65536, dtype=np.uint16)
    back, want = D.half_bits_to_float(codes), codes.view(np.float16).astype(np.float32)
    assert np.array_equal(np.isnan(back), np.isnan(want)) and np.array_equal(back[~np.isnan(want)], want[~np.isnan(want)])
    vals = np.arange(0, 0x7C00, dtype=np.uint16).view(np.float16).astype(np.float64)
    mid = ((vals[:-1] + vals[1:]) / 2).astype(np.float32)
    assert np.array_equal(D.float_to_half_bits(mid), mid.astype(np.float16).view(np.uint16))
    bf = torch.from_numpy(x.copy()).to(torch.bfloat16).view(torch.uint16).numpy()
    assert np.array_equal(D.float_to_bf16_bits(x)[~nan], bf[~nan]) and (D.float_to_bf16_bits(x)[nan] == 0x7FC0).all()
    assert D.float_to_bf16_bits(x.reshape(5, -1)).shape == (5, x.size // 5)
    for fmt, tdt, nan_code in ((D.DType.F8E4M3, torch.float8_e4m3fn, 0x7F), (D.DType.F8E5M2, torch.float8_e5m2, 0x7E)):
        mx = D.FP8_MAX[fmt]
        got = D.fp8_encode(x, fmt)
        inr = np.isfinite(x) & (np.abs(x) <= mx)
        assert np.array_equal(got[inr], torch.from_numpy(x.copy()).to(tdt).view(torch.uint8).numpy()[inr])
        big = ~nan & (np.abs(x) > mx)
        dec = D.fp8_decode(got[big], fmt)
        assert (np.abs(dec) == mx).all() and np.array_equal(np.signbit(dec), np.signbit(x[big])) and (got[nan] == nan_code).all()
        c8 = np.arange(256, dtype=np.uint8)
        q, r = torch.from_numpy(c8).view(tdt).float().numpy(), D.fp8_decode(c8, fmt)
        assert np.array_equal(np.isnan(r), np.isnan(q)) and np.array_equal(r[~np.isnan(q)], q[~np.isnan(q)])
        fin = np.sort(q[np.isfinite(q) & (q >= 0)]).astype(np.float64)
        mid = ((fin[:-1] + fin[1:]) / 2).astype(np.float32)
        assert np.array_equal(D.fp8_encode(mid, fmt), torch.from_numpy(mid).to(tdt).view(torch.uint8).numpy())
