"""Block-scaled FP8 (MX) reference path on CPU: scale selection, atom layout, round trips, the linear layer."""
import torch

from nexus_b200.ops import _lowp as L


def test_scale_is_smallest_power_of_two_without_saturation():
    x = torch.tensor([[448.0] + [0.0] * 31 + [449.0] + [0.0] * 31 + [1e-3] * 32 + [0.0] * 32])
    q, s = L.mx_quantize_reference(x)
    e = s[L.mx_scale_index(1, 128)][0].tolist()
    assert e == [127, 128, 127 - 18, 127]      # 448 -> 2^0, 449 -> 2^1, 1e-3/448 = 2^-18.77 -> 2^-18, zeros -> 2^0
    assert float(q[0, 0].float()) == 448.0 and float(q[0, 32].float()) == 224.0
    assert s.numel() == 512 and (s == 127).sum() == 512 - 2


def test_atom_layout_and_round_trip():
    idx = L.mx_scale_index(300, 200)
    assert idx.shape == (300, 7) and idx.unique().numel() == idx.numel()
    assert int(idx[0, 0]) == 0 and int(idx[1, 0]) == 16 and int(idx[32, 0]) == 4 and int(idx[0, 1]) == 1
    assert int(idx[0, 4]) == 512 and int(idx[128, 0]) == 2 * 512          # two column atoms per row block
    torch.manual_seed(0)
    x = torch.randn(300, 200) * torch.logspace(-3, 3, 200)
    for dt, tol in ((torch.float8_e4m3fn, 0.04), (torch.float8_e5m2, 0.08)):
        for tr in (False, True):
            q, s = L.mx_quantize(x, dt, transpose=tr)
            want = x.t() if tr else x
            assert q.shape == want.shape and s.numel() == L.mx_scale_bytes(*want.shape)
            assert (L.mx_dequantize(q, s) - want).norm() / want.norm() < tol


def test_mx_gemm_and_linear_reference():
    torch.manual_seed(1)
    a, b = torch.randn(70, 96), torch.randn(50, 96)
    aq, asf = L.mx_quantize(a)
    bq, bsf = L.mx_quantize(b)
    y = L.mx_gemm(aq, asf, bq, bsf, out_dtype=torch.float32)
    assert (y - a @ b.t()).norm() / (a @ b.t()).norm() < 0.05
    hq, hs = L.mx_gemm(aq, asf, bq, bsf, act="relu", out_dtype=torch.float8_e4m3fn)
    assert (L.mx_dequantize(hq, hs) - torch.relu(a @ b.t())).norm() / torch.relu(a @ b.t()).norm() < 0.06
    x = torch.randn(3, 5, 64, requires_grad=True)
    w = torch.randn(32, 64, requires_grad=True)
    L.mx_linear(x, w).square().sum().backward()
    x2, w2 = x.detach().clone().requires_grad_(), w.detach().clone().requires_grad_()
    torch.nn.functional.linear(x2, w2).square().sum().backward()
    assert (x.grad - x2.grad).norm() / x2.grad.norm() < 0.1 and (w.grad - w2.grad).norm() / w2.grad.norm() < 0.1


def test_language_model_under_mxfp8_linear_precision():
    from nexus_b200.fused.ops import linear_precision
    from nexus_b200.lm.config import preset
    from nexus_b200.lm.model import build
    cfg = preset("llama2-7b")
    cfg.n_layer, cfg.d_model, cfg.n_head, cfg.n_kv_head, cfg.d_ff, cfg.vocab_size, cfg.max_position = 2, 64, 4, 4, 192, 128, 64
    model = build(cfg)
    toks = torch.randint(0, 128, (2, 32))
    native = model.loss(toks)
    with linear_precision("mxfp8"):
        low = model.loss(toks)
        low.backward()
    assert abs(float(low) - float(native)) < 0.05 * abs(float(native))
    grads = [p.grad for p in model.parameters() if p.grad is not None]
    assert grads and all(torch.isfinite(g).all() for g in grads)
    model.zero_grad()
    native.backward()


def test_weight_forms_are_quantised_once_per_version():
    torch.manual_seed(2)
    w = torch.randn(32, 64, requires_grad=True)
    x = torch.randn(8, 64)
    L.mx_weight_cache.enabled = True
    h0, m0 = L.mx_weight_cache.hits, L.mx_weight_cache.misses
    for _ in range(3):                                       # three micro-batches between two optimizer steps
        L.mx_linear(x.clone().requires_grad_(), w).sum().backward()
    assert L.mx_weight_cache.misses - m0 == 2               # the stored form and the transposed form
    assert L.mx_weight_cache.hits - h0 == 4
    with torch.no_grad():
        w.mul_(0.5)                                          # the optimizer step bumps the version
    y = L.mx_linear(x, w)
    assert L.mx_weight_cache.misses - m0 == 3
    assert (y - x @ w.t()).norm() / (x @ w.t()).norm() < 0.06
    w.data.mul_(2.0)                                         # invisible to the version counter: needs invalidate()
    L.mx_weight_cache.invalidate()
    y = L.mx_linear(x, w)
    assert (y - x @ w.t()).norm() / (x @ w.t()).norm() < 0.06
    L.mx_weight_cache.enabled = False
    L.mx_weight_cache.invalidate()
