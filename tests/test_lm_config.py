import pytest

from nexus_b200.lm import config as C


def test_presets_and_parameter_counts():
    assert set(["gpt2-124m", "gpt2-350m", "gpt2-774m", "gpt2-1.5b", "llama2-7b", "llama3-8b", "mistral-7b", "qwen2-0.5b",
                "qwen2-1.5b", "qwen2-7b", "tinyllama-1.1b", "moe-124m"]) <= set(C.preset_names())
    assert C.count_parameters(C.preset("gpt2-124m")) == 124439808
    assert C.count_parameters(C.preset("llama2-7b")) == 6738415616
    assert C.count_parameters(C.preset("llama3-8b")) == 8030261248
    moe = C.preset("moe-124m")
    assert C.count_active_parameters(moe) < C.count_parameters(moe)


def test_json_round_trip_and_overrides():
    c = C.preset("mistral-7b")
    c.rope_scaling.type, c.rope_scaling.factor = "yarn", 4.0
    d = C.from_json(C.to_json(c))
    assert d == c
    e = C.apply_overrides(c, '{"n_layer": 2, "rope_scaling": {"factor": 2.0}}')
    assert e.n_layer == 2 and e.rope_scaling.factor == 2.0 and c.n_layer == 32
    with pytest.raises(C.ConfigError):
        C.from_json('{"no_such_key": 1}')


@pytest.mark.parametrize("field,value", [("n_head", 5), ("norm", "batchnorm"), ("resid_dropout", 1.0),
                                          ("vocab_pad_multiple", 0), ("n_kv_head", 5)])
def test_validate_rejects(field, value):
    c = C.preset("gpt2-124m")
    setattr(c, field, value)
    with pytest.raises(C.ConfigError):
        C.validate(c)


def test_moe_validation():
    c = C.preset("moe-124m")
    c.bias = True
    with pytest.raises(C.ConfigError):
        C.validate(c)
    c = C.preset("moe-124m")
    c.moe_top_k = 99
    with pytest.raises(C.ConfigError):
        C.validate(c)


def test_cpu_inference_weight_modes_and_native_attention():
    """`prepare_cpu_inference`: the packed no-grad forward (native GEMMs + blocked attention) follows the autograd
    forward; BF16 / INT8 / INT4 shrink the weights and stay within their quantisation error; generation runs."""
    import torch
    from nexus_b200.lm.config import preset
    from nexus_b200.lm.model import LanguageModel
    cfg = preset("nano")
    m = LanguageModel(cfg)
    toks = torch.randint(0, cfg.vocab_size, (2, 24), generator=torch.Generator().manual_seed(0))
    with torch.enable_grad():
        ref = m.logits(toks).detach()
    sizes = {}
    for mode, tol in (("f32", 2e-4), ("bf16", 2e-2), ("int8", 6e-2), ("int4", 0.5)):
        m.prepare_cpu_inference(mode)
        assert m.cpu_weight_mode() == mode
        sizes[mode] = m.cpu_inference_weight_bytes()
        with torch.no_grad():
            got = m.logits(toks)
        rel = ((got - ref).norm() / ref.norm()).item()
        assert rel < tol, (mode, rel)
    assert sizes["f32"] > sizes["bf16"] > sizes["int8"] > sizes["int4"] > 0
    with torch.no_grad():
        out = m.generate(toks[:1, :4], 5)
    assert out.shape[-1] == 9
    with pytest.raises(ValueError):
        m.prepare_cpu_inference("fp4")


def test_cpu_flash_attention_matches_math_attention_with_every_option():
    import numpy as np
    import torch
    from nexus_b200 import cpu
    from nexus_b200.fused.ops import attention_reference
    g = torch.Generator().manual_seed(3)
    q = torch.randn(2, 70, 4, 16, generator=g)
    k = torch.randn(2, 100, 2, 16, generator=g)
    v = torch.randn(2, 100, 2, 16, generator=g)
    slopes = torch.tensor([0.1, 0.2, 0.3, 0.4])
    for kw in ({"causal": True}, {"causal": False}, {"causal": True, "window": 33}, {"causal": True, "softcap": 20.0},
               {"causal": True, "alibi_slopes": slopes}):
        want = attention_reference(q, k, v, **kw)
        got, lse = cpu.flash_attention(q.numpy(), k.numpy(), v.numpy(), causal=kw.get("causal", True),
                                       window=kw.get("window", 0), softcap=kw.get("softcap", 0.0),
                                       alibi=None if "alibi_slopes" not in kw else slopes.numpy())
        assert np.abs(got - want.numpy()).max() < 1e-4, kw
        assert lse.shape == (2, 4, 70) and np.isfinite(lse).all()
    a = cpu.flash_attention(q.numpy(), k.numpy(), v.numpy(), threads=1)[0]
    b = cpu.flash_attention(q.numpy(), k.numpy(), v.numpy(), threads=4)[0]
    assert np.array_equal(a, b)           # the work split does not change a single bit
