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
