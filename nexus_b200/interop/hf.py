"""Hugging Face llama / mistral / qwen2 checkpoints <-> `lm.LanguageModel`.

Name / layout table (HF weights are [out, in], as here):
  model.embed_tokens.weight                      <-> wte
  model.layers.L.input_layernorm.weight          <-> h.L.norm1.weight
  model.layers.L.self_attn.{q,k,v}_proj.weight   <-> rows of h.L.attn.qkv.weight (q | k | v)   (+ .bias for qwen2)
  model.layers.L.self_attn.o_proj.weight         <-> h.L.attn.o.weight
  model.layers.L.post_attention_layernorm.weight <-> h.L.norm2.weight
  model.layers.L.mlp.{gate,up}_proj.weight       <-> rows of h.L.mlp.up.weight (gate | up)
  model.layers.L.mlp.down_proj.weight            <-> h.L.mlp.down.weight
  model.norm.weight                              <-> norm_f.weight
  lm_head.weight                                 <-> lm_head (absent when embeddings are tied)
With equal head counts the fused QKV of this model is interleaved per [3, H, D]; the split handles both.
Parity: include/nexus/interop/hf.hpp, src/interop/hf.cpp of the reference."""
from __future__ import annotations

import json
import os
from typing import Dict

import torch

from ..lm.config import LmConfig, RopeScaling
from ..lm.model import LanguageModel
from .safetensors import load_file, save_file

SUPPORTED = ("llama", "mistral", "qwen2")


def config_from_hf(hf: dict) -> LmConfig:
    mt = hf.get("model_type", "llama")
    if mt not in SUPPORTED:
        raise ValueError(f"unsupported model_type {mt!r} (supported: {SUPPORTED})")
    rs = hf.get("rope_scaling") or {}
    kind = rs.get("rope_type", rs.get("type", "none"))
    scaling = RopeScaling(type={"default": "none"}.get(kind, kind), factor=float(rs.get("factor", 1.0)),
                          original_max_position=int(rs.get("original_max_position_embeddings", 0)),
                          low_freq_factor=float(rs.get("low_freq_factor", 1.0)),
                          high_freq_factor=float(rs.get("high_freq_factor", 4.0)))
    return LmConfig(name=mt, vocab_size=hf["vocab_size"], n_layer=hf["num_hidden_layers"], d_model=hf["hidden_size"],
                    n_head=hf["num_attention_heads"], n_kv_head=hf.get("num_key_value_heads", hf["num_attention_heads"]),
                    head_dim=hf.get("head_dim", 0) or 0, d_ff=hf["intermediate_size"],
                    max_position=hf.get("max_position_embeddings", 2048), norm="rmsnorm",
                    norm_eps=hf.get("rms_norm_eps", 1e-6), mlp="swiglu", pos="rope",
                    rope_theta=float(hf.get("rope_theta", 10000.0)), rope_scaling=scaling,
                    tie_embeddings=bool(hf.get("tie_word_embeddings", False)), bias=False, qkv_bias=(mt == "qwen2"),
                    window=int(hf.get("sliding_window") or 0) if mt == "mistral" else 0)


def config_to_hf(cfg: LmConfig, model_type: str = "llama") -> dict:
    if cfg.norm != "rmsnorm" or cfg.mlp != "swiglu" or cfg.pos != "rope" or cfg.bias:
        raise ValueError("only RMSNorm + SwiGLU + RoPE models without linear biases map to the llama family")
    out = {"model_type": model_type, "architectures": [{"llama": "LlamaForCausalLM", "mistral": "MistralForCausalLM",
                                                       "qwen2": "Qwen2ForCausalLM"}[model_type]],
           "vocab_size": cfg.vocab_size, "num_hidden_layers": cfg.n_layer, "hidden_size": cfg.d_model,
           "num_attention_heads": cfg.n_head, "num_key_value_heads": cfg.kv_heads(), "intermediate_size": cfg.d_ff,
           "max_position_embeddings": cfg.max_position, "rms_norm_eps": cfg.norm_eps, "rope_theta": cfg.rope_theta,
           "tie_word_embeddings": cfg.tie_embeddings, "hidden_act": "silu", "torch_dtype": "float32"}
    if cfg.head_dim:
        out["head_dim"] = cfg.head_dim
    if cfg.rope_scaling.type != "none":
        out["rope_scaling"] = {"rope_type": cfg.rope_scaling.type, "factor": cfg.rope_scaling.factor,
                               "original_max_position_embeddings": cfg.rope_scaling.original_max_position,
                               "low_freq_factor": cfg.rope_scaling.low_freq_factor,
                               "high_freq_factor": cfg.rope_scaling.high_freq_factor}
    if model_type == "mistral" and cfg.window:
        out["sliding_window"] = cfg.window
    return out


def _split_qkv(w: torch.Tensor, cfg: LmConfig):
    H, Hk, D = cfg.n_head, cfg.kv_heads(), cfg.hdim()
    if H == Hk:     # stored as [3, H, D] blocks == q | k | v rows
        return w[: H * D], w[H * D: 2 * H * D], w[2 * H * D:]
    return w[: H * D], w[H * D: (H + Hk) * D], w[(H + Hk) * D:]


def to_hf_state(model: LanguageModel) -> Dict[str, torch.Tensor]:
    cfg, sd = model.config, model.state_dict()
    out = {"model.embed_tokens.weight": sd["wte"], "model.norm.weight": sd["norm_f.weight"]}
    if not cfg.tie_embeddings:
        out["lm_head.weight"] = sd["lm_head"]
    F = cfg.d_ff
    for l in range(cfg.n_layer):
        p, h = f"h.{l}.", f"model.layers.{l}."
        q, k, v = _split_qkv(sd[p + "attn.qkv.weight"], cfg)
        out[h + "self_attn.q_proj.weight"], out[h + "self_attn.k_proj.weight"], out[h + "self_attn.v_proj.weight"] = q, k, v
        if p + "attn.qkv.bias" in sd:
            bq, bk, bv = _split_qkv(sd[p + "attn.qkv.bias"], cfg)
            out[h + "self_attn.q_proj.bias"], out[h + "self_attn.k_proj.bias"], out[h + "self_attn.v_proj.bias"] = bq, bk, bv
        out[h + "self_attn.o_proj.weight"] = sd[p + "attn.o.weight"]
        out[h + "input_layernorm.weight"] = sd[p + "norm1.weight"]
        out[h + "post_attention_layernorm.weight"] = sd[p + "norm2.weight"]
        up = sd[p + "mlp.up.weight"]
        out[h + "mlp.gate_proj.weight"], out[h + "mlp.up_proj.weight"] = up[:F], up[F:]
        out[h + "mlp.down_proj.weight"] = sd[p + "mlp.down.weight"]
    return {k: v.detach().clone().contiguous() for k, v in out.items()}


def from_hf_state(cfg: LmConfig, hf: Dict[str, torch.Tensor]) -> LanguageModel:
    model = LanguageModel(cfg)
    sd = {}
    need = lambda k: hf[k] if k in hf else (_ for _ in ()).throw(KeyError(f"missing tensor {k}"))   # noqa: E731
    sd["wte"] = need("model.embed_tokens.weight")
    sd["norm_f.weight"] = need("model.norm.weight")
    if not cfg.tie_embeddings:
        sd["lm_head"] = hf.get("lm_head.weight", sd["wte"])
    for l in range(cfg.n_layer):
        p, h = f"h.{l}.", f"model.layers.{l}."
        sd[p + "attn.qkv.weight"] = torch.cat([need(h + f"self_attn.{n}_proj.weight") for n in "qkv"], 0)
        if cfg.qkv_bias:
            sd[p + "attn.qkv.bias"] = torch.cat([need(h + f"self_attn.{n}_proj.bias") for n in "qkv"], 0)
        sd[p + "attn.o.weight"] = need(h + "self_attn.o_proj.weight")
        sd[p + "norm1.weight"] = need(h + "input_layernorm.weight")
        sd[p + "norm2.weight"] = need(h + "post_attention_layernorm.weight")
        sd[p + "mlp.up.weight"] = torch.cat([need(h + "mlp.gate_proj.weight"), need(h + "mlp.up_proj.weight")], 0)
        sd[p + "mlp.down.weight"] = need(h + "mlp.down_proj.weight")
    own = model.state_dict()
    for k, v in sd.items():
        if own[k].shape != v.shape:
            raise ValueError(f"{k}: shape {tuple(v.shape)} does not match the config ({tuple(own[k].shape)})")
    model.load_state_dict({k: v.to(own[k].dtype) for k, v in sd.items()}, strict=False)
    return model


def export_hf(model: LanguageModel, directory: str, model_type: str = "llama") -> None:
    os.makedirs(directory, exist_ok=True)
    with open(os.path.join(directory, "config.json"), "w") as f:
        json.dump(config_to_hf(model.config, model_type), f, indent=2)
    save_file(to_hf_state(model), os.path.join(directory, "model.safetensors"), {"format": "pt"})


def import_hf(directory: str) -> LanguageModel:
    with open(os.path.join(directory, "config.json")) as f:
        cfg = config_from_hf(json.load(f))
    tensors: Dict[str, torch.Tensor] = {}
    index = os.path.join(directory, "model.safetensors.index.json")
    if os.path.exists(index):
        with open(index) as f:
            files = sorted(set(json.load(f)["weight_map"].values()))
    else:
        files = ["model.safetensors"]
    for name in files:
        tensors.update(load_file(os.path.join(directory, name)))
    return from_hf_state(cfg, tensors)
