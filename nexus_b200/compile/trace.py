"""Tracer: builds the forward graph of a decoder LM from its config, from token ids to the shifted
cross-entropy loss, over meta values (shapes only).  The traced graph is unfused: Linear, Bias, Gelu, Add,
LayerNorm / RmsNorm, SplitQKV + Attention, GatedSplit + Silu + Mul appear as separate nodes, so that the
rewrite patterns have something to find.
Parity: include/nexus/compile/trace.hpp:20-70, src/compile/trace.cpp of the reference."""
from __future__ import annotations

from ..lm.config import LmConfig
from .ir import Dim, Graph, Value

B, T = Dim.of("B"), Dim.of("T")


class Builder:
    def __init__(self, name: str = "lm"):
        self.g = Graph(name)

    def linear(self, x: Value, w: Value, out_features: int) -> Value:
        (y,) = self.g.add("Linear", [x, w], [x.shape[:-1] + (Dim.of(out_features),)])
        return y

    def bias(self, x: Value, b: Value) -> Value:
        return self.g.add("Bias", [x, b], [x.shape])[0]

    def unary(self, op: str, x: Value, **attrs) -> Value:
        return self.g.add(op, [x], [x.shape], **attrs)[0]

    def binary(self, op: str, a: Value, b: Value) -> Value:
        return self.g.add(op, [a, b], [a.shape])[0]

    def norm(self, cfg: LmConfig, x: Value, prefix: str, d: int) -> Value:
        w = self.g.param(prefix + ".weight", [d])
        if cfg.norm == "layernorm":
            b = self.g.param(prefix + ".bias", [d])
            return self.g.add("LayerNorm", [x, w, b], [x.shape], eps=cfg.norm_eps)[0]
        return self.g.add("RmsNorm", [x, w], [x.shape], eps=cfg.norm_eps)[0]


def trace_lm(cfg: LmConfig) -> Graph:
    if cfg.moe_experts > 0:
        raise NotImplementedError("trace_lm covers dense models")
    bd = Builder(cfg.name or "lm")
    g = bd.g
    d, H, Hk, D, F = cfg.d_model, cfg.n_head, cfg.kv_heads(), cfg.hdim(), cfg.d_ff
    tokens = g.input("tokens", [B, T])
    wte = g.param("wte", [cfg.padded_vocab() if hasattr(cfg, "padded_vocab") else cfg.vocab_size, d])
    ins = [tokens, wte]
    if cfg.pos == "learned":
        ins.append(g.param("wpe", [cfg.max_position, d]))
    (x,) = g.add("Embedding", ins, [[B, T, d]])
    for l in range(cfg.n_layer):
        p = f"h.{l}."
        h = bd.norm(cfg, x, p + "norm1", d) if cfg.prenorm else x
        qkv = bd.linear(h, g.param(p + "attn.qkv.weight", [(H + 2 * Hk) * D, d]), (H + 2 * Hk) * D)
        if cfg.bias or cfg.qkv_bias:
            qkv = bd.bias(qkv, g.param(p + "attn.qkv.bias", [(H + 2 * Hk) * D]))
        q, k, v = g.add("SplitQKV", [qkv], [[B, T, H, D], [B, T, Hk, D], [B, T, Hk, D]], heads=H, kv_heads=Hk)
        if cfg.pos == "rope":
            q = bd.unary("Rope", q, theta=cfg.rope_theta)
            k = bd.unary("Rope", k, theta=cfg.rope_theta)
        (a,) = g.add("Attention", [q, k, v], [[B, T, H * D]], causal=True, window=cfg.window)
        a = bd.linear(a, g.param(p + "attn.o.weight", [d, H * D]), d)
        if cfg.bias:
            a = bd.bias(a, g.param(p + "attn.o.bias", [d]))
        x = bd.binary("Add", x, a)
        if not cfg.prenorm:
            x = bd.norm(cfg, x, p + "norm1", d)
        h = bd.norm(cfg, x, p + "norm2", d) if cfg.prenorm else x
        mult = 2 if cfg.gated_mlp() else 1
        u = bd.linear(h, g.param(p + "mlp.up.weight", [mult * F, d]), mult * F)
        if cfg.bias:
            u = bd.bias(u, g.param(p + "mlp.up.bias", [mult * F]))
        if cfg.gated_mlp():
            gate, up = g.add("GatedSplit", [u], [[B, T, F], [B, T, F]])
            act = bd.unary("Silu" if cfg.mlp == "swiglu" else "Gelu", gate)
            u = bd.binary("Mul", act, up)
        else:
            u = bd.unary("Gelu", u)
        m = bd.linear(u, g.param(p + "mlp.down.weight", [d, F]), d)
        if cfg.bias:
            m = bd.bias(m, g.param(p + "mlp.down.bias", [d]))
        x = bd.binary("Add", x, m)
        if not cfg.prenorm:
            x = bd.norm(cfg, x, p + "norm2", d)
    x = bd.norm(cfg, x, "norm_f", d)
    head = wte if cfg.tie_embeddings else g.param("lm_head", [wte.shape[0].coef, d])
    logits = bd.linear(x, head, wte.shape[0].coef)
    (loss,) = g.add("CrossEntropyShifted", [logits, tokens], [[]], vocab=cfg.vocab_size)
    g.outputs = [loss]
    return g
