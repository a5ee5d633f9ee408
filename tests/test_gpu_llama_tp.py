"""`models.llama_tp.LlamaTpModel` on one GPU (the code path that is the oracle of the multi-GPU runs) against a plain
PyTorch FP32 implementation of the same decoder: loss, every gradient, and one AdamW step."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _reference_loss(cfg, W, tokens):
    """FP32 PyTorch: RMSNorm, rotate-half RoPE, causal attention, SwiGLU, untied head, shifted cross-entropy."""
    B, T = tokens.shape
    H, Hk, D, d = cfg.n_head, cfg.kv_heads(), cfg.hdim(), cfg.d_model
    x = W["wte"][tokens.long()]
    half = D // 2
    inv = 1.0 / (cfg.rope_theta ** (torch.arange(half, dtype=torch.float64, device=x.device) * 2 / D))
    ang = torch.arange(T, dtype=torch.float32, device=x.device)[:, None] * inv.float()[None]
    cos, sin = ang.cos()[None, :, None, :], ang.sin()[None, :, None, :]

    def rms(v, g):
        return v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + cfg.norm_eps) * g

    def rope(t):
        a, b = t[..., :half], t[..., half:]
        return torch.cat([a * cos - b * sin, b * cos + a * sin], -1)

    for l in range(cfg.n_layer):
        h = rms(x, W["norm1"][l])
        q = rope((h @ W["q_w"][l].t()).view(B, T, H, D))
        k = rope((h @ W["k_w"][l].t()).view(B, T, Hk, D))
        v = (h @ W["v_w"][l].t()).view(B, T, Hk, D)
        rep = H // Hk
        k, v = k.repeat_interleave(rep, 2), v.repeat_interleave(rep, 2)
        att = torch.einsum("bthd,bshd->bhts", q, k) / math.sqrt(D)
        att = att.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool, device=x.device), 1), float("-inf"))
        o = torch.einsum("bhts,bshd->bthd", att.softmax(-1), v).reshape(B, T, H * D)
        x = x + o @ W["o_w"][l].t()
        h = rms(x, W["norm2"][l])
        x = x + (torch.nn.functional.silu(h @ W["gate_w"][l].t()) * (h @ W["up_w"][l].t())) @ W["down_w"][l].t()
    logits = rms(x, W["normf"]) @ W["head"].t()
    return torch.nn.functional.cross_entropy(logits[:, :-1].reshape(-1, logits.shape[-1]), tokens[:, 1:].reshape(-1).long())


def _tiny_config():
    from nexus_b200.lm.config import LmConfig
    return LmConfig(name="tiny-llama", vocab_size=512, n_layer=2, d_model=256, n_head=4, n_kv_head=2, d_ff=512,
                    max_position=256, norm="rmsnorm", mlp="swiglu", pos="rope", tie_embeddings=False, bias=False)


def test_single_rank_loss_and_gradients_match_pytorch():
    from nexus_b200.models.llama_tp import LlamaTpModel
    from nexus_b200.ops import _cuda as K
    cfg = _tiny_config()
    full = LlamaTpModel.random_full_weights(cfg, seed=3)
    for k in ("norm1", "norm2", "normf"):
        full[k] = full[k] + 0.1 * torch.randn(full[k].shape, generator=torch.Generator().manual_seed(5))
    model = LlamaTpModel(cfg, device="cuda", full_weights=full)
    tokens = torch.randint(0, cfg.vocab_size, (2, 256), dtype=torch.int32, device="cuda",
                           generator=torch.Generator(device="cuda").manual_seed(1))
    loss = float(model.forward_backward(tokens).item())
    torch.cuda.synchronize()
    K.check_status()
    # the reference sees the BF16-rounded weights the kernels read
    W = {k: v.cuda().bfloat16().float().requires_grad_(True) if not k.startswith("norm") else v.cuda().requires_grad_(True)
         for k, v in full.items()}
    ref = _reference_loss(cfg, W, tokens)
    ref.backward()
    assert abs(loss - float(ref)) < 2e-2, (loss, float(ref))
    got = model.gather_full("grads")
    for name in W:
        a, b = got[name], W[name].grad
        rel = (a - b).norm().item() / max(b.norm().item(), 1e-12)
        assert rel < 4e-2, (name, rel)


def test_single_rank_training_reduces_the_loss():
    from nexus_b200.models.gpt import AdamWConfig
    from nexus_b200.models.llama_tp import LlamaTpModel
    from nexus_b200.ops import _cuda as K
    cfg = _tiny_config()
    model = LlamaTpModel(cfg, device="cuda", seed=9)
    model.set_optimizer(AdamWConfig(lr=2e-3, grad_clip=1.0))
    tokens = torch.randint(0, cfg.vocab_size, (2, 256), dtype=torch.int32, device="cuda")
    losses = []
    for _ in range(8):
        losses.append(float(model.forward_backward(tokens).item()))
        model.optimizer_step()
    torch.cuda.synchronize()
    K.check_status()
    assert losses[-1] < losses[0] - 0.5, losses
    st = model.read_opt_state()
    assert st.step == 8 and st.grad_norm > 0
