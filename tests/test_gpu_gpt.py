"""End-to-end GPT-2 on the sm_100a kernels: loss and every parameter gradient against a PyTorch
FP32 reference of the same network; optimizer steps reduce the loss; trainer + CUDA graph path."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def small_cfg():
    from nexus_b200.lm.config import preset
    cfg = preset("gpt2-124m")
    cfg.n_layer, cfg.d_model, cfg.n_head, cfg.d_ff, cfg.vocab_size, cfg.max_position = 2, 128, 2, 512, 500, 128
    return cfg


def torch_reference(P, tok, cfg):
    F = torch.nn.functional
    bf = lambda t: t.bfloat16().float()
    B, T = tok.shape
    C, H = cfg.d_model, cfg.n_head
    x = bf(P["wte"])[tok.long()] + bf(P["wpe"])[None, :T]
    for l in range(cfg.n_layer):
        h = F.layer_norm(x, (C,), P["ln1_w"][l], P["ln1_b"][l])
        qkv = h @ bf(P["qkv_w"][l]).t() + bf(P["qkv_b"][l])
        q, k, v = qkv.view(B, T, 3, H, C // H).permute(2, 0, 3, 1, 4)
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True).permute(0, 2, 1, 3).reshape(B, T, C)
        x = x + a @ bf(P["attproj_w"][l]).t() + bf(P["attproj_b"][l])
        h = F.layer_norm(x, (C,), P["ln2_w"][l], P["ln2_b"][l])
        h = F.gelu(h @ bf(P["fc_w"][l]).t() + bf(P["fc_b"][l]), approximate="tanh")
        x = x + h @ bf(P["fcproj_w"][l]).t() + bf(P["fcproj_b"][l])
    x = F.layer_norm(x, (C,), P["lnf_w"], P["lnf_b"])
    logits = x @ bf(P["wte"])[: cfg.vocab_size].t()
    return F.cross_entropy(logits[:, :-1].reshape(-1, cfg.vocab_size), tok.long()[:, 1:].reshape(-1))


def test_gpt_loss_and_grads_match_reference():
    from nexus_b200.models.gpt import PARAM_ORDER, GptModel
    from nexus_b200.ops import _cuda as K
    torch.manual_seed(0)
    cfg = small_cfg()
    m = GptModel(cfg)
    tok = torch.randint(0, cfg.vocab_size, (2, 128), dtype=torch.int32, device="cuda")
    loss = m.forward_backward(tok).item()
    K.check_status()
    P = {n: m.p[n].float().clone().requires_grad_(True) for n in PARAM_ORDER}
    ref = torch_reference(P, tok, cfg)
    ref.backward()
    assert abs(loss - ref.item()) < 2e-2
    for n in PARAM_ORDER:
        g, r = m.g[n].float(), P[n].grad
        if n == "wte":
            g, r = g[: cfg.vocab_size], r[: cfg.vocab_size]
        assert (g - r).norm() <= 5e-2 * r.norm(), n


def test_gpt_training_reduces_loss_and_trainer_graph_matches_eager():
    from nexus_b200.train.lm_trainer import AdamW, ArrayTokens, LanguageTrainerBuilder
    cfg = small_cfg()
    data = np.random.default_rng(0).integers(0, cfg.vocab_size, size=128 * 8, dtype=np.int32)

    def run(graph):
        tr = (LanguageTrainerBuilder(cfg).data(ArrayTokens(data)).optimizer(AdamW(lr=1e-3))
              .micro_batch(2).seq_len(128).global_batch_tokens(2 * 128 * 2).seed(7).log_every(0)
              .compile(graph).build())
        tr.train(6)
        return [r.loss for r in tr.history]

    eager, graph = run(False), run(True)
    assert eager[-1] < eager[0]
    assert np.allclose(eager, graph, rtol=2e-3, atol=2e-3)
