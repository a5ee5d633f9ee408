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
    assert abs(loss - ref.item()) < 2e-3          # measured: 4e-6 .. 4e-5 over seeds
    for n in PARAM_ORDER:
        g, r = m.g[n].float(), P[n].grad
        if n == "wte":
            g, r = g[: cfg.vocab_size], r[: cfg.vocab_size]
        assert (g - r).norm() <= 1.5e-2 * r.norm(), n   # measured: 0.3 % .. 0.6 % per tensor (BF16 activations)


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


def _tiny_cfg():
    from nexus_b200.lm.config import preset
    cfg = preset("gpt2-124m")
    cfg.n_layer, cfg.d_model, cfg.n_head, cfg.d_ff, cfg.vocab_size, cfg.max_position = 3, 128, 2, 512, 500, 128
    return cfg


@pytest.mark.parametrize("mode,every", [("selective", 2), ("full", 2), ("every_k", 2)])
def test_recompute_modes_give_the_same_gradients_with_fewer_saved_bytes(mode, every):
    from nexus_b200.models.gpt import GptModel
    from nexus_b200.ops import _cuda as K
    """Every recompute mode re-runs the same kernels on the same inputs: loss and gradients equal the keep-everything
    run bit for bit (deterministic embedding), and the activation buffers shrink."""
    cfg = _tiny_cfg()
    tokens = torch.randint(0, cfg.vocab_size, (2, 128), dtype=torch.int32, device="cuda",
                           generator=torch.Generator(device="cuda").manual_seed(3))
    base = GptModel(cfg, device="cuda", seed=5)
    base.deterministic_embedding = True
    other = GptModel(cfg, device="cuda", seed=5, recompute=mode, recompute_every=every)
    other.deterministic_embedding = True
    l0 = float(base.forward_backward(tokens).item())
    l1 = float(other.forward_backward(tokens).item())
    torch.cuda.synchronize()
    K.check_status()
    assert l0 == l1
    rel = (other.grads - base.grads).norm().item() / base.grads.norm().item()
    # "full" re-runs the very same kernels (only the split-K summation order is free); "selective" redoes the GELU from
    # the BF16 pre-activation instead of the FP32 accumulator, a rounding-level difference
    assert rel < (1e-2 if mode == "selective" else 2e-3), rel
    assert other.activation_bytes() < base.activation_bytes()
    assert [other.layer_mode(l) for l in range(3)] == {"selective": ["selective"] * 3, "full": ["full"] * 3,
                                                       "every_k": ["full", "none", "full"]}[mode]


def test_eight_bit_and_offloaded_optimizers_track_fp32_adamw():
    from nexus_b200.models.gpt import AdamWConfig, GptModel
    from nexus_b200.ops import _cuda as K
    """Three optimizer kinds on the same model and data: the CPU (offloaded) AdamW follows the device AdamW closely
    (same operation order; BF16 gradient transfer), the 8-bit one follows within the quantisation error, and all
    reduce the loss."""
    cfg = _tiny_cfg()
    tokens = torch.randint(0, cfg.vocab_size, (2, 128), dtype=torch.int32, device="cuda",
                           generator=torch.Generator(device="cuda").manual_seed(4))
    runs = {}
    for kind, kw in (("adamw", {}), ("adamw8bit", {}), ("zero_offload", {"offload_grad_dtype": "f32"}),
                     ("adamw", {"master": "cast_per_forward"})):
        m = GptModel(cfg, device="cuda", seed=6, optimizer=kind, **kw)
        m.deterministic_embedding = True
        m.set_optimizer(AdamWConfig(lr=1e-3))
        losses = []
        for _ in range(6):
            losses.append(float(m.forward_backward(tokens).item()))
            m.optimizer_step()
        torch.cuda.synchronize()
        K.check_status()
        runs[kind + kw.get("master", "")] = (losses, m.optimizer_tensors()["params"].float().clone())
        assert losses[-1] < losses[0] - 0.3, (kind, losses)
    ref_losses, ref_p = runs["adamw"]
    init = GptModel(cfg, device="cuda", seed=6).params.cpu()
    upd = (ref_p - init).norm().item()
    off_losses, off_p = runs["zero_offload"]
    assert max(abs(a - b) for a, b in zip(ref_losses, off_losses)) < 2e-2
    assert (off_p - ref_p).norm().item() / upd < 0.1
    q_losses, q_p = runs["adamw8bit"]
    assert max(abs(a - b) for a, b in zip(ref_losses, q_losses)) < 0.15
    c_losses, c_p = runs["adamwcast_per_forward"]
    assert max(abs(a - b) for a, b in zip(ref_losses, c_losses)) < 2e-2
    dev_bytes, host_bytes = GptModel(cfg, device="cuda", optimizer="zero_offload").optimizer_state_bytes()
    assert host_bytes > 0 and dev_bytes < 12 * init.numel()


def test_dynamic_loss_scale_on_the_device():
    """The loss scale lives in the device-resident optimizer state: the loss gradient is multiplied by it inside the
    cross-entropy kernel, the norm kernel unscales and flags non-finite gradients, AdamW skips such a step (and still
    clears the gradients), and the update kernel halves the scale after an overflow and doubles it after
    `growth_interval` clean steps.  No host read takes part."""
    from nexus_b200.models.gpt import AdamWConfig, GptModel
    from nexus_b200.ops import _cuda as K
    cfg = _tiny_cfg()
    tokens = torch.randint(0, cfg.vocab_size, (2, 128), dtype=torch.int32, device="cuda",
                           generator=torch.Generator(device="cuda").manual_seed(4))

    def state(m):
        return K.unpack_opt_state(bytes(m.opt_state.cpu().numpy().tobytes()))

    # a power-of-two scale changes nothing but the exponent of the BF16 gradients: same training as without it
    ref = GptModel(cfg, device="cuda", seed=6)
    dyn = GptModel(cfg, device="cuda", seed=6, dynamic_loss_scale=True, loss_scale_init=1024.0, loss_scale_growth_interval=3)
    for m in (ref, dyn):
        m.deterministic_embedding = True
        m.set_optimizer(AdamWConfig(lr=1e-3))
    la, lb = [], []
    for _ in range(4):
        la.append(float(ref.forward_backward(tokens).item())); ref.optimizer_step()
        lb.append(float(dyn.forward_backward(tokens).item())); dyn.optimizer_step()
    assert max(abs(a - b) for a, b in zip(la, lb)) < 2e-2
    upd = (ref.params - GptModel(cfg, device="cuda", seed=6).params).norm().item()
    assert (ref.params - dyn.params).norm().item() / upd < 5e-2
    st = state(dyn)
    assert st.skipped == 0 and st.step == 4 and st.loss_scale == 2048.0       # doubled once after three clean steps

    # an absurd scale overflows the gradients: the step is skipped, the weights stay, the scale is halved, the
    # gradients are cleared, and training goes on once the scale is small enough
    big = GptModel(cfg, device="cuda", seed=6, dynamic_loss_scale=True, loss_scale_init=2.0 ** 126)
    big.set_optimizer(AdamWConfig(lr=1e-3))
    before = big.params.clone()
    big.forward_backward(tokens, grad_scale=2.0 ** 12)      # scale x weight is past the FP32 range: infinite gradients
    big.optimizer_step()
    st = state(big)
    assert st.found_inf == 1 and st.skipped == 1 and st.step == 0 and st.loss_scale == 2.0 ** 125
    assert torch.equal(big.params, before) and float(big.grads.abs().max()) == 0.0
    torch.cuda.synchronize()
    K.check_status()


def test_unimplemented_modes_are_refused_not_ignored():
    from nexus_b200.models.gpt import GptModel
    cfg = _tiny_cfg()
    for kw in ({"optimizer": "adamw8bit_fused"}, {"master": "none"}, {"compute_dtype": "f16"}, {"recompute": "sometimes"}):
        with pytest.raises(ValueError):
            GptModel(cfg, device="cuda", **kw)


@pytest.mark.parametrize("chunk_rows", [128, 256, 300])
def test_chunked_head_and_loss_match_the_single_pass(chunk_rows):
    from nexus_b200.models.gpt import GptModel
    from nexus_b200.ops import _cuda as K
    """LM head + cross-entropy + head backward over groups of whole sequences: same loss and gradients as one pass over
    all rows (only the summation order of the embedding gradient and of the loss differs), a smaller logits buffer,
    and `loss()` / `forward()` still see every row."""
    cfg = _tiny_cfg()
    tokens = torch.randint(0, cfg.vocab_size, (4, 128), dtype=torch.int32, device="cuda",
                           generator=torch.Generator(device="cuda").manual_seed(11))
    base = GptModel(cfg, device="cuda", seed=5, ce_chunk_rows=0)
    base.deterministic_embedding = True
    other = GptModel(cfg, device="cuda", seed=5, ce_chunk_rows=chunk_rows)
    other.deterministic_embedding = True
    assert other._head_group(4, 128) == {128: 1, 256: 2, 300: 2}[chunk_rows]
    l0 = float(base.forward_backward(tokens).item())
    l1 = float(other.forward_backward(tokens).item())
    torch.cuda.synchronize()
    K.check_status()
    assert abs(l0 - l1) < 1e-5 * abs(l0), (l0, l1)
    rel = (other.grads - base.grads).norm().item() / base.grads.norm().item()
    assert rel < 2e-3, rel
    assert other._acts["logits"].shape[0] == other._head_group(4, 128) * 128 < base._acts["logits"].shape[0]
    assert abs(other.loss(tokens) - base.loss(tokens)) < 1e-5 * abs(l0)
    full, ref = other.forward(tokens), base.forward(tokens)
    assert full.shape == ref.shape and torch.allclose(full.float(), ref.float(), atol=1e-2, rtol=1e-2)
    # a second micro-step accumulates the loss like the single pass does
    a0 = float(base.forward_backward(tokens, accumulate_loss=True, loss_weight=0.5).item())
    a1 = float(other.forward_backward(tokens, accumulate_loss=True, loss_weight=0.5).item())
    assert abs(a0 - a1) < 1e-5 * abs(a0)
