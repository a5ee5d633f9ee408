import math

import numpy as np
import pytest
import torch

from nexus_b200 import nn
from nexus_b200.data import DataLoader
from nexus_b200.lm import LanguageModel, preset
from nexus_b200.train import (AdamW, ArrayTokens, EpochStats, LanguageTrainer, LanguageTrainerBuilder, NanOptions,
                              ParamGroupPolicy, ParamGroupRule, SyntheticTokens, TokenRows, TrainerBuilder, WarmupCosine,
                              read_tensorboard_scalars)
from nexus_b200.train.callbacks import EarlyStopping


def nano_tokens():
    return np.random.Generator(np.random.PCG64(20261024)).integers(0, 256, size=8 * 128 * 4, dtype=np.int32)


def test_nano_config_trains_on_cpu_and_round_trips_through_nxs2(tmp_path):
    """4 layers, d 128, 4 heads, FFN 512 GELU, LayerNorm, learned positions, tied embeddings, vocab 256,
    seq 128, batch 8, AdamW lr 3e-4, FP32 on CPU."""
    cfg = preset("nano")
    assert (cfg.n_layer, cfg.d_model, cfg.n_head, cfg.d_ff, cfg.vocab_size, cfg.tie_embeddings) == (4, 128, 4, 512, 256, True)
    model = LanguageModel(cfg)
    tr = (LanguageTrainerBuilder(model).data(ArrayTokens(nano_tokens())).optimizer(AdamW(lr=3e-4))
          .micro_batch(8).seq_len(128).global_batch_tokens(8 * 128).precision("f32").execution_policy("cpu")
          .log_every(0).build())
    s = tr.train(6)
    losses = [r.loss for r in tr.history]
    assert s.steps == 6 and losses[-1] < losses[0] and all(math.isfinite(l) for l in losses)
    p = str(tmp_path / "nano.nxs")
    model.save_nxs(p)
    again = LanguageModel.load_nxs(p)
    t = torch.from_numpy(nano_tokens()[: 2 * 128].reshape(2, 128)).long()
    assert torch.equal(again.loss(t), model.loss(t))
    for (n1, a), (n2, b) in zip(model.named_parameters(), again.named_parameters()):
        assert n1 == n2 and torch.equal(a, b)


def test_accumulation_equals_one_big_batch_and_param_groups():
    cfg = preset("nano")
    cfg.n_layer, cfg.d_model, cfg.d_ff, cfg.max_position = 1, 32, 64, 16
    data = np.random.default_rng(0).integers(0, 256, size=16 * 8, dtype=np.int32)

    def run(micro, policy=None):
        tr = (LanguageTrainerBuilder(LanguageModel(cfg)).data(ArrayTokens(data)).optimizer(AdamW(lr=1e-3), policy)
              .micro_batch(micro).seq_len(16).global_batch_tokens(8 * 16).precision("f32").execution_policy("cpu")
              .log_every(0).build())
        tr.train(2)
        return tr
    a, b = run(8), run(2)
    assert b.accum == 4
    for p, q in zip(a.backend.params, b.backend.params):
        assert torch.allclose(p, q, atol=2e-6)
    pol = ParamGroupPolicy(decay_embeddings=False, rules=[ParamGroupRule("h.0.mlp", lr_scale=0.5, weight_decay_scale=0.0)])
    c = run(8, pol)
    names = c.backend.names
    assert c.backend.wd[names.index("wte")] == 0.0 and c.backend.wd[names.index("h.0.attn.qkv.weight")] == 1.0
    assert c.backend.wd[names.index("h.0.attn.qkv.bias")] == 0.0
    assert c.backend.lrs[names.index("h.0.mlp.up.weight")] == 0.5 and c.backend.wd[names.index("h.0.mlp.up.weight")] == 0.0


def test_loggers_schedule_eval_and_legacy_save_resume(tmp_path):
    cfg = preset("nano")
    cfg.n_layer, cfg.d_model, cfg.d_ff, cfg.max_position = 1, 32, 64, 16

    def build():
        return (LanguageTrainerBuilder(LanguageModel(cfg)).data(SyntheticTokens(256, 1), SyntheticTokens(256, 2))
                .optimizer(AdamW(lr=1e-3)).schedule(WarmupCosine(2, 10, 0.1)).micro_batch(2).seq_len(16)
                .precision("f32").execution_policy("cpu").eval_every(2, 1).log_every(1)
                .log_csv(str(tmp_path / "a.csv")).log_jsonl(str(tmp_path / "a.jsonl"))
                .log_tensorboard(str(tmp_path / "tb")).log_wandb(str(tmp_path / "wb")).build())
    tr = build()
    tr.train(4)
    assert tr.history[0].lr == pytest.approx(1e-3 / 3) and math.isfinite(tr.history[1].val_loss)
    assert len(open(tmp_path / "a.csv").read().splitlines()) == 5
    ev = read_tensorboard_scalars(tr.loggers[2].path)
    assert [e for e in ev if e[1] == "train/loss"][0][2] == pytest.approx(tr.history[0].loss, rel=1e-6)
    tr.save(str(tmp_path / "legacy.bin"))
    tr.train(2)
    want = [r.loss for r in tr.history[4:]]
    tr2 = build()
    tr2.resume(str(tmp_path / "legacy.bin"))
    tr2.train(2)
    assert [r.loss for r in tr2.history] == want          # bit-exact continuation
    assert tr.score_choices([1, 2, 3], [[4, 5], [6, 7]]) in (0, 1)


def test_nan_policy_skip_stop_and_spike_detector():
    cfg = preset("nano")
    cfg.n_layer, cfg.d_model, cfg.d_ff, cfg.max_position = 1, 32, 64, 16

    def build(policy):
        tr = (LanguageTrainerBuilder(LanguageModel(cfg)).data(SyntheticTokens(256, 1)).optimizer(AdamW(lr=1e-3))
              .micro_batch(2).seq_len(16).precision("f32").execution_policy("cpu").log_every(0)
              .nan_policy(NanOptions(policy=policy)).build())
        return tr
    tr = build("skip")
    tr.train(1)
    with torch.no_grad():
        tr.backend.params[0][0, 0] = float("nan")
    s = tr.train(1)
    assert tr.history[-1].skipped and tr.nan_events[-1].action == "skip" and "wte" in tr.nan_events[-1].where
    tr = build("stop")
    with torch.no_grad():
        tr.backend.params[0][0, 0] = float("nan")
    assert tr.train(3).stopped and len(tr.history) == 1
    tr = build("skip")
    tr._recent = [2.0 + 0.01 * (i % 3) for i in range(20)]
    from nexus_b200.train.lm_trainer import StepRecord
    tr._detect_spike(StepRecord(20, 9.0, 0, 0, 0, 0, 0, 0, 0, False))
    assert tr.spikes and tr.spikes[0].loss == 9.0


def test_classic_trainer_fit_early_stopping_and_nxs(tmp_path):
    torch.manual_seed(0)
    x = torch.randn(256, 2)
    y = (x[:, 0] * x[:, 1] > 0).long()
    model = nn.Sequential().add(nn.Linear(2, 16, True)).add(nn.ReLU()).add(nn.Linear(16, 2, True))
    tr = (TrainerBuilder(model).adamw(lr=2e-2, weight_decay=0.0).loss(0.0).gradient_clip_norm(1.0)
          .gradient_accumulation(2).callback(EarlyStopping(patience=50)).build())
    hist = tr.fit(DataLoader(x.numpy(), y.numpy(), 32, shuffle=True), DataLoader(x.numpy(), y.numpy(), 64), epochs=30)
    assert isinstance(hist[0], EpochStats) and hist[-1].train_loss < hist[0].train_loss and hist[-1].metrics["accuracy"] > 0.8
    p = str(tmp_path / "t.nxs")
    tr.save_nxs(p)
    model2 = nn.Sequential().add(nn.Linear(2, 16, True)).add(nn.ReLU()).add(nn.Linear(16, 2, True))
    tr2 = TrainerBuilder(model2).adamw(lr=2e-2, weight_decay=0.0).callback(EarlyStopping(patience=50)).build()
    tr2.load_nxs(p)
    assert tr2.epoch == tr.epoch and tr2.global_step == tr.global_step and tr2.optimizer.steps == tr.optimizer.steps
    assert torch.equal(model2(x), model(x)) and torch.equal(tr2.optimizer.m[0], tr.optimizer.m[0])
    assert nn.Sequential.load_nxs(p)(x).shape == (256, 2)      # the same file loads as a plain model


def test_legacy_language_trainer():
    cfg = preset("nano")
    cfg.n_layer, cfg.d_model, cfg.d_ff, cfg.max_position = 1, 32, 64, 16
    lt = LanguageTrainer(LanguageModel(cfg), lr=3e-3)
    vals = np.random.default_rng(1).integers(0, 256, size=4 * 16 * 3)
    losses = lt.fit(TokenRows(vals, 4, 16), epochs=3)
    assert len(losses) == 3 and losses[-1] < losses[0]


def test_in_process_data_parallel_step_equals_one_replica_on_the_whole_batch():
    """Three replicas, each on a third of the batch, gradients averaged: the same update as one model on the whole
    batch (mean loss over rows); the loop profile accounts for the time."""
    import copy
    from nexus_b200 import nn as nn_
    from nexus_b200.loss import CrossEntropy
    from nexus_b200.optim import SGD
    from nexus_b200.train import DataParallelStep, DataParallelTrainer, LoopProfile, all_reduce_mean
    torch.manual_seed(0)
    base = nn_.Sequential(nn_.Linear(4, 8, True), nn_.ReLU(), nn_.Linear(8, 3, True))
    single = copy.deepcopy(base)
    reps = [copy.deepcopy(base), copy.deepcopy(base), copy.deepcopy(base)]
    with torch.no_grad():                                  # replicas start different: construction must broadcast
        for p in reps[1].parameters():
            p.add_(1.0)
    x, y = torch.randn(6, 4), torch.randint(0, 3, (6,))
    step = DataParallelStep(reps, CrossEntropy().forward_backward, SGD(list(reps[0].parameters()), lr=0.1))
    o1 = SGD(list(single.parameters()), lr=0.1)
    for _ in range(3):
        got = step.step(x, y)
        pred = single(x)
        loss, grad = CrossEntropy().forward_backward(pred, y)
        o1.zero_grad()
        pred.backward(grad)
        o1.step()
        assert abs(got - float(loss)) < 1e-5
    for a, b, c in zip(single.parameters(), reps[0].parameters(), reps[2].parameters()):
        assert torch.allclose(a, b, atol=1e-5) and torch.equal(b, c)
    pr = step.profile
    assert pr.steps == 3 and pr.wall_s >= pr.optimizer_s > 0 and "forward_s=" in pr.report() and "%" in pr.report()
    tr = DataParallelTrainer(reps, CrossEntropy().forward_backward, SGD(list(reps[0].parameters()), lr=0.1))
    hist = tr.fit([(x, y), (x, y)], epochs=2)
    assert len(hist) == 2 and hist[1] < hist[0] and tr.profile.batches == 4
    ranks = [[1.0, 3.0], [3.0, 5.0]]
    all_reduce_mean(ranks)
    assert ranks == [[2.0, 4.0], [2.0, 4.0]] and LoopProfile().report().startswith("batches=0")


def test_nano_cpu_training_reproduces_the_stored_losses():
    """Regression anchor: the nano decoder (4 layers, d 128, vocabulary 256, 8 x 128 tokens, AdamW 3e-4) trained for
    six steps on CPU FP32 from fixed seeds gives the loss and gradient-norm sequence stored beside the tests.  A change
    of model maths, initialisation, loss, clipping or optimizer order shows up here first.  The tolerance leaves room
    for a different BLAS summation order on another CPU, nothing more."""
    import json
    import os
    torch.manual_seed(1234)
    cfg = preset("nano")
    toks = np.random.default_rng(7).integers(0, 256, size=8 * 128 * 6, dtype=np.int32)
    tr = (LanguageTrainerBuilder(LanguageModel(cfg)).data(ArrayTokens(toks)).optimizer(AdamW(lr=3e-4)).micro_batch(8)
          .seq_len(128).global_batch_tokens(8 * 128).precision("f32").execution_policy("cpu").log_every(0).build())
    tr.train(6)
    gold = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "nano_cpu_fp32_losses.json")))
    for got, want in zip(tr.history, zip(gold["loss"], gold["grad_norm"])):
        assert got.loss == pytest.approx(want[0], rel=2e-5) and got.grad_norm == pytest.approx(want[1], rel=2e-4)
    assert len(tr.history) == len(gold["loss"]) == 6


def test_native_event_file_encoding(tmp_path):
    """CRC32C known answers, a scalar record checked byte by byte against the TFRecord / protobuf wire format, and the
    reader refusing damaged files."""
    import struct
    from nexus_b200 import _native
    from nexus_b200.train.loggers import TensorBoardLogger, crc32c, masked_crc32c
    assert crc32c(b"123456789") == 0xE3069283 and crc32c(b"") == 0 and crc32c(bytes(32)) == 0x8A9136AA
    c = crc32c(b"abc")
    assert masked_crc32c(b"abc") == (((c >> 15) | (c << 17)) + 0xA282EAD8) & 0xFFFFFFFF
    rec = _native.tb_scalar_record(2.5, 300, "loss", 1.5)
    (n,) = struct.unpack_from("<Q", rec, 0)
    body = rec[12:12 + n]
    assert len(rec) == 16 + n and struct.unpack_from("<I", rec, 8)[0] == masked_crc32c(rec[:8])
    assert struct.unpack_from("<I", rec, 12 + n)[0] == masked_crc32c(body)
    value = b"\x0a\x04loss" + b"\x15" + struct.pack("<f", 1.5)                  # Value{1: tag, 2: simple_value}
    summary = b"\x0a" + bytes([len(value)]) + value                              # Summary{1: Value}
    want = b"\x09" + struct.pack("<d", 2.5) + b"\x10\xac\x02" + b"\x2a" + bytes([len(summary)]) + summary
    assert body == want                                                          # Event{1: wall_time, 2: step, 5: summary}
    lg = TensorBoardLogger(str(tmp_path))
    for i in range(3):
        lg.scalar("a/b", i * 0.5, i)
    lg.flush()
    assert read_tensorboard_scalars(lg.path) == [(0, "a/b", 0.0), (1, "a/b", 0.5), (2, "a/b", 1.0)]
    raw = bytearray(open(lg.path, "rb").read())
    raw[-6] ^= 1
    bad = tmp_path / "bad.tfevents"
    bad.write_bytes(bytes(raw))
    with pytest.raises(ValueError, match="checksum"):
        read_tensorboard_scalars(str(bad))
    bad.write_bytes(bytes(raw[:-3]))
    with pytest.raises(ValueError, match="truncated"):
        read_tensorboard_scalars(str(bad))
