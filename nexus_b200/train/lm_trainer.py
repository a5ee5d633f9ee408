"""Language-model trainer: ``LanguageTrainerBuilder(...).data(...).optimizer(...).build().train(n)``.

One optimizer step = ``accum`` micro-steps (token-weighted: ``w_i = valid_i / sum(valid)``, global
over data-parallel ranks, gradients SUM-reduced) -> global-norm clip + AdamW -> one host/device
sync.  Around that: LR schedule, parameter groups (matrices decay, biases/norms do not; prefix
rules), evaluation, NaN policy (skip / stop / rollback with layer diagnosis), loss-spike detector
(median + k*1.4826*MAD), tokens/s and MFU, loggers, durable checkpoints and watchdog beats.

Parity: include/nexus/train/lm_trainer.hpp:73-552 and src/train/lm_trainer.cpp:1127-1700 of the
reference (builder surface, `LmBackend` interface, loop order, MFU formula).
"""
from __future__ import annotations

import math
import statistics
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence

import numpy as np
import torch

from .schedule import ConstantLr, LrSchedule


# ----------------------------------------------------------------------------------- configuration
@dataclass
class AdamW:
    lr: float = 6.0e-4
    beta1: float = 0.9
    beta2: float = 0.95
    eps: float = 1.0e-8
    weight_decay: float = 0.1


@dataclass
class ParamGroupRule:
    prefix: str
    lr_scale: float = 1.0
    weight_decay_scale: float = -1.0  # < 0: decided by the policy


@dataclass
class ParamGroupPolicy:
    decay: str = "matrices_only"  # "matrices_only" (nanoGPT rule) | "all" | "none"
    decay_embeddings: bool = True
    rules: List[ParamGroupRule] = field(default_factory=list)


@dataclass
class NanOptions:
    policy: str = "skip"  # "skip" | "stop" | "rollback"
    diagnose: bool = True
    snapshot_every: int = 100
    rollback_lr_factor: float = 0.5
    max_rollbacks: int = 3
    max_consecutive_skips: int = 16


@dataclass
class SpikeOptions:
    enabled: bool = True
    window: int = 64
    k: float = 6.0
    min_steps: int = 16


@dataclass
class LmParamInfo:
    name: str
    numel: int
    rank: int = 1
    embedding: bool = False


@dataclass
class LmStepResult:
    loss: float = float("nan")
    grad_norm: float = float("nan")
    skipped: bool = False
    micro_losses: List[float] = field(default_factory=list)
    loss_scale: float = 1.0


@dataclass
class LmNonFinite:
    found: bool = False
    where: str = ""


@dataclass
class StepRecord:
    step: int
    loss: float
    lr: float
    grad_norm: float
    tokens_per_s: float
    mfu: float
    step_ms: float
    data_ms: float
    peak_memory: int
    skipped: bool
    val_loss: float = float("nan")


@dataclass
class SpikeEvent:
    step: int
    loss: float
    median: float
    threshold: float
    sample_index: int = 0


@dataclass
class NanEvent:
    step: int
    where: str
    action: str


@dataclass
class TrainSummary:
    steps: int = 0
    final_loss: float = float("nan")
    tokens: int = 0
    seconds: float = 0.0
    stopped: bool = False
    skipped_steps: int = 0
    rollbacks: int = 0


# -------------------------------------------------------------------------------------- data sources
class TokenSource:
    """Yields rows of ``seq_len`` token ids; ``global_cursor`` makes resume and resharding exact."""

    def next_rows(self, rows: int, seq_len: int) -> np.ndarray:
        raise NotImplementedError

    def global_cursor(self) -> int:
        return 0

    def seek(self, cursor: int) -> None:
        pass


class SyntheticTokens(TokenSource):
    """Uniform random tokens in [0, vocab) from a counter-based stream (row index -> content)."""

    def __init__(self, vocab: int, seed: int = 0, rank: int = 0, world: int = 1):
        self.vocab, self.seed, self.rank, self.world = vocab, seed, rank, world
        self.cursor = 0

    def next_rows(self, rows: int, seq_len: int) -> np.ndarray:
        out = np.empty((rows, seq_len), dtype=np.int32)
        for r in range(rows):
            idx = (self.cursor + r) * self.world + self.rank
            rng = np.random.Generator(np.random.Philox(key=self.seed, counter=[idx, 0, 0, 0]))
            out[r] = rng.integers(0, self.vocab, size=seq_len, dtype=np.int32)
        self.cursor += rows
        return out

    def global_cursor(self) -> int:
        return self.cursor * self.world

    def seek(self, cursor: int) -> None:
        self.cursor = cursor // self.world


class ArrayTokens(TokenSource):
    """Walks a flat token array in windows of ``seq_len`` (wraps around), strided over ranks."""

    def __init__(self, tokens: Sequence[int], rank: int = 0, world: int = 1):
        self.tokens = np.asarray(tokens, dtype=np.int32)
        self.rank, self.world = rank, world
        self.cursor = 0

    def next_rows(self, rows: int, seq_len: int) -> np.ndarray:
        n = len(self.tokens)
        if n < seq_len:
            raise ValueError("ArrayTokens: fewer tokens than seq_len")
        out = np.empty((rows, seq_len), dtype=np.int32)
        nwin = max(1, n // seq_len)
        for r in range(rows):
            w = ((self.cursor + r) * self.world + self.rank) % nwin
            out[r] = self.tokens[w * seq_len: w * seq_len + seq_len]
        self.cursor += rows
        return out

    def global_cursor(self) -> int:
        return self.cursor * self.world

    def seek(self, cursor: int) -> None:
        self.cursor = cursor // self.world


class ShardTokens(TokenSource):
    """Token shards written by ``nexus_b200.tools.tokenize`` (NXTK files), memory-mapped and read by the native
    reader (`csrc/host/token_data.cpp`): windows of ``seq_len`` tokens numbered across the shards, optionally in a
    keyed per-epoch permutation, rank ``r`` of ``w`` taking the rows ``cursor * w + r``; a worker thread keeps
    ``prefetch`` batches decoded ahead.  The global cursor is the whole state (resume, resharding)."""

    def __init__(self, paths, seq_len: int, rank: int = 0, world: int = 1, seed: int = 0, shuffle: bool = False,
                 prefetch: int = 2):
        from .. import _native
        if isinstance(paths, (str, bytes)) or hasattr(paths, "__fspath__"):
            paths = [paths]
        self.paths = [str(p) for p in paths]
        self.seq_len = seq_len
        self._r = _native.TokenShards(self.paths, seq_len, rank, world, seed, shuffle, prefetch)

    def next_rows(self, rows: int, seq_len: int) -> np.ndarray:
        return self._r.next_rows(rows, seq_len)

    def next_into(self, ptr: int, rows: int, seq_len: int) -> None:
        """Decodes the next ``rows`` rows straight into caller memory (``rows * seq_len`` int32 at ``ptr``)."""
        if seq_len != self.seq_len:
            raise ValueError("ShardTokens: seq_len differs from the one the windows were cut for")
        self._r.next_into(ptr, rows)

    def global_cursor(self) -> int:
        return self._r.global_cursor()

    def seek(self, cursor: int) -> None:
        self._r.seek(cursor)

    def windows(self) -> int:
        return self._r.windows()

    def vocab(self) -> int:
        return self._r.vocab()


# ------------------------------------------------------------------------------------------ backend
class LmBackend:
    """What the trainer needs from a model + optimizer implementation."""

    def device(self) -> str: raise NotImplementedError
    def parameters(self) -> List[LmParamInfo]: raise NotImplementedError
    def set_param_scales(self, weight_decay: List[float], lr: List[float]) -> None: raise NotImplementedError
    def micro_batch(self) -> int: raise NotImplementedError
    def seq_len(self) -> int: raise NotImplementedError
    def vocab(self) -> int: raise NotImplementedError
    def reshape(self, micro_batch: int, seq_len: int) -> None: raise NotImplementedError
    def micro_step(self, tokens: np.ndarray, grad_weight: float, index: int, count: int) -> None: raise NotImplementedError
    def optimizer_step(self, optimizer: AdamW, lr: float, clip: float) -> None: raise NotImplementedError
    def finish_step(self) -> LmStepResult: raise NotImplementedError
    def eval_loss(self, tokens: np.ndarray) -> float: raise NotImplementedError
    def token_losses(self, tokens: np.ndarray) -> np.ndarray: raise NotImplementedError
    def diagnose(self, tokens: np.ndarray) -> LmNonFinite: return LmNonFinite()
    def save_state(self) -> bytes: raise NotImplementedError
    def load_state(self, blob: bytes) -> None: raise NotImplementedError
    def layer_norms(self): return []
    def peak_memory_bytes(self) -> int: return 0
    def reset_peak_memory(self) -> None: pass
    def peak_flops(self) -> float: return 0.0
    def flops_per_token(self, seq_len: int) -> float: return 0.0
    def attach_process_group(self, group, options=None) -> None: raise RuntimeError("backend has no data-parallel path")
    def broadcast_parameters(self) -> None: pass
    def attach_fsdp(self, group, options=None) -> None: raise RuntimeError("backend has no FSDP path")
    def data_parallel_group(self): return None
    def set_rng(self, seed: int, offset: int) -> None: pass
    def state_layout(self) -> str: return "replicated"
    def load_resharded_state(self, blobs: List[bytes]) -> None: raise RuntimeError("backend cannot reshard")
    def compile(self, enabled: bool, mode: str = "default") -> None: pass


def valid_targets(tokens: np.ndarray) -> int:
    """Shifted next-token targets: every position but the last of each row."""
    return int(tokens.shape[0] * (tokens.shape[1] - 1))


# ------------------------------------------------------------------------------------------ trainer
class LanguageTrainerBuilder:
    def __init__(self, model=None):
        self._model = model
        self._source = self._val = None
        self._opt, self._policy = AdamW(), ParamGroupPolicy()
        self._schedule = LrSchedule(ConstantLr())
        self._global_batch_tokens = 0
        self._micro_batch, self._seq_len = 1, 0
        self._clip = 1.0
        self._precision, self._master = "bf16", "fp32"
        self._recompute = "none"
        self._recompute_every = 2
        self._ce_chunk_rows = None
        self._optimizer_kind = "adamw"
        self._eval_every, self._eval_batches, self._log_every = 0, 4, 1
        self._seed = 1234
        self._deterministic = False
        self._compile, self._compile_mode = False, "default"
        self._nan, self._spike = NanOptions(), SpikeOptions()
        self._histogram_every = 0
        self._loggers: List = []
        self._after_backward: Optional[Callable] = None
        self._pg = self._ddp_options = None
        self._fsdp_pg = self._fsdp_options = None
        self._parallel_pg = self._parallel_cfg = None
        self._ckpt = None
        self._watchdog = None
        self._backend: Optional[LmBackend] = None
        self._device = "cuda" if torch.cuda.is_available() else "cpu"

    # fluent setters (names follow the reference builder)
    def data(self, source: TokenSource, val: Optional[TokenSource] = None): self._source, self._val = source, val; return self
    def optimizer(self, opt: AdamW, policy: Optional[ParamGroupPolicy] = None):
        self._opt = opt
        if policy is not None:
            self._policy = policy
        return self
    def schedule(self, s): self._schedule = s if isinstance(s, LrSchedule) else LrSchedule(s); return self
    def global_batch_tokens(self, n: int): self._global_batch_tokens = n; return self
    def micro_batch(self, n: int): self._micro_batch = n; return self
    def seq_len(self, n: int): self._seq_len = n; return self
    def grad_clip(self, c: float): self._clip = c; return self
    def precision(self, p: str, master: str = "fp32"): self._precision, self._master = p.lower(), master.lower(); return self
    def recompute(self, r: str, every: int = 2): self._recompute, self._recompute_every = r, every; return self
    def optimizer_kind(self, kind: str): self._optimizer_kind = kind; return self
    def ce_chunk_rows(self, rows: int):
        """GPU model backend: run the LM head and the loss over groups of whole sequences of at most ``rows`` rows
        (0: one pass), so that only one group's logits are alive."""
        self._ce_chunk_rows = int(rows); return self
    def dynamic_loss_scale(self, enabled: bool = True, init: float = 65536.0, growth_interval: int = 2000):
        """Device-resident dynamic loss scale of the GPU model backend (off by default; BF16 rarely needs it)."""
        self._dynamic_loss_scale = (bool(enabled), float(init), int(growth_interval))
        return self
    def eval_every(self, n: int, batches: int = 4): self._eval_every, self._eval_batches = n, batches; return self
    def log_every(self, n: int): self._log_every = n; return self
    def execution_policy(self, device: str): self._device = device; return self
    def seed(self, s: int): self._seed = s; return self
    def deterministic(self, d: bool = True): self._deterministic = d; return self
    def compile(self, enabled: bool = True, mode: str = "default"): self._compile, self._compile_mode = enabled, mode; return self
    def nan_policy(self, o: NanOptions): self._nan = o; return self
    def spike_detector(self, o: SpikeOptions): self._spike = o; return self
    def histogram_every(self, n: int): self._histogram_every = n; return self
    def logger(self, lg): self._loggers.append(lg); return self
    def log_console(self):
        from .loggers import ConsoleLogger
        return self.logger(ConsoleLogger())
    def log_csv(self, path):
        from .loggers import CsvLogger
        return self.logger(CsvLogger(path))
    def log_jsonl(self, path):
        from .loggers import JsonlLogger
        return self.logger(JsonlLogger(path))
    def log_tensorboard(self, logdir):
        from .loggers import TensorBoardLogger
        return self.logger(TensorBoardLogger(logdir))
    def log_wandb(self, run_dir):
        from .loggers import WandbOfflineLogger
        return self.logger(WandbOfflineLogger(run_dir))
    def after_backward(self, hook): self._after_backward = hook; return self
    def process_group(self, pg, options=None): self._pg, self._ddp_options = pg, options; return self
    def fsdp(self, pg, options=None): self._fsdp_pg, self._fsdp_options = pg, options; return self
    def parallel(self, pg, cfg): self._parallel_pg, self._parallel_cfg = pg, cfg; return self
    def checkpointing(self, options): self._ckpt = options; return self
    def watchdog(self, wd): self._watchdog = wd; return self
    def backend(self, b: LmBackend): self._backend = b; return self

    def build(self) -> "LanguageModelTrainer":
        if self._source is None:
            raise ValueError("LanguageTrainerBuilder: data(source) is required")
        if self._seq_len <= 0:
            raise ValueError("LanguageTrainerBuilder: seq_len is required")
        return LanguageModelTrainer(self)


def _make_backend(b: LanguageTrainerBuilder) -> LmBackend:
    if b._backend is not None:
        return b._backend
    model = b._model
    from ..lm.config import LmConfig
    if b._parallel_pg is not None:
        from ..parallel.parallel_backend import ParallelLmBackend
        return ParallelLmBackend(model, b._parallel_pg, b._parallel_cfg, b._micro_batch, b._seq_len, device=b._device)
    use_gpu = str(b._device).startswith("cuda") and torch.cuda.is_available()
    if isinstance(model, LmConfig):
        cfg = model
        if use_gpu and cfg.norm == "layernorm" and cfg.mlp == "gelu" and cfg.pos == "learned" and cfg.tie_embeddings \
                and cfg.bias and b._precision == "bf16":
            from .gpt_backend import GptLmBackend
            master = {"fp32": "fp32", "cast_per_forward": "cast_per_forward", "castperforward": "cast_per_forward"}.get(
                b._master, b._master)   # anything else ("none", ...) is refused by the model with a clear message
            return GptLmBackend(cfg, b._micro_batch, b._seq_len, device=b._device, seed=b._seed,
                                deterministic=b._deterministic, recompute=b._recompute,
                                recompute_every=b._recompute_every, optimizer=b._optimizer_kind, master=master,
                                dynamic_loss_scale=getattr(b, "_dynamic_loss_scale", (False, 65536.0, 2000)),
                                ce_chunk_rows=b._ce_chunk_rows)
        from ..lm.model import LanguageModel
        model = LanguageModel(cfg)
    from .torch_backend import TorchLmBackend
    return TorchLmBackend(model, b._micro_batch, b._seq_len, device=b._device, precision=b._precision,
                          recompute=b._recompute, seed=b._seed)


class LanguageModelTrainer:
    def __init__(self, b: LanguageTrainerBuilder):
        self.b = b
        self.backend = _make_backend(b)
        self.source, self.val = b._source, b._val
        self.opt, self.schedule, self.clip = b._opt, b._schedule, b._clip
        self.micro, self.T = b._micro_batch, b._seq_len
        self.pg = b._pg or b._fsdp_pg
        self.dp = self.pg.size() if self.pg is not None else 1
        self.rank = self.pg.rank() if self.pg is not None else 0
        if b._parallel_pg is not None:
            dpg = self.backend.data_parallel_group()
            self.pg = dpg
            self.dp = dpg.size() if dpg is not None else 1
            self.rank = b._parallel_pg.rank()
        per_micro = self.micro * self.T * self.dp
        gbt = b._global_batch_tokens or per_micro
        if gbt % per_micro != 0:
            raise ValueError("global_batch_tokens must be a multiple of micro_batch * seq_len * dp")
        self.accum = gbt // per_micro
        self.tokens_per_step = gbt
        # checkpoint manager is created BEFORE any collective (rank 0 cleans stale temp dirs)
        self.ckpt = None
        if b._ckpt is not None:
            from ..ckpt.checkpoint import CheckpointManager
            self.ckpt = CheckpointManager(b._ckpt, rank=self.rank, world=self.dp)
        self._apply_param_groups()
        if b._fsdp_pg is not None:
            self.backend.attach_fsdp(b._fsdp_pg, b._fsdp_options)
        elif b._pg is not None and self.dp > 1:
            self.backend.attach_process_group(b._pg, b._ddp_options)
            self.backend.broadcast_parameters()
        if b._compile:
            self.backend.compile(True, b._compile_mode)
        self.loggers = b._loggers if self.rank == 0 else []
        self.step = 0
        self.lr_factor = 1.0
        self.rng_offset = 0
        self.history: List[StepRecord] = []
        self.spikes: List[SpikeEvent] = []
        self.nan_events: List[NanEvent] = []
        self._recent: List[float] = []
        self._snapshot = None
        self._snapshot_step = -1
        self._consec_skips = 0
        self._rollbacks = 0
        self._prefetched = None
        self.watchdog = b._watchdog
        self.tokens_seen = 0

    # --------------------------------------------------------------------------- param groups
    def _apply_param_groups(self) -> None:
        infos = self.backend.parameters()
        pol = self.b._policy
        wd, lr = [], []
        for p in infos:
            if pol.decay == "all":
                d = 1.0
            elif pol.decay == "none":
                d = 0.0
            else:
                d = 1.0 if p.rank >= 2 else 0.0
            if p.embedding and not pol.decay_embeddings:
                d = 0.0
            s = 1.0
            for r in pol.rules:
                if p.name.startswith(r.prefix):
                    s = r.lr_scale
                    if r.weight_decay_scale >= 0.0:
                        d = r.weight_decay_scale
            wd.append(d)
            lr.append(s)
        self.backend.set_param_scales(wd, lr)

    # ------------------------------------------------------------------------------- data
    def _fetch(self) -> List[np.ndarray]:
        return [self.source.next_rows(self.micro, self.T) for _ in range(self.accum)]

    # ------------------------------------------------------------------------------- loop
    def train(self, max_steps: int) -> TrainSummary:
        t_begin = time.perf_counter()
        summary = TrainSummary()
        target = self.step + max_steps
        while self.step < target:
            t0 = time.perf_counter()
            batches = self._prefetched if self._prefetched is not None else self._fetch()
            self._prefetched = None
            data_ms = (time.perf_counter() - t0) * 1e3
            valid = [valid_targets(m) for m in batches]
            total_valid = sum(valid)
            if self.pg is not None and self.dp > 1:
                total_valid = int(self.pg.all_reduce_scalar(total_valid, "sum"))
            if total_valid <= 0:
                raise RuntimeError("no valid targets in this step")
            for i, m in enumerate(batches):
                self.backend.set_rng(self.b._seed, self.rng_offset)
                self.rng_offset += 1
                self.backend.micro_step(m, valid[i] / total_valid, i, self.accum)
            if self.b._after_backward is not None:
                self.b._after_backward(self)
            lr = self.opt.lr * self.schedule.factor(self.step) * self.lr_factor
            self.backend.optimizer_step(self.opt, lr, self.clip)
            self._prefetched = self._fetch()  # host prefetch while the device runs
            res = self.backend.finish_step()   # the single host/device sync of the step
            step_ms = (time.perf_counter() - t0) * 1e3
            if self.watchdog is not None:
                self.watchdog.beat(self.step, step_ms)
            loss = res.loss
            if self.pg is not None and self.dp > 1:
                loss = float(self.pg.all_reduce_scalar(loss, "sum"))
            tok_s = self.tokens_per_step / (step_ms * 1e-3)
            peak = self.backend.peak_flops()
            mfu = (self.backend.flops_per_token(self.T) * tok_s / (peak * self.dp)) if peak > 0 else float("nan")
            bad = res.skipped or not math.isfinite(loss)
            rec = StepRecord(self.step, loss, lr, res.grad_norm, tok_s, mfu, step_ms, data_ms,
                             self.backend.peak_memory_bytes(), bad)
            stop = False
            if bad:
                stop = self._handle_nan(batches, rec, summary)
            else:
                self._consec_skips = 0
                self._detect_spike(rec)
                if self.b._nan.policy == "rollback" and self.step % max(1, self.b._nan.snapshot_every) == 0:
                    self._snapshot, self._snapshot_step = self.backend.save_state(), self.step
            if self.b._eval_every > 0 and self.val is not None and (self.step + 1) % self.b._eval_every == 0:
                rec.val_loss = self.evaluate(self.b._eval_batches)
            self.history.append(rec)
            self.tokens_seen += self.tokens_per_step
            if self.b._log_every > 0 and self.step % self.b._log_every == 0:
                for lg in self.loggers:
                    lg.log(rec)
            self.step += 1
            if self.ckpt is not None and self.ckpt.due(self.step):
                self.save_checkpoint()
            summary.final_loss = loss
            if stop:
                summary.stopped = True
                break
        if self.ckpt is not None:
            self.ckpt.wait()
        for lg in self.loggers:
            lg.flush()
        summary.steps = self.step
        summary.tokens = self.tokens_seen
        summary.seconds = time.perf_counter() - t_begin
        summary.rollbacks = self._rollbacks
        summary.skipped_steps = sum(1 for r in self.history if r.skipped)
        return summary

    # ------------------------------------------------------------------------ anomaly handling
    def _handle_nan(self, batches, rec: StepRecord, summary: TrainSummary) -> bool:
        opts = self.b._nan
        where = ""
        if opts.diagnose:
            for m in batches:
                d = self.backend.diagnose(m)
                if d.found:
                    where = d.where
                    break
        if opts.policy == "stop":
            self.nan_events.append(NanEvent(self.step, where, "stop"))
            return True
        if opts.policy == "rollback" and self._snapshot is not None and self._rollbacks < opts.max_rollbacks:
            self.backend.load_state(self._snapshot)
            self.lr_factor *= opts.rollback_lr_factor
            self._rollbacks += 1
            self.nan_events.append(NanEvent(self.step, where, "rollback"))
            return False
        self._consec_skips += 1
        self.nan_events.append(NanEvent(self.step, where, "skip"))
        return self._consec_skips > opts.max_consecutive_skips

    def _detect_spike(self, rec: StepRecord) -> None:
        o = self.b._spike
        if o.enabled and len(self._recent) >= max(o.min_steps, 2):
            med = statistics.median(self._recent)
            mad = statistics.median([abs(x - med) for x in self._recent])
            thr = med + o.k * 1.4826 * mad
            if mad > 0 and rec.loss > thr:
                self.spikes.append(SpikeEvent(rec.step, rec.loss, med, thr, self.source.global_cursor()))
        self._recent.append(rec.loss)
        if len(self._recent) > o.window:
            self._recent.pop(0)

    # ------------------------------------------------------------------------------ evaluation
    def evaluate(self, batches: int = 4) -> float:
        src = self.val if self.val is not None else self.source
        tot, cnt = 0.0, 0
        for _ in range(batches):
            m = src.next_rows(self.micro, self.T)
            v = valid_targets(m)
            tot += self.backend.eval_loss(m) * v
            cnt += v
        if self.pg is not None and self.dp > 1:
            tot = float(self.pg.all_reduce_scalar(tot, "sum"))
            cnt = int(self.pg.all_reduce_scalar(cnt, "sum"))
        return tot / max(cnt, 1)

    def score_choices(self, context: Sequence[int], choices: Sequence[Sequence[int]]) -> int:
        """HellaSwag-style scoring: index of the continuation with the lowest mean token loss."""
        best, best_loss = 0, float("inf")
        for i, ch in enumerate(choices):
            seq = list(context) + list(ch)
            seq = (seq + [0] * self.T)[: self.T]
            rows = np.tile(np.asarray(seq, dtype=np.int32), (self.micro, 1))
            tl = self.backend.token_losses(rows).reshape(self.micro, self.T)[0]
            lo, hi = max(len(context) - 1, 0), min(len(context) + len(ch) - 1, self.T - 1)
            l = float(np.mean(tl[lo:hi])) if hi > lo else float("inf")
            if l < best_loss:
                best, best_loss = i, l
        return best

    # ------------------------------------------------------------------------------ persistence
    def trainer_state(self) -> dict:
        cursor = self.source.global_cursor()
        if self._prefetched is not None:  # the prefetched batch already advanced the source: rewind one step
            cursor -= self.accum * self.micro * self.dp
        return {"step": self.step, "lr_factor": self.lr_factor, "rng_seed": self.b._seed,
                "rng_offset": self.rng_offset, "train_cursor": cursor,
                "val_cursor": self.val.global_cursor() if self.val is not None else 0,
                "world": self.dp, "rank": self.rank, "tokens_seen": self.tokens_seen,
                "schedule_step": self.step, "accum_steps": self.accum, "micro_batch": self.micro,
                "seq_len": self.T, "global_batch_tokens": self.accum * self.micro * self.T * self.dp}

    def load_trainer_state(self, st: dict) -> None:
        self.step = int(st["step"])
        self.lr_factor = float(st.get("lr_factor", 1.0))
        self.rng_offset = int(st.get("rng_offset", 0))
        self.tokens_seen = int(st.get("tokens_seen", 0))
        self.source.seek(int(st.get("train_cursor", 0)))
        if self.val is not None:
            self.val.seek(int(st.get("val_cursor", 0)))
        self._prefetched = None

    def save_checkpoint(self) -> None:
        if self.ckpt is None:
            raise RuntimeError("checkpointing(options) was not configured")
        st = self.trainer_state()
        self.ckpt.save(self.step, st, self.backend.save_state(), layout=self.backend.state_layout())

    def resume_latest(self) -> bool:
        """Loads the newest complete checkpoint; reshards when the world size changed."""
        if self.ckpt is None:
            raise RuntimeError("checkpointing(options) was not configured")
        loaded = self.ckpt.load_latest()
        if loaded is None:
            return False
        if loaded.resharded:
            self.backend.load_resharded_state(loaded.backend_blobs)
        else:
            self.backend.load_state(loaded.backend_blobs[self.rank])
        self.load_trainer_state(loaded.state)
        return True

    def save(self, path: str) -> None:
        """Legacy single-file save (``path.rank<r>`` when multi-rank)."""
        import pickle
        p = path if self.dp == 1 else f"{path}.rank{self.rank}"
        with open(p, "wb") as f:
            pickle.dump({"state": self.trainer_state(), "backend": self.backend.save_state()}, f)

    def resume(self, path: str) -> None:
        import pickle
        p = path if self.dp == 1 else f"{path}.rank{self.rank}"
        with open(p, "rb") as f:
            d = pickle.load(f)
        self.backend.load_state(d["backend"])
        self.load_trainer_state(d["state"])
