"""`GptModel` behind the `LmBackend` interface: pinned double-buffered token upload, one device
sync per optimizer step, optional whole-step CUDA graph (inputs, every micro-step, optimizer and
the result tail are captured once and replayed; learning rate and micro-step weights are refreshed
from pinned host memory), data-parallel gradient all-reduce over NCCL.

Parity: include/nexus/cuda/lm_backend.hpp:52-141 and src/cuda/lm_backend.cpp:211-700 of the
reference (`GptLmBackend`).  The reference moves DDP gradients through the host; here they stay
on the device (NCCL / NVLink).
"""
from __future__ import annotations

import io
import os
from typing import List, Optional

import numpy as np
import torch

from ..lm.config import LmConfig
from ..models.gpt import PARAM_ORDER, AdamWConfig, GptModel
from ..ops import _cuda as K
from .lm_trainer import AdamW, LmBackend, LmNonFinite, LmParamInfo, LmStepResult

# Dense BF16 tensor peak per device, FLOP/s, keyed by compute capability major (MFU denominator).
PEAK_BF16_FLOPS = {10: 2.25e15, 9: 0.989e15, 8: 0.312e15}


class GptLmBackend(LmBackend):
    def __init__(self, config: LmConfig, micro_batch: int, seq_len: int, device="cuda", seed: int = 1234,
                 deterministic: bool = False, recompute: str = "none", recompute_every: int = 2,
                 optimizer: str = "adamw", master: str = "fp32", compute_dtype: str = "bf16",
                 dynamic_loss_scale=(False, 65536.0, 2000), ce_chunk_rows: Optional[int] = None):
        self.dev = torch.device(device)
        if self.dev.index is None:
            self.dev = torch.device("cuda", torch.cuda.current_device())
        torch.cuda.set_device(self.dev)
        # unknown or unimplemented modes raise inside GptModel: nothing is silently ignored
        self.model = GptModel(config, device=self.dev, seed=seed, recompute=recompute, recompute_every=recompute_every,
                              optimizer=optimizer, master=master, compute_dtype=compute_dtype,
                              dynamic_loss_scale=dynamic_loss_scale[0], loss_scale_init=dynamic_loss_scale[1],
                              loss_scale_growth_interval=dynamic_loss_scale[2], ce_chunk_rows=ce_chunk_rows)
        self.model.deterministic_embedding = deterministic
        self.B, self.T = micro_batch, seq_len
        self._host_tokens = [torch.empty((micro_batch, seq_len), dtype=torch.int32).pin_memory() for _ in range(2)]
        self._dev_tokens: List[torch.Tensor] = []
        self._copy_events = [None, None]
        self._slot = 0
        self._losses_dev = None
        self._result_host = torch.zeros(8, dtype=torch.float32).pin_memory()
        self._opt_cfg: Optional[AdamWConfig] = None
        self._pg = None
        self._sharded = None
        self._scales = None
        self._graph = None
        self._graph_enabled = False
        self._graph_key = None
        self._pending: List[tuple] = []
        self._loss_total = torch.zeros(1, dtype=torch.float32, device=self.dev)
        self.h2d_bytes = 0
        self.d2h_bytes = 0

    # -------------------------------------------------------------------------------- interface
    def device(self) -> str: return str(self.dev)
    def micro_batch(self) -> int: return self.B
    def seq_len(self) -> int: return self.T
    def vocab(self) -> int: return self.model.V

    def parameters(self) -> List[LmParamInfo]:
        m = self.model
        return [LmParamInfo(n, int(np.prod(m.shapes[n])), 2 if n.endswith("_w") and not n.startswith("ln") or n in ("wte", "wpe") else 1,
                            n in ("wte", "wpe")) for n in PARAM_ORDER]

    def set_param_scales(self, weight_decay, lr) -> None:
        self._scales = (list(weight_decay), list(lr))
        if self._sharded is not None:
            self._sharded.set_param_scales(weight_decay, lr)
        m = self.model
        segs = [(m.offsets[n], int(np.prod(m.shapes[n])), float(weight_decay[i]), float(lr[i]))
                for i, n in enumerate(PARAM_ORDER)]
        m.chunks = K.make_chunks(segs, device=self.dev)

    def reshape(self, micro_batch: int, seq_len: int) -> None:
        if (micro_batch, seq_len) != (self.B, self.T):
            self.__init_buffers(micro_batch, seq_len)

    def __init_buffers(self, B, T):
        self.B, self.T = B, T
        self._host_tokens = [torch.empty((B, T), dtype=torch.int32).pin_memory() for _ in range(2)]
        self._dev_tokens = []
        self._graph = None

    def _upload(self, tokens: np.ndarray, index: int) -> torch.Tensor:
        """Pinned host buffer (double-buffered) -> device, on the compute stream."""
        while len(self._dev_tokens) <= index:
            self._dev_tokens.append(torch.empty((self.B, self.T), dtype=torch.int32, device=self.dev))
        slot = self._slot
        self._slot ^= 1
        ev = self._copy_events[slot]
        if ev is not None:
            ev.synchronize()  # the previous copy out of this pinned buffer has finished
        host = self._host_tokens[slot]
        host.copy_(torch.from_numpy(np.ascontiguousarray(tokens, dtype=np.int32)))
        self._dev_tokens[index].copy_(host, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self._copy_events[slot] = ev
        self.h2d_bytes += host.numel() * 4
        return self._dev_tokens[index]

    def micro_step(self, tokens: np.ndarray, grad_weight: float, index: int, count: int) -> None:
        dev_tokens = self._upload(tokens, index)
        if self._graph_enabled:
            self._pending.append((index, grad_weight))
            if index == count - 1:
                self._count = count
            return
        self._ddp_arm(index == count - 1)
        self.model.forward_backward(dev_tokens, grad_scale=grad_weight, accumulate_loss=index > 0,
                                    loss_weight=grad_weight)
        if index == count - 1:
            self._ddp_finish()

    def optimizer_step(self, optimizer: AdamW, lr: float, clip: float) -> None:
        cfg = AdamWConfig(lr=lr, beta1=optimizer.beta1, beta2=optimizer.beta2, eps=optimizer.eps,
                          weight_decay=optimizer.weight_decay, grad_clip=clip)
        m = self.model
        if self._opt_cfg is None or (cfg.beta1, cfg.beta2, cfg.eps, cfg.weight_decay, cfg.grad_clip) != \
                (self._opt_cfg.beta1, self._opt_cfg.beta2, self._opt_cfg.eps, self._opt_cfg.weight_decay,
                 self._opt_cfg.grad_clip):
            m.set_optimizer(cfg)
            self._opt_cfg = cfg
        m.set_lr(lr)
        if self._graph_enabled:
            self._run_graph()
            return
        self._opt_step()

    def _ddp_arm(self, last_micro_step: bool) -> None:
        """Buckets are reduced only during the last micro-step of an accumulation window."""
        if getattr(self, "_ddp", None) is not None:
            self._ddp["armed"] = bool(last_micro_step)

    def _ddp_finish(self) -> None:
        """After the last backward pass: the optimizer's stream waits for the last bucket (bucketed form), or the
        whole gradient buffer is all-reduced at once (NCCL form)."""
        if self._pg is None or self._sharded is not None:
            return
        d = getattr(self, "_ddp", None)
        if d is not None:
            torch.cuda.current_stream().wait_event(d["done"])
            d["armed"] = False
            return
        self._pg.all_reduce_tensor(self.model.grads, "sum")

    def _opt_step(self) -> None:
        if self._sharded is not None:
            self._sharded.step()
        else:
            self.model.optimizer_step()

    def attach_fsdp(self, group, options=None) -> None:
        """Shards master weights, moments and the gradient reduction over ``group`` using the fused
        peer-memory kernels (reduce-scatter + norm exchange + AdamW + all-gather, no NCCL in the step)."""
        from ..parallel.symm import FusedShardedOptimizer, SymmetricWorkspace
        if self.model.optimizer_kind != "adamw" or self.model.master_mode != "fp32":
            raise ValueError("the sharded optimizer implements FP32-master AdamW; it cannot be combined with "
                             f"optimizer='{self.model.optimizer_kind}' / master='{self.model.master_mode}'")
        if self.model.dynamic_loss_scale:
            raise ValueError("the sharded optimizer does not run the loss-scale update; use dynamic_loss_scale with "
                             "data parallelism (attach_process_group) or on one GPU")
        self._pg_fsdp = group
        group.broadcast_tensor(self.model.params, 0)
        self.model.refresh_shadow()
        self._ws = SymmetricWorkspace(group)
        self._sharded = FusedShardedOptimizer(self.model, self._ws)
        if self._scales is not None:
            self._sharded.set_param_scales(*self._scales)

    def state_layout(self) -> str:
        return f"fsdp:2:{self._ws.n}" if self._sharded is not None else "replicated"

    def finish_step(self) -> LmStepResult:
        """One small D2H copy (loss, grad norm, found_inf) + one synchronisation."""
        m = self.model
        st = m.opt_state
        gn_off, fi_off = K.OptState.grad_norm.offset, K.OptState.found_inf.offset
        self._result_host[0:1].copy_(m.loss_buf, non_blocking=True)
        self._result_host[1:2].copy_(st[gn_off: gn_off + 4].view(torch.float32), non_blocking=True)
        self._result_host[2:3].copy_(st[fi_off: fi_off + 4].view(torch.int32).to(torch.float32), non_blocking=True)
        torch.cuda.current_stream().synchronize()
        self.d2h_bytes += 12
        K.check_status(self.dev)
        loss, gn, fi = (float(x) for x in self._result_host[:3])
        return LmStepResult(loss=loss, grad_norm=gn, skipped=fi != 0.0)

    def device_step(self, tokens_dev: torch.Tensor, lr: float) -> None:
        """One full optimizer step on tokens that already live on the device (no host traffic, no sync)."""
        m = self.model
        if self._opt_cfg is None:
            self._opt_cfg = AdamWConfig(lr=lr)
            m.set_optimizer(self._opt_cfg)
        world = self._ws.n if self._sharded is not None else (self._pg.size() if self._pg is not None else 1)
        self._ddp_arm(True)
        m.forward_backward(tokens_dev, grad_scale=1.0 / world)
        self._ddp_finish()
        self._opt_step()

    # ------------------------------------------------------------------------------- CUDA graph
    def compile(self, enabled: bool, mode: str = "default") -> None:
        self._graph_enabled = enabled
        self._graph = None

    def _run_graph(self) -> None:
        m = self.model
        count = self._count
        weights = [w for _, w in sorted(self._pending)]
        self._pending = []
        key = (count, tuple(weights))
        if self._graph is None or self._graph_key != key:
            # warm-up on a side stream (allocations, lazy module loading), then capture
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                self._graph_body(count, weights)
                K.scratch(1, "gemm_splitk", self.dev)
            torch.cuda.current_stream().wait_stream(s)
            torch.cuda.synchronize()
            # undo the warm-up's optimizer update: restore from a snapshot
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._graph_body(count, weights)
            self._graph, self._graph_key = g, key
            return  # the warm-up run already performed this step
        self._graph.replay()

    def _graph_body(self, count: int, weights) -> None:
        m = self.model
        for i in range(count):
            self._ddp_arm(i == count - 1)
            m.forward_backward(self._dev_tokens[i], grad_scale=weights[i], accumulate_loss=i > 0,
                               loss_weight=weights[i])
        self._ddp_finish()
        self._opt_step()

    # ------------------------------------------------------------------------------- evaluation
    def eval_loss(self, tokens: np.ndarray) -> float:
        t = torch.from_numpy(np.ascontiguousarray(tokens, dtype=np.int32)).to(self.dev)
        return self.model.loss(t)

    def token_losses(self, tokens: np.ndarray) -> np.ndarray:
        t = torch.from_numpy(np.ascontiguousarray(tokens, dtype=np.int32)).to(self.dev)
        logits = self.model.forward(t)[:, : self.model.V].float()
        tgt = torch.roll(t.long(), -1, dims=1).reshape(-1)
        l = torch.nn.functional.cross_entropy(logits, tgt, reduction="none").reshape(t.shape)
        l[:, -1] = 0.0
        return l.reshape(-1).cpu().numpy()

    def diagnose(self, tokens: np.ndarray) -> LmNonFinite:
        m = self.model
        for n in PARAM_ORDER:
            if int(K.count_nonfinite(m.p[n].reshape(-1)).item()):
                return LmNonFinite(True, f"param:{n}")
        for n in PARAM_ORDER:
            if int(K.count_nonfinite(m.g[n].reshape(-1)).item()):
                return LmNonFinite(True, f"grad:{n}")
        t = torch.from_numpy(np.ascontiguousarray(tokens, dtype=np.int32)).to(self.dev)
        m.forward(t)
        a = m._acts
        for l in range(m.L):
            for key in ("ln1", "qkv", "atty", "ln2", "fch"):
                if int(K.count_nonfinite(a[key][l].reshape(-1)).item()):
                    return LmNonFinite(True, f"activation:h{l}.{key}")
        return LmNonFinite(False, "")

    def layer_norms(self):
        m = self.model
        return [(n, float(m.p[n].norm()), float(m.g[n].norm())) for n in PARAM_ORDER]

    # ------------------------------------------------------------------------------------ state
    def save_state(self) -> bytes:
        """This rank's training state.  Replicated layout: the full FP32 master, both moments and the device
        optimizer state.  Sharded layout (after `attach_fsdp`): the live FP32 master and moments are the
        shards owned by the fused optimizer, so exactly those are written with their offset and count; the
        flat `model.params/m/v` buffers are not current in that mode and are never written."""
        m = self.model
        buf = io.BytesIO()
        if self._sharded is not None:
            sh = self._sharded
            torch.save({"layout": "fsdp", "world": sh.ws.n, "rank": sh.ws.rank, "off": sh.off, "count": sh.count,
                        "num_params": m.num_params, "master": sh.master.cpu(), "m": sh.m.cpu(), "v": sh.v.cpu(),
                        "opt": m.opt_state.cpu(), "step_count": m.step_count}, buf)
        elif m.optimizer_kind == "adamw":
            torch.save({"layout": "replicated", "params": m.params.cpu(), "m": m.m.cpu(), "v": m.v.cpu(),
                        "opt": m.opt_state.cpu(), "step_count": m.step_count}, buf)
        else:
            torch.save({"layout": "replicated", "kind": m.optimizer_kind, "tensors": m.optimizer_tensors(),
                        "opt": m.opt_state.cpu(), "step_count": m.step_count}, buf)
        return buf.getvalue()

    @staticmethod
    def _full_state(blobs):
        """Full (params, m, v, opt, step_count) on the host from one replicated blob or from every rank's shard."""
        ds = [torch.load(io.BytesIO(b), map_location="cpu") for b in blobs]
        first = ds[0]
        if first.get("layout", "replicated") == "replicated":
            return first["params"], first["m"], first["v"], first["opt"], first["step_count"]
        world = first["world"]
        if len(ds) != world or sorted(d["rank"] for d in ds) != list(range(world)):
            raise ValueError(f"sharded state needs the blobs of all {world} ranks, got {len(ds)}")
        n = first["num_params"]
        full = [torch.zeros(n, dtype=torch.float32) for _ in range(3)]
        covered = 0
        for d in ds:
            lo, cnt = d["off"], d["count"]
            for dst, key in zip(full, ("master", "m", "v")):
                dst[lo: lo + cnt] = d[key]
            covered += cnt
        if covered != n:
            raise ValueError(f"sharded state covers {covered} of {n} parameters")
        return full[0], full[1], full[2], first["opt"], first["step_count"]

    def _install_full_state(self, params, m_, v_, opt, step_count) -> None:
        m = self.model
        m.opt_state.copy_(opt)
        m.step_count = step_count
        if self._sharded is not None:
            sh = self._sharded
            sl = slice(sh.off, sh.off + sh.count)
            sh.master.copy_(params[sl])
            sh.m.copy_(m_[sl])
            sh.v.copy_(v_[sl])
            sh.install_weights(params.to(m.device))
        else:
            m.params.copy_(params)
            m.m.copy_(m_)
            m.v.copy_(v_)
            m.refresh_shadow()
        m.grads.zero_()

    def load_state(self, blob: bytes) -> None:
        """Restores what `save_state` wrote on this rank.  A shard written under the same sharding goes straight
        back into the fused optimizer's buffers and the BF16 weights / FP32 norm-and-bias tail are rebuilt from the
        gathered master (a collective: every rank of the group loads at the same point)."""
        d = torch.load(io.BytesIO(blob), map_location="cpu")
        m = self.model
        if d.get("layout", "replicated") == "fsdp":
            sh = self._sharded
            if sh is None or (sh.ws.n, sh.off, sh.count) != (d["world"], d["off"], d["count"]):
                raise ValueError("this blob is one shard of an fsdp:%d state; use load_resharded_state with every "
                                 "rank's blob to load it under a different layout" % d["world"])
            sh.master.copy_(d["master"])
            sh.m.copy_(d["m"])
            sh.v.copy_(d["v"])
            m.opt_state.copy_(d["opt"])
            m.step_count = d["step_count"]
            sh.install_weights(sh.gather_master())
            m.grads.zero_()
            return
        if "tensors" in d:
            if d.get("kind") != m.optimizer_kind:
                raise ValueError(f"state was written by optimizer '{d.get('kind')}', this model uses '{m.optimizer_kind}'")
            m.load_optimizer_tensors(d["tensors"])
            m.opt_state.copy_(d["opt"])
            m.step_count = d["step_count"]
            m.grads.zero_()
            return
        self._install_full_state(d["params"], d["m"], d["v"], d["opt"], d["step_count"])

    def load_resharded_state(self, blobs) -> None:
        """Loads a state written under another layout / world size: ``blobs`` holds every old rank's blob (one is
        enough when the old layout was replicated); the full vectors are rebuilt on the host and this rank keeps
        what its own layout owns."""
        self._install_full_state(*self._full_state(list(blobs)))

    def peak_memory_bytes(self) -> int: return int(torch.cuda.max_memory_allocated(self.dev))
    def reset_peak_memory(self) -> None: torch.cuda.reset_peak_memory_stats(self.dev)

    def peak_flops(self) -> float:
        major = torch.cuda.get_device_capability(self.dev)[0]
        return PEAK_BF16_FLOPS.get(major, 0.0)

    def flops_per_token(self, seq_len: int) -> float: return self.model.flops_per_token(seq_len)

    # ------------------------------------------------------------------------------ data parallel
    def attach_process_group(self, group, options=None) -> None:
        """Data-parallel gradient averaging over ``group``.  With ``options.bucketed`` (default when the group has
        peer-mapped memory) the gradients live in a symmetric buffer and are reduced bucket by bucket while the
        backward pass is still being executed: the model's backward hook fires after the head, after every layer and
        after the embedding; every ``options.bucket_layers`` layers the finished gradient ranges are all-reduced in
        place by the peer-memory kernel (two-shot, FP32) on a second stream that waits on an event of the compute
        stream; the optimizer waits for the last bucket.  Otherwise one NCCL all-reduce of the whole buffer follows the
        backward pass.  Parity: the staged, bucketed DDP of the reference's GPU backend
        (src/cuda/lm_backend.cpp:211-290, include/nexus/dist/ddp.hpp:36-110), which moves buckets through host memory."""
        self._pg = group
        self._ddp = None
        bucketed = getattr(options, "bucketed", None)
        if bucketed is None:
            bucketed = group.size() > 1 and str(self.dev).startswith("cuda") and getattr(group, "group", None) is not None \
                and os.environ.get("NEXUS_DDP_BUCKETED", "1") == "1"
        if not bucketed or group.size() == 1:
            return
        from ..parallel.symm import SymmetricWorkspace
        m = self.model
        ws = SymmetricWorkspace(group)
        gsym = ws.alloc(m.num_params, torch.float32)
        gsym.local.zero_()
        m.rebind_buffers(grads=gsym.local)
        self._ddp = {"ws": ws, "grads": gsym, "stream": torch.cuda.Stream(device=self.dev),
                     "bucket_layers": max(1, int(getattr(options, "bucket_layers", 4) or 4)), "pending": None,
                     "done": torch.cuda.Event(), "buckets": 0}
        m.set_backward_hook(self._ddp_hook)
        torch.cuda.synchronize()
        group.barrier()

    def _ddp_ranges(self, stage: int):
        """Gradient ranges (offset, count) that are complete once ``stage`` has been enqueued and belong to its bucket."""
        m, d = self.model, self._ddp
        bl = d["bucket_layers"]
        if stage == m.STAGE_HEAD:
            lo = m.offsets["lnf_w"]
            return [(lo, m.num_params - lo)]                       # lnf_w, lnf_b (and the padding after them)
        if stage == m.STAGE_EMBEDDING:
            return [(m.offsets["wte"], m.offsets["qkv_w"] - m.offsets["wte"])]   # wte, wpe
        if stage % bl == 0:                                         # layers [stage, min(stage + bl, L)) are complete
            return m.layer_grad_ranges(stage, min(stage + bl, m.L))
        return []

    def _ddp_hook(self, stage: int) -> None:
        d = self._ddp
        if not d.get("armed", False):
            return
        ranges = self._ddp_ranges(stage)
        if not ranges:
            return
        from ..parallel.symm import _table
        import ctypes as C
        ws, g = d["ws"], d["grads"]
        n, r = ws.n, ws.rank
        ev = torch.cuda.Event()
        ev.record()                                   # the stage's gradient kernels are in the compute stream
        with torch.cuda.stream(d["stream"]):
            d["stream"].wait_event(ev)
            ws.barrier()                              # every rank has produced this bucket
            for off, cnt in ranges:
                if cnt % 8 != 0 or off % 4 != 0:
                    raise ValueError("bucketed data parallelism needs gradient slices of a multiple of 8 elements "
                                     "that start on a 16-byte boundary; set NEXUS_DDP_BUCKETED=0 for this model")
                cnt8 = cnt
                per = (-(-cnt8 // n) + 7) // 8 * 8
                lo = min(cnt8, r * per)
                mine = max(0, min(per, cnt8 - lo))
                if mine > 0 and g.multicast:      # the sum is formed inside NVSwitch
                    K._check(K.lib().nx_comm_allreduce_multimem(C.c_void_p(g.multicast), C.c_int(K._DT[torch.float32]),
                                                                C.c_int64(off + lo), C.c_int64(mine), C.c_float(1.0),
                                                                K._stream()), "nx_comm_allreduce_multimem")
                elif mine > 0:
                    K._check(K.lib().nx_comm_allreduce_shard(C.byref(g.table), C.c_int(K._DT[torch.float32]), C.c_int(n),
                                                             C.byref(g.table), C.c_int(K._DT[torch.float32]), C.c_int(n),
                                                             C.c_int64(off + lo), C.c_int64(mine), C.c_float(1.0),
                                                             K._stream()), "nx_comm_allreduce_shard")
            ws.barrier()                              # the sums are in every rank's buffer
            d["done"].record()
        d["buckets"] += 1

    def broadcast_parameters(self) -> None:
        if self._pg is not None:
            self._pg.broadcast_tensor(self.model.params, 0)
            self.model.refresh_shadow()

    def data_parallel_group(self): return self._pg
