"""ZeRO-0/1/2/3, FSDP and HSDP on flat parameter units.

Every unit (one transformer block, or the whole model) is flattened; rank r owns the shard
``[r*S, (r+1)*S)`` with ``S = ceil(N/dp)`` (zero padded) of the FP32 master weights and AdamW
moments.  All stages use the SAME reduce-scatter + all-gather pattern, so the trained weights are
bit-identical across stages:

* stage 0/1/2: parameters stay materialised; gradients are reduce-scattered to shards after
  backward, the shard is updated, updated parameters are all-gathered.
* stage 3 (FullShard): a unit's parameters exist only between its all-gather and the end of its
  forward (and again backward); gathers are prefetched one unit ahead with at most
  ``limit_all_gathers`` in flight; gradients are reduce-scattered and freed as soon as the unit's
  backward finishes.
* HSDP: shards inside a replica group, gradient shards all-reduced across replicas.

Mixed precision: gather and reduce in BF16, FP32 master shard.  The optimizer step computes the
global gradient norm from shard square sums (all-reduced in FP64), clips, runs AdamW on the shard.
State can be saved sharded and re-loaded under a different world size (`load_resharded`).
``trace()`` returns the ordered event log used by ordering tests.  Optimizer state / parameter
shards can be offloaded to an `NvmeStore`.

Parity: include/nexus/dist/fsdp.hpp:8-158, include/nexus/dist/fsdp_options.hpp:20-51 and
src/dist/fsdp.cpp:260-568 of the reference.
"""
from __future__ import annotations

import io
import math
from dataclasses import dataclass
from typing import Callable, List, Optional

import numpy as np
import torch

from ..fused.ops import adamw_multi_tensor


@dataclass
class FsdpOptions:
    stage: int = 3                 # 0..3 (3 = FullShard)
    unit: str = "per_block"        # "per_block" | "whole"
    limit_all_gathers: int = 2
    prefetch: bool = True
    mixed_precision: bool = False  # gather / reduce in BF16
    replica_group = None           # HSDP: process group across replicas
    nvme = None                    # NvmeStore for optimizer state offload
    comm: str = "auto"             # "nccl": collectives of the process group; "fused": on GPUs a unit's shards are
                                   # gathered by peer loads and its gradients reduce-scattered by an owner pull over
                                   # symmetric memory (no NCCL call per unit); "auto": fused when that is available


class _Unit:
    def __init__(self, name: str, params: List[torch.nn.Parameter], module, dp: int, rank: int):
        self.name, self.params, self.module = name, params, module
        self.numels = [p.numel() for p in params]
        self.shapes = [p.shape for p in params]
        self.N = sum(self.numels)
        self.S = (self.N + dp - 1) // dp
        dev = params[0].device
        full = torch.zeros(self.S * dp, dtype=torch.float32, device=dev)
        off = 0
        for p in params:
            full[off: off + p.numel()].copy_(p.detach().reshape(-1).float())
            off += p.numel()
        self.master = full[rank * self.S: (rank + 1) * self.S].clone()
        self.m = torch.zeros_like(self.master)
        self.v = torch.zeros_like(self.master)
        self.grad_shard = torch.zeros_like(self.master)
        self.gathered = True
        self.pending = None
        self.ready = 0


class FsdpEngine:
    def __init__(self, model: torch.nn.Module, group, options: Optional[FsdpOptions] = None):
        self.model, self.pg, self.o = model, group, options or FsdpOptions()
        self.dp, self.rank = group.size(), group.rank()
        self.units: List[_Unit] = []
        self.events: List[str] = []
        self.steps = 0
        self._build_units()
        self._ws = None
        self._setup_fused()
        group.barrier()
        for u in self.units:  # rank 0's initial values everywhere
            full = self._gather_master(u)
            self._unpack(u, full)
        self._install_hooks()
        if self.o.stage == 3:
            for u in self.units:
                self._release(u)

    # ------------------------------------------------------------------------------------ units
    def _build_units(self) -> None:
        blocks = getattr(self.model, "h", None)
        seen = set()
        if self.o.unit == "per_block" and blocks is not None:
            for i, blk in enumerate(blocks):
                ps = [p for p in blk.parameters() if p.requires_grad]
                seen.update(id(p) for p in ps)
                if ps:
                    self.units.append(_Unit(f"h{i}", ps, blk, self.dp, self.rank))
        rest = [p for p in self.model.parameters() if p.requires_grad and id(p) not in seen]
        if rest:
            self.units.insert(0, _Unit("root", rest, None, self.dp, self.rank))

    def _setup_fused(self) -> None:
        """Symmetric-memory plumbing of the fused form: one persistent shard slot per unit (1 / dp of the unit, in the
        gather dtype) and two rotating full-size gradient buffers shared by all units."""
        dev = self.units[0].master.device if self.units else torch.device("cpu")
        want = self.o.comm
        ok = dev.type == "cuda" and self.dp > 1 and hasattr(self.pg, "dist")      # a torch (NCCL) process group
        if want == "nccl" or (want == "auto" and not ok):
            return
        if not ok:
            raise ValueError("FsdpOptions.comm='fused' needs CUDA parameters and a torch process group")
        from .symm import SymmetricWorkspace
        self._ws = SymmetricWorkspace(self.pg)
        self._gdt = torch.bfloat16 if self.o.mixed_precision else torch.float32
        for u in self.units:
            u.S8 = (u.S + 7) // 8 * 8                        # 16-byte vectors in both dtypes
            u.shard_sym = self._ws.alloc(u.S8, self._gdt)
            u.shard_sym.local.zero_()
        big = max(u.S8 for u in self.units) * self.dp
        self._gsym = [self._ws.alloc(big, self._gdt) for _ in range(2)]
        self._gnext = 0
        torch.cuda.synchronize()

    def comm(self) -> str:
        return "fused" if self._ws is not None else "nccl"

    def trace(self) -> List[str]:
        return list(self.events)

    def layout(self) -> str:
        return f"fsdp:{self.o.stage}:{self.dp}"

    # ---------------------------------------------------------------------------- gather / free
    def _gather_master(self, u: _Unit, dtype=torch.float32) -> torch.Tensor:
        if self._ws is not None and dtype == self._gdt:
            return self._gather_fused(u)
        src = u.master.to(dtype) if dtype != torch.float32 else u.master
        out = torch.empty(u.S * self.dp, dtype=dtype, device=src.device)
        self.pg.all_gather_tensor(out, src.contiguous())
        return out

    def _gather_fused(self, u: _Unit) -> torch.Tensor:
        """This rank's shard goes into its symmetric slot (cast to the gather dtype); after the barrier one kernel
        reads every rank's slot over peer memory into the unit's full buffer."""
        import ctypes as C
        from ..ops import _cuda as K
        ws = self._ws
        u.shard_sym.local[: u.S].copy_(u.master)
        ws.barrier()
        full = torch.empty(u.S8 * self.dp, dtype=self._gdt, device=u.master.device)
        K._check(K.lib().nx_comm_gather_shards(C.byref(u.shard_sym.table), C.c_int(self.dp),
                                               C.c_int64(u.S8 * full.element_size()), K._p(full), K._stream()),
                 "nx_comm_gather_shards")
        ws.barrier()                                   # the slots may be rewritten
        if u.S8 == u.S:
            return full
        return full.view(self.dp, u.S8)[:, : u.S].reshape(-1)

    def _unpack(self, u: _Unit, full: torch.Tensor) -> None:
        off = 0
        with torch.no_grad():
            for p, n, shp in zip(u.params, u.numels, u.shapes):
                p.data = full[off: off + n].view(shp).to(p.dtype if p.data.numel() else torch.float32)
                off += n
        u.gathered = True

    def _gather(self, u: _Unit, why: str) -> None:
        if u.gathered:
            return
        self.events.append(f"gather:{u.name}:{why}")
        dt = torch.bfloat16 if self.o.mixed_precision else torch.float32
        full = self._gather_master(u, dt)
        self._unpack(u, full.float() if dt != torch.float32 else full)

    def _release(self, u: _Unit) -> None:
        if self.o.stage != 3 or not u.gathered:
            return
        self.events.append(f"release:{u.name}")
        for p in u.params:
            p.data = torch.empty(0, dtype=p.dtype, device=p.device)
        u.gathered = False

    # ------------------------------------------------------------------------------------ hooks
    def _install_hooks(self) -> None:
        self._sync = True
        order = {id(u): i for i, u in enumerate(self.units)}
        for u in self.units:
            if u.module is not None and self.o.stage == 3:
                u.module.register_forward_pre_hook(lambda m, a, u=u: self._pre_forward(u))
                u.module.register_forward_hook(lambda m, a, out, u=u: self._post_forward(u))
                u.module.register_full_backward_pre_hook(lambda m, g, u=u: self._gather(u, "bwd"))
            for p in u.params:
                p.register_post_accumulate_grad_hook(lambda t, u=u: self._on_grad(u))

    def _pre_forward(self, u: _Unit) -> None:
        self._gather(u, "fwd")
        if self.o.prefetch:
            i = self.units.index(u)
            inflight = sum(1 for x in self.units if x.gathered and x.module is not None)
            if i + 1 < len(self.units) and inflight < self.o.limit_all_gathers:
                self._gather(self.units[i + 1], "prefetch")

    def _post_forward(self, u: _Unit) -> None:
        if torch.is_grad_enabled():
            # parameters are needed again in backward: saved tensors hold views of the gathered buffer,
            # so the unit stays resident until its backward finished (freed in _launch_reduce)
            return
        self._release(u)

    def _on_grad(self, u: _Unit) -> None:
        u.ready += 1
        if u.ready == len(u.params):
            u.ready = 0
            if self._sync or self.o.stage == 3:
                self._launch_reduce(u)

    def _launch_reduce(self, u: _Unit) -> None:
        self.events.append(f"reduce:{u.name}")
        dt = torch.bfloat16 if self.o.mixed_precision else torch.float32
        flat = torch.zeros(u.S * self.dp, dtype=dt, device=u.master.device)
        off = 0
        for p, n in zip(u.params, u.numels):
            if p.grad is not None:
                flat[off: off + n].copy_(p.grad.reshape(-1).to(dt))
            off += n
        if self._ws is not None:
            shard = self._reduce_fused(u, flat)
        else:
            shard = torch.empty(u.S, dtype=dt, device=flat.device)
            self.pg.reduce_scatter_tensor(shard, flat, "sum")
        if self.o.replica_group is not None:
            self.o.replica_group.all_reduce_tensor(shard, "sum")
        u.grad_shard.add_(shard.float())
        for p in u.params:
            p.grad = None
        if u.module is not None:
            self._release(u)

    def _reduce_fused(self, u: _Unit, flat: torch.Tensor) -> torch.Tensor:
        """Reduce-scatter by owner pull: the unit's flat gradients go into one of two rotating symmetric buffers, and
        after the barrier this rank sums its own shard range over every rank's buffer (rank order, FP32 math)."""
        import ctypes as C
        from ..ops import _cuda as K
        from .symm import _table
        ws = self._ws
        g = self._gsym[self._gnext]
        self._gnext ^= 1
        ws.barrier()                                   # the readers of this buffer's previous use are done
        g.local[: flat.numel()].copy_(flat)
        ws.barrier()                                   # every rank's gradients are in place
        lo = self.rank * u.S
        # the kernel works on multiples of 8 elements: widen the range to the enclosing aligned window and cut
        a0 = lo // 8 * 8
        cnt = min(((lo + u.S + 7) // 8 * 8), (flat.numel() + 7) // 8 * 8) - a0
        win = torch.zeros(cnt, dtype=self._gdt, device=flat.device)
        own = _table([win.data_ptr() - a0 * win.element_size()])   # the kernel indexes outputs by global offset
        K._check(K.lib().nx_comm_allreduce_shard(C.byref(g.table), C.c_int(K._DT[self._gdt]), C.c_int(self.dp),
                                                 C.byref(own), C.c_int(K._DT[self._gdt]), C.c_int(1),
                                                 C.c_int64(a0), C.c_int64(cnt), C.c_float(1.0), K._stream()),
                 "nx_comm_allreduce_shard")
        return win[lo - a0: lo - a0 + u.S]

    # ------------------------------------------------------------------------------------- step
    def forward_backward(self, loss_fn: Callable[[], torch.Tensor], weight: float, sync: bool = True) -> torch.Tensor:
        self._sync = sync
        if self.o.stage == 3:
            for u in self.units:
                if u.module is None:
                    self._gather(u, "fwd")
        loss = loss_fn()
        (loss * weight).backward()
        if sync or self.o.stage == 3:
            for u in self.units:  # units whose parameters got no gradient this step
                if any(p.grad is not None for p in u.params):
                    u.ready = 0
                    self._launch_reduce(u)
            if self.o.stage == 3:
                for u in self.units:
                    self._release(u)
        return loss.detach()

    def step(self, opt, lr: float, clip: float, wd_scales=None, lr_scales=None):
        sq = sum(float(u.grad_shard.double().pow(2).sum()) for u in self.units)
        sq = float(self.pg.all_reduce_scalar(sq, "sum"))
        norm = math.sqrt(sq) if math.isfinite(sq) else float("nan")
        if not math.isfinite(norm):
            for u in self.units:
                u.grad_shard.zero_()
            return norm, True
        self.steps += 1
        pidx = {id(p): i for i, p in enumerate(p for p in self.model.parameters())}
        for u in self.units:
            # per-segment decay / LR scales: split the shard at parameter boundaries
            lo, hi = self.rank * u.S, (self.rank + 1) * u.S
            off = 0
            ps, gs, ms, vs, wds, lrs = [], [], [], [], [], []
            for p, n in zip(u.params, u.numels):
                a, b = max(lo, off), min(hi, off + n)
                if a < b:
                    sl = slice(a - lo, b - lo)
                    ps.append(u.master[sl]); gs.append(u.grad_shard[sl]); ms.append(u.m[sl]); vs.append(u.v[sl])
                    i = pidx.get(id(p), 0)
                    wds.append(1.0 if wd_scales is None else wd_scales[i] if i < len(wd_scales) else 1.0)
                    lrs.append(1.0 if lr_scales is None else lr_scales[i] if i < len(lr_scales) else 1.0)
                off += n
            if ps:
                adamw_multi_tensor(ps, gs, ms, vs, self.steps, lr, opt.beta1, opt.beta2, opt.eps, opt.weight_decay,
                                   clip, wds, lrs, grad_sq_sum=sq)
            u.grad_shard.zero_()
            if self.o.nvme is not None:
                self.o.nvme.write(f"{u.name}.m.rank{self.rank}", u.m.cpu().numpy().tobytes())
                self.o.nvme.write(f"{u.name}.v.rank{self.rank}", u.v.cpu().numpy().tobytes())
            if self.o.stage < 3:
                self.events.append(f"gather:{u.name}:params")
                self._unpack(u, self._gather_master(u))
                u.gathered = True
        return norm, False

    def full_parameters(self) -> List[torch.Tensor]:
        """All parameters materialised in FP32 (test helper)."""
        out = []
        for u in self.units:
            full = self._gather_master(u)
            off = 0
            for n, shp in zip(u.numels, u.shapes):
                out.append(full[off: off + n].view(shp).clone())
                off += n
        return out

    # ------------------------------------------------------------------------------ persistence
    def save_state(self) -> bytes:
        buf = io.BytesIO()
        torch.save({"dp": self.dp, "rank": self.rank, "steps": self.steps,
                    "units": [{"name": u.name, "N": u.N, "S": u.S, "master": u.master.cpu(), "m": u.m.cpu(),
                               "v": u.v.cpu()} for u in self.units]}, buf)
        return buf.getvalue()

    def load_state(self, blob: bytes) -> None:
        d = torch.load(io.BytesIO(blob), map_location="cpu")
        if d["dp"] != self.dp:
            raise RuntimeError("load_state: world size changed; use load_resharded")
        self.steps = d["steps"]
        for u, s in zip(self.units, d["units"]):
            u.master.copy_(s["master"]); u.m.copy_(s["m"]); u.v.copy_(s["v"])
        self._after_load()

    def load_resharded(self, blobs: List[bytes]) -> None:
        """Rebuilds this rank's shards from the shards of every old rank (any old world size)."""
        olds = sorted((torch.load(io.BytesIO(b), map_location="cpu") for b in blobs), key=lambda d: d["rank"])
        self.steps = olds[0]["steps"]
        for ui, u in enumerate(self.units):
            for key in ("master", "m", "v"):
                full = torch.cat([o["units"][ui][key] for o in olds])[: u.N]
                pad = torch.zeros(u.S * self.dp)
                pad[: u.N] = full
                getattr(u, key).copy_(pad[self.rank * u.S: (self.rank + 1) * u.S])
        self._after_load()

    def _after_load(self) -> None:
        for u in self.units:
            self._unpack(u, self._gather_master(u))
            if self.o.stage == 3 and u.module is not None:
                self._release(u)
