"""Symmetric (peer-mapped) device memory and the fused compute+communication paths built on it.

Every rank allocates buffers of identical layout through ``torch.distributed._symmetric_memory``
(the allocation / handle exchange plumbing) and maps all peers' copies; the kernels of
``csrc/cuda/comm_kernels.cu`` and the distributed GEMM then read and write peers directly over
NVLink 5 / NVSwitch.  Cross-GPU ordering uses flag arrays with bounded device-side waits.

`FusedShardedOptimizer` is the FSDP/ZeRO path of the flat GPT model: gradient reduce-scatter by
owner-pull in a fixed order, global-norm exchange, AdamW on the owned shard and the all-gather of
the updated BF16 weights, as four kernels and no NCCL call.

Parity (behaviour): FsdpEngine::step of src/dist/fsdp.cpp:474-568 in the reference (norm ->
all-reduce -> clip -> AdamW on the shard -> all-gather), which runs on CPU ranks there.
"""
from __future__ import annotations

import ctypes as C
import math
import os
from typing import List, Optional

import numpy as np
import torch

from ..ops import _cuda as K

MAX_PEERS = 8


class PeerTable(C.Structure):
    _fields_ = [("ptr", C.c_void_p * MAX_PEERS)]


class GemmDist(C.Structure):
    _fields_ = [("a_ptrs", C.c_void_p * MAX_PEERS), ("b_ptrs", C.c_void_p * MAX_PEERS),
                ("out_ptrs", C.c_void_p * MAX_PEERS), ("n_ranks", C.c_int32), ("rank", C.c_int32),
                ("a_sharded", C.c_int32), ("b_sharded", C.c_int32), ("out_scatter", C.c_int32)]


def _table(ptrs: List[int]) -> PeerTable:
    t = PeerTable()
    for i, p in enumerate(ptrs):
        t.ptr[i] = p
    return t


class SymmetricBuffer:
    """One symmetric allocation: ``local`` is this rank's tensor, ``ptrs[q]`` rank q's device address."""

    def __init__(self, local: torch.Tensor, ptrs: List[int], multicast: int = 0):
        self.local, self.ptrs = local, ptrs
        self.table = _table(ptrs)
        # NVSwitch multicast address of the allocation (0: the fabric or the driver offers none): one address that
        # stands for the same offset in every rank's copy, for the in-switch reductions (`multimem_all_reduce`)
        self.multicast = int(multicast)

    def offset_table(self, byte_offset: int) -> PeerTable:
        return _table([p + byte_offset for p in self.ptrs])


class SymmetricWorkspace:
    """Allocator of symmetric buffers for one process group + the group's flag array and barrier."""

    def __init__(self, pg):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        self.pg, self.symm_mem = pg, symm_mem
        self.rank, self.n = pg.rank(), pg.size()
        if self.n > MAX_PEERS:
            raise ValueError(f"at most {MAX_PEERS} ranks per symmetric group")
        self.group = pg.group if pg.group is not None else dist.group.WORLD
        self.device = pg.device
        try:
            symm_mem.enable_symm_mem_for_group(self.group.group_name)
        except Exception:
            pass
        # barrier generation, advanced on the device by every barrier-bearing kernel (graph-replay safe)
        self.counter = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.flags = self.alloc(MAX_PEERS, torch.int32)
        self.flags.local.zero_()
        self.slots = self.alloc(MAX_PEERS, torch.float64)
        self.slots.local.zero_()
        torch.cuda.synchronize()
        pg.barrier()

    def alloc(self, numel: int, dtype: torch.dtype) -> SymmetricBuffer:
        t = self.symm_mem.empty(int(numel), dtype=dtype, device=self.device)
        hdl = self.symm_mem.rendezvous(t, self.group)
        ptrs = [int(p) for p in hdl.buffer_ptrs]
        mc = 0
        if os.environ.get("NEXUS_B200_MULTIMEM", "1") != "0":
            try:
                mc = int(hdl.multicast_ptr) if getattr(hdl, "multicast_ptr", None) else 0
            except Exception:
                mc = 0
        return SymmetricBuffer(t, ptrs, mc)

    def check(self, op: str, *fields) -> None:
        """Validate mode of the process group (``NEXUS_DIST_DEBUG=1``): before a communicating kernel is launched, the
        ranks compare what they are about to launch (op name, sizes, dtypes) on the host and a difference raises a
        named ``DistError`` here, where the kernel would otherwise wait for a peer until its bounded wait gives up.
        Skipped while a CUDA graph is being captured (a host exchange cannot be captured)."""
        if getattr(self.pg, "validate", False) and not torch.cuda.is_current_stream_capturing():
            self.pg.check_call(op, *fields)

    def barrier(self) -> None:
        """Device-side barrier over the group on the current stream (bounded wait)."""
        K._check(K.lib().nx_comm_barrier(C.byref(self.flags.table), C.c_int(self.rank), C.c_int(self.n),
                                         K._p(self.counter), K._p(K.status_word(self.device)), K._stream()),
                 "nx_comm_barrier")


class FusedShardedOptimizer:
    """ZeRO-style sharded AdamW for a `GptModel` over symmetric memory (no NCCL in the step)."""

    def __init__(self, model, ws: SymmetricWorkspace):
        self.model, self.ws = model, ws
        n, r = ws.n, ws.rank
        N = model.num_params
        self.S = (math.ceil(N / n) + 63) // 64 * 64
        self.off = min(N, r * self.S)
        self.count = max(0, min(self.S, N - self.off))
        dev = model.device
        # gradients and the BF16 shadow move into symmetric memory so that peers can reach them
        self.grads = ws.alloc(N, torch.float32)
        self.shadow = ws.alloc(N, torch.bfloat16)
        self.grads.local.zero_()
        self.shadow.local.copy_(model.params_lp)
        model.rebind_buffers(params_lp=self.shadow.local, grads=self.grads.local)
        # the 1-D parameters (norm scales, biases) are read by the model in FP32: they live in a
        # symmetric FP32 buffer that the optimizer kernel of their owner fills on every rank
        self.tail_off = model.fp32_tail_offset()
        self.tail = ws.alloc(max(N - self.tail_off, 4), torch.float32)
        self.tail.local[: N - self.tail_off].copy_(model.params[self.tail_off:])
        model.rebind_fp32_tail(self.tail.local[: N - self.tail_off])
        sl = slice(self.off, self.off + self.count)
        self.master = model.params[sl].clone()
        self.m = torch.zeros(self.count, dtype=torch.float32, device=dev)
        self.v = torch.zeros(self.count, dtype=torch.float32, device=dev)
        self.gshard = torch.empty(max(self.count, 4), dtype=torch.float32, device=dev)
        nparts = int(K.lib().nx_comm_reduce_partials(C.c_int64(max(self.count, 1))))
        self.partials = torch.zeros(max(nparts, 1), dtype=torch.float64, device=dev)
        self.nparts = nparts
        self.chunks = None
        self.set_param_scales(None, None)
        torch.cuda.synchronize()
        ws.pg.barrier()

    def set_param_scales(self, weight_decay, lr) -> None:
        from ..models.gpt import DECAY, PARAM_ORDER
        m = self.model
        segs = []
        for i, name in enumerate(PARAM_ORDER):
            a, cnt = m.offsets[name], math.prod(m.shapes[name])
            lo, hi = max(a, self.off), min(a + cnt, self.off + self.count)
            if lo < hi:
                wd = (1.0 if name in DECAY else 0.0) if weight_decay is None else float(weight_decay[i])
                segs.append((lo, hi - lo, wd, 1.0 if lr is None else float(lr[i])))
        self.chunks = K.make_chunks(segs, device=m.device) if segs else None

    def step(self) -> None:
        ws, m, L = self.ws, self.model, K.lib()
        n, r = ws.n, ws.rank
        st = K._stream()
        status = K._p(K.status_word(m.device))
        # NEXUS_B200_SHARDED_MULTIMEM=1: the reduce-scatter and the all-gather go through NVSwitch (1 / n of the
        # gradients enters a GPU instead of (n - 1) / n, every result leaves it once).  Opt-in: equal results on two
        # GPUs, where it measured 0.5 ms per step slower than the peer-load form (20.83 against 20.34 ms); the in-switch
        # all-reduce only wins from four ranks up and this path has not been timed there.
        mc = bool(os.environ.get("NEXUS_B200_SHARDED_MULTIMEM", "0") == "1" and self.grads.multicast
                  and self.shadow.multicast and self.tail.multicast)
        ws.check("sharded_optimizer_step", self.grads.local.numel(), mc)
        ws.barrier()  # every rank has finished its backward pass
        if self.count > 0 and mc:
            K._check(L.nx_comm_reduce_shard_multimem(C.c_void_p(self.grads.multicast), C.c_int64(self.off),
                                                     C.c_int64(self.count), C.c_float(1.0), K._p(self.gshard),
                                                     K._p(self.partials), st), "nx_comm_reduce_shard_multimem")
        elif self.count > 0:
            K._check(L.nx_comm_reduce_shard(C.byref(self.grads.table), C.c_int(n), C.c_int64(self.off),
                                            C.c_int64(self.count), C.c_float(1.0), K._p(self.gshard),
                                            K._p(self.partials), st), "nx_comm_reduce_shard")
        K._check(L.nx_comm_norm_exchange(K._p(self.partials), C.c_int(self.nparts if self.count > 0 else 0),
                                         C.byref(ws.slots.table), C.byref(ws.flags.table), C.c_int(r), C.c_int(n),
                                         K._p(ws.counter), K._p(m.opt_state), status, st), "nx_comm_norm_exchange")
        m.grads.zero_()  # every peer has finished reading this rank's gradients
        if self.count > 0 and self.chunks is not None and mc:
            K._check(L.nx_comm_adamw_allgather_multimem(K._p(self.master), K._p(self.gshard), K._p(self.m), K._p(self.v),
                                                        C.c_void_p(self.shadow.multicast), C.c_void_p(self.tail.multicast),
                                                        C.byref(self.shadow.table), C.c_int(n),
                                                        C.c_int64(self.tail_off), C.c_int64(self.off),
                                                        K._p(self.chunks), C.c_int(self.chunks.nchunks),
                                                        K._p(m.opt_state), st), "nx_comm_adamw_allgather_multimem")
        elif self.count > 0 and self.chunks is not None:
            K._check(L.nx_comm_adamw_allgather(K._p(self.master), K._p(self.gshard), K._p(self.m), K._p(self.v),
                                               C.byref(self.shadow.table), C.byref(self.tail.table),
                                               C.c_int64(self.tail_off), C.c_int(n), C.c_int64(self.off),
                                               K._p(self.chunks), C.c_int(self.chunks.nchunks), K._p(m.opt_state),
                                               st), "nx_comm_adamw_allgather")
        ws.barrier()  # updated weights are visible on every rank
        m.step_count += 1

    def install_weights(self, full_master: torch.Tensor) -> None:
        """Rebuilds what the model reads (BF16 shadow, FP32 norm / bias tail) and the flat FP32 copy from a full
        master vector, e.g. after a checkpoint load."""
        m = self.model
        N = m.num_params
        full = full_master[:N].to(m.device, torch.float32)
        m.params.copy_(full)
        self.shadow.local.copy_(full)
        self.tail.local[: N - self.tail_off].copy_(full[self.tail_off:])

    def gather_master(self) -> torch.Tensor:
        """Full FP32 master vector (for checkpoints / tests) through NCCL."""
        out = torch.zeros(self.S * self.ws.n, dtype=torch.float32, device=self.model.device)
        pad = torch.zeros(self.S, dtype=torch.float32, device=self.model.device)
        pad[: self.count] = self.master
        self.ws.pg.all_gather_tensor(out, pad)
        return out[: self.model.num_params]


def fused_all_reduce(ws: SymmetricWorkspace, src: SymmetricBuffer, dst: SymmetricBuffer, count: int, *,
                     scale: float = 1.0, one_shot: Optional[bool] = None, multimem: Optional[bool] = None) -> None:
    """All-reduce (sum * scale) of ``src`` over the group into ``dst`` on every rank, with the dtype
    conversion fused into the reduction (e.g. BF16-compressed gradients in, FP32 out).  Two-shot
    (each rank reduces one slice and stores it to every rank) for large buffers, one-shot (each rank
    reduces the whole buffer for itself) for small ones; when both sides have one dtype and the allocation has an
    NVSwitch multicast address, the large form is reduced inside the switch (`multimem_all_reduce`; ``multimem=False``
    keeps the peer-load kernel).  ``count`` must be a multiple of 8."""
    n, r = ws.n, ws.rank
    if count % 8:
        raise ValueError("fused_all_reduce: count must be a multiple of 8 elements")
    ws.check("fused_all_reduce", count, src.local.dtype, dst.local.dtype, scale, one_shot, multimem)
    if one_shot is None:
        one_shot = count * src.local.element_size() <= (256 << 10)
    # same dtype on both sides and a multicast address: let NVSwitch do the sum (in place in `src`, then one local
    # copy when the result is wanted elsewhere); small buffers keep the one-shot form, which needs no second hop
    if multimem is None:
        multimem = not one_shot
    if multimem and src.multicast and src.local.dtype == dst.local.dtype and \
            src.local.dtype in (torch.float32, torch.bfloat16):
        multimem_all_reduce(ws, src, count, scale=scale)
        if dst is not src:
            dst.local[:count].copy_(src.local[:count])
        return
    dt_in, dt_out = K._DT[src.local.dtype], K._DT[dst.local.dtype]
    L = K.lib()
    ws.barrier()
    if one_shot:
        own = _table([dst.ptrs[r]])
        K._check(L.nx_comm_allreduce_shard(C.byref(src.table), C.c_int(dt_in), C.c_int(n), C.byref(own), C.c_int(dt_out),
                                           C.c_int(1), C.c_int64(0), C.c_int64(count), C.c_float(scale), K._stream()),
                 "nx_comm_allreduce_shard")
    else:
        per = (-(-count // n) + 7) // 8 * 8
        off = min(count, r * per)
        cnt = max(0, min(per, count - off))
        if cnt > 0:
            K._check(L.nx_comm_allreduce_shard(C.byref(src.table), C.c_int(dt_in), C.c_int(n), C.byref(dst.table),
                                               C.c_int(dt_out), C.c_int(n), C.c_int64(off), C.c_int64(cnt),
                                               C.c_float(scale), K._stream()), "nx_comm_allreduce_shard")
    ws.barrier()


def multimem_all_reduce(ws: SymmetricWorkspace, buf: SymmetricBuffer, count: int, *, offset: int = 0,
                        scale: float = 1.0) -> bool:
    """In-place all-reduce (sum * scale) of ``buf.local[offset : offset + count]`` over the group, reduced inside
    NVSwitch: every rank asks the switch for the sum of its slice (``multimem.ld_reduce``) and stores it into every
    rank's copy (``multimem.st``), so each byte crosses a GPU's links once per direction whatever the group size.
    FP32 or BF16 buffers; ``offset`` and ``count`` multiples of 8 elements.  Returns False (nothing done) when the
    allocation has no multicast address; the caller then uses ``fused_all_reduce``."""
    if not buf.multicast:
        return False
    ws.check("multimem_all_reduce", count, offset, buf.local.dtype, scale)
    if offset % 8 or count % 8:
        raise ValueError("multimem_all_reduce: offset and count must be multiples of 8 elements")
    n, r = ws.n, ws.rank
    per = (-(-count // n) + 7) // 8 * 8
    lo = min(count, r * per)
    mine = max(0, min(per, count - lo))
    ws.barrier()                                   # every rank's values are in its copy
    if mine > 0:
        K._check(K.lib().nx_comm_allreduce_multimem(C.c_void_p(buf.multicast), C.c_int(K._DT[buf.local.dtype]),
                                                    C.c_int64(offset + lo), C.c_int64(mine), C.c_float(scale),
                                                    K._stream()), "nx_comm_allreduce_multimem")
    ws.barrier()                                   # every slice has been written everywhere
    return True


def gemm_dist(ws: SymmetricWorkspace, a: torch.Tensor, b: torch.Tensor, out: torch.Tensor, *,
              a_peers: Optional[SymmetricBuffer] = None, b_peers: Optional[SymmetricBuffer] = None,
              out_peers: Optional[SymmetricBuffer] = None, a_mn: bool = False, b_mn: bool = False,
              a_shard: str = "rows", b_shard: str = "rows", scatter: str = "add_f32", accumulate: bool = False,
              bias=None, act=None, m: Optional[int] = None, n: Optional[int] = None, k: Optional[int] = None,
              a_offset: int = 0, b_offset: int = 0) -> torch.Tensor:
    """out = epilogue(A @ B^T) on the tcgen05 GEMM with operands and/or output spread over the group.

    ``a`` / ``b`` are this rank's (local) operands: K-major ``[rows, K]`` by default, MN-major ``[K, rows]`` with
    ``a_mn`` / ``b_mn``.  ``a_peers`` / ``b_peers`` name the symmetric buffer that holds every rank's part of that
    operand (``a_offset`` / ``b_offset``: element offset of the part inside the buffer):

    * ``*_shard="rows"`` (K-major): rank q holds row block q; tiles are fetched from their owners (all-gather -> GEMM);
    * ``*_shard="k"`` (MN-major): rank q holds K rows block q: the contraction dimension is spread over the ranks
      (weight gradients under sequence parallelism).

    ``out_peers``: GEMM -> reduce-scatter.  ``scatter="add_f32"`` adds partial tiles into the owner's FP32 buffer;
    ``scatter="slots"`` stores them as BF16 into slot ``rank`` of the owner's ``[n][M/n][N]`` buffer (sum them with
    `sum_slots` after a barrier: deterministic, half the NVLink bytes).  ``accumulate`` adds into ``out`` (beta = 1)."""
    g = K.GemmArgs()
    kk = k if k is not None else (a.shape[0] if a_mn else a.shape[1])
    a_rows = a.shape[1] if a_mn else a.shape[0]
    b_rows = b.shape[1] if b_mn else b.shape[0]
    a_mode = 0 if a_peers is None else (1 if a_shard == "rows" else 2)
    b_mode = 0 if b_peers is None else (1 if b_shard == "rows" else 2)
    M = m if m is not None else (a_rows * ws.n if a_mode == 1 else a_rows)
    N = n if n is not None else (b_rows * ws.n if b_mode == 1 else b_rows)
    if k is None and (a_mode == 2 or b_mode == 2):
        kk = (a.shape[0] if a_mode == 2 else b.shape[0]) * ws.n
    g.a, g.b, g.out = a.data_ptr(), b.data_ptr(), out.data_ptr()
    g.lda, g.ldb, g.ldo = a.stride(0), b.stride(0), out.stride(0)
    g.m, g.n, g.k, g.batch = M, N, kk, 1
    g.a_mn_major, g.b_mn_major = int(a_mn), int(b_mn)
    g.in_dtype, g.out_dtype = K._DT[a.dtype], K._DT[out.dtype]
    g.accumulate = int(accumulate)
    if bias is not None:
        g.bias, g.bias_dtype = bias.data_ptr(), K._DT[bias.dtype]
    g.act, g.alpha, g.split_k = K.ACT[act], 1.0, 1
    g.status = K.status_word(a.device).data_ptr()
    d = GemmDist()
    d.n_ranks, d.rank = ws.n, ws.rank
    ea, eb = a.element_size(), b.element_size()
    for q in range(ws.n):
        if a_peers is not None:
            d.a_ptrs[q] = a_peers.ptrs[q] + a_offset * ea
        if b_peers is not None:
            d.b_ptrs[q] = b_peers.ptrs[q] + b_offset * eb
        if out_peers is not None:
            d.out_ptrs[q] = out_peers.ptrs[q]
    d.a_sharded, d.b_sharded = a_mode, b_mode
    d.out_scatter = 0 if out_peers is None else (1 if scatter == "add_f32" else 2)
    K._check(K.lib().nx_gemm_dist(C.byref(g), C.byref(d), K._stream()), "nx_gemm_dist")
    return out


class GemmAg(C.Structure):
    _fields_ = [("gather", C.c_void_p * MAX_PEERS), ("flags", C.c_void_p * MAX_PEERS), ("counter", C.c_void_p),
                ("n_ranks", C.c_int32), ("rank", C.c_int32), ("copier_ctas", C.c_int32)]


class GatherSite:
    """Flags and generation counter shared by the all-gather GEMMs of one group whose row blocks have ``rows_per_rank``
    rows (any number of gather buffers can use one site, one call at a time)."""

    def __init__(self, ws: SymmetricWorkspace, rows_per_rank: int):
        if rows_per_rank % 256:
            raise ValueError("all-gather GEMM: rows per rank must be a multiple of 256")
        self.ws, self.rows = ws, rows_per_rank
        self.flags = ws.alloc(ws.n * (rows_per_rank // 128), torch.int32)
        self.flags.local.zero_()
        self.counter = torch.zeros(1, dtype=torch.int32, device=ws.device)
        torch.cuda.synchronize()
        ws.pg.barrier()


def gemm_ag(site: GatherSite, gather: SymmetricBuffer, b: torch.Tensor, out: torch.Tensor, *, k: int,
            b_mn: bool = False, bias=None, act=None, aux_out=None, copier_ctas: int = 8) -> torch.Tensor:
    """out[M, N] = epilogue(all-gather(A)[M, k] @ B^T) as ONE kernel.  ``gather`` is the group's peer-mapped gather
    buffer ([M, k] BF16 on every rank); this rank has already written its own row block ``rank`` into its local copy.
    Copier CTAs of the kernel push that block to every peer while the tensor-core CTAs work through the rows in their
    order of arrival; on return (stream order) this rank's copy holds the complete gathered A.  The caller separates
    two uses of the same gather buffer by ``ws.barrier()`` (peers may still be reading the old contents)."""
    ws = site.ws
    M = site.rows * ws.n
    ws.check("gemm_ag", M, k, tuple(b.shape), b_mn, out.dtype, act)
    a = gather.local.view(M, k)
    g = K.GemmArgs()
    g.a, g.b, g.out = a.data_ptr(), b.data_ptr(), out.data_ptr()
    g.lda, g.ldb, g.ldo = k, b.stride(0), out.stride(0)
    g.m, g.n, g.k, g.batch = M, (b.shape[1] if b_mn else b.shape[0]), k, 1
    g.a_mn_major, g.b_mn_major = 0, int(b_mn)
    g.in_dtype, g.out_dtype = K._DT[a.dtype], K._DT[out.dtype]
    if bias is not None:
        g.bias, g.bias_dtype = bias.data_ptr(), K._DT[bias.dtype]
    if aux_out is not None:
        g.aux_out, g.ld_aux = aux_out.data_ptr(), aux_out.stride(0)
    g.act, g.alpha, g.split_k = K.ACT[act], 1.0, 1
    g.status = K.status_word(a.device).data_ptr()
    d = GemmAg()
    for q in range(ws.n):
        d.gather[q] = gather.ptrs[q]
        d.flags[q] = site.flags.ptrs[q]
    d.counter = site.counter.data_ptr()
    d.n_ranks, d.rank, d.copier_ctas = ws.n, ws.rank, copier_ctas
    L = K.lib()
    K._check(L.nx_gemm_ag(C.byref(g), C.byref(d), K._stream()), "nx_gemm_ag")
    K._check(L.nx_comm_bump(K._p(site.counter), K._stream()), "nx_comm_bump")
    return out


class GemmRs(C.Structure):
    _fields_ = [("slots", C.c_void_p * MAX_PEERS), ("done", C.c_void_p), ("n_ranks", C.c_int32), ("rank", C.c_int32),
                ("copier_ctas", C.c_int32), ("copy_own", C.c_int32)]


def gemm_rs(ws: SymmetricWorkspace, a: torch.Tensor, b: torch.Tensor, partial: torch.Tensor, slots: SymmetricBuffer,
            done: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False, copier_ctas: int = 8,
            copy_own: bool = False) -> None:
    """GEMM -> reduce-scatter as ONE kernel: ``partial[M, N] = a @ b^T`` (BF16, local scratch) on the CTA-pair kernel,
    whose copier CTAs push every finished 256-row block into slot ``rank`` of the owner's ``slots`` buffer
    ([n][M/n][N] BF16).  ``done``: int32 [M / 256] scratch.  Follow with ``ws.barrier()`` and `sum_slots`; precede
    with ``ws.barrier()`` when the owners may still be reading the previous contents of their slots.  Unless
    ``copy_own``, the block this rank owns stays in ``partial`` only: pass `sum_slots` ``own=partial[rank block]``."""
    M = a.shape[1] if a_mn else a.shape[0]
    ws.check("gemm_rs", tuple(a.shape), tuple(b.shape), a_mn, b_mn, partial.dtype, copy_own)
    g = K.GemmArgs()
    g.a, g.b, g.out = a.data_ptr(), b.data_ptr(), partial.data_ptr()
    g.lda, g.ldb, g.ldo = a.stride(0), b.stride(0), partial.stride(0)
    g.m, g.n, g.k, g.batch = M, (b.shape[1] if b_mn else b.shape[0]), (a.shape[0] if a_mn else a.shape[1]), 1
    g.a_mn_major, g.b_mn_major = int(a_mn), int(b_mn)
    g.in_dtype, g.out_dtype = K._DT[a.dtype], K._DT[partial.dtype]
    g.act, g.alpha, g.split_k = K.ACT[None], 1.0, 1
    g.status = K.status_word(a.device).data_ptr()
    d = GemmRs()
    for q in range(ws.n):
        d.slots[q] = slots.ptrs[q]
    d.done = done.data_ptr()
    d.n_ranks, d.rank, d.copier_ctas, d.copy_own = ws.n, ws.rank, copier_ctas, int(copy_own)
    done.zero_()
    K._check(K.lib().nx_gemm_rs(C.byref(g), C.byref(d), K._stream()), "nx_gemm_rs")


def sum_slots(slots: torch.Tensor, n: int, rows: int, cols: int, out: torch.Tensor, *, residual=None,
              out_lp: Optional[torch.Tensor] = None, own: Optional[torch.Tensor] = None, own_rank: int = 0) -> torch.Tensor:
    """out = residual + sum of the n BF16 slots ``slots[q][rows][cols]`` in rank order (the owner's half of the slot
    form of GEMM -> reduce-scatter); ``out_lp`` receives a BF16 copy.  ``own`` ([rows, cols] BF16) stands in for slot
    ``own_rank`` (this rank's own partial sums, which never left its memory)."""
    K._check(K.lib().nx_comm_sum_slots(K._p(slots), C.c_int(n), C.c_int(rows), C.c_int(cols), C.c_int64(cols),
                                       K._p(residual), C.c_int(K._DT[residual.dtype] if residual is not None else 0),
                                       C.c_int64(residual.stride(0) if residual is not None else 0), K._p(out),
                                       C.c_int(K._DT[out.dtype]), C.c_int64(out.stride(0)), K._p(out_lp),
                                       C.c_int64(out_lp.stride(0) if out_lp is not None else 0), K._p(own),
                                       C.c_int(own_rank), K._stream()),
             "nx_comm_sum_slots")
    return out


def moe_dispatch(ws, x, token_of, expert_of, slot_of, bufs: SymmetricBuffer, local_experts: int, capacity: int,
                 row_scale=None, rows_per_token: int = 1):
    rows = expert_of.numel()
    ws.check("moe_dispatch", x.shape[1], local_experts, capacity, rows_per_token, x.dtype)
    K._check(K.lib().nx_moe_dispatch(K._p(x), K._p(token_of), K._p(expert_of), K._p(slot_of), C.byref(bufs.table),
                                     C.c_int(rows), C.c_int(x.shape[1]), C.c_int(local_experts),
                                     C.c_int(capacity), C.c_int(ws.rank), C.c_int(ws.n), K._p(row_scale),
                                     C.c_int(rows_per_token), K._stream()), "nx_moe_dispatch")


def moe_combine(ws, bufs: SymmetricBuffer, expert, slot, gate, y, local_experts: int, capacity: int):
    tokens, top_k = expert.shape
    ws.check("moe_combine", top_k, y.shape[1], local_experts, capacity, y.dtype)
    K._check(K.lib().nx_moe_combine(C.byref(bufs.table), K._p(expert), K._p(slot), K._p(gate), K._p(y),
                                    C.c_int(tokens), C.c_int(top_k), C.c_int(y.shape[1]), C.c_int(local_experts),
                                    C.c_int(capacity), K._stream()), "nx_moe_combine")


# ---------------------------------------------------------------------------------------------- context parallel
class RingAttention:
    """Ring attention (forward and backward) over symmetric memory: every rank publishes its K/V chunk once; each step
    runs ONE attention kernel whose TMA loads read the owner's K/V straight from peer memory (plain,
    non-multicast loads) and whose epilogue merges the chunk into the running FP32 output / LSE.
    Layouts: ``contiguous`` (rank r holds tokens [r*Tl, (r+1)*Tl)) or ``zigzag`` (rank r holds chunks
    r and 2n-1-r of 2n, which balances the causal work).  Parity: src/dist/context_parallel.cpp
    (ring_attention_forward) of the reference, which exchanges blocks with send_recv on CPU ranks."""

    def __init__(self, ws: SymmetricWorkspace, B: int, Tl: int, Hkv: int, D: int, layout: str = "contiguous"):
        if layout not in ("contiguous", "zigzag"):
            raise ValueError("layout must be 'contiguous' or 'zigzag'")
        if layout == "zigzag" and Tl % 2:
            raise ValueError("zigzag needs an even local length")
        self.ws, self.layout, self.shape = ws, layout, (B, Tl, Hkv, D)
        n = B * Tl * Hkv * D
        self.k_sym = ws.alloc(n, torch.bfloat16)
        self.v_sym = ws.alloc(n, torch.bfloat16)
        hdl_k = ws.symm_mem.rendezvous(self.k_sym.local, ws.group)
        hdl_v = ws.symm_mem.rendezvous(self.v_sym.local, ws.group)
        self.k_peer = [hdl_k.get_buffer(q, (B, Tl, Hkv, D), torch.bfloat16) for q in range(ws.n)]
        self.v_peer = [hdl_v.get_buffer(q, (B, Tl, Hkv, D), torch.bfloat16) for q in range(ws.n)]

    def forward(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = True):
        """q [B, Tl, H, D], k/v [B, Tl, Hkv, D] (this rank's tokens).  Returns (o BF16, lse FP32 [B, H, Tl])."""
        ws, n, r = self.ws, self.ws.n, self.ws.rank
        B, Tl, H, D = q.shape
        ws.check("ring_attention_forward", tuple(q.shape), tuple(k.shape), causal, self.layout)
        self.k_sym.local.view(self.shape).copy_(k)
        self.v_sym.local.view(self.shape).copy_(v)
        ws.barrier()                                   # every rank's K/V chunk is published
        dev = q.device
        if not causal or self.layout == "contiguous":
            acc_o = torch.zeros((B, Tl, H, D), dtype=torch.float32, device=dev)
            acc_l = torch.full((B, H, Tl), float("-inf"), dtype=torch.float32, device=dev)
            out = torch.empty_like(q)
            for s in range(n):
                src = (r - s) % n                      # own chunk first, then around the ring
                if causal and src > r:
                    continue                           # entirely in the future
                K.attention_fwd(q, self.k_peer[src], self.v_peer[src], causal=causal and src == r, out=out,
                                merge_o=acc_o, merge_lse=acc_l)
            ws.barrier()                               # nobody reads this rank's K/V any more
            return out, acc_l
        # zigzag: rank x holds chunk x (first half of its tokens) and chunk 2n-1-x (second half)
        half = Tl // 2
        acc = [(torch.zeros((B, half, H, D), dtype=torch.float32, device=dev),
                torch.full((B, H, half), float("-inf"), dtype=torch.float32, device=dev)) for _ in range(2)]
        o_half = [torch.empty((B, half, H, D), dtype=torch.bfloat16, device=dev) for _ in range(2)]
        for s in range(n):
            src = (r - s) % n
            kk, vv = self.k_peer[src], self.v_peer[src]
            for qi, qc in enumerate((r, 2 * n - 1 - r)):
                for ki, kc in enumerate((src, 2 * n - 1 - src)):
                    if kc > qc:
                        continue
                    K.attention_fwd(q[:, qi * half: (qi + 1) * half], kk[:, ki * half: (ki + 1) * half],
                                    vv[:, ki * half: (ki + 1) * half], causal=(kc == qc), out=o_half[qi],
                                    merge_o=acc[qi][0], merge_lse=acc[qi][1])
        ws.barrier()
        return torch.cat(o_half, dim=1), torch.cat([acc[0][1], acc[1][1]], dim=2)


    # ------------------------------------------------------------------ backward
    def _grad_buffers(self):
        """Symmetric BF16 buffer [n owners][dk | dv][B, Tl, Hkv, D]: slot j collects what this rank's queries
        contribute to the keys / values of rank j; the owners pull and sum their slots at the end."""
        if not hasattr(self, "g_sym"):
            B, Tl, Hkv, D = self.shape
            self.slot = 2 * B * Tl * Hkv * D
            self.g_sym = self.ws.alloc(self.ws.n * self.slot, torch.bfloat16)
        return self.g_sym

    def backward(self, q, k, v, o, lse, d_o, causal: bool = True):
        """Gradients of ``forward``.  q/o/d_o [B, Tl, H, D], k/v [B, Tl, Hkv, D], lse [B, H, Tl] as returned by
        ``forward`` (the log-sum-exp over ALL keys, so every chunk's probabilities come out right).  Each step
        runs the two backward kernels on one rank's K/V chunk read from peer memory; dQ accumulates locally in
        FP32, the chunk's dK/dV go into that owner's slot of a symmetric buffer, and after a barrier every rank
        sums its own slot over the peers with the fused reduce kernel.  Returns (dq, dk, dv) in BF16.
        Parity: src/dist/context_parallel.cpp (ring_attention_backward) of the reference."""
        ws, n, r = self.ws, self.ws.n, self.ws.rank
        B, Tl, H, D = q.shape
        Hkv = self.shape[2]
        g = self._grad_buffers()
        self.k_sym.local.view(self.shape).copy_(k)
        self.v_sym.local.view(self.shape).copy_(v)
        g.local.zero_()
        ws.barrier()                                   # K/V published; nobody still reads the previous slots
        slots = g.local.view(n, 2, B, Tl, Hkv, D)
        dq_acc = torch.zeros((B, Tl, H, D), dtype=torch.float32, device=q.device)
        if not causal or self.layout == "contiguous":
            dq_p = torch.empty_like(q)
            for s in range(n):
                src = (r - s) % n
                if causal and src > r:
                    continue
                K.attention_bwd(q, self.k_peer[src], self.v_peer[src], o, lse, d_o, causal=causal and src == r,
                                dq=dq_p, dk=slots[src, 0], dv=slots[src, 1])
                dq_acc += dq_p
        else:
            half = Tl // 2
            dq_p = torch.empty((B, half, H, D), dtype=q.dtype, device=q.device)
            dk_p = torch.empty((B, half, Hkv, D), dtype=q.dtype, device=q.device)
            dv_p = torch.empty_like(dk_p)
            for s in range(n):
                src = (r - s) % n
                kk, vv = self.k_peer[src], self.v_peer[src]
                for qi, qc in enumerate((r, 2 * n - 1 - r)):
                    qs = slice(qi * half, (qi + 1) * half)
                    for ki, kc in enumerate((src, 2 * n - 1 - src)):
                        if kc > qc:
                            continue
                        ks = slice(ki * half, (ki + 1) * half)
                        K.attention_bwd(q[:, qs], kk[:, ks], vv[:, ks], o[:, qs], lse[:, :, qs].contiguous(),
                                        d_o[:, qs], causal=(kc == qc), dq=dq_p, dk=dk_p, dv=dv_p)
                        dq_acc[:, qs] += dq_p
                        slots[src, 0][:, ks] += dk_p
                        slots[src, 1][:, ks] += dv_p
        ws.barrier()                                   # every rank's slots are complete
        dkv = torch.empty((2, B, Tl, Hkv, D), dtype=torch.bfloat16, device=q.device)
        own = _table([dkv.data_ptr() - r * self.slot * 2])   # the kernel indexes outputs by global offset
        K._check(K.lib().nx_comm_allreduce_shard(C.byref(g.table), C.c_int(K._DT[torch.bfloat16]), C.c_int(n),
                                                 C.byref(own), C.c_int(K._DT[torch.bfloat16]), C.c_int(1),
                                                 C.c_int64(r * self.slot), C.c_int64(self.slot), C.c_float(1.0),
                                                 K._stream()), "nx_comm_allreduce_shard")
        ws.barrier()                                   # slots may be overwritten again
        return dq_acc.to(q.dtype), dkv[0], dkv[1]


class _RingAttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, ring, causal):
        o, lse = ring.forward(q, k, v, causal)
        ctx.ring, ctx.causal = ring, causal
        ctx.save_for_backward(q, k, v, o, lse)
        return o

    @staticmethod
    def backward(ctx, d_o):
        q, k, v, o, lse = ctx.saved_tensors
        dq, dk, dv = ctx.ring.backward(q, k, v, o, lse, d_o.contiguous(), ctx.causal)
        return dq, dk, dv, None, None


def ring_attention_autograd(ws: SymmetricWorkspace, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                            layout: str = "contiguous", causal: bool = True) -> torch.Tensor:
    """Differentiable ring attention over the group of ``ws`` (q [B, Tl, H, D], k / v [B, Tl, Hkv, D], BF16, this rank's
    tokens in the given layout): `RingAttention.forward` / `.backward` under one autograd node.  The symmetric K / V
    and gradient buffers are kept per shape on the workspace.  Used by `ParallelLm` on GPUs when cp > 1."""
    B, Tl, Hkv, D = k.shape
    cache = ws.__dict__.setdefault("_rings", {})
    key = (B, Tl, Hkv, D, layout)
    ring = cache.get(key)
    if ring is None:
        ring = cache[key] = RingAttention(ws, B, Tl, Hkv, D, layout)
    return _RingAttnFn.apply(q.contiguous(), k.contiguous(), v.contiguous(), ring, causal)


class _VocabParallelCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, targets, ws, vocab_start, ignore_index):
        rows, vl = logits.shape
        lf = logits.float()
        lmax = lf.max(dim=1).values
        lse_local = torch.exp(lf - lmax[:, None]).sum(dim=1)
        local_t = targets.long() - vocab_start
        mine = (local_t >= 0) & (local_t < vl)
        tlogit = torch.where(mine, lf.gather(1, local_t.clamp(0, vl - 1)[:, None])[:, 0], torch.zeros_like(lmax))
        stats = torch.stack([lmax, lse_local, tlogit], dim=1).contiguous()
        cache = ws.__dict__.setdefault("_vocab_ce", {})
        if cache.get("rows") != rows:
            cache["rows"] = rows
            cache["table"] = ws.alloc(ws.n * rows * 3, torch.float32)
        merged = torch.empty((rows, 3), dtype=torch.float32, device=logits.device)
        ws.barrier()                         # the previous call's tables have been read by everyone
        K._check(K.lib().nx_vocab_ce_exchange(K._p(stats), C.byref(cache["table"].table), C.byref(ws.flags.table),
                                              C.c_int(ws.rank), C.c_int(ws.n), C.c_int(rows), K._p(ws.counter),
                                              K._p(merged), K._p(K.status_word(ws.device)), K._stream()),
                 "nx_vocab_ce_exchange")
        lse = merged[:, 0] + torch.log(merged[:, 1])
        valid = targets != ignore_index
        n_valid = valid.sum().clamp(min=1)
        loss = ((lse - merged[:, 2]) * valid).sum() / n_valid
        ctx.save_for_backward(logits, lse, local_t, mine & valid, valid, n_valid)
        return loss

    @staticmethod
    def backward(ctx, g):
        logits, lse, local_t, hit, valid, n_valid = ctx.saved_tensors
        p = torch.exp(logits.float() - lse[:, None]) * valid[:, None]
        p[hit.nonzero()[:, 0], local_t[hit]] -= 1.0
        return (p * (g / n_valid)).to(logits.dtype), None, None, None, None


def vocab_parallel_cross_entropy(ws: SymmetricWorkspace, logits: torch.Tensor, targets: torch.Tensor,
                                 vocab_start: int, ignore_index: int = -100) -> torch.Tensor:
    """Mean cross-entropy when the vocabulary dimension of the logits is split over the ranks.

    ``logits`` [rows, V / n] holds columns [vocab_start, vocab_start + V / n) of the full logits; ``targets``
    [rows] are global token ids.  Each rank reduces its columns to (max, sum-exp, target logit) per row; ONE kernel
    stores the three numbers into every peer's table, waits on the flag barrier and merges them (max of maxima,
    rescaled sum, sum of target logits), so the full logits never exist anywhere.  Differentiable in ``logits``.
    Parity: src/dist/parallel_lm.cpp (vocab-parallel loss) of the reference."""
    return _VocabParallelCE.apply(logits, targets, ws, int(vocab_start), int(ignore_index))


def _a2a_heads(ws: SymmetricWorkspace, x: torch.Tensor, buf: SymmetricBuffer, mode: int) -> None:
    """mode 0: [B, Tl, H, D] of every rank -> [B, n * Tl, H / n, D] in each rank's ``buf``; mode 1: the way back."""
    if mode == 0:
        B, Tl, H, D = x.shape
    else:
        B, T, Hl, D = x.shape
        Tl, H = T // ws.n, Hl * ws.n
    K._check(K.lib().nx_comm_a2a_heads(K._p(x.contiguous()), C.byref(buf.table), C.c_int(B), C.c_int(Tl), C.c_int(H),
                                       C.c_int(D), C.c_int(ws.rank), C.c_int(ws.n), C.c_int(mode), K._stream()),
             "nx_comm_a2a_heads")


def _ulysses_bufs(ws: SymmetricWorkspace, tag: str, numel: int, count: int) -> List[SymmetricBuffer]:
    cache = ws.__dict__.setdefault("_ulysses", {})
    bufs = cache.setdefault((tag, numel), [])
    while len(bufs) < count:
        bufs.append(ws.alloc(numel, torch.bfloat16))
    return bufs


class _UlyssesFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, ws, causal):
        n = ws.n
        B, Tl, H, D = q.shape
        Hkv = k.shape[2]
        gq_b, back_b = _ulysses_bufs(ws, "q", q.numel(), 2)
        gk_b, gv_b = _ulysses_bufs(ws, "kv", k.numel(), 2)
        ws.barrier()                                   # the previous call's readers are done
        _a2a_heads(ws, q, gq_b, 0)
        _a2a_heads(ws, k, gk_b, 0)
        _a2a_heads(ws, v, gv_b, 0)
        ws.barrier()
        gq = gq_b.local.view(B, n * Tl, H // n, D).clone()
        gk = gk_b.local.view(B, n * Tl, Hkv // n, D).clone()
        gv = gv_b.local.view(B, n * Tl, Hkv // n, D).clone()
        o, lse = K.attention_fwd(gq, gk, gv, causal=causal)
        _a2a_heads(ws, o, back_b, 1)
        ws.barrier()
        out = back_b.local.view(B, Tl, H, D).clone()
        ctx.ws, ctx.causal = ws, causal
        ctx.save_for_backward(gq, gk, gv, o, lse)
        return out

    @staticmethod
    def backward(ctx, d_out):
        ws, n = ctx.ws, ctx.ws.n
        gq, gk, gv, o, lse = ctx.saved_tensors
        B, T, Hl, D = gq.shape
        Tl, Hkvl = T // n, gk.shape[2]
        bq0, bq1 = _ulysses_bufs(ws, "q", gq.numel(), 2)
        bk0, bk1 = _ulysses_bufs(ws, "kv", gk.numel(), 2)
        ws.barrier()
        _a2a_heads(ws, d_out, bq0, 0)                  # dO: sequence shards -> head shards
        ws.barrier()
        g_do = bq0.local.view(B, T, Hl, D).clone()
        dq, dk, dv = K.attention_bwd(gq, gk, gv, o, lse, g_do, causal=ctx.causal)
        ws.barrier()                                   # every rank has taken its dO out of the buffer
        _a2a_heads(ws, dq, bq1, 1)
        _a2a_heads(ws, dk, bk0, 1)
        _a2a_heads(ws, dv, bk1, 1)
        ws.barrier()
        gdq = bq1.local.view(B, Tl, Hl * n, D).clone()
        gdk = bk0.local.view(B, Tl, Hkvl * n, D).clone()
        gdv = bk1.local.view(B, Tl, Hkvl * n, D).clone()
        return gdq, gdk, gdv, None, None


def ulysses_attention(ws: SymmetricWorkspace, q, k, v, causal: bool = True):
    """DeepSpeed-Ulysses attention over symmetric memory: heads <-> sequence all-to-all by peer stores,
    local causal flash attention over the full sequence on H/n heads, all-to-all back.
    q [B, Tl, H, D], k / v [B, Tl, Hkv, D] BF16 with H and Hkv divisible by n.  Returns o [B, Tl, H, D];
    differentiable (the backward sends dO the same way, runs the local backward kernels and returns dQ, dK, dV)."""
    if q.shape[2] % ws.n or k.shape[2] % ws.n:
        raise ValueError("ulysses_attention: heads and kv heads must be divisible by the group size")
    return _UlyssesFn.apply(q, k, v, ws, causal)
