"""Communication backend: one `ProcessGroup` interface, two transports.

* `TorchProcessGroup` — one process per GPU over ``torch.distributed`` (NCCL on NVLink 5 / NVSwitch
  for device tensors, gloo for host tensors and for the CPU-rank tests).
* `ThreadWorld` / `ThreadProcessGroup` — N ranks as N threads of one process exchanging tensors
  through in-memory mailboxes; every distributed engine can be tested without a cluster.

Both offer: ``all_reduce``, ``reduce_scatter``, ``all_gather``, ``broadcast``, ``all_to_all_v``,
``send``/``recv``/``send_recv``, ``barrier``, ``new_group``, ``all_reduce_hierarchical``; reduce ops
sum/avg/max/min/product; asynchronous `Work` handles; a per-group timeout that raises `DistTimeout`
and marks the group broken; and a validate mode (``NEXUS_DIST_DEBUG=1``) that compares a
fingerprint (sequence number, op, dtype, element count, root) of every collective across ranks and
turns a would-be deadlock into a named `DistError`.

Parity: include/nexus/dist/process_group.hpp:43-177, src/dist/process_group.cpp:465-885 and
include/nexus/dist/store.hpp of the reference (thread + tcp transports; no NCCL there).
"""
from __future__ import annotations

import os
import threading
import time
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Sequence

import torch

REDUCE_OPS = ("sum", "avg", "max", "min", "product")


class DistError(RuntimeError):
    pass


class DistTimeout(DistError):
    pass


@dataclass
class GroupOptions:
    timeout_s: float = 60.0
    validate: Optional[bool] = None  # None: read NEXUS_DIST_DEBUG


class Work:
    """Handle of an asynchronous collective."""

    def __init__(self, waiter: Optional[Callable[[float], bool]] = None):
        self._waiter = waiter
        self._done = waiter is None
        self.started = time.perf_counter()
        self.finished = self.started if self._done else None

    def is_completed(self) -> bool:
        return self._done

    def wait(self, timeout: Optional[float] = None) -> bool:
        if not self._done:
            ok = self._waiter(timeout)
            if ok:
                self._done = True
                self.finished = time.perf_counter()
            return ok
        return True


def _reduce_pair(a: torch.Tensor, b: torch.Tensor, op: str) -> torch.Tensor:
    if op in ("sum", "avg"):
        return a + b
    if op == "max":
        return torch.maximum(a, b)
    if op == "min":
        return torch.minimum(a, b)
    if op == "product":
        return a * b
    raise ValueError(f"unknown reduce op {op}")


class ProcessGroup:
    """Interface + helpers shared by both transports."""

    def __init__(self, options: Optional[GroupOptions] = None):
        self.options = options or GroupOptions()
        v = self.options.validate
        self.validate = (os.environ.get("NEXUS_DIST_DEBUG", "0") == "1") if v is None else v
        self.broken = False
        self._seq = 0

    # -- to be provided by transports
    def rank(self) -> int: raise NotImplementedError
    def size(self) -> int: raise NotImplementedError
    def all_reduce_tensor(self, t: torch.Tensor, op: str = "sum") -> torch.Tensor: raise NotImplementedError
    def reduce_scatter_tensor(self, out: torch.Tensor, inp: torch.Tensor, op: str = "sum") -> torch.Tensor: raise NotImplementedError
    def all_gather_tensor(self, out: torch.Tensor, inp: torch.Tensor) -> torch.Tensor: raise NotImplementedError
    def broadcast_tensor(self, t: torch.Tensor, root: int = 0) -> torch.Tensor: raise NotImplementedError
    def all_to_all_v(self, send: List[torch.Tensor]) -> List[torch.Tensor]: raise NotImplementedError
    def send(self, t: torch.Tensor, dst: int, tag: int = 0) -> None: raise NotImplementedError
    def recv(self, t: torch.Tensor, src: int, tag: int = 0) -> torch.Tensor: raise NotImplementedError
    def barrier(self) -> None: raise NotImplementedError
    def new_group(self, ranks: Sequence[int]) -> Optional["ProcessGroup"]: raise NotImplementedError
    def destroy(self) -> None: pass

    # -- shared
    def _check_alive(self) -> None:
        if self.broken:
            raise DistError("process group is broken (an earlier collective failed or timed out)")

    def send_recv(self, send_t: torch.Tensor, dst: int, recv_t: torch.Tensor, src: int, tag: int = 0) -> torch.Tensor:
        """Simultaneous exchange (deadlock-free on both transports)."""
        if self.rank() % 2 == 0 or dst == src == self.rank():
            self.send(send_t, dst, tag)
            self.recv(recv_t, src, tag)
        else:
            tmp = send_t.clone()
            self.recv(recv_t, src, tag)
            self.send(tmp, dst, tag)
        return recv_t

    def all_reduce_scalar(self, value, op: str = "sum"):
        dt = torch.int64 if isinstance(value, int) and not isinstance(value, bool) else torch.float64
        t = torch.tensor([value], dtype=dt)
        t = self._scalar_device(t)
        self.all_reduce_tensor(t, op)
        v = t.cpu().item()
        return int(v) if dt == torch.int64 else float(v)

    def _scalar_device(self, t: torch.Tensor) -> torch.Tensor:
        return t

    def all_reduce_hierarchical(self, t: torch.Tensor, local_size: int, op: str = "sum") -> torch.Tensor:
        """intra-node reduce-scatter -> inter-node all-reduce -> intra-node all-gather."""
        n, r = self.size(), self.rank()
        if local_size <= 1 or n % local_size != 0 or local_size == n or t.numel() % local_size != 0:
            return self.all_reduce_tensor(t, op)
        node, local = r // local_size, r % local_size
        intra = self._cached_group(("intra", local_size), [list(range(k * local_size, (k + 1) * local_size))
                                                           for k in range(n // local_size)])
        inter = self._cached_group(("inter", local_size), [list(range(l, n, local_size)) for l in range(local_size)])
        flat = t.reshape(-1)
        shard = torch.empty(flat.numel() // local_size, dtype=t.dtype, device=t.device)
        red = "sum" if op == "avg" else op
        intra.reduce_scatter_tensor(shard, flat, red)
        inter.all_reduce_tensor(shard, red)
        intra.all_gather_tensor(flat, shard)
        if op == "avg":
            flat.div_(n)
        return t

    def _cached_group(self, key, partitions: List[List[int]]):
        cache = self.__dict__.setdefault("_subgroups", {})
        if key not in cache:
            mine = None
            for ranks in partitions:  # every rank creates every sub-group, in the same order
                g = self.new_group(ranks)
                if self.rank() in ranks:
                    mine = g
            cache[key] = mine
        return cache[key]

    def fingerprint(self, op: str, t: Optional[torch.Tensor], root: int = -1) -> str:
        self._seq += 1
        return f"{self._seq}:{op}:{None if t is None else t.dtype}:{0 if t is None else t.numel()}:{root}"

    def check_call(self, op: str, *fields) -> None:
        """Validate mode only: compares (sequence number, ``op``, ``fields``) across the ranks and raises ``DistError``
        on the first difference.  Callers that launch their own communicating kernels (the symmetric-memory ops) use
        it before the launch, so a mismatched call becomes a named host error instead of a device-side time-out."""
        if not self.validate:
            return
        self._seq += 1
        self._exchange_fingerprint(f"{self._seq}:{op}:" + ":".join(str(f) for f in fields))

    def _exchange_fingerprint(self, fp: str) -> None:
        raise NotImplementedError


# ================================================================================================
# torch.distributed transport
# ================================================================================================
class TorchProcessGroup(ProcessGroup):
    def __init__(self, group=None, device: Optional[str] = None, options: Optional[GroupOptions] = None):
        super().__init__(options)
        import torch.distributed as dist
        self.dist = dist
        self.group = group
        self.device = torch.device(device) if device is not None else torch.device("cpu")
        self._ranks = dist.get_process_group_ranks(group) if group is not None else list(range(dist.get_world_size()))
        self._fp_group = None

    def rank(self) -> int: return self.dist.get_rank(self.group)
    def size(self) -> int: return self.dist.get_world_size(self.group)
    def global_rank(self, r: int) -> int: return self._ranks[r]

    def _op(self, op: str):
        R = self.dist.ReduceOp
        return {"sum": R.SUM, "avg": R.SUM, "max": R.MAX, "min": R.MIN, "product": R.PRODUCT}[op]

    def _validate(self, op: str, t, root: int = -1) -> None:
        if not self.validate:
            return
        fp = self.fingerprint(op, t, root)
        self._exchange_fingerprint(fp)

    def _exchange_fingerprint(self, fp: str) -> None:
        gathered = [None] * self.size()
        self.dist.all_gather_object(gathered, fp, group=self.group)
        if any(g != gathered[0] for g in gathered):
            self.broken = True
            raise DistError(f"mismatched collective across ranks: {gathered}")

    def _run(self, fn):
        self._check_alive()
        try:
            return fn()
        except RuntimeError as e:
            self.broken = True
            if "timeout" in str(e).lower() or "timed out" in str(e).lower():
                raise DistTimeout(str(e)) from e
            raise DistError(str(e)) from e

    def _scalar_device(self, t):
        return t.to(self.device) if self.device.type == "cuda" else t

    def all_reduce_tensor(self, t, op="sum"):
        self._validate("all_reduce", t)
        self._run(lambda: self.dist.all_reduce(t, self._op(op), group=self.group))
        if op == "avg":
            t.div_(self.size())
        return t

    def all_reduce_async(self, t, op="sum") -> Work:
        self._validate("all_reduce", t)
        w = self._run(lambda: self.dist.all_reduce(t, self._op(op), group=self.group, async_op=True))
        return Work(lambda timeout: (w.wait(), True)[1])

    def reduce_scatter_tensor(self, out, inp, op="sum"):
        self._validate("reduce_scatter", inp)
        self._run(lambda: self.dist.reduce_scatter_tensor(out, inp, self._op(op), group=self.group))
        if op == "avg":
            out.div_(self.size())
        return out

    def all_gather_tensor(self, out, inp):
        self._validate("all_gather", inp)
        self._run(lambda: self.dist.all_gather_into_tensor(out, inp, group=self.group))
        return out

    def broadcast_tensor(self, t, root=0):
        self._validate("broadcast", t, root)
        self._run(lambda: self.dist.broadcast(t, self.global_rank(root), group=self.group))
        return t

    def all_to_all_v(self, send: List[torch.Tensor]) -> List[torch.Tensor]:
        n = self.size()
        dev = send[0].device
        counts = torch.tensor([s.numel() for s in send], dtype=torch.int64, device=dev)
        rcounts = torch.empty_like(counts)
        self._run(lambda: self.dist.all_to_all_single(rcounts, counts, group=self.group))
        rc = rcounts.tolist()
        recv = [torch.empty(c, dtype=send[0].dtype, device=dev) for c in rc]
        if dev.type == "cuda" or True:
            inp = torch.cat([s.reshape(-1) for s in send]) if send else torch.empty(0)
            out = torch.empty(sum(rc), dtype=send[0].dtype, device=dev)
            self._run(lambda: self.dist.all_to_all_single(out, inp, rc, [s.numel() for s in send], group=self.group))
            recv = list(out.split(rc))
        return recv

    def send(self, t, dst, tag=0):
        self._run(lambda: self.dist.send(t, self.global_rank(dst), group=self.group, tag=tag))

    def recv(self, t, src, tag=0):
        self._run(lambda: self.dist.recv(t, self.global_rank(src), group=self.group, tag=tag))
        return t

    def isend(self, t, dst, tag=0) -> Work:
        w = self._run(lambda: self.dist.isend(t, self.global_rank(dst), group=self.group, tag=tag))
        return Work(lambda timeout: (w.wait(), True)[1])

    def irecv(self, t, src, tag=0) -> Work:
        w = self._run(lambda: self.dist.irecv(t, self.global_rank(src), group=self.group, tag=tag))
        return Work(lambda timeout: (w.wait(), True)[1])

    def send_recv(self, send_t, dst, recv_t, src, tag=0):
        ops = [self.dist.P2POp(self.dist.isend, send_t, self.global_rank(dst), self.group, tag),
               self.dist.P2POp(self.dist.irecv, recv_t, self.global_rank(src), self.group, tag)]
        for w in self._run(lambda: self.dist.batch_isend_irecv(ops)):
            w.wait()
        return recv_t

    def barrier(self):
        self._run(lambda: self.dist.barrier(group=self.group))

    def new_group(self, ranks):
        import datetime
        g = self.dist.new_group([self.global_rank(r) for r in ranks],
                                timeout=datetime.timedelta(seconds=self.options.timeout_s))
        if self.rank() not in ranks:
            return None
        return TorchProcessGroup(g, str(self.device), self.options)

    def destroy(self):
        if self.group is None and self.dist.is_initialized():
            self.dist.destroy_process_group()


def init_process_group(backend: Optional[str] = None, device: Optional[str] = None,
                       options: Optional[GroupOptions] = None) -> TorchProcessGroup:
    """Reads RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT (as set by ``nexus-run`` or torchrun)."""
    import datetime
    import torch.distributed as dist
    options = options or GroupOptions()
    if backend is None:
        backend = "nccl" if (device or "").startswith("cuda") else "gloo"
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        kw = {}
        if backend == "nccl" and device is not None:
            kw["device_id"] = torch.device(device)
        dist.init_process_group(backend, timeout=datetime.timedelta(seconds=options.timeout_s), **kw)
    return TorchProcessGroup(None, device or "cpu", options)


# ================================================================================================
# in-process transport: N ranks = N threads
# ================================================================================================
class _Shared:
    """State shared by the ranks of one thread group."""

    def __init__(self, n: int, timeout_s: float):
        self.n, self.timeout_s = n, timeout_s
        self.cond = threading.Condition()
        self.slots: Dict[tuple, list] = {}
        self.mail: Dict[tuple, list] = {}
        self.broken = False
        self.children: Dict[tuple, "_Shared"] = {}
        self.next_child = 0

    def rendezvous(self, key, rank: int, value, combine: Callable[[list], object]):
        """Every rank deposits `value`; the last arrival runs `combine(values)`; all get the result."""
        deadline = time.monotonic() + self.timeout_s
        with self.cond:
            if self.broken:
                raise DistError("process group is broken")
            ent = self.slots.setdefault(key, [dict(), None, 0])
            ent[0][rank] = value
            if len(ent[0]) == self.n:
                try:
                    ent[1] = ("ok", combine([ent[0][r] for r in range(self.n)]))
                except Exception as e:  # surfaced on every rank
                    ent[1] = ("err", e)
                self.cond.notify_all()
            while ent[1] is None:
                left = deadline - time.monotonic()
                if left <= 0 or self.broken:
                    self.broken = True
                    self.cond.notify_all()
                    raise DistTimeout(f"collective {key} timed out after {self.timeout_s}s "
                                      f"({len(ent[0])}/{self.n} ranks arrived)")
                self.cond.wait(left)
            ent[2] += 1
            res = ent[1]
            if ent[2] == self.n:
                del self.slots[key]
        if res[0] == "err":
            raise res[1]
        return res[1]


class ThreadProcessGroup(ProcessGroup):
    def __init__(self, shared: _Shared, rank: int, options: Optional[GroupOptions] = None):
        super().__init__(options)
        self.s, self._rank = shared, rank
        self._n = 0  # per-rank op counter: the k-th collective of every rank meets in slot k

    def rank(self): return self._rank
    def size(self): return self.s.n

    def _collect(self, op: str, value, combine, t=None, root=-1):
        self._check_alive()
        self._n += 1
        fp = self.fingerprint(op, t, root) if self.validate else None

        def comb(vals):
            if self.validate:
                fps = [v[1] for v in vals]
                if any(f != fps[0] for f in fps):
                    raise DistError(f"mismatched collective across ranks: {fps}")
            return combine([v[0] for v in vals])
        try:
            return self.s.rendezvous(("c", self._n), self._rank, (value, fp), comb)
        except DistError:
            self.broken = True
            raise

    def _exchange_fingerprint(self, fp: str) -> None:
        self._check_alive()
        self._n += 1

        def comb(vals):
            if any(v != vals[0] for v in vals):
                raise DistError(f"mismatched collective across ranks: {list(vals)}")
            return None
        try:
            self.s.rendezvous(("c", self._n), self._rank, fp, comb)
        except DistError:
            self.broken = True
            raise

    def all_reduce_tensor(self, t, op="sum"):
        def combine(vals):
            acc = vals[0].clone().float() if vals[0].dtype in (torch.float16, torch.bfloat16) else vals[0].clone()
            for v in vals[1:]:
                acc = _reduce_pair(acc, v.to(acc.dtype), op)
            if op == "avg":
                acc = acc / len(vals)
            return acc
        res = self._collect("all_reduce", t.detach().clone(), combine, t)
        t.copy_(res.to(t.dtype))
        return t

    def all_reduce_async(self, t, op="sum") -> Work:
        self.all_reduce_tensor(t, op)
        return Work()

    def reduce_scatter_tensor(self, out, inp, op="sum"):
        n = self.size()
        if inp.numel() != out.numel() * n:
            raise ValueError("reduce_scatter: input must hold size() chunks of the output's size")

        def combine(vals):
            acc = vals[0].clone().float() if vals[0].dtype in (torch.float16, torch.bfloat16) else vals[0].clone()
            for v in vals[1:]:
                acc = _reduce_pair(acc, v.to(acc.dtype), op)
            if op == "avg":
                acc = acc / len(vals)
            return acc
        res = self._collect("reduce_scatter", inp.detach().reshape(-1).clone(), combine, inp)
        out.copy_(res.view(n, -1)[self._rank].view(out.shape).to(out.dtype))
        return out

    def all_gather_tensor(self, out, inp):
        res = self._collect("all_gather", inp.detach().reshape(-1).clone(), lambda vals: torch.cat(vals), inp)
        out.copy_(res.view(out.shape))
        return out

    def broadcast_tensor(self, t, root=0):
        res = self._collect("broadcast", t.detach().clone(), lambda vals: vals[root], t, root)
        t.copy_(res)
        return t

    def all_to_all_v(self, send):
        if len(send) != self.size():
            raise ValueError("all_to_all_v: one tensor per destination rank")
        res = self._collect("all_to_all_v", [s.detach().clone() for s in send], lambda vals: vals, None)
        return [res[src][self._rank] for src in range(self.size())]

    def _mail_key(self, src, dst, tag): return (src, dst, tag)

    def send(self, t, dst, tag=0):
        self._check_alive()
        with self.s.cond:
            self.s.mail.setdefault(self._mail_key(self._rank, dst, tag), []).append(t.detach().clone())
            self.s.cond.notify_all()

    def recv(self, t, src, tag=0):
        self._check_alive()
        key = self._mail_key(src, self._rank, tag)
        deadline = time.monotonic() + self.s.timeout_s
        with self.s.cond:
            while not self.s.mail.get(key):
                left = deadline - time.monotonic()
                if left <= 0 or self.s.broken:
                    self.broken = self.s.broken = True
                    self.s.cond.notify_all()
                    raise DistTimeout(f"recv from rank {src} (tag {tag}) timed out")
                self.s.cond.wait(left)
            msg = self.s.mail[key].pop(0)
        t.copy_(msg.view(t.shape))
        return t

    def isend(self, t, dst, tag=0) -> Work:
        self.send(t, dst, tag)
        return Work()

    def irecv(self, t, src, tag=0) -> Work:
        return Work(lambda timeout: (self.recv(t, src, tag), True)[1])

    def send_recv(self, send_t, dst, recv_t, src, tag=0):
        self.send(send_t, dst, tag)  # mailboxes never block the sender
        return self.recv(recv_t, src, tag)

    def barrier(self):
        self._collect("barrier", 0, lambda vals: 0)

    def new_group(self, ranks):
        ranks = list(ranks)
        key = tuple(ranks)
        # every member of the parent calls new_group in the same order (like the torch transport)
        child = self._collect("new_group", key, lambda vals: self._make_child(vals))
        if self._rank not in ranks:
            return None
        return ThreadProcessGroup(child, ranks.index(self._rank), self.options)

    def _make_child(self, keys):
        k = keys[0]
        if any(x != k for x in keys):
            raise DistError("new_group called with different rank lists")
        self.s.next_child += 1
        if self.s.next_child > 63:
            raise DistError("too many sub-groups (max 63)")
        return _Shared(len(k), self.s.timeout_s)


class ThreadWorld:
    """Runs ``fn(pg)`` on ``n`` threads, one rank each; re-raises the first failure."""

    def __init__(self, n: int, options: Optional[GroupOptions] = None):
        self.n = n
        self.options = options or GroupOptions(timeout_s=30.0)
        self.shared = _Shared(n, self.options.timeout_s)

    def group(self, rank: int) -> ThreadProcessGroup:
        return ThreadProcessGroup(self.shared, rank, self.options)

    def run(self, fn: Callable[[ThreadProcessGroup], object]) -> list:
        results, errors = [None] * self.n, [None] * self.n

        def target(r):
            try:
                results[r] = fn(self.group(r))
            except BaseException as e:
                errors[r] = e
                with self.shared.cond:
                    self.shared.broken = True
                    self.shared.cond.notify_all()
        threads = [threading.Thread(target=target, args=(r,), daemon=True) for r in range(self.n)]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        # a rank's own failure outranks the DistErrors it caused on the ranks that waited for it
        real = [e for e in errors if e is not None and not isinstance(e, DistError)]
        first = real[0] if real else next((e for e in errors if e is not None), None)
        if first is not None:
            raise first
        return results


def run_threads(n: int, fn: Callable[[ThreadProcessGroup], object], options: Optional[GroupOptions] = None) -> list:
    return ThreadWorld(n, options).run(fn)
