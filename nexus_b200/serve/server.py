"""In-process continuous-batching server over the paged-KV inference engine.

Every ``step`` (1) preempts the newest running requests while decode blocks are short (their KV is
freed and they re-prefill later), (2) admits waiting requests under the token budget, the running limit
and the free-block count, (3) runs ONE engine forward over [one decode token per running request] +
[the full prompt of every admitted request], (4) samples with a per-request Philox offset (the
request's own token index, so draws do not depend on the batch), (5) streams tokens, finishes requests
on a stop token / ``max_new`` and records TTFT / TPOT / latency.

Pipelined decode (``Config.pipeline_decode``, on by default on the kernel path): while nothing can be admitted and nothing has to be
preempted, step n + 1 is launched before the tokens of step n have been read.  The engine feeds each sequence the token
its last sampling call left on the device, the host reads the tokens one step late (streaming callbacks, stop tokens,
statistics), and a request that turns out to have stopped at step n has its step n + 1 token dropped.  The host-side
scheduling of a step then overlaps the device's work on the previous one.

Parity: include/nexus/cuda/serve.hpp:39-97 and src/cuda/serve.cpp (`Server::step`) of the reference.
"""
from __future__ import annotations

import threading
import time
from collections import deque
from concurrent.futures import Future
from dataclasses import dataclass, field
from typing import Callable, Deque, List, Optional, Sequence

from ..infer.engine import Chunk, Engine, SamplingParams

__all__ = ["Config", "Request", "Result", "Metrics", "Server"]


@dataclass
class Config:
    max_batch_tokens: int = 2048
    max_running: int = 64
    pipeline_decode: Optional[bool] = None   # launch the next decode step before reading this one's tokens
                                             # (None: on the kernel path only; True also on the reference path)


@dataclass
class Request:
    prompt: Sequence[int] = ()
    max_new: int = 16
    sampling: SamplingParams = field(default_factory=lambda: SamplingParams(temperature=0.0))
    stop_token: Optional[int] = None
    on_token: Optional[Callable[[int, int], None]] = None   # (request id, token)


@dataclass
class Result:
    id: int = -1
    tokens: List[int] = field(default_factory=list)
    ttft_ms: float = 0.0
    tpot_ms: float = 0.0
    latency_ms: float = 0.0
    preemptions: int = 0


@dataclass
class Metrics:
    steps: int = 0
    completed: int = 0
    preemptions: int = 0
    prompt_tokens: int = 0
    output_tokens: int = 0
    ttft_ms_sum: float = 0.0
    tpot_ms_sum: float = 0.0
    latency_ms_sum: float = 0.0
    busy_ms: float = 0.0
    pipelined_steps: int = 0     # decode steps launched before the previous step's tokens were read

    def mean_ttft_ms(self) -> float:
        return self.ttft_ms_sum / max(1, self.completed)

    def mean_tpot_ms(self) -> float:
        return self.tpot_ms_sum / max(1, self.completed)

    def throughput_tokens_per_s(self) -> float:
        return self.output_tokens / max(1e-9, self.busy_ms * 1e-3)


class _Live:
    __slots__ = ("id", "req", "future", "seq", "out", "t_submit", "t_first", "t_last", "preemptions", "next_token",
                 "launched", "zombie")

    def __init__(self, rid: int, req: Request):
        self.id, self.req, self.future = rid, req, Future()
        self.seq = -1
        self.out: List[int] = []
        self.t_submit = time.perf_counter()
        self.t_first = self.t_last = 0.0
        self.preemptions = 0
        self.next_token: Optional[int] = None   # sampled, not yet in the KV cache
        self.launched = 0      # tokens sampled or being sampled by a step in flight
        self.zombie = False    # finished while a later step that still contains it was in flight


class Server:
    def __init__(self, engine: Engine, config: Optional[Config] = None):
        self.engine = engine
        self.cfg = config or Config()
        self.cfg.max_running = min(self.cfg.max_running, engine.cfg.max_seqs)
        self.cfg.max_batch_tokens = min(self.cfg.max_batch_tokens, engine.cfg.max_tokens)
        self.waiting: Deque[_Live] = deque()
        self.running: List[_Live] = []
        self.metrics = Metrics()
        self._next_id = 0
        self._lock = threading.Lock()
        self._wake = threading.Condition(self._lock)
        self._thread: Optional[threading.Thread] = None
        self._stop = False
        self._inflight = None      # (PendingTokens, [requests]) of the decode step whose tokens have not been read

    # ------------------------------------------------------------------ submission
    def submit(self, req: Request) -> Future:
        """Queues a request; the future resolves to a ``Result``."""
        if len(req.prompt) == 0:
            raise ValueError("empty prompt")
        if len(req.prompt) + 1 > self.engine.ctx:
            raise ValueError("prompt longer than the context window")
        if len(req.prompt) > self.cfg.max_batch_tokens:
            raise ValueError("prompt longer than the per-step token budget")
        with self._wake:
            live = _Live(self._next_id, req)
            self._next_id += 1
            self.waiting.append(live)
            self._wake.notify()
        return live.future

    def pending(self) -> int:
        with self._lock:
            return len(self.waiting) + len(self.running) + (1 if self._inflight is not None else 0)

    # ------------------------------------------------------------------ one scheduling step
    def step(self) -> int:
        """Runs one forward; returns the number of tokens processed (0: nothing to do)."""
        eng, cfg = self.engine, self.cfg
        t0 = time.perf_counter()
        with self._lock:
            n_pipe = self._pipelined_step()
            if n_pipe is not None:
                return n_pipe
            self._drain()
            # 1. every running request needs room for one more token: preempt the newest while short
            def decode_need() -> int:
                return sum(eng.blocks_needed(r.seq, 1) for r in self.running)
            need = decode_need()                     # walked once per step unless something is preempted
            while self.running and need > eng.free_blocks():
                victim = self.running.pop()          # newest admitted
                eng.free_sequence(victim.seq)
                victim.seq = -1
                victim.preemptions += 1
                self.metrics.preemptions += 1
                self.waiting.appendleft(victim)      # re-prefills prompt + generated tokens later
                need = decode_need()
            budget = cfg.max_batch_tokens - len(self.running)
            free = eng.free_blocks() - need
            admitted: List[_Live] = []
            bs = eng.block_size()
            # 2. admission in arrival order (no overtaking: keeps latency fair)
            while self.waiting and len(self.running) + len(admitted) < cfg.max_running:
                cand = self.waiting[0]
                n = len(cand.req.prompt) + len(cand.out)
                need = -(-(n + 1) // bs)
                if n > budget or need > free:
                    break
                self.waiting.popleft()
                budget -= n
                free -= need
                admitted.append(cand)
            if not self.running and not admitted:
                if self.waiting and not self.running:
                    head = self.waiting[0]
                    if -(-(len(head.req.prompt) + len(head.out) + 1) // bs) > eng.total_blocks():
                        self.waiting.popleft()
                        head.future.set_exception(RuntimeError("request does not fit in the KV cache"))
                return 0
            # 3. one packed batch: decode tokens first, then prompts
            chunks: List[Chunk] = []
            order: List[_Live] = []
            for r in self.running:
                chunks.append(Chunk(r.seq, [r.next_token], 1, True))
                order.append(r)
            for r in admitted:
                r.seq = eng.add_sequence()
                toks = list(r.req.prompt)
                if r.out:   # preempted earlier: prompt (prompt counters), then its own output so far
                    chunks.append(Chunk(r.seq, toks, 0, False))
                    chunks.append(Chunk(r.seq, list(r.out), 1, True))
                else:
                    chunks.append(Chunk(r.seq, toks, 1, False))
                order.append(r)
                self.metrics.prompt_tokens += len(toks)
            eng.forward(chunks)
            params = [r.req.sampling for r in order]
            offsets = [len(r.req.prompt) + len(r.out) for r in order]
            toks = eng.sample(params, [r.seq for r in order], offsets)
            self.running.extend(admitted)
            for r in order:
                r.launched = len(r.out) + 1
            self._consume(order, toks)
            self.metrics.steps += 1
            self.metrics.busy_ms += (time.perf_counter() - t0) * 1e3
            return eng.last_step().tokens

    def _consume(self, order: List[_Live], toks: List[int]) -> None:
        """Books one sampled token per request of ``order``: streaming, stop conditions, results."""
        eng = self.engine
        now = time.perf_counter()
        done: List[_Live] = []
        for r, t in zip(order, toks):
            if r.zombie:                 # stopped one step earlier; this token was drawn past its end
                eng.free_sequence(r.seq)
                r.seq = -1
                continue
            r.out.append(t)
            r.next_token = t
            if r.t_first == 0.0:
                r.t_first = now
            r.t_last = now
            self.metrics.output_tokens += 1
            if r.req.on_token is not None:
                r.req.on_token(r.id, t)
            full = len(r.req.prompt) + len(r.out) >= eng.ctx
            if len(r.out) >= r.req.max_new or t == r.req.stop_token or full:
                done.append(r)
        for r in done:
            self.running.remove(r)
            if r.launched > len(r.out):  # a step in flight still works on this sequence: free it when that step is read
                r.zombie = True
            else:
                eng.free_sequence(r.seq)
            res = Result(r.id, list(r.out), (r.t_first - r.t_submit) * 1e3,
                         (r.t_last - r.t_first) * 1e3 / max(1, len(r.out) - 1), (now - r.t_submit) * 1e3,
                         r.preemptions)
            m = self.metrics
            m.completed += 1
            m.ttft_ms_sum += res.ttft_ms
            m.tpot_ms_sum += res.tpot_ms
            m.latency_ms_sum += res.latency_ms
            r.future.set_result(res)

    def _drain(self) -> None:
        """Reads the tokens of the step in flight, if any."""
        if self._inflight is not None:
            pend, order = self._inflight
            self._inflight = None
            self._consume(order, self.engine.collect(pend))

    def _pipelined_step(self) -> Optional[int]:
        """Launches the next decode step before the tokens of the one in flight are read.  Returns None when the
        situation needs the ordinary step (something to admit, blocks short, nothing to continue)."""
        eng, cfg = self.engine, self.cfg
        on = getattr(eng, "fast", False) if cfg.pipeline_decode is None else cfg.pipeline_decode
        if not (on and self.running):
            return None
        bs = eng.block_size()
        if self.waiting and len(self.running) < cfg.max_running:
            cand = self.waiting[0]
            n = len(cand.req.prompt) + len(cand.out)
            if n <= cfg.max_batch_tokens - len(self.running) and -(-(n + 1) // bs) <= eng.free_blocks():
                return None                                   # the head of the queue can be admitted: ordinary step
        cont = [r for r in self.running
                if r.launched < r.req.max_new and len(r.req.prompt) + r.launched < eng.ctx]
        if not cont:
            return None
        if sum(eng.blocks_needed(r.seq, 1) for r in cont) > eng.free_blocks():
            return None                                       # preemption is decided with every token known
        t0 = time.perf_counter()
        chunks = [Chunk(r.seq, [0], 1, True) for r in cont]
        eng.forward(chunks, device_tokens=True)
        offsets = [len(r.req.prompt) + r.launched for r in cont]
        pend = eng.sample([r.req.sampling for r in cont], [r.seq for r in cont], offsets, pending=True)
        for r in cont:
            r.launched += 1
        prev, self._inflight = self._inflight, (pend, cont)
        if prev is not None:
            self._consume(prev[1], eng.collect(prev[0]))
        self.metrics.steps += 1
        self.metrics.pipelined_steps += 1
        self.metrics.busy_ms += (time.perf_counter() - t0) * 1e3
        return len(cont)

    def run_until_idle(self, max_steps: int = 1 << 30) -> None:
        for _ in range(max_steps):
            if self.pending() == 0:
                return
            self.step()

    # ------------------------------------------------------------------ background loop
    def start(self) -> None:
        if self._thread is not None:
            return
        self._stop = False
        self._thread = threading.Thread(target=self._loop, name="nexus-serve", daemon=True)
        self._thread.start()

    def stop(self) -> None:
        with self._wake:
            self._stop = True
            self._wake.notify_all()
        if self._thread is not None:
            self._thread.join()
            self._thread = None

    def _loop(self) -> None:
        while True:
            with self._wake:
                while not self._stop and not self.waiting and not self.running:
                    self._wake.wait(timeout=0.05)
                if self._stop:
                    return
            if self.step() == 0:
                time.sleep(0.001)
