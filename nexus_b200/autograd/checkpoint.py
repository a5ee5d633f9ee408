"""Non-reentrant activation checkpointing on saved-tensor hooks: inside ``checkpoint(fn, *inputs)``
every tensor autograd wants to save is replaced by its index; the first unpack during backward
re-runs ``fn`` under the same hooks in "recompute" mode and hands the saved tensors back by index.
Nested checkpoints work because each frame owns its own storage.  `SavedBytesCounter` measures
what autograd keeps alive.

Parity: src/autograd/checkpoint.cpp:39-117 of the reference.
"""
from __future__ import annotations

from typing import Callable, List

import torch


class _Frame:
    def __init__(self, fn, inputs):
        self.fn, self.inputs = fn, inputs
        self.count = 0
        self.recomputed: List[torch.Tensor] = []
        self.done = False
        self.rng_cpu = torch.get_rng_state()
        self.rng_cuda = torch.cuda.get_rng_state() if torch.cuda.is_available() and torch.cuda.is_initialized() else None


class _StopRecompute(Exception):
    pass


def checkpoint(fn: Callable, *inputs):
    """Runs ``fn(*inputs)`` without keeping its intermediate activations."""
    if not torch.is_grad_enabled():
        return fn(*inputs)
    frame = _Frame(fn, inputs)

    def pack(t: torch.Tensor):
        idx = frame.count
        frame.count += 1
        return idx

    def unpack(idx: int) -> torch.Tensor:
        if not frame.done:
            total = frame.count
            seen = {"n": 0}

            def pack2(t):
                frame.recomputed.append(t.detach())
                seen["n"] += 1
                if seen["n"] >= total:
                    raise _StopRecompute()
                return None

            def unpack2(_):
                raise RuntimeError("checkpoint: backward through the recomputation is not supported")

            cpu_now = torch.get_rng_state()
            torch.set_rng_state(frame.rng_cpu)
            if frame.rng_cuda is not None:
                cuda_now = torch.cuda.get_rng_state()
                torch.cuda.set_rng_state(frame.rng_cuda)
            try:
                with torch.enable_grad(), torch.autograd.graph.saved_tensors_hooks(pack2, unpack2):
                    detached = [x.detach().requires_grad_(x.requires_grad) if isinstance(x, torch.Tensor) else x
                                for x in frame.inputs]
                    frame.fn(*detached)
            except _StopRecompute:
                pass
            finally:
                torch.set_rng_state(cpu_now)
                if frame.rng_cuda is not None:
                    torch.cuda.set_rng_state(cuda_now)
            frame.done = True
        return frame.recomputed[idx]

    with torch.autograd.graph.saved_tensors_hooks(pack, unpack):
        return fn(*inputs)


class SavedBytesCounter:
    """Context manager counting the bytes autograd saves for backward inside the block."""

    def __init__(self):
        self.bytes = 0
        self.tensors = 0
        self._ctx = None

    def __enter__(self):
        def pack(t):
            self.bytes += t.numel() * t.element_size()
            self.tensors += 1
            return t

        self._ctx = torch.autograd.graph.saved_tensors_hooks(pack, lambda t: t)
        self._ctx.__enter__()
        return self

    def __exit__(self, *exc):
        return self._ctx.__exit__(*exc)
