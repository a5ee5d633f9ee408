"""Parallelism and communication: process groups, DDP, ZeRO/FSDP, DeviceMesh/DTensor, tensor /
sequence / pipeline / context / expert parallelism, watchdog, launcher glue, symmetric-memory kernels."""
from .ddp import DdpEngine, DdpOptions, DdpStepStats, plan_buckets, scaled_lr  # noqa: F401
from .fsdp import FsdpEngine, FsdpOptions  # noqa: F401
from .process_group import (DistError, DistTimeout, GroupOptions, ProcessGroup, ThreadProcessGroup,  # noqa: F401
                            ThreadWorld, TorchProcessGroup, Work, init_process_group, run_threads)
from .watchdog import LocalBoard, StoreBoard, Watchdog, WatchdogEvent, WatchdogOptions  # noqa: F401
