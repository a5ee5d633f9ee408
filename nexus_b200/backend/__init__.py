"""Backend abstraction: drivers, registry, CUDA->HIP source translation, StableHLO / GSPMD / PJRT."""
from .driver import (ELEMENTWISE, AllocatorStats, CpuDriver, CudaDriver, DeviceInfo, Driver, FallbackPolicy,  # noqa: F401
                     FallbackStats, Kind, Operation, Registry, UnavailableDriver, fallback_policy, fallback_stats,
                     parse_kind, require_cpu_fallback, reset_fallback_stats, set_fallback_policy)
from .hip import HipDriver, hipify_source  # noqa: F401
from .pjrt import PjrtDriver, StableHloModule, sharding_annotation  # noqa: F401
