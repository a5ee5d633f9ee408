"""Core types: dtypes and promotion, FP8 / half host conversions, devices, shapes, the memory gate and
runtime wrappers, strided tensors over shared storage with the flat op dispatcher, and host/device
mirrors."""
from .device import (DeviceKind, DeviceRef, ExecutionPolicy, MemorySpace, Shape, global_seed,  # noqa: F401
                     set_global_seed)
from .dtype import (ALL_DTYPES, FP8_MAX, DType, Fp8DelayedScaling, TensorError, bf16_bits_to_float,  # noqa: F401
                    float_to_bf16_bits, float_to_half_bits, fp8_decode, fp8_encode, from_torch, half_bits_to_float,
                    is_float8, is_floating, is_integral, parse_dtype, promote, size_of, to_string, to_torch)
from .memory import (AllocationCounters, DeviceBuffer, Event, MemoryGate, Stream, cuda_check, current_device,  # noqa: F401
                     gate)
from .mirrored import MirroredTensor, MirrorState  # noqa: F401
from .tensor import Op, Storage, Tensor, UNARY_FNS, add, dispatch, matmul, mul, register, unary  # noqa: F401
