"""Graph compiler: IR, tracer, passes, JIT code generation for fused clusters, executor / CompiledLm."""
from . import passes  # noqa: F401
from .codegen import FusedKernel, cluster_source, compile_cpu, compile_cuda  # noqa: F401
from .executor import CompiledLm, CompileOptions, Executor, autotune, compile_lm  # noqa: F401
from .ir import Dim, Graph, Node, Value  # noqa: F401
from .trace import Builder, trace_lm  # noqa: F401
