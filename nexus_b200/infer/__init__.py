"""Paged-KV inference engine (GPT-2 family): block allocator with copy-on-write, packed prefill/decode
steps, decode CUDA graphs, single-kernel sampler, speculative decoding and weight / KV quantisation."""
from .engine import (Chunk, Engine, EngineConfig, GenerateStats, Gpt2Weights, QuantOptions, SamplingParams,  # noqa: F401
                     SpecStats, StepStats, generate, load_gpt2, speculative_generate)
from .sampling import sample_reference  # noqa: F401
