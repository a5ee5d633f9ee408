"""Interoperability: safetensors, Hugging Face llama-family checkpoints, GGUF v3, ONNX export, DLPack."""
from . import dlpack, gguf, hf, safetensors  # noqa: F401
from .hf import export_hf, import_hf  # noqa: F401
from .safetensors import SafetensorsError, SafetensorsFile, load_file, save_file  # noqa: F401
