"""Builds the reference arm: the reference's own single-GPU GPT training path, compiled from its
unmodified sources for sm_100, driven by ``ref_gpt_driver.cpp``.

The reference has no Python package at its root and its CMake project stops at five empty git submodules, so
``pip install`` cannot produce it.  Its ``src/cuda`` training path (``cuda::GptModel`` / ``cuda::GptTrainer`` on
cuBLASLt and its FlashAttention-2 kernels) depends on none of those submodules; this script copies exactly the
files that path needs into ``baseline/_ref/`` (byte for byte), compiles them with ``g++ -std=c++20`` and
``nvcc -gencode arch=compute_100,code=sm_100`` and links ``baseline/_ref/lib/libnexus_ref_gpt.so`` (loaded by
``bench.py --impl reference`` through ctypes) and the command-line form ``baseline/_ref/bin/ref_gpt_bench``.  Unused functions of
``src/fused/training.cpp`` (the CPU autograd forms) are dropped by ``--gc-sections`` instead of pulling in the
rest of the CPU library.

    python baseline/build_ref.py [--reference /path/to/reference] [--force]
"""
from __future__ import annotations

import hashlib
import json
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"
BIN = OUT / "bin" / "ref_gpt_bench"
LIB = OUT / "lib" / "libnexus_ref_gpt.so"

HOST_SOURCES = [
    "src/cuda/gpt.cpp", "src/cuda/gemm_lt.cpp", "src/cuda/caching_allocator.cpp", "src/cuda/runtime.cpp",
    "src/cuda/cast_cache.cpp", "src/prof/prof.cpp", "src/cpu/adam_avx2.cpp", "src/cpu/threads.cpp",
    "src/cpu/features.cpp", "src/attention/cpu.cpp", "src/fused/training.cpp",
]
CUDA_SOURCES = [
    "src/cuda/kernels_train.cu", "src/cuda/flash_attention.cu", "src/cuda/kernels_norm.cu",
    "src/cuda/kernels_elementwise.cu",
]
EXTRA_FILES = ["src/cuda/common.cuh"]
INCLUDE_TREES = ["include", "lib/NexusTrain/include"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", shutil.which("nvcc")):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found")


def _run(cmd):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("command failed: %s\n%s\n%s" % (" ".join(map(str, cmd)), r.stdout[-4000:], r.stderr[-4000:]))


def _sha(path: Path) -> str:
    return hashlib.sha256(path.read_bytes()).hexdigest()


def copy_sources(ref: Path) -> dict:
    """Copies the needed files unmodified and returns {relative path: sha256} of what was copied."""
    manifest = {}
    for rel in HOST_SOURCES + CUDA_SOURCES + EXTRA_FILES:
        dst = OUT / rel
        dst.parent.mkdir(parents=True, exist_ok=True)
        shutil.copyfile(ref / rel, dst)
        manifest[rel] = _sha(dst)
    for tree in INCLUDE_TREES:
        dst = OUT / tree
        if dst.exists():
            shutil.rmtree(dst)
        shutil.copytree(ref / tree, dst)
    return manifest


def build(ref: Path | None = None, force: bool = False, verbose: bool = True) -> Path:
    # the reference checkout: given, or $NEXUS_REFERENCE, or a `reference` directory beside this repository
    ref = Path(ref or os.environ.get("NEXUS_REFERENCE") or HERE.parent.parent / "reference")
    driver = HERE / "ref_gpt_driver.cpp"
    if LIB.exists() and BIN.exists() and not force and LIB.stat().st_mtime >= driver.stat().st_mtime:
        return LIB
    if not (ref / "src" / "cuda" / "gpt.cpp").exists():
        raise RuntimeError(f"reference sources not found under {ref}")
    manifest = copy_sources(ref)
    obj = OUT / "obj"
    obj.mkdir(parents=True, exist_ok=True)
    (OUT / "bin").mkdir(parents=True, exist_ok=True)
    (OUT / "lib").mkdir(parents=True, exist_ok=True)
    cuda_home = Path(_nvcc()).resolve().parent.parent
    inc = ["-I", str(OUT / "include"), "-I", str(OUT / "lib/NexusTrain/include"), "-I", str(OUT / "src/cuda"),
           "-I", str(cuda_home / "include")]
    cmds, objs = [], []
    for rel in HOST_SOURCES:
        o = obj / (rel.replace("/", "_") + ".o")
        objs.append(o)
        cmds.append(["g++", "-std=c++20", "-O2", "-mavx2", "-mfma", "-mf16c", "-fPIC", "-ffunction-sections",
                     "-fdata-sections", "-DNEXUS_ENABLE_CUDA=1", "-DNEXUS_HAS_CUDA_KERNELS=1", *inc, "-c",
                     str(OUT / rel), "-o", str(o)])
    for rel in CUDA_SOURCES:
        o = obj / (rel.replace("/", "_") + ".o")
        objs.append(o)
        cmds.append([_nvcc(), "-std=c++20", "-O3", "-gencode", "arch=compute_100,code=sm_100", "-Xcompiler", "-fPIC",
                     "-DNEXUS_ENABLE_CUDA=1", "-DNEXUS_HAS_CUDA_KERNELS=1", *inc, "-c", str(OUT / rel), "-o", str(o)])
    o_lib, o_main = obj / "ref_gpt_driver.o", obj / "ref_gpt_driver_main.o"
    for o, extra in ((o_lib, []), (o_main, ["-DREF_DRIVER_MAIN"])):
        cmds.append(["g++", "-std=c++20", "-O2", "-fPIC", "-DNEXUS_ENABLE_CUDA=1", "-DNEXUS_HAS_CUDA_KERNELS=1", *extra,
                     *inc, "-c", str(driver), "-o", str(o)])
    with ThreadPoolExecutor(max_workers=8) as ex:
        list(ex.map(_run, cmds))
    lib = cuda_home / "lib64"
    link = ["-L", str(lib), f"-Wl,-rpath,{lib}", "-lcudart", "-lcublasLt", "-lcublas", "-lpthread"]
    _run(["g++", "-Wl,--gc-sections", "-o", str(BIN), str(o_main), *map(str, objs), *link])
    # the shared library keeps only what the exported C entry points reach (version script + gc-sections)
    vs = obj / "exports.map"
    vs.write_text("{ global: nexus_ref_gpt_*; local: *; };\n")
    _run(["g++", "-shared", "-Wl,--gc-sections", f"-Wl,--version-script={vs}", "-o", str(LIB), str(o_lib),
          *map(str, objs), *link])
    (OUT / "MANIFEST.json").write_text(json.dumps({"reference": str(ref), "files": manifest}, indent=1))
    if verbose:
        print("built", LIB, "and", BIN)
    return LIB


if __name__ == "__main__":
    ref_arg = None
    if "--reference" in sys.argv:
        ref_arg = sys.argv[sys.argv.index("--reference") + 1]
    build(ref_arg, force="--force" in sys.argv)
