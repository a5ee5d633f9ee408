"""In-tree native build: every ``.cu`` under ``csrc/cuda`` is compiled for sm_100a into
``lib/libnexus_b200_cuda.so`` and every ``.cpp`` under ``csrc/host`` into the pybind11 module
``_native``.  Plain ``nvcc`` / ``g++`` invocations, run in parallel, rebuilt only when a source or
header is newer than the object; nothing is installed outside the package directory.

``python -m nexus_b200._build`` builds everything; ``--force`` rebuilds from scratch.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB_DIR = PKG / "lib"
OBJ_DIR = PKG / "lib" / "obj"
CUDA_LIB = LIB_DIR / "libnexus_b200_cuda.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-Wall", "-pthread", "-ffp-contract=off"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", shutil.which("nvcc")):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found")


def _newest_header(dirs) -> float:
    t = 0.0
    for d in dirs:
        for pat in ("*.h", "*.cuh", "*.hpp"):
            for f in Path(d).glob(pat):
                t = max(t, f.stat().st_mtime)
    return t


def _run(cmd) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("command failed: %s\n%s\n%s" % (" ".join(map(str, cmd)), r.stdout, r.stderr))


def _compile_many(jobs, force: bool) -> bool:
    """jobs: (src, obj, cmd).  Returns True when anything was rebuilt."""
    todo = []
    for src, obj, cmd, dep_time in jobs:
        if force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, dep_time):
            todo.append(cmd)
    if todo:
        with ThreadPoolExecutor(max_workers=min(8, len(todo))) as ex:
            list(ex.map(_run, todo))
    return bool(todo)


def cuda_sources():
    return sorted((CSRC / "cuda").glob("*.cu"))


def host_sources():
    return sorted((CSRC / "host").glob("*.cpp"))


def native_module_path() -> Path:
    return PKG / ("_native" + sysconfig.get_config_var("EXT_SUFFIX"))


def build_cuda(force: bool = False, verbose: bool = False) -> Path:
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    nvcc = _nvcc()
    hdr = _newest_header([CSRC / "cuda"])
    jobs = []
    for src in cuda_sources():
        obj = OBJ_DIR / (src.stem + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-I", str(CSRC / "cuda"), "-c", str(src), "-o", str(obj)]
        jobs.append((src, obj, cmd, hdr))
    rebuilt = _compile_many(jobs, force)
    if rebuilt or not CUDA_LIB.exists():
        objs = [str(j[1]) for j in jobs]
        _run([nvcc, "-shared", "-o", str(CUDA_LIB), *objs, "-gencode", "arch=compute_100a,code=sm_100a",
              "-cudart", "static"])
        if verbose:
            print("linked", CUDA_LIB)
    return CUDA_LIB


def build_cuda_debug(verbose: bool = False) -> Path:
    """The kernel library with the debug-build bounds checks of the tile index arithmetic compiled in
    (`-DNX_DEBUG_BOUNDS`: a coordinate that leaves its tensor is recorded in the status word and the access is
    skipped).  Built on demand into `lib/libnexus_b200_cuda_dbg.so`; `NEXUS_B200_DEBUG_BOUNDS=1` makes
    `ops._cuda.lib()` load it instead of the release library."""
    out = CUDA_LIB.parent / "libnexus_b200_cuda_dbg.so"
    srcs = cuda_sources()
    newest = max([s.stat().st_mtime for s in srcs] + [_newest_header([CSRC / "cuda"])])
    if not out.exists() or out.stat().st_mtime < newest:
        dbg = OBJ_DIR / "dbg"
        dbg.mkdir(parents=True, exist_ok=True)
        cmds = [[_nvcc(), *NVCC_FLAGS, "-DNX_DEBUG_BOUNDS", "-I", str(CSRC / "cuda"), "-c", str(s), "-o",
                 str(dbg / (s.stem + ".o"))] for s in srcs]
        with ThreadPoolExecutor(max_workers=8) as ex:
            list(ex.map(_run, cmds))
        _run([_nvcc(), "-shared", "-o", str(out), *[str(dbg / (s.stem + ".o")) for s in srcs], "-gencode",
              "arch=compute_100a,code=sm_100a", "-cudart", "static"])
        if verbose:
            print("linked", out)
    return out


def build_gemm_profile(verbose: bool = False) -> Path:
    """Instrumented GEMM library (`-DNX_PROFILE_MMA`), built on demand by `python -m nexus_b200.bench.mma_profile`;
    not part of `build_all` and never loaded by the framework itself."""
    out = CUDA_LIB.parent / "libnexus_b200_gemm_prof.so"
    src = CSRC / "cuda" / "gemm_sm100.cu"
    if not out.exists() or out.stat().st_mtime < max(src.stat().st_mtime, _newest_header([CSRC / "cuda"])):
        _run([_nvcc(), *NVCC_FLAGS, "-DNX_PROFILE_MMA", "-I", str(CSRC / "cuda"), "-shared", "-Xcompiler", "-fPIC",
              str(src), "-o", str(out), "-cudart", "static", "-lcuda"])
        if verbose:
            print("linked", out)
    return out


def build_host(force: bool = False, verbose: bool = False) -> Path:
    import pybind11

    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    out = native_module_path()
    hdr = _newest_header([CSRC / "host"])
    inc = ["-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"], "-I", str(CSRC / "host")]
    jobs = []
    for src in host_sources():
        obj = OBJ_DIR / ("host_" + src.stem + ".o")
        cmd = ["g++", *CXX_FLAGS, *inc, "-c", str(src), "-o", str(obj)]
        jobs.append((src, obj, cmd, hdr))
    if not jobs:
        return out
    rebuilt = _compile_many(jobs, force)
    if rebuilt or not out.exists():
        _run(["g++", "-shared", "-o", str(out), *[str(j[1]) for j in jobs], "-pthread"])
        if verbose:
            print("linked", out)
    return out


SANITIZERS = {"asan": ["-fsanitize=address,undefined", "-fno-sanitize-recover=undefined"], "tsan": ["-fsanitize=thread"]}


def build_host_sanitized(kind: str = "asan", verbose: bool = False) -> Path:
    """A second build of the host module with AddressSanitizer + UBSan (``asan``) or ThreadSanitizer (``tsan``), written
    to ``build/sanitized/<kind>/`` beside the package.  It is loaded instead of the regular module when ``NEXUS_B200_NATIVE`` names it and
    the matching runtime is preloaded::

        NEXUS_B200_NATIVE=$(python -m nexus_b200._build --sanitize asan) \
        LD_PRELOAD=$(gcc -print-file-name=libasan.so) ASAN_OPTIONS=detect_leaks=0 python -m pytest tests/test_kv_sched.py
    """
    import pybind11

    flags = SANITIZERS[kind]
    odir = PKG.parent / "build" / "sanitized" / kind      # objects and module: outside the package, rebuilt on demand
    odir.mkdir(parents=True, exist_ok=True)
    out = odir / native_module_path().name
    inc = ["-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"], "-I", str(CSRC / "host")]
    base = [f for f in CXX_FLAGS if f != "-O2"] + ["-O1", "-g", "-fno-omit-frame-pointer", *flags]
    hdr = _newest_header([CSRC / "host"])
    jobs = [(src, odir / (src.stem + ".o"), ["g++", *base, *inc, "-c", str(src), "-o", str(odir / (src.stem + ".o"))], hdr)
            for src in host_sources()]
    rebuilt = _compile_many(jobs, False)
    if rebuilt or not out.exists():
        _run(["g++", "-shared", "-o", str(out), *[str(j[1]) for j in jobs], "-pthread", *flags])
        if verbose:
            print("linked", out, file=sys.stderr)
    return out


def build_tools(force: bool = False, verbose: bool = False):
    """Stand-alone native executables (launcher)."""
    outs = []
    tdir = CSRC / "tools"
    if not tdir.exists():
        return outs
    bindir = PKG / "bin"
    bindir.mkdir(exist_ok=True)
    for src in sorted(tdir.glob("*.cpp")):
        out = bindir / src.stem.replace("_", "-")
        if force or not out.exists() or out.stat().st_mtime < src.stat().st_mtime:
            _run(["g++", "-O2", "-std=c++17", "-pthread", "-o", str(out), str(src)])
            if verbose:
                print("built", out)
        outs.append(out)
    return outs


def build_all(force: bool = False, verbose: bool = False):
    return build_cuda(force, verbose), build_host(force, verbose), build_tools(force, verbose), build_cuda_debug(verbose)


if __name__ == "__main__":
    if "--sanitize" in sys.argv:
        print(build_host_sanitized(sys.argv[sys.argv.index("--sanitize") + 1], verbose=True))
    else:
        build_all(force="--force" in sys.argv, verbose=True)
        print("ok")
