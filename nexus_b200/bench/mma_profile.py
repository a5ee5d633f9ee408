"""Where the tcgen05-issuing thread of the GEMM spends its time (profiling build of the kernel).

    python -m nexus_b200.bench.mma_profile

For each shape: CUDA-event time of one launch and, averaged over the persistent CTAs, the share of the MMA
thread's cycles spent waiting for a free TMEM accumulator (epilogue behind), waiting for TMA data (loads
behind), and between a stage's arrival and the commit of its four MMAs - the issue blocks while the
tensor-core queue is full, so this share is the time the tensor core itself needs per k-block.  A second line gives the first epilogue warp's cycles per tile (from
"accumulator ready" to "accumulator released") and how much of that it waited for TMEM loads and for a free
staging tile of the tiled stores.
"""
from __future__ import annotations

import ctypes as C
import sys

import numpy as np
import torch

from .. import _build
from ..ops import _cuda as K

SHAPES = [(16384, 2304, 64), (16384, 2304, 768), (16384, 3072, 768), (16384, 768, 3072), (8192, 8192, 8192)]


def plain(shape) -> int:
    """`--plain M N K`: four launches of the product kernel on one shape (the target of a profiler capture)."""
    m, n, k = shape
    a = torch.randn(m, k, device="cuda").bfloat16()
    b = torch.randn(n, k, device="cuda").bfloat16()
    bias = torch.randn(n, device="cuda").bfloat16()
    for _ in range(4):
        K.gemm(a, b, bias=bias)
    K.check_status()
    return 0


def main() -> int:
    """The first shape has a single k-block per tile: its epilogue runs with next to no tensor-core or TMA-load
    traffic beside it, which shows the epilogue's own cost."""
    lib = C.CDLL(str(_build.build_gemm_profile()))
    K._lib = lib                    # route gemm() through the instrumented library
    for m, n, k in SHAPES:
        a = torch.randn(m, k, device="cuda").bfloat16()
        b = torch.randn(n, k, device="cuda").bfloat16()
        bias = torch.randn(n, device="cuda").bfloat16()
        for _ in range(3):
            K.gemm(a, b, bias=bias)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        K.gemm(a, b, bias=bias)
        e1.record()
        torch.cuda.synchronize()
        buf = (C.c_longlong * (256 * 8))()
        lib.nx_gemm_prof_read(buf)
        r = np.array(buf[:], dtype=np.int64).reshape(256, 8)
        r = r[r[:, 4] > 0]
        tot, acc, tma, issue, nkb, nt = (r[:, i].mean() for i in range(6))
        print(f"{m}x{n}x{k}: {e0.elapsed_time(e1) * 1e3:8.1f} us | accumulator wait {acc / tot * 100:4.1f} % | "
              f"TMA wait {tma / tot * 100:4.1f} % | issue-to-commit {issue / tot * 100:4.1f} % | "
              f"{tot / nkb:6.0f} cycles per k-block ({nt:.1f} tiles, {nkb:.0f} k-blocks per CTA)", flush=True)
        lib.nx_gemm_prof_read_epilogue(buf)
        e = np.array(buf[:], dtype=np.int64).reshape(256, 8)
        e = e[e[:, 3] > 0]
        busy, ld, slot, tiles, bias_c, stage, fence, issue = (e[:, i].sum() for i in range(8))
        print(f"    first epilogue warp: {busy / tiles:6.0f} cycles per tile, of which TMEM-load wait {ld / tiles:5.0f}, "
              f"store-slot wait {slot / tiles:5.0f}, bias {bias_c / tiles:5.0f}, staging {stage / tiles:5.0f}, "
              f"proxy fence {fence / tiles:5.0f}, store issue {issue / tiles:5.0f}; mainloop {tot / nt:6.0f} cycles per tile",
              flush=True)
    K.check_status()
    return 0


if __name__ == "__main__":
    if len(sys.argv) == 5 and sys.argv[1] == "--plain":
        sys.exit(plain([int(x) for x in sys.argv[2:5]]))
    sys.exit(main())
