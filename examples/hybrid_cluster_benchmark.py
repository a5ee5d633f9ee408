"""CPU GEMM (deterministic thread pool), the same product through the GPU tensor-core GEMM when a B200 is present,
and a two-rank all-reduce mean over the in-process thread world.  Prints a small table; exits non-zero when a
result is wrong.  Counterpart of apps/hybrid_cluster_benchmark of the reference."""
import os
import sys
import time

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from nexus_b200 import cpu  # noqa: E402
from nexus_b200.parallel.process_group import run_threads  # noqa: E402


def timed(fn, repeats: int = 4) -> float:
    fn()
    t0 = time.perf_counter()
    for _ in range(repeats):
        fn()
    return (time.perf_counter() - t0) / repeats


def main() -> int:
    n = 256
    a = np.full((n, n), 0.01, dtype=np.float32)
    b = np.full((n, n), 0.02, dtype=np.float32)
    c = cpu.gemm_nt(a, b)
    flops = 2.0 * n ** 3
    rows = [("CPU GEMM", timed(lambda: cpu.gemm_nt(a, b)))]
    ok = bool(np.allclose(c, n * 0.01 * 0.02, rtol=1e-5))
    if torch.cuda.is_available():
        from nexus_b200.ops import _cuda as K
        ga, gb = torch.from_numpy(a).cuda().bfloat16(), torch.from_numpy(b).cuda().bfloat16()

        def gpu():
            K.gemm(ga, gb)
            torch.cuda.synchronize()
        rows.append(("GPU GEMM (tcgen05)", timed(gpu)))
        ok &= bool(torch.allclose(K.gemm(ga, gb).float().cpu(), torch.from_numpy(c), rtol=2e-2))

    def rank_fn(pg):
        t = torch.tensor([[2.0, 8.0, 4.0], [6.0, 0.0, 2.0]][pg.rank()])
        return pg.all_reduce_tensor(t, "sum") / pg.size()
    means = run_threads(2, rank_fn)
    ok &= abs(float(means[0][0]) - 4.0) < 1e-5 and abs(float(means[1][2]) - 3.0) < 1e-5
    print("| operation | time us | GFLOPS |")
    for name, sec in rows:
        print(f"| {name} | {sec * 1e6:.1f} | {flops / sec / 1e9:.1f} |")
    print(f"allreduce_mean={float(means[0][0])}")
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
