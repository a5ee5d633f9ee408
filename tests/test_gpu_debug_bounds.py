"""The debug build of the kernel library (tile-index bounds checks compiled in, `-DNX_DEBUG_BOUNDS`) runs the same GEMM
and attention problems as the release build, including ragged edges, without recording an out-of-range coordinate."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CODE = r"""
import sys, torch
sys.path.insert(0, %r)
from nexus_b200.ops import _cuda as K
assert K.lib()._name.endswith("libnexus_b200_cuda_dbg.so")
torch.manual_seed(0)
for (m, n, k) in ((512, 768, 256), (300, 520, 72), (129, 257, 64), (4096, 2304, 768)):
    a = torch.randn(m, k, device="cuda").bfloat16(); b = torch.randn(n, k, device="cuda").bfloat16()
    out = K.gemm(a, b)
    ref = a.float() @ b.float().t()
    assert (out.float() - ref).abs().max() <= 2e-2 * ref.abs().max(), (m, n, k)
    dw = K.gemm(a, a, a_mn=True, b_mn=True, out_dtype=torch.float32)
    assert (dw - a.float().t() @ a.float()).abs().max() <= 2e-2 * dw.abs().max()
q, k_, v = (torch.randn(2, 200, 4, 64, device="cuda").bfloat16() for _ in range(3))
o, lse = K.attention_fwd(q, k_, v, causal=True)
torch.cuda.synchronize()
K.check_status()
print("DEBUG_BOUNDS_OK")
"""


def test_debug_bounds_library_runs_clean():
    env = dict(os.environ, NEXUS_B200_DEBUG_BOUNDS="1")
    r = subprocess.run([sys.executable, "-c", CODE % ROOT], capture_output=True, text=True, env=env, timeout=300)
    assert "DEBUG_BOUNDS_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
