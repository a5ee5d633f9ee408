"""The allocation-free column-sum entry point, called through its exported C symbol.

Some hosts of this library cannot allocate device memory while they run (all HBM already belongs to
their own arena, or an allocation's implicit synchronisation is not acceptable on their hot path).
`nx_colsum_static` serves them: it keeps its partial sums in a fixed array inside the library.  The
test runs it twice in a row on different inputs (the array keeps the first call's contents) and
compares each result with the regular entry point, which takes caller-provided scratch.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call_static(lib, dy, out, accumulate=0):
    fn = lib.nx_colsum_static
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_int64, C.c_int, C.c_void_p]
    dtype = 0 if dy.dtype == torch.bfloat16 else 1
    return fn(dy.data_ptr(), dtype, out.data_ptr(), dy.shape[0], dy.shape[1], dy.stride(0), accumulate,
              torch.cuda.current_stream().cuda_stream)


def test_colsum_static_matches_regular_entry_point_twice():
    from nexus_b200.ops import _cuda as K
    lib = K.lib()
    torch.manual_seed(0)
    first = torch.randn(3000, 768, device="cuda").bfloat16()
    second = torch.randn(517, 1000, device="cuda")          # different shape and dtype on purpose
    for dy in (first, second):
        want = K.colsum(dy)
        got = torch.full((dy.shape[1],), float("nan"), device="cuda")
        assert _call_static(lib, dy, got) == 0
        torch.cuda.synchronize()
        assert (got - want).abs().max().item() <= 1e-4 * max(want.abs().max().item(), 1.0)
        ref = dy.float().sum(0)
        assert (got - ref).abs().max().item() <= 1e-4 * max(ref.abs().max().item(), 1.0)
    # accumulate into an existing output
    base = torch.randn(768, device="cuda")
    got = base.clone()
    assert _call_static(lib, first, got, accumulate=1) == 0
    torch.cuda.synchronize()
    want = base + K.colsum(first)
    assert (got - want).abs().max().item() <= 1e-4 * max(want.abs().max().item(), 1.0)


def test_colsum_static_strided_odd_width_and_tall_inputs():
    """A BF16 view whose row stride exceeds its width and whose width is not a multiple of 8 (the scalar path),
    and an input tall enough to use all 64 row chunks of the built-in array."""
    from nexus_b200.ops import _cuda as K
    lib = K.lib()
    torch.manual_seed(1)
    wide = torch.randn(700, 1024, device="cuda").bfloat16()
    view = wide[:, 3:3 + 501]                                  # ld 1024 > cols 501, 501 % 8 != 0, unaligned start
    tall = torch.randn(16384 + 777, 264, device="cuda").bfloat16()
    for dy in (view, tall, view):                              # the repeat runs on the tall call's leftovers
        got = torch.full((dy.shape[1],), float("nan"), device="cuda")
        assert _call_static(lib, dy, got) == 0
        torch.cuda.synchronize()
        ref = dy.float().sum(0)
        assert (got - ref).abs().max().item() <= 1e-4 * max(ref.abs().max().item(), 1.0)
        want = K.colsum(dy)
        assert (got - want).abs().max().item() <= 1e-4 * max(want.abs().max().item(), 1.0)


def test_colsum_static_rejects_oversize():
    from nexus_b200.ops import _cuda as K
    lib = K.lib()
    lib.nx_colsum_static_max_cols.restype = C.c_int
    limit = lib.nx_colsum_static_max_cols()
    assert limit == 8192
    dy = torch.zeros(4, limit + 8, device="cuda")
    out = torch.zeros(limit + 8, device="cuda")
    assert _call_static(lib, dy, out) == -5
