"""Native host bookkeeping of the paged-KV engine: block pool, copy-on-write, truncation and batch packing."""
import os
import time

import numpy as np
import pytest

from nexus_b200 import _native


def _plan(s, chunks, device_tokens=False, max_tokens=4096):
    seqs = [c[0] for c in chunks]
    toks = [list(c[1]) for c in chunks]
    flat = [t for c in toks for t in c] if not device_tokens else [0] * len(chunks)
    return s.plan(seqs, [len(t) for t in toks], flat, [c[2] for c in chunks], [int(c[3]) for c in chunks], device_tokens,
                  max_tokens)


def _rows(s, width):
    h = np.full((6, width), 77, dtype=np.int32)
    s.write(h.ctypes.data, width)
    return h


def test_prefill_decode_packing_and_padding():
    s = _native.KvScheduler(16, 4, 8, 64)
    a, b = s.add(), s.add()
    assert (a, b) == (0, 1) and s.free_blocks() == 16 and s.live_sequences() == 2
    p = _plan(s, [(a, [5, 6, 7, 8, 9], 1, False), (b, [1, 2, 3], 1, False)])
    assert p["tokens"] == 8 and p["logit_rows"] == 2 and p["prefill_tokens"] == 8 and p["decode_tokens"] == 0
    assert p["runs"] == [("flash", 0, 5, a), ("flash", 5, 8, b)] and p["logit_seq"] == [a, b] and p["out_rows"] == []
    assert sorted(p["tables"]) == [a, b] and p["cows"] == [] and p["patches"] == []
    assert s.blocks(a) == [0, 1] and s.blocks(b) == [2] and s.free_blocks() == 13
    h = _rows(s, 16)
    assert h[0, :8].tolist() == [5, 6, 7, 8, 9, 1, 2, 3] and h[1, :8].tolist() == [0, 1, 2, 3, 4, 0, 1, 2]
    assert h[2, :8].tolist() == [0, 1, 2, 3, 4, 8, 9, 10] and h[3, :8].tolist() == [a] * 5 + [b] * 3
    assert h[4, :8].tolist() == [1, 2, 3, 4, 5, 1, 2, 3] and h[5, :2].tolist() == [4, 7]
    assert (h[[0, 1, 3, 4], 8:] == 0).all() and (h[2, 8:] == -1).all() and (h[5, 2:] == 0).all()
    assert s.n_prompt(a) == 5 and s.length(a) == 5 and s.tokens(b) == [1, 2, 3]
    # decode step: adjacent one-token chunks merge into one paged run; output rows are reported
    p = _plan(s, [(a, [11], 1, True), (b, [12], 1, True)])
    assert p["runs"] == [("paged", 0, 2, -1)] and p["decode_tokens"] == 2 and p["out_rows"] == [0, 1]
    assert p["tables"] == [] and s.n_prompt(a) == 5 and s.tokens(a)[-1] == 11
    # a cached-prefix continuation (several tokens onto a non-empty sequence) is a paged run counted as prefill
    p = _plan(s, [(a, [1, 2, 3], 3, False)])
    assert p["runs"] == [("paged", 0, 3, -1)] and p["prefill_tokens"] == 3 and p["logit_rows"] == 3 and s.blocks(a) == [0, 1, 3]
    with pytest.raises(ValueError):
        s.write(0, 16)
    with pytest.raises(ValueError):
        h = np.zeros((6, 2), dtype=np.int32)
        s.write(h.ctypes.data, 2)


def test_fork_copy_on_write_truncate_and_free():
    s = _native.KvScheduler(8, 4, 4, 32)
    a = s.add()
    _plan(s, [(a, [1, 2, 3, 4, 5, 6], 1, False)])                  # blocks [0, 1], second one half full
    f = s.fork(a)
    assert s.blocks(f) == [0, 1] and s.refcount(0) == s.refcount(1) == 2 and s.tokens(f) == s.tokens(a)
    assert s.blocks_needed(f, 1) == 1 and s.blocks_needed(f, 3) == 2 and s.blocks_needed(f, 0) == 0
    p = _plan(s, [(f, [9], 1, True)])
    assert p["cows"] == [(1, 2)] and p["tables"] == [f] and s.blocks(f) == [0, 2] and s.blocks(a) == [0, 1]
    assert s.refcount(1) == 1 and s.refcount(2) == 1 and s.refcount(0) == 2
    assert _rows(s, 1)[2, 0] == 2 * 4 + 2                                 # position 6 lands in the copied block
    p = _plan(s, [(a, [8], 1, True)])                                     # the original now owns block 1 alone: no copy
    assert p["cows"] == [] and p["tables"] == []
    removed, n_out = s.truncate(f, 5)
    assert removed == [6, 9] and n_out == 1 and s.length(f) == 5 and s.n_prompt(f) == 5 and s.blocks(f) == [0, 2]
    removed, n_out = s.truncate(f, 2)
    assert removed == [3, 4, 5] and n_out == 0 and s.blocks(f) == [0] and s.n_prompt(f) == 2 and s.free_blocks() == 6
    assert s.truncate(f, 2) == ([], 0)
    with pytest.raises(ValueError):
        s.truncate(f, 3)
    s.free(a)
    assert s.refcount(0) == 1 and s.free_blocks() == 7 and not s.live(a)
    s.free(f)
    assert s.free_blocks() == 8 and s.live_sequences() == 0
    with pytest.raises(KeyError):
        s.length(a)
    with pytest.raises(KeyError):
        s.fork(a)
    assert s.live_sequences() == 0                                         # the refused fork took no slot


def test_device_fed_tokens_limits_and_exhaustion():
    s = _native.KvScheduler(2, 4, 2, 6)
    a = s.add()
    _plan(s, [(a, [1, 2, 3], 1, False)])
    p = _plan(s, [(a, [0], 1, True)], device_tokens=True)
    assert p["patches"] == [(a, 3)] and s.tokens(a) == [1, 2, 3, -1]
    assert s.patch(a, 3, 42) and s.tokens(a)[-1] == 42 and not s.patch(a, 3, 43) and not s.patch(1, 0, 1)
    with pytest.raises(ValueError, match="one-token"):
        _plan(s, [(a, [0, 0], 1, True)], device_tokens=True)
    with pytest.raises(ValueError, match="context length"):
        _plan(s, [(a, [1, 2, 3], 1, False)])
    with pytest.raises(ValueError, match="max_tokens"):
        _plan(s, [(a, [1, 2], 1, False)], max_tokens=1)
    b = s.add()
    with pytest.raises(RuntimeError, match="max_seqs"):
        s.add()
    _plan(s, [(b, [1], 1, False)])
    with pytest.raises(RuntimeError, match="exhausted"):
        _plan(s, [(b, [1, 2, 3, 4], 1, False)])
    with pytest.raises(ValueError):
        s.plan([a], [1, 1], [0], [1], [0], False, 8)


def test_packing_a_large_decode_step_is_fast():
    """256 one-token chunks: plan + write stay far below a millisecond (the Python loops they replace took several)."""
    n = 256
    s = _native.KvScheduler(n * 70, 16, n, 2048)
    ids = [s.add() for _ in range(n)]
    _plan(s, [(i, list(range(700)), 1, False) for i in ids], max_tokens=n * 700)
    h = np.zeros((6, n), dtype=np.int32)
    seqs, counts, flat, ones = ids, [1] * n, [3] * n, [1] * n
    best = 1e9
    for _ in range(20):
        t0 = time.perf_counter()
        s.plan(seqs, counts, flat, ones, ones, False, 8192)
        s.write(h.ctypes.data, n)
        best = min(best, time.perf_counter() - t0)
    if not os.environ.get("NEXUS_B200_NATIVE"):          # an instrumented (sanitizer) build is not timed
        assert best < 2e-3, best
    assert h[1, 0] == 719 and h[4, 0] == 720


def test_a_refused_step_changes_nothing():
    """Every failure of `plan` (pool exhausted by a later chunk, context overflow, too many tokens, unknown sequence) is
    found before the first change: lengths, token lists, block lists, reference counts and the free count stay put."""
    s = _native.KvScheduler(4, 4, 4, 12)
    a, b = s.add(), s.add()
    _plan(s, [(a, [1, 2, 3, 4, 5], 1, False), (b, [1, 2], 1, False)])             # a: 2 blocks, b: 1 block, 1 free
    f = s.fork(b)

    def state():
        return ([(s.length(i), s.tokens(i), s.blocks(i), s.n_prompt(i)) for i in (a, b, f)], s.free_blocks(),
                [s.refcount(i) for i in range(4)], _rows(s, 8).tolist())
    before = state()
    bad = [
        ([(a, [9, 9, 9, 9], 1, True), (f, [7], 1, True)], RuntimeError),                      # a new block for a and a CoW copy, one free block
        ([(a, [9], 1, True), (b, list(range(11)), 1, False)], ValueError),                    # context length on the second chunk
        ([(a, [9], 1, True), (b, [1, 2], 1, False)], ValueError),                             # max_tokens (see below)
        ([(a, [9], 1, True), (3, [1], 1, False)], KeyError),                                   # unknown sequence
        ([(a, [9], 1, True), (a, list(range(7)), 1, True)], ValueError),                       # the same sequence twice: 6 + 7 > 12
    ]
    for chunks, err in bad:
        with pytest.raises(err):
            _plan(s, chunks, max_tokens=2 if err is ValueError and len(chunks[1][1]) == 2 else 4096)
        assert state() == before
    # two sequences sharing a partial block append in one step: only the first copies, the second then owns the block
    g = _native.KvScheduler(3, 4, 3, 12)
    x = g.add()
    _plan(g, [(x, [1, 2], 1, False)])
    y = g.fork(x)
    p = _plan(g, [(x, [3], 1, True), (y, [4], 1, True)])
    assert p["cows"] == [(0, 1)] and g.blocks(x) == [1] and g.blocks(y) == [0] and g.free_blocks() == 1
    # the same sequence twice in one step is fine when it fits: blocks are counted once
    p = _plan(s, [(a, [9], 1, True), (a, [8, 7], 1, True)])
    assert s.length(a) == 8 and s.tokens(a)[-3:] == [9, 8, 7] and s.blocks(a) == [0, 1] and p["tokens"] == 3
    p = _plan(s, [(f, [5], 1, True)])
    assert p["cows"] == [(2, 3)] and s.free_blocks() == 0
    with pytest.raises(RuntimeError):
        _plan(s, [(b, [1, 2, 3], 1, True)])                                                   # would need a new block
    assert s.length(b) == 2
    _plan(s, [(b, [1, 2], 1, True)])                                                          # exactly fills its block
    assert s.length(b) == 4 and s.refcount(2) == 1
