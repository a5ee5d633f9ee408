"""Native memory-mapped token shard reader: window numbering across shards, rank striding, the keyed per-epoch
permutation, resume by global cursor, the read-ahead thread, and refusal of malformed files."""
import struct
import threading

import numpy as np
import pytest

from nexus_b200 import _native
from nexus_b200.tools.tokenize import write_shard
from nexus_b200.train import ArrayTokens, ShardTokens


def _shards(tmp_path, sizes, vocab=50000, seed=0):
    rng = np.random.default_rng(seed)
    paths, arrays = [], []
    for i, n in enumerate(sizes):
        a = rng.integers(0, vocab, size=n)
        p = tmp_path / f"s{i}.bin"
        write_shard(str(p), a, vocab)
        paths.append(str(p))
        arrays.append(a.astype(np.int32))
    return paths, arrays


def _windows(arrays, T):
    return np.concatenate([a[: len(a) // T * T].reshape(-1, T) for a in arrays if len(a) >= T])


@pytest.mark.parametrize("prefetch", [0, 3])
def test_sequential_windows_across_shards_match_the_arrays(tmp_path, prefetch):
    T = 16
    paths, arrays = _shards(tmp_path, [16 * 5 + 7, 9, 16 * 3, 16 * 2 + 15])
    want = _windows(arrays, T)
    src = ShardTokens(paths, T, prefetch=prefetch)
    assert src.windows() == len(want) == 10 and src.vocab() == 50000
    got = np.concatenate([src.next_rows(4, T) for _ in range(5)])      # 20 rows: two epochs
    assert got.dtype == np.int32 and np.array_equal(got, np.concatenate([want, want]))
    assert src.global_cursor() == 20
    # one shard, no shuffle: the same walk as the in-memory source
    one = ShardTokens(paths[0], T, rank=1, world=2, prefetch=prefetch)
    ref = ArrayTokens(arrays[0], rank=1, world=2)
    for _ in range(4):
        assert np.array_equal(one.next_rows(3, T), ref.next_rows(3, T))
    assert one.global_cursor() == ref.global_cursor()


def test_wide_vocabulary_shards_are_read_as_u32(tmp_path):
    T = 8
    paths, arrays = _shards(tmp_path, [8 * 6], vocab=200000)
    assert arrays[0].max() > 65535
    src = ShardTokens(paths, T, prefetch=1)
    assert np.array_equal(src.next_rows(6, T), arrays[0].reshape(6, T)) and src.vocab() == 200000


def test_shuffle_is_a_permutation_per_epoch_and_ranks_partition_it(tmp_path):
    T = 4
    paths, arrays = _shards(tmp_path, [4 * 37, 4 * 20 + 3])
    want = _windows(arrays, T)
    total = len(want)
    key = {tuple(r): i for i, r in enumerate(want)}
    assert len(key) == total                                           # windows are distinct, so rows identify them
    world = 3
    seen = [[] for _ in range(2)]
    readers = [ShardTokens(paths, T, rank=r, world=world, seed=7, shuffle=True, prefetch=2) for r in range(world)]
    per_rank = 2 * total // world                                      # two epochs exactly: 2 * 57 = 114 = 3 * 38
    rows = [rd.next_rows(per_rank, T) for rd in readers]
    for c in range(per_rank):
        for r in range(world):
            g = c * world + r
            seen[g // total].append(key[tuple(rows[r][c])])
    assert sorted(seen[0]) == sorted(seen[1]) == list(range(total))    # every window once per epoch
    assert seen[0] != list(range(total)) and seen[0] != seen[1]        # shuffled, and differently each epoch
    other = ShardTokens(paths, T, seed=8, shuffle=True).next_rows(total, T)
    same = ShardTokens(paths, T, seed=7, shuffle=True).next_rows(total, T)
    assert np.array_equal(same, np.stack([want[i] for i in seen[0]])) and not np.array_equal(other, same)
    # the bijection itself, on awkward sizes
    for n in (1, 2, 3, 5, 17, 64, 1000):
        assert sorted(_native.permute_index(i, n, 12345) for i in range(n)) == list(range(n))


@pytest.mark.parametrize("prefetch", [0, 2])
def test_seek_resumes_exactly_and_reshards(tmp_path, prefetch):
    T = 8
    paths, _ = _shards(tmp_path, [8 * 50])
    a = ShardTokens(paths, T, seed=3, shuffle=True, prefetch=prefetch)
    head = [a.next_rows(4, T) for _ in range(3)]
    cur = a.global_cursor()
    tail = [a.next_rows(4, T) for _ in range(3)]
    b = ShardTokens(paths, T, seed=3, shuffle=True, prefetch=prefetch)
    b.seek(cur)
    assert all(np.array_equal(x, y) for x, y in zip(tail, [b.next_rows(4, T) for _ in range(3)]))
    a.seek(0)                                                           # rewinding a reader with batches in flight
    assert all(np.array_equal(x, y) for x, y in zip(head, [a.next_rows(4, T) for _ in range(3)]))
    # the same 24 global rows read by two ranks from the cursor of a one-rank job
    two = [ShardTokens(paths, T, rank=r, world=2, seed=3, shuffle=True, prefetch=prefetch) for r in range(2)]
    for t in two:
        t.seek(cur)
    inter = np.empty((12, T), dtype=np.int32)
    inter[0::2], inter[1::2] = two[0].next_rows(6, T), two[1].next_rows(6, T)
    assert np.array_equal(inter, np.concatenate(tail))
    # a different batch size mid-stream restarts the read-ahead at the right row
    c = ShardTokens(paths, T, seed=3, shuffle=True, prefetch=prefetch)
    mixed = np.concatenate([c.next_rows(4, T), c.next_rows(8, T), c.next_rows(2, T), c.next_rows(10, T)])
    assert np.array_equal(mixed, np.concatenate(head + tail))


def test_next_into_fills_caller_memory_and_read_ahead_runs_off_the_interpreter_lock(tmp_path):
    T = 32
    paths, arrays = _shards(tmp_path, [32 * 64])
    src = ShardTokens(paths, T, prefetch=4)
    buf = np.zeros((8, T), dtype=np.int32)
    src.next_into(buf.ctypes.data, 8, T)
    assert np.array_equal(buf, arrays[0][: 8 * T].reshape(8, T))
    with pytest.raises(ValueError):
        src.next_into(buf.ctypes.data, 8, T + 1)
    # two consumers on two readers in parallel threads: no deadlock, each sees its own stream in order
    out = {}

    def work(name, rank):
        rd = ShardTokens(paths, T, rank=rank, world=2, prefetch=3)
        out[name] = np.concatenate([rd.next_rows(2, T) for _ in range(40)])
    th = [threading.Thread(target=work, args=(f"t{r}", r)) for r in range(2)]
    for t in th:
        t.start()
    for t in th:
        t.join(timeout=30)
        assert not t.is_alive()
    want = _windows(arrays, T)
    for r in range(2):
        idx = [(c * 2 + r) % len(want) for c in range(80)]
        assert np.array_equal(out[f"t{r}"], want[idx])
    from nexus_b200.data.loader import GpuTokenLoader
    ld = GpuTokenLoader(ShardTokens(paths, T), 4, T, device="cpu")
    first = ld.next().clone()
    second = ld.next().clone()
    ld.close()
    assert np.array_equal(first.numpy(), want[:4]) and np.array_equal(second.numpy(), want[4:8])


def test_malformed_shards_are_refused(tmp_path):
    good, _ = _shards(tmp_path, [64])
    bad = tmp_path / "bad.bin"
    bad.write_bytes(b"NOPE" + bytes(32))
    with pytest.raises(RuntimeError, match="not an NXTK"):
        ShardTokens([good[0], str(bad)], 8)
    short = tmp_path / "short.bin"
    short.write_bytes(b"NXTK" + struct.pack("<IIQ", 1, 1000, 500) + bytes(100))      # claims 500 tokens, holds 50
    with pytest.raises(RuntimeError, match="truncated"):
        ShardTokens(str(short), 8)
    v2 = tmp_path / "v2.bin"
    v2.write_bytes(b"NXTK" + struct.pack("<IIQ", 2, 1000, 4) + bytes(8))
    with pytest.raises(RuntimeError, match="version"):
        ShardTokens(str(v2), 2)
    with pytest.raises(RuntimeError, match="cannot open"):
        ShardTokens(str(tmp_path / "missing.bin"), 8)
    with pytest.raises(ValueError, match="seq_len tokens"):
        ShardTokens(good, 128)
    with pytest.raises(ValueError):
        ShardTokens(good, 8, rank=2, world=2)
    with pytest.raises(ValueError):
        ShardTokens(good, 8).next_rows(2, 4)


def test_trainer_on_shards_matches_the_in_memory_source(tmp_path):
    """The LM trainer fed from mapped shards takes the same steps as one fed from the same tokens in memory."""
    import torch
    from nexus_b200.lm.config import preset
    from nexus_b200.lm.model import LanguageModel
    from nexus_b200.train import AdamW, LanguageTrainerBuilder
    cfg = preset("nano")
    cfg.n_layer, cfg.d_model, cfg.d_ff, cfg.max_position = 1, 32, 64, 16
    data = np.random.default_rng(0).integers(0, 256, size=16 * 24)
    write_shard(str(tmp_path / "d.bin"), data, 256)

    def run(source):
        torch.manual_seed(0)
        tr = (LanguageTrainerBuilder(LanguageModel(cfg)).data(source).optimizer(AdamW(lr=1e-3)).micro_batch(4).seq_len(16)
              .global_batch_tokens(8 * 16).precision("f32").execution_policy("cpu").log_every(0).build())
        tr.train(3)
        return [r.loss for r in tr.history], source.global_cursor()
    a = run(ShardTokens(str(tmp_path / "d.bin"), 16))
    b = run(ArrayTokens(data.astype(np.int32)))
    assert a == b and a[1] >= 24
