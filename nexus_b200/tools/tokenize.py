"""`nexus_tokenize`: byte-level BPE training and tokenisation of text files into NXTK token shards.

A shard is ``"NXTK"`` | u32 version = 1 | u32 vocab | u64 count | u16 or u32 token ids (u16 when the
vocabulary fits).  The tokenizer starts from the 256 bytes and merges the most frequent adjacent pair
(ties: lowest pair) until the vocabulary size is reached; merges are stored as JSON.

    python -m nexus_b200.tools.tokenize train --vocab 512 --out tok.json corpus.txt
    python -m nexus_b200.tools.tokenize encode --tokenizer tok.json --out shard.nxtk corpus.txt

Parity: tools/nexus_tokenize/main.cpp of the reference."""
from __future__ import annotations

import argparse
import json
import struct
import sys
from collections import Counter
from typing import Dict, List, Tuple

import numpy as np

MAGIC = b"NXTK"


class ByteBpe:
    def __init__(self, merges: List[Tuple[int, int]] = ()):
        self.merges = [tuple(m) for m in merges]
        self.rank: Dict[Tuple[int, int], int] = {m: i for i, m in enumerate(self.merges)}

    @property
    def vocab_size(self) -> int:
        return 256 + len(self.merges)

    @staticmethod
    def train(data: bytes, vocab_size: int) -> "ByteBpe":
        if vocab_size < 256:
            raise ValueError("vocabulary must hold at least the 256 bytes")
        ids = list(data)
        merges: List[Tuple[int, int]] = []
        while 256 + len(merges) < vocab_size and len(ids) > 1:
            counts = Counter(zip(ids, ids[1:]))
            (pair, n) = min(counts.items(), key=lambda kv: (-kv[1], kv[0]))
            if n < 2:
                break
            new = 256 + len(merges)
            merges.append(pair)
            out, i = [], 0
            while i < len(ids):
                if i + 1 < len(ids) and ids[i] == pair[0] and ids[i + 1] == pair[1]:
                    out.append(new)
                    i += 2
                else:
                    out.append(ids[i])
                    i += 1
            ids = out
        return ByteBpe(merges)

    def encode(self, data: bytes) -> List[int]:
        ids = list(data)
        while len(ids) > 1:
            best = min(((self.rank.get(p, 1 << 30), i) for i, p in enumerate(zip(ids, ids[1:]))), default=(1 << 30, -1))
            if best[0] == 1 << 30:
                break
            pair = self.merges[best[0]]
            new = 256 + best[0]
            out, i = [], 0
            while i < len(ids):
                if i + 1 < len(ids) and ids[i] == pair[0] and ids[i + 1] == pair[1]:
                    out.append(new)
                    i += 2
                else:
                    out.append(ids[i])
                    i += 1
            ids = out
        return ids

    def decode(self, ids) -> bytes:
        table: Dict[int, bytes] = {i: bytes([i]) for i in range(256)}
        for k, (a, b) in enumerate(self.merges):
            table[256 + k] = table[a] + table[b]
        return b"".join(table[int(i)] for i in ids)

    def save(self, path: str) -> None:
        with open(path, "w") as f:
            json.dump({"type": "byte-bpe", "merges": self.merges}, f)

    @staticmethod
    def load(path: str) -> "ByteBpe":
        with open(path) as f:
            return ByteBpe([tuple(m) for m in json.load(f)["merges"]])


def write_shard(path: str, ids, vocab: int) -> None:
    arr = np.asarray(ids, dtype=np.uint16 if vocab <= 65536 else np.uint32)
    with open(path, "wb") as f:
        f.write(MAGIC + struct.pack("<IIQ", 1, vocab, arr.size))
        f.write(arr.tobytes())


def read_shard(path: str):
    with open(path, "rb") as f:
        head = f.read(20)
        if head[:4] != MAGIC:
            raise ValueError("not an NXTK shard")
        version, vocab, count = struct.unpack("<IIQ", head[4:])
        if version != 1:
            raise ValueError(f"NXTK version {version}")
        dt = np.uint16 if vocab <= 65536 else np.uint32
        data = np.frombuffer(f.read(), dtype=dt)
    if data.size != count:
        raise ValueError("NXTK shard is truncated")
    return data, vocab


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="nexus_tokenize")
    sub = ap.add_subparsers(dest="cmd", required=True)
    t = sub.add_parser("train")
    t.add_argument("--vocab", type=int, default=512)
    t.add_argument("--out", required=True)
    t.add_argument("files", nargs="+")
    e = sub.add_parser("encode")
    e.add_argument("--tokenizer", required=True)
    e.add_argument("--out", required=True)
    e.add_argument("files", nargs="+")
    a = ap.parse_args(argv)
    data = b"".join(open(p, "rb").read() for p in a.files)
    if a.cmd == "train":
        tok = ByteBpe.train(data, a.vocab)
        tok.save(a.out)
        print(f"{tok.vocab_size} tokens ({len(tok.merges)} merges)")
    else:
        tok = ByteBpe.load(a.tokenizer)
        ids = tok.encode(data)
        write_shard(a.out, ids, tok.vocab_size)
        print(f"{len(data)} bytes -> {len(ids)} tokens")
    return 0


if __name__ == "__main__":
    sys.exit(main())
