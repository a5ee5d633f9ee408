"""TCP key-value store for rendezvous and heartbeats: `set`, blocking `get`, `add`, `check`, `wait`,
`barrier`.  Wire format of a request: ``[u8 cmd][u32 key length][key][u64 value length][value]``; replies
are ``[u8 status][u64 length][payload]``.  Rank 0 runs the server inside its own process.  Server (accept thread,
one thread per connection) and client are native (`csrc/host/store.cpp`); a client call blocks without holding the
interpreter lock.
Parity: include/nexus/dist/store.hpp, src/dist/store.cpp of the reference."""
from __future__ import annotations

import struct
from typing import Optional, Sequence

from .. import _native

SET, GET, ADD, CHECK, WAIT = 1, 2, 3, 4, 5
OK, MISSING, TIMEOUT = 0, 1, 2


class TcpStore:
    def __init__(self, host: str = "127.0.0.1", port: int = 29500, is_server: bool = False, world_size: int = 1,
                 timeout_s: float = 60.0):
        self.world, self.timeout = world_size, timeout_s
        self.server = None
        if is_server:
            self.server = _native.StoreServer(host, int(port))
            port = self.server.port
        self.host, self.port = host, int(port)
        try:
            self._client = _native.StoreClient(host, self.port, float(timeout_s))
        except RuntimeError as e:
            raise TimeoutError(str(e)) from None
        self._barriers = 0

    def _call(self, cmd: int, key: str, value: bytes = b""):
        try:
            return self._client.call(cmd, key, value)
        except RuntimeError as e:
            raise ConnectionError(str(e)) from None

    def set(self, key: str, value) -> None:
        self._call(SET, key, value if isinstance(value, bytes) else str(value).encode())

    def get(self, key: str, timeout_s: Optional[float] = None) -> bytes:
        st, val = self._call(GET, key, struct.pack("<d", self.timeout if timeout_s is None else timeout_s))
        if st != OK:
            raise TimeoutError(f"store key {key!r} was not set in time")
        return val

    def add(self, key: str, delta: int = 1) -> int:
        _, val = self._call(ADD, key, struct.pack("<q", delta))
        return struct.unpack("<q", val)[0]

    def check(self, keys: Sequence[str]) -> bool:
        return all(self._call(CHECK, k)[0] == OK for k in keys)

    def wait(self, keys: Sequence[str], timeout_s: Optional[float] = None) -> None:
        for k in keys:
            st, _ = self._call(WAIT, k, struct.pack("<d", self.timeout if timeout_s is None else timeout_s))
            if st != OK:
                raise TimeoutError(f"store key {k!r} was not set in time")

    def barrier(self, name: str = "barrier", timeout_s: Optional[float] = None) -> None:
        """All `world_size` clients must call it the same number of times."""
        self._barriers += 1
        tag = f"{name}/{self._barriers}"
        if self.add(tag + "/count", 1) == self.world:
            self.set(tag + "/done", b"1")
        self.wait([tag + "/done"], timeout_s)

    def close(self) -> None:
        self._client.close()
        if self.server is not None:
            self.server.shutdown()
