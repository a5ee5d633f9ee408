"""TCP key-value store for rendezvous and heartbeats: `set`, blocking `get`, `add`, `check`, `wait`,
`barrier`.  Wire format of a request: ``[u8 cmd][u32 key length][key][u64 value length][value]``; replies
are ``[u8 status][u64 length][payload]``.  Rank 0 runs the server thread inside its own process.
Parity: include/nexus/dist/store.hpp, src/dist/store.cpp of the reference."""
from __future__ import annotations

import socket
import struct
import threading
import time
from typing import Dict, List, Optional, Sequence

SET, GET, ADD, CHECK, WAIT = 1, 2, 3, 4, 5
OK, MISSING, TIMEOUT = 0, 1, 2


def _recv_exact(sock: socket.socket, n: int) -> bytes:
    buf = bytearray()
    while len(buf) < n:
        chunk = sock.recv(n - len(buf))
        if not chunk:
            raise ConnectionError("store connection closed")
        buf.extend(chunk)
    return bytes(buf)


class _Server(threading.Thread):
    def __init__(self, host: str, port: int):
        super().__init__(name="nexus-store", daemon=True)
        self.sock = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
        self.sock.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
        self.sock.bind((host, port))
        self.sock.listen(128)
        self.port = self.sock.getsockname()[1]
        self.data: Dict[bytes, bytes] = {}
        self.cv = threading.Condition()
        self.stop = False

    def run(self) -> None:
        while not self.stop:
            try:
                conn, _ = self.sock.accept()
            except OSError:
                return
            threading.Thread(target=self._serve, args=(conn,), daemon=True).start()

    def _reply(self, conn, status: int, payload: bytes = b"") -> None:
        conn.sendall(struct.pack("<BQ", status, len(payload)) + payload)

    def _serve(self, conn: socket.socket) -> None:
        try:
            while True:
                cmd, klen = struct.unpack("<BI", _recv_exact(conn, 5))
                key = _recv_exact(conn, klen)
                (vlen,) = struct.unpack("<Q", _recv_exact(conn, 8))
                val = _recv_exact(conn, vlen) if vlen else b""
                if cmd == SET:
                    with self.cv:
                        self.data[key] = val
                        self.cv.notify_all()
                    self._reply(conn, OK)
                elif cmd in (GET, WAIT):
                    (timeout,) = struct.unpack("<d", val) if len(val) == 8 else (300.0,)
                    deadline = time.monotonic() + timeout
                    with self.cv:
                        while key not in self.data:
                            left = deadline - time.monotonic()
                            if left <= 0:
                                break
                            self.cv.wait(left)
                        got = self.data.get(key)
                    if got is None:
                        self._reply(conn, TIMEOUT)
                    else:
                        self._reply(conn, OK, got if cmd == GET else b"")
                elif cmd == ADD:
                    (delta,) = struct.unpack("<q", val)
                    with self.cv:
                        cur = int(self.data.get(key, b"0")) + delta
                        self.data[key] = str(cur).encode()
                        self.cv.notify_all()
                    self._reply(conn, OK, struct.pack("<q", cur))
                elif cmd == CHECK:
                    with self.cv:
                        self._reply(conn, OK if key in self.data else MISSING)
                else:
                    return
        except (ConnectionError, OSError, struct.error):
            pass
        finally:
            conn.close()

    def shutdown(self) -> None:
        self.stop = True
        try:
            self.sock.close()
        except OSError:
            pass


class TcpStore:
    def __init__(self, host: str = "127.0.0.1", port: int = 29500, is_server: bool = False, world_size: int = 1,
                 timeout_s: float = 60.0):
        self.world, self.timeout = world_size, timeout_s
        self.server: Optional[_Server] = None
        if is_server:
            self.server = _Server(host, port)
            self.server.start()
            port = self.server.port
        self.host, self.port = host, port
        deadline = time.monotonic() + timeout_s
        while True:
            try:
                self.sock = socket.create_connection((host, port), timeout=timeout_s)
                self.sock.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
                break
            except OSError:
                if time.monotonic() > deadline:
                    raise TimeoutError(f"no store at {host}:{port}")
                time.sleep(0.05)
        self._lock = threading.Lock()
        self._barriers = 0

    def _call(self, cmd: int, key: str, value: bytes = b""):
        k = key.encode()
        with self._lock:
            self.sock.sendall(struct.pack("<BI", cmd, len(k)) + k + struct.pack("<Q", len(value)) + value)
            status, n = struct.unpack("<BQ", _recv_exact(self.sock, 9))
            return status, (_recv_exact(self.sock, n) if n else b"")

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
        try:
            self.sock.close()
        except OSError:
            pass
        if self.server is not None:
            self.server.shutdown()
