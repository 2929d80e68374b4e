"""A small RESP2 client for the control plane's store (or any Redis server).

Only what PeerAgent, the cache service and the obs tools need: strings, hashes, lists,
streams, scans, expiry, publish. Replies come back as ``str`` (UTF-8), ``int``, ``None``
or nested lists, like ``redis-py`` with ``decode_responses=True``. One socket per client,
guarded by a lock; blocking commands (``blpop``, ``xread`` with ``block``) should use a
dedicated client (``clone()``), as the listener threads do.
"""

from __future__ import annotations

import socket
import threading
from typing import Any, Iterable


class RespError(RuntimeError):
    pass


class RespClient:
    def __init__(self, host: str = "127.0.0.1", port: int = 6379, timeout: float | None = None):
        self.host, self.port, self.timeout = host, int(port), timeout
        self._sock: socket.socket | None = None
        self._buf = b""
        self._lock = threading.Lock()

    @classmethod
    def from_address(cls, address: str, **kw) -> "RespClient":
        """``host:port`` or ``redis://host:port[/db]``."""
        a = address
        if "://" in a:
            a = a.split("://", 1)[1]
        a = a.split("/", 1)[0]
        host, _, port = a.rpartition(":")
        return cls(host or "127.0.0.1", int(port or 6379), **kw)

    def clone(self) -> "RespClient":
        return RespClient(self.host, self.port, self.timeout)

    # -- wire -------------------------------------------------------------------------
    def _connect(self) -> None:
        if self._sock is None:
            s = socket.create_connection((self.host, self.port), timeout=5.0)
            s.settimeout(self.timeout)
            s.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
            self._sock, self._buf = s, b""

    def close(self) -> None:
        with self._lock:
            if self._sock is not None:
                try:
                    self._sock.close()
                finally:
                    self._sock = None

    def _readline(self) -> bytes:
        while b"\r\n" not in self._buf:
            chunk = self._sock.recv(65536)
            if not chunk:
                raise ConnectionError("store connection closed")
            self._buf += chunk
        line, self._buf = self._buf.split(b"\r\n", 1)
        return line

    def _readn(self, n: int) -> bytes:
        while len(self._buf) < n + 2:
            chunk = self._sock.recv(max(65536, n + 2 - len(self._buf)))
            if not chunk:
                raise ConnectionError("store connection closed")
            self._buf += chunk
        data, self._buf = self._buf[:n], self._buf[n + 2:]
        return data

    def _reply(self) -> Any:
        line = self._readline()
        kind, rest = line[:1], line[1:]
        if kind == b"+":
            return rest.decode()
        if kind == b"-":
            raise RespError(rest.decode())
        if kind == b":":
            return int(rest)
        if kind == b"$":
            n = int(rest)
            return None if n < 0 else self._readn(n).decode("utf-8", "surrogateescape")
        if kind == b"*":
            n = int(rest)
            return None if n < 0 else [self._reply() for _ in range(n)]
        raise RespError(f"unexpected reply {line!r}")

    def execute(self, *args: Any) -> Any:
        out = [b"*%d\r\n" % len(args)]
        for a in args:
            b = a if isinstance(a, bytes) else str(a).encode("utf-8", "surrogateescape")
            out.append(b"$%d\r\n%s\r\n" % (len(b), b))
        with self._lock:
            try:
                self._connect()
                self._sock.sendall(b"".join(out))
                return self._reply()
            except (OSError, ConnectionError):
                if self._sock is not None:
                    self._sock.close()
                    self._sock = None
                raise

    # -- commands ----------------------------------------------------------------------
    def ping(self) -> bool:
        return self.execute("PING") == "PONG"

    def set(self, key, value, ex: int | None = None, px: int | None = None, nx: bool = False):
        args = ["SET", key, value]
        if ex is not None:
            args += ["EX", int(ex)]
        if px is not None:
            args += ["PX", int(px)]
        if nx:
            args.append("NX")
        return self.execute(*args) == "OK"

    def get(self, key):
        return self.execute("GET", key)

    def mget(self, keys: Iterable[str]):
        keys = list(keys)
        return self.execute("MGET", *keys) if keys else []

    def delete(self, *keys):
        return self.execute("DEL", *keys) if keys else 0

    def exists(self, *keys):
        return self.execute("EXISTS", *keys)

    def expire(self, key, seconds):
        return self.execute("EXPIRE", key, int(seconds)) == 1

    def pexpire(self, key, ms):
        return self.execute("PEXPIRE", key, int(ms)) == 1

    def ttl(self, key):
        return self.execute("TTL", key)

    def pttl(self, key):
        return self.execute("PTTL", key)

    def incr(self, key):
        return self.execute("INCR", key)

    def keys(self, pattern="*"):
        return self.execute("KEYS", pattern)

    def scan_iter(self, match="*", count=100):
        cursor = 0
        while True:
            cursor, keys = self.execute("SCAN", cursor, "MATCH", match, "COUNT", count)
            yield from keys
            cursor = int(cursor)
            if cursor == 0:
                return

    def hset(self, key, field=None, value=None, mapping: dict | None = None):
        args = []
        if field is not None:
            args += [field, value]
        for k, v in (mapping or {}).items():
            args += [k, v]
        return self.execute("HSET", key, *args)

    def hget(self, key, field):
        return self.execute("HGET", key, field)

    def hgetall(self, key) -> dict:
        flat = self.execute("HGETALL", key) or []
        return dict(zip(flat[::2], flat[1::2]))

    def hdel(self, key, *fields):
        return self.execute("HDEL", key, *fields)

    def lpush(self, key, *values):
        return self.execute("LPUSH", key, *values)

    def rpush(self, key, *values):
        return self.execute("RPUSH", key, *values)

    def lpop(self, key):
        return self.execute("LPOP", key)

    def llen(self, key):
        return self.execute("LLEN", key)

    def blpop(self, keys, timeout: float = 0):
        keys = [keys] if isinstance(keys, str) else list(keys)
        res = self.execute("BLPOP", *keys, timeout)
        return tuple(res) if res else None

    def xadd(self, key, fields: dict, id: str = "*", maxlen: int | None = None, approximate: bool = True):
        args = ["XADD", key]
        if maxlen is not None:
            args += ["MAXLEN", "~" if approximate else "=", int(maxlen)]
        args.append(id)
        for k, v in fields.items():
            args += [k, v]
        return self.execute(*args)

    def xlen(self, key):
        return self.execute("XLEN", key)

    def xread(self, streams: dict, count: int | None = None, block: int | None = None):
        """``streams`` maps key -> last seen id. Returns ``[(key, [(id, {field: value}), ...]), ...]``."""
        args = ["XREAD"]
        if count:
            args += ["COUNT", int(count)]
        if block is not None:
            args += ["BLOCK", int(block)]
        args.append("STREAMS")
        args += list(streams.keys()) + list(streams.values())
        res = self.execute(*args)
        out = []
        for key, entries in res or []:
            out.append((key, [(eid, dict(zip(flat[::2], flat[1::2]))) for eid, flat in entries]))
        return out

    def publish(self, channel, message):
        return self.execute("PUBLISH", channel, message)

    def flushall(self):
        return self.execute("FLUSHALL")
