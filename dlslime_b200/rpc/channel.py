"""One RPC channel = the buffers and the C++ session between this agent and one peer.

Buffers (names as in the reference, ``dlslime/rpc/proxy.py:23,88-121``): the send staging buffer
``rpc:send:{peer}``, the receive mailbox ``rpc:mailbox:{local}:{peer}`` of ``slot_count`` slots of
``slot_size`` bytes, and the peer's mailbox ``rpc:mailbox:{peer}:{local}`` which is looked up in the
control-plane store (polled for up to 30 s, since the peer may still be starting). Slot geometry
comes from ``agent._rpc_buffer_size`` and ``agent._rpc_max_inflight`` and must match on both sides;
the length of the peer's mailbox is checked against it.
"""

from __future__ import annotations

import ctypes
import time

from .. import _slime_c
from .errors import RpcError

MAILBOX_WAIT_S = 30.0


class GrowableBuffer:
    """Page-aligned host buffer registered with an agent under a fixed name."""

    def __init__(self, agent, name: str, nbytes: int):
        self.agent, self.name, self.nbytes = agent, name, int(nbytes)
        self._raw = ctypes.create_string_buffer(self.nbytes + 4096)
        base = ctypes.addressof(self._raw)
        self.ptr = (base + 4095) & ~4095
        self.handle = agent.register_memory_region(name, self.ptr, 0, self.nbytes)

    def close(self) -> None:
        try:
            self.agent.unregister_memory_region(self.name)
        except Exception:
            pass


class RpcChannel:
    def __init__(self, agent, peer_alias: str, for_server: bool, slot_size: int | None = None, slot_count: int | None = None):
        conn = agent._get_connection(peer_alias)
        if conn.state != "connected":
            raise RpcError(f"connect to {peer_alias!r} first: agent.connect_to({peer_alias!r}).wait()")
        self.agent, self.peer, self.conn = agent, peer_alias, conn
        self.slot_count = int(slot_count or agent._rpc_max_inflight)
        self.slot_size = int(slot_size or max(4096, agent._rpc_buffer_size // self.slot_count))
        self.send_buf = GrowableBuffer(agent, f"rpc:send:{peer_alias}", self.slot_size)
        self.recv_buf = GrowableBuffer(agent, f"rpc:mailbox:{agent.alias}:{peer_alias}", self.slot_size * self.slot_count)
        remote_name = f"rpc:mailbox:{peer_alias}:{agent.alias}"
        deadline = time.monotonic() + MAILBOX_WAIT_S
        while True:
            info = agent.get_mr_info(peer_alias, remote_name, conn.peer_key)
            if info is not None:
                break
            if time.monotonic() > deadline:
                raise RpcError(f"peer {peer_alias!r} did not publish its RPC mailbox within {MAILBOX_WAIT_S} s")
            time.sleep(0.005)
        if int(info["length"]) != self.slot_size * self.slot_count:
            raise RpcError(f"RPC mailbox geometry differs: peer has {info['length']} bytes, expected "
                           f"{self.slot_size} x {self.slot_count}")
        send_h = agent.get_handle(conn, self.send_buf.name)
        recv_h = agent.get_handle(conn, self.recv_buf.name)
        remote_h = agent.get_handle(conn, remote_name, remote=True)
        # a pure client with a single slot needs no pump thread: call() waits for its own reply
        pump = for_server or self.slot_count > 1
        self.session = _slime_c.rpc.RpcSession(conn.endpoint, send_h, self.send_buf.ptr, recv_h, self.recv_buf.ptr, remote_h,
                                               self.slot_size, self.slot_count, pump)

    def close(self) -> None:
        try:
            self.session.close()
        finally:
            self.send_buf.close()
            self.recv_buf.close()


def get_or_create_channel(agent, peer_alias: str, for_server: bool = False, **kw) -> RpcChannel:
    ch = agent._rpc_channels.get(peer_alias)
    if ch is None or ch.session.closed:
        ch = agent._rpc_channels[peer_alias] = RpcChannel(agent, peer_alias, for_server, **kw)
    return ch
