"""Value types of the PeerAgent runtime.

``ResourceKey`` generalises the reference's ``RdmaResourceKey`` (``dlslime/peer_agent/_agent.py:44-51``
in the reference) from RDMA NIC ports to any link a region can be reached through: an RDMA
port (``RoCE`` / ``IB``), the TCP fallback (``TCP``) or an NVLink peer mapping (``NVLink``).
The Redis suffix format ``{device}:{ib_port}:{link_type}`` is unchanged.
"""

from __future__ import annotations

import threading
from dataclasses import dataclass, field
from typing import Any, Optional


@dataclass(frozen=True)
class ResourceKey:
    device: str
    ib_port: int = 1
    link_type: str = "TCP"

    def redis_suffix(self) -> str:
        return f"{self.device}:{self.ib_port}:{self.link_type}"


RdmaResourceKey = ResourceKey  # name used by the reference


@dataclass
class LogicalMemoryRegion:
    name: str
    ptr: int
    offset: int
    length: int


@dataclass
class MaterializedMemoryRegion:
    name: str
    key: ResourceKey
    handler: int
    info: dict


@dataclass
class DirectedConnection:
    """One agent-to-agent link over one pair of resources."""

    local_alias: str
    peer_alias: str
    local_key: ResourceKey
    peer_key: ResourceKey
    qp_num: int = 1
    profile: str = "default"
    endpoint: Any = None
    state: str = "pending"  # pending | connecting | connected | failed | closed
    remote_handles: dict = field(default_factory=dict)  # mr name -> (remote handle, cached info)
    peer_digest: str = ""  # fingerprint of the endpoint description this link was connected to
    lock: threading.Lock = field(default_factory=threading.Lock)

    @property
    def conn_id(self) -> str:
        return (f"{self.local_alias}:{self.local_key.device}:port{self.local_key.ib_port}->"
                f"{self.peer_alias}:{self.peer_key.device}:port{self.peer_key.ib_port}#qp{self.qp_num}")

    def mirror_id(self) -> str:
        """The id the peer uses for the same link."""
        return (f"{self.peer_alias}:{self.peer_key.device}:port{self.peer_key.ib_port}->"
                f"{self.local_alias}:{self.local_key.device}:port{self.local_key.ib_port}#qp{self.qp_num}")

    def meta(self) -> dict:
        return {"conn_id": self.conn_id, "src": self.local_alias, "dst": self.peer_alias,
                "src_device": self.local_key.device, "dst_device": self.peer_key.device,
                "ib_port": self.local_key.ib_port, "qp_num": self.qp_num, "link_type": self.local_key.link_type,
                "profile": self.profile}


class PeerConnection:
    """Handle returned by ``PeerAgent.connect_to``; ``wait()`` blocks until the link is up."""

    def __init__(self, agent, conn_id: str):
        self._agent, self._conn_id = agent, conn_id

    def _connection(self) -> DirectedConnection:
        return self._agent._connections[self._conn_id]

    @property
    def peer_alias(self) -> str:
        return self._connection().peer_alias

    def wait(self, timeout: float = 60.0) -> "PeerConnection":
        self._agent._wait_connected(self._conn_id, timeout)
        return self

    def is_connected(self) -> bool:
        return self._connection().state == "connected"

    @property
    def conn_id(self) -> str:
        return self._conn_id

    @property
    def local_nic(self) -> str:
        return self._connection().local_key.device

    @property
    def remote_nic(self) -> str:
        return self._connection().peer_key.device

    @property
    def state(self) -> str:
        return self._connection().state

    @property
    def endpoint(self) -> Optional[Any]:
        return self._connection().endpoint

    def __repr__(self) -> str:
        return f"PeerConnection({self._conn_id!r}, state={self.state})"
