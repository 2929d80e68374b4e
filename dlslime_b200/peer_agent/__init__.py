"""PeerAgent runtime: registration, discovery, handshake and named I/O on top of any endpoint."""

from ._agent import PeerAgent, start_peer_agent
from ._types import DirectedConnection, PeerConnection, RdmaResourceKey, ResourceKey

__all__ = ["PeerAgent", "start_peer_agent", "PeerConnection", "DirectedConnection", "ResourceKey", "RdmaResourceKey"]
