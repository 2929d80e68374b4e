"""SlimeRPC: method calls between PeerAgents over one-sided mailbox writes."""

from .errors import RemoteRpcError, RpcError, RpcTimeoutError
from .proxy import RpcFuture, ServiceProxy, proxy, wait_all
from .registry import MethodRegistry, method
from .rnr import SoftRnrMonitor
from .service import serve, serve_once

__all__ = ["method", "proxy", "serve", "serve_once", "wait_all", "RpcError", "RemoteRpcError", "RpcTimeoutError",
           "SoftRnrMonitor", "MethodRegistry", "RpcFuture", "ServiceProxy"]
