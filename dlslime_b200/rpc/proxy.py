"""Client side: ``proxy(agent, peer, ServiceClass).method(args).wait()``."""

from __future__ import annotations

import pickle
from typing import Any, Iterable

from .. import _slime_c
from .channel import get_or_create_channel
from .errors import RemoteRpcError, RpcError, RpcTimeoutError
from .registry import MethodInfo, MethodRegistry


class RpcFuture:
    """Result of one call. ``wait(timeout)`` returns the value, raises what the handler raised
    (as :class:`RemoteRpcError`) or :class:`RpcTimeoutError`."""

    def __init__(self, session, cfut, info: MethodInfo):
        self._session, self._cfut, self._info = session, cfut, info

    def done(self) -> bool:
        return self._cfut.done()

    def wait(self, timeout: float | None = None) -> Any:
        try:
            data = self._cfut.wait() if timeout is None else self._cfut.wait_for(timeout)
        except RuntimeError as e:
            raise RpcError(str(e)) from None
        if data is None:
            self._session.detach_request(self._cfut.request_id)
            raise RpcTimeoutError(f"RPC {self._info.name!r} got no reply within {timeout} s")
        if self._cfut.is_remote_exception:
            try:
                exc = pickle.loads(data)
            except Exception:
                exc = {"type": "RemoteError", "message": repr(data[:200]), "traceback": ""}
            raise RemoteRpcError(exc.get("type", "Exception"), exc.get("message", ""), exc.get("traceback", ""))
        return self._info.loads_result(data)


class _BoundMethod:
    def __init__(self, channel, info: MethodInfo):
        self._channel, self._info = channel, info

    def __call__(self, *args, **kwargs) -> RpcFuture:
        payload = self._info.dumps_args(args, kwargs)
        session = self._channel.session
        if len(payload) > session.payload_capacity:
            raise RpcError(f"RPC {self._info.name!r}: {len(payload)} argument bytes exceed the slot capacity of "
                           f"{session.payload_capacity}; raise agent._rpc_buffer_size or lower agent._rpc_max_inflight")
        try:
            cfut = session.call(self._info.tag, payload)
        except RuntimeError as e:
            raise RpcError(str(e)) from None
        return RpcFuture(session, cfut, self._info)


class ServiceProxy:
    def __init__(self, channel, registry: MethodRegistry):
        self._channel, self._registry = channel, registry
        for name, info in registry.by_name.items():
            setattr(self, name, _BoundMethod(channel, info))

    def close(self) -> None:
        self._channel.close()


def proxy(agent, peer_alias: str, service_cls: type, **channel_kw) -> ServiceProxy:
    """A client stub for ``service_cls`` served by ``peer_alias`` (which must already be connected)."""
    return ServiceProxy(get_or_create_channel(agent, peer_alias, for_server=False, **channel_kw), MethodRegistry(service_cls))


def wait_all(futures: Iterable[RpcFuture], timeout: float | None = None) -> list:
    return [f.wait(timeout) for f in futures]


WIRE_VERSION = _slime_c.rpc.WIRE_VERSION
