"""Server side: ``serve(agent, service_object, peer_alias)``.

The loop polls the C++ session for requests and runs handlers on a thread pool of
``SLIME_RPC_SERVER_WORKERS`` (default 1) threads. Handlers of one service object are
serialised by a lock unless marked ``parallel``. An exception in a handler travels back as a
pickled ``{"type", "message", "traceback"}`` with the EXC flag; a ``None`` result is an empty reply.
"""

from __future__ import annotations

import ctypes
import os
import pickle
import threading
import traceback
from concurrent.futures import ThreadPoolExecutor

from .. import _slime_c
from ..logging import get_logger
from .channel import get_or_create_channel
from .registry import MethodRegistry

log = get_logger("rpc.service")
EXC_BIT = _slime_c.rpc.EXC_BIT


def _dispatch(session, registry: MethodRegistry, service, lock: threading.Lock, req) -> None:
    info = registry.by_tag.get(req.base_tag)
    try:
        if info is None:
            raise LookupError(f"no RPC method with tag {req.base_tag}")
        if info.inplace:
            view = (ctypes.c_char * req.payload_nbytes).from_address(req.payload_ptr) if req.payload_nbytes else b""

            def writer(ptr: int, cap: int) -> int:
                if info.parallel:
                    return int(info.fn(service, memoryview(view), ptr, cap))
                with lock:
                    return int(info.fn(service, memoryview(view), ptr, cap))

            session.post_reply_inplace(info.tag, req.request_id, req.slot_id, writer)
            return
        data = ctypes.string_at(req.payload_ptr, req.payload_nbytes) if req.payload_nbytes else b""
        args, kwargs = info.loads_args(data)
        if info.parallel:
            result = info.fn(service, *args, **kwargs)
        else:
            with lock:
                result = info.fn(service, *args, **kwargs)
        session.post_reply(info.tag, req.request_id, req.slot_id, info.dumps_result(result))
    except Exception as e:
        payload = pickle.dumps({"type": type(e).__name__, "message": str(e), "traceback": traceback.format_exc()},
                               protocol=pickle.HIGHEST_PROTOCOL)
        try:
            session.post_reply((req.base_tag) | EXC_BIT, req.request_id, req.slot_id, payload[: session.payload_capacity])
        except Exception:
            log.exception("could not deliver the error reply of request %s", req.request_id)


def serve(agent, service, peer_alias: str, stop_event: threading.Event | None = None, poll_timeout: float = 0.1, **channel_kw) -> None:
    """Serve ``service`` to ``peer_alias`` until ``stop_event`` is set or the session closes. Blocks."""
    channel = get_or_create_channel(agent, peer_alias, for_server=True, **channel_kw)
    registry = MethodRegistry(type(service))
    lock = threading.Lock()
    workers = int(os.environ.get("SLIME_RPC_SERVER_WORKERS", "1") or 1)
    with ThreadPoolExecutor(max_workers=max(1, workers), thread_name_prefix=f"rpc-{agent.alias}") as pool:
        while not channel.session.closed and not (stop_event is not None and stop_event.is_set()):
            req = channel.session.poll_request(poll_timeout)
            if req is None:
                continue
            if workers <= 1:
                _dispatch(channel.session, registry, service, lock, req)
            else:
                pool.submit(_dispatch, channel.session, registry, service, lock, req)


def serve_once(agent, service, peer_alias: str, timeout: float = 30.0, **channel_kw) -> bool:
    """Handle exactly one request; returns False when none arrived within ``timeout``."""
    channel = get_or_create_channel(agent, peer_alias, for_server=True, **channel_kw)
    req = channel.session.poll_request(timeout)
    if req is None:
        return False
    _dispatch(channel.session, MethodRegistry(type(service)), service, threading.Lock(), req)
    return True
