"""DLSlimeCache service: slab directory (C++), registered cache memory, HTTP front-end.

The service stores no payload itself: ``POST /store`` allocates slabs and returns a manifest
whose ``source_offset`` fields are offsets inside the service's registered region ``"cache"``;
the client then moves the bytes with one-sided endpoint writes, and reads them back after
``POST /query``. Routes and JSON follow the reference (``dlslime/cache/service.py:117-177`` in
the reference): ``GET /healthz, /stats, /peer-agent``; ``POST /store, /query, /delete``; errors
are ``{"error": msg}`` with 400 / 404 / 503. The cache memory may live on a GPU
(``device="cuda:N"``), in which case clients reach it over NVLink.
"""

from __future__ import annotations

import ctypes
import json
import socket
import threading
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from typing import Any

from .. import _slime_c
from ..logging import get_logger
from ..nanoctrl.client import NanoCtrlClient
from .types import (DEFAULT_CACHE_MR_NAME, DEFAULT_MEMORY_SIZE, DEFAULT_SERVICE_ID, DEFAULT_SLAB_SIZE, assignment_from_json,
                    manifest_to_json, stats_to_json)

log = get_logger("cache.service")
_cache = _slime_c.cache


def resolve_host_for_registration(host: str) -> str:
    return socket.gethostname() if host in {"", "0.0.0.0", "::"} else host


class CacheService:
    """In-process cache service object; ``peer_agent`` is a composed dependency, not a base class."""

    def __init__(self, peer_agent: Any | None = None, *, slab_size: int = DEFAULT_SLAB_SIZE,
                 memory_size: int = DEFAULT_MEMORY_SIZE, cache_mr_name: str = DEFAULT_CACHE_MR_NAME, device: str | None = None):
        self.cache = _cache.CacheServer(slab_size=slab_size, memory_size=memory_size)
        self.peer_agent = peer_agent
        self.cache_mr_name = cache_mr_name
        self.cache_storage = None
        self.cache_mr_handle = None
        self.device = device
        if peer_agent is not None and memory_size > 0:
            if device and device.startswith("cuda"):
                import torch

                self.cache_storage = torch.zeros(memory_size, dtype=torch.uint8, device=device)
                ptr = self.cache_storage.data_ptr()
            else:
                self.cache_storage = ctypes.create_string_buffer(memory_size)
                ptr = ctypes.addressof(self.cache_storage)
            self.cache_mr_handle = peer_agent.register_memory_region(cache_mr_name, ptr, 0, memory_size)

    @property
    def slab_size(self) -> int:
        return int(self.cache.slab_size())

    @property
    def memory_size(self) -> int:
        return int(self.cache.memory_size())

    def store_assignments(self, peer_agent_id: str, assignments: list):
        return self.cache.store_assignments(peer_agent_id, assignments)

    def query_assignments(self, peer_agent_id: str, version: int):
        return self.cache.query_assignments(peer_agent_id, int(version))

    def delete_assignments(self, peer_agent_id: str, version: int) -> bool:
        return bool(self.cache.delete_assignments(peer_agent_id, int(version)))

    def stats(self):
        return self.cache.stats()

    def peer_agent_info(self) -> dict[str, Any]:
        if self.peer_agent is None:
            raise RuntimeError("cache service was started without a PeerAgent")
        alias = str(getattr(self.peer_agent, "alias", ""))
        if not alias:
            raise RuntimeError("cache service PeerAgent has no alias")
        if self.cache_mr_handle is None:
            raise RuntimeError("cache service was started without preallocated cache memory")
        return {"peer_agent_id": alias, "cache_mr_name": self.cache_mr_name, "cache_mr_handle": self.cache_mr_handle,
                "nanoctrl_url": getattr(self.peer_agent, "nanoctrl_url", None),
                "scope": getattr(self.peer_agent, "_scope", None) or None, "slab_size": self.slab_size,
                "memory_size": self.memory_size, "resource": self.peer_agent.get_resource(), "device": self.device}


class _Handler(BaseHTTPRequestHandler):
    service: CacheService = None  # set on the subclass created by CacheHttpServer
    protocol_version = "HTTP/1.1"

    def log_message(self, fmt, *args):  # quiet by default
        log.debug("%s " + fmt, self.address_string(), *args)

    def _send(self, status: int, body: dict) -> None:
        data = json.dumps(body).encode()
        self.send_response(status)
        self.send_header("Content-Type", "application/json")
        self.send_header("Content-Length", str(len(data)))
        self.end_headers()
        self.wfile.write(data)

    def _body(self) -> dict:
        n = int(self.headers.get("Content-Length") or 0)
        raw = self.rfile.read(n) if n else b"{}"
        body = json.loads(raw or b"{}")
        if not isinstance(body, dict):
            raise ValueError("request body must be a JSON object")
        return body

    def do_GET(self):
        try:
            if self.path == "/healthz":
                return self._send(200, {"ok": True})
            if self.path == "/stats":
                return self._send(200, stats_to_json(self.service.stats()))
            if self.path == "/peer-agent":
                try:
                    return self._send(200, self.service.peer_agent_info())
                except RuntimeError as e:
                    return self._send(503, {"error": str(e)})
            return self._send(404, {"error": f"no such route: {self.path}"})
        except Exception as e:
            return self._send(500, {"error": str(e)})

    def do_POST(self):
        try:
            body = self._body()
        except Exception as e:
            return self._send(400, {"error": f"bad request body: {e}"})
        try:
            if self.path == "/store":
                assigns = [assignment_from_json(a) for a in body.get("assignments", [])]
                m = self.service.store_assignments(str(body.get("peer_agent_id", "")), assigns)
                return self._send(200, manifest_to_json(m))
            if self.path == "/query":
                m = self.service.query_assignments(str(body.get("peer_agent_id", "")), int(body.get("version", 0)))
                if m is None:
                    return self._send(404, {"error": "no such assignment manifest"})
                return self._send(200, manifest_to_json(m))
            if self.path == "/delete":
                ok = self.service.delete_assignments(str(body.get("peer_agent_id", "")), int(body.get("version", 0)))
                return self._send(200, {"deleted": ok})
            return self._send(404, {"error": f"no such route: {self.path}"})
        except (ValueError, KeyError, TypeError) as e:
            return self._send(400, {"error": str(e)})
        except RuntimeError as e:
            return self._send(400, {"error": str(e)})
        except Exception as e:
            return self._send(500, {"error": str(e)})


class CacheHttpServer:
    """Threaded HTTP server in front of a :class:`CacheService`."""

    def __init__(self, service: CacheService, host: str = "127.0.0.1", port: int = 0):
        handler = type("BoundCacheHandler", (_Handler,), {"service": service})
        self.httpd = ThreadingHTTPServer((host, port), handler)
        self.httpd.daemon_threads = True
        self.host, self.port = host, self.httpd.server_address[1]
        self._thread: threading.Thread | None = None

    @property
    def url(self) -> str:
        return f"http://{'127.0.0.1' if self.host in ('', '0.0.0.0') else self.host}:{self.port}"

    def start(self) -> "CacheHttpServer":
        self._thread = threading.Thread(target=self.httpd.serve_forever, name="cache-http", daemon=True)
        self._thread.start()
        return self

    def serve_forever(self) -> None:
        self.httpd.serve_forever()

    def stop(self) -> None:
        self.httpd.shutdown()
        self.httpd.server_close()
        if self._thread is not None:
            self._thread.join(timeout=2.0)


class NanoCtrlRegistration:
    """Registers the cache service as entity ``cache:0`` (kind ``cache``) and keeps it alive."""

    def __init__(self, ctrl: str, host: str, port: int, scope: str | None = None, service_id: str = DEFAULT_SERVICE_ID,
                 p2p_host: str | None = None, p2p_port: int | None = None):
        self.client = NanoCtrlClient(ctrl, scope=scope)
        self.service_id = service_id
        self.endpoint = {"host": resolve_host_for_registration(host), "port": int(port), "protocol": "http"}
        self.metadata = {"p2p_host": p2p_host, "p2p_port": p2p_port}

    def register(self) -> None:
        self.client.register(self.service_id, "cache", endpoint=self.endpoint, metadata=self.metadata)

    def start(self, interval: float = 15.0) -> None:
        self.register()
        self.client.start_heartbeat(self.service_id, interval=interval, on_not_found=self.register)

    def stop(self) -> None:
        self.client.stop_heartbeat()
        try:
            self.client.unregister(self.service_id)
        except Exception:
            pass


class CacheServer:
    """Everything a cache process needs: PeerAgent, service, HTTP server and NanoCtrl registration.

    Called the way the reference's ``dlslime.cache.CacheServer`` is called (nothing but ``slab_size`` / ``memory_size``,
    by keyword or as the two positional numbers) it returns the slab directory itself, which is what that name means
    there (``dlslime/cache/__init__.py:23`` in the reference); the directory is also ``dlslime_b200.cache.CacheDirectory``.
    """

    def __new__(cls, ctrl=None, *args, **kw):
        process_keys = {"host", "port", "scope", "alias", "device", "metadata_only"}
        if (ctrl is None or isinstance(ctrl, int)) and not (process_keys & kw.keys()):
            numbers = ([ctrl] if isinstance(ctrl, int) else []) + list(args)
            return _cache.CacheServer(*numbers, **kw)
        return super().__new__(cls)

    def __init__(self, ctrl: str | None = None, *, host: str = "127.0.0.1", port: int = 0, slab_size: int = DEFAULT_SLAB_SIZE,
                 memory_size: int = DEFAULT_MEMORY_SIZE, scope: str | None = None, alias: str | None = None,
                 device: str | None = None, metadata_only: bool = False):
        self.agent = None
        if ctrl and not metadata_only:
            from ..peer_agent import PeerAgent

            self.agent = PeerAgent(nanoctrl_url=ctrl, alias=alias, scope=scope, device=device if device and device.startswith("cuda") else None)
        self.service = CacheService(self.agent, slab_size=slab_size, memory_size=memory_size, device=device)
        self.http = CacheHttpServer(self.service, host, port).start()
        self.registration = NanoCtrlRegistration(ctrl, host if host not in ("", "0.0.0.0") else "127.0.0.1", self.http.port, scope) if ctrl else None
        if self.registration:
            self.registration.start()

    @property
    def url(self) -> str:
        return self.http.url

    def stop(self) -> None:
        if self.registration:
            self.registration.stop()
        self.http.stop()
        if self.agent is not None:
            self.agent.shutdown()
