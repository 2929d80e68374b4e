"""Client of a DLSlimeCache service: HTTP for the directory, endpoint I/O for the bytes.

``store / query / load / delete`` mirror the reference's client (``dlslime/cache/client.py:119-208``
in the reference). ``put`` and ``get`` add the data movement: ``put`` asks the directory for slabs
and writes the local bytes into them, ``get`` reads them back. In a manifest ``target_offset`` is the
offset in the client's region and ``source_offset`` the offset in the cache region; the named tuples
handed to the PeerAgent are therefore ``(local_region, "cache", target_offset, source_offset, length)``
(local offset first, remote offset second), which ``tests/test_cache.py`` pins.
"""

from __future__ import annotations

import json
import urllib.error
import urllib.request
from typing import Any

from .._slime_c import Assignment
from ..nanoctrl.client import NanoCtrlClient
from .types import DEFAULT_SERVICE_ID, assignment_to_json

_OPENER = urllib.request.build_opener(urllib.request.ProxyHandler({}))


def _request(url: str, path: str, body: dict | None, timeout: float) -> dict[str, Any]:
    data = None if body is None else json.dumps(body).encode()
    req = urllib.request.Request(url.rstrip("/") + path, data=data, headers={"Content-Type": "application/json"},
                                 method="GET" if body is None else "POST")
    try:
        with _OPENER.open(req, timeout=timeout) as rsp:
            return json.loads(rsp.read() or b"{}")
    except urllib.error.HTTPError as e:
        text = e.read().decode(errors="replace")
        try:
            msg = json.loads(text).get("error", text)
        except Exception:
            msg = text
        raise RuntimeError(f"{path} failed with HTTP {e.code}: {msg}") from None


def post_json(url: str, path: str, body: dict, *, timeout: float = 5.0) -> dict[str, Any]:
    return _request(url, path, body, timeout)


def get_json(url: str, path: str, *, timeout: float = 5.0) -> dict[str, Any]:
    return _request(url, path, None, timeout)


def discover_cache_url(ctrl: str, scope: str | None = None, service_id: str | None = DEFAULT_SERVICE_ID) -> str:
    client = NanoCtrlClient(ctrl, scope=scope)
    info = client.get_entity_info(service_id) if service_id else None
    if info is None:
        caches = client.list_entities(kind="cache")
        if not caches:
            raise RuntimeError("No NanoCtrl service with kind='cache' found")
        info = caches[0]
    ep = info.get("endpoint") or {}
    return f"http://{ep['host']}:{int(ep['port'])}"


class CacheClient:
    def __init__(self, url: str | None = None, *, peer_agent: Any | None = None, ctrl: str | None = None,
                 scope: str | None = None, service_id: str | None = DEFAULT_SERVICE_ID, timeout: float = 5.0):
        if url is None:
            if ctrl is None:
                raise ValueError("CacheClient requires either url or ctrl")
            url = discover_cache_url(ctrl, scope, service_id)
        self.url = url.rstrip("/")
        self.peer_agent = peer_agent
        self.timeout = timeout
        self._server_info: dict | None = None

    def server_peer_agent(self) -> dict[str, Any]:
        try:
            return get_json(self.url, "/peer-agent", timeout=self.timeout)
        except RuntimeError as e:
            if "HTTP 503" in str(e):
                raise RuntimeError("cache service did not publish a usable PeerAgent; start it with a control-plane "
                                   "address and a non-zero --memory-size") from e
            raise

    def connect_to_server(self, *, peer_agent: Any | None = None, alias: str | None = None, ctrl: str | None = None,
                          scope: str | None = None, local_device: str | None = None, peer_device: str | None = None,
                          ib_port: int = 1, qp_num: int = 1, timeout_sec: float = 60.0, link_type: str | None = None) -> dict[str, Any]:
        info = self.server_peer_agent()
        agent = peer_agent or self.peer_agent
        if agent is None or not hasattr(agent, "connect_to"):
            url = ctrl or info.get("nanoctrl_url")
            if not url:
                raise RuntimeError("cache service did not publish a NanoCtrl address")
            from ..peer_agent import PeerAgent

            agent = PeerAgent(nanoctrl_url=url, alias=alias, device=local_device, scope=scope if scope is not None else info.get("scope"))
        self.peer_agent = agent
        agent.connect_to(str(info["peer_agent_id"]), local_device=local_device, peer_device=peer_device, ib_port=ib_port,
                         qp_num=qp_num, link_type=link_type).wait(timeout=timeout_sec)
        self._server_info = info
        return info

    @staticmethod
    def peer_agent_id(peer_agent: Any | None) -> str:
        alias = getattr(peer_agent, "alias", None)
        if not alias:
            raise ValueError("peer_agent_id must be provided when no peer_agent.alias is available")
        return str(alias)

    def default_peer_agent_id(self) -> str:
        return self.peer_agent_id(self.peer_agent)

    def store(self, assignments: list[Assignment], *, peer_agent: Any | None = None, peer_agent_id: str | None = None) -> dict[str, Any]:
        owner = peer_agent_id or self.peer_agent_id(peer_agent or self.peer_agent)
        return post_json(self.url, "/store", {"peer_agent_id": owner, "assignments": [assignment_to_json(a) for a in assignments]},
                         timeout=self.timeout)

    def query(self, peer_agent_id: str, version: int) -> dict[str, Any]:
        return post_json(self.url, "/query", {"peer_agent_id": peer_agent_id, "version": int(version)}, timeout=self.timeout)

    def load(self, peer_agent_id: str, version: int) -> dict[str, Any]:
        return self.query(peer_agent_id, version)

    def delete(self, peer_agent_id: str, version: int) -> bool:
        return bool(post_json(self.url, "/delete", {"peer_agent_id": peer_agent_id, "version": int(version)}, timeout=self.timeout)["deleted"])

    def stats(self) -> dict[str, Any]:
        return get_json(self.url, "/stats", timeout=self.timeout)

    # -- data movement -----------------------------------------------------------------------
    def _tuples(self, local_region: str, manifest: dict) -> list[tuple]:
        cache_mr = (self._server_info or self.server_peer_agent())["cache_mr_name"]
        return [(local_region, cache_mr, int(a["target_offset"]), int(a["source_offset"]), int(a["length"]))
                for a in manifest["assignments"]]

    def put(self, local_region: str, extents: list[tuple[int, int]], timeout: float = 30.0) -> dict[str, Any]:
        """Store ``[(local_offset, length), ...]`` of ``local_region`` in the cache; returns the manifest."""
        if self._server_info is None:
            self.connect_to_server()
        manifest = self.store([Assignment(0, 0, int(off), 0, int(n)) for off, n in extents])
        fut = self.peer_agent.write(self._server_info["peer_agent_id"], self._tuples(local_region, manifest))
        status = fut.wait(timeout)
        if status != 0:
            raise RuntimeError(f"cache put failed with status {status}")
        return manifest

    def get(self, local_region: str, peer_agent_id: str, version: int, timeout: float = 30.0) -> dict[str, Any]:
        """Read a stored batch back into the offsets of ``local_region`` it came from."""
        if self._server_info is None:
            self.connect_to_server()
        manifest = self.query(peer_agent_id, version)
        fut = self.peer_agent.read(self._server_info["peer_agent_id"], self._tuples(local_region, manifest))
        status = fut.wait(timeout)
        if status != 0:
            raise RuntimeError(f"cache get failed with status {status}")
        return manifest
