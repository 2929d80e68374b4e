"""Client of a DLSlimeCache service: HTTP for the directory, endpoint I/O for the bytes.

The public surface follows the reference's client (``dlslime/cache/client.py:119-208`` in the
reference): ``store / query / load / delete / stats``, ``server_peer_agent`` and
``connect_to_server``. ``put`` and ``get`` add the data movement: ``put`` asks the directory for
slabs and writes the local bytes into them, ``get`` reads them back. In a manifest
``target_offset`` is the offset in the client's region and ``source_offset`` the offset in the
cache region; the named tuples handed to the PeerAgent are therefore
``(local_region, "cache", target_offset, source_offset, length)`` (local offset first, remote
offset second), which ``tests/test_cache_service.py`` pins.

Layout of this module: ``_Http`` is the only place that talks HTTP (one opener without proxies,
JSON in and out, server-side errors turned into ``RuntimeError("<path> failed with HTTP <code>: ...")``);
``_locate`` turns a control-plane record into a base URL; ``CacheClient`` holds one ``_Http`` and,
once connected, the description of the server's PeerAgent.
"""

from __future__ import annotations

import json
import urllib.error
import urllib.request
from typing import Any, Iterable

from .._slime_c import Assignment
from ..nanoctrl.client import NanoCtrlClient
from .types import DEFAULT_SERVICE_ID, assignment_to_json


class _Http:
    """JSON over HTTP against one base URL."""

    _opener = urllib.request.build_opener(urllib.request.ProxyHandler({}))  # never through an environment proxy

    def __init__(self, base: str, timeout: float):
        self.base, self.timeout = base.rstrip("/"), timeout

    def call(self, path: str, body: dict | None = None, timeout: float | None = None) -> dict[str, Any]:
        payload = json.dumps(body).encode() if body is not None else None
        req = urllib.request.Request(self.base + path, data=payload, method="POST" if body is not None else "GET",
                                     headers={"Content-Type": "application/json"})
        try:
            with self._opener.open(req, timeout=self.timeout if timeout is None else timeout) as rsp:
                raw = rsp.read()
        except urllib.error.HTTPError as err:
            raise RuntimeError(f"{path} failed with HTTP {err.code}: {self._reason(err)}") from None
        return json.loads(raw) if raw else {}

    @staticmethod
    def _reason(err: urllib.error.HTTPError) -> str:
        text = err.read().decode(errors="replace")
        try:
            doc = json.loads(text)
        except ValueError:
            return text
        return doc.get("error", text) if isinstance(doc, dict) else text


def post_json(url: str, path: str, body: dict, *, timeout: float = 5.0) -> dict[str, Any]:
    return _Http(url, timeout).call(path, body)


def get_json(url: str, path: str, *, timeout: float = 5.0) -> dict[str, Any]:
    return _Http(url, timeout).call(path)


def _locate(record: dict) -> str | None:
    """Base URL of a cache entity record, or None when the record carries no usable endpoint."""
    endpoint = record.get("endpoint") if isinstance(record, dict) else None
    if not isinstance(endpoint, dict):
        return None
    host, port = endpoint.get("host"), endpoint.get("port")
    try:
        port = int(port)
    except (TypeError, ValueError):
        return None
    if not host or not 0 < port < 65536:
        return None
    return f"http://{host}:{port}"


def discover_cache_url(ctrl: str, scope: str | None = None, service_id: str | None = DEFAULT_SERVICE_ID) -> str:
    """Ask the control plane where a cache service listens: the entity ``service_id`` when it exists and is usable,
    else the first usable entity of kind ``cache``."""
    directory = NanoCtrlClient(ctrl, scope=scope)
    candidates: list[dict] = []
    if service_id:
        named = directory.get_entity_info(service_id)
        if named is not None:
            candidates.append(named)
    if not candidates:
        candidates = list(directory.list_entities(kind="cache"))
    for record in candidates:
        url = _locate(record)
        if url is not None:
            return url
    what = f"entity {service_id!r} or any entity" if service_id else "an entity"
    raise RuntimeError(f"the control plane at {ctrl} lists no usable cache service ({what} of kind 'cache' with an endpoint)")


class CacheClient:
    def __init__(self, url: str | None = None, *, peer_agent: Any | None = None, ctrl: str | None = None,
                 scope: str | None = None, service_id: str | None = DEFAULT_SERVICE_ID, timeout: float = 5.0):
        if url is None and ctrl is None:
            raise ValueError("CacheClient requires either url or ctrl")
        self.url = (url or discover_cache_url(ctrl, scope, service_id)).rstrip("/")
        self.peer_agent = peer_agent
        self.timeout = timeout
        self._http = _Http(self.url, timeout)
        self._server_info: dict | None = None

    # -- the service's PeerAgent -------------------------------------------------------------------
    def server_peer_agent(self) -> dict[str, Any]:
        """The description the service publishes of its PeerAgent (alias, cache region name, control plane)."""
        try:
            return self._http.call("/peer-agent")
        except RuntimeError as err:
            if " HTTP 503" not in str(err):
                raise
            raise RuntimeError("the cache service runs without a data plane (HTTP 503 on /peer-agent): start it with a "
                               "control-plane address and a non-zero --memory-size") from err

    def _agent_for(self, info: dict, given: Any | None, *, alias, ctrl, scope, device) -> Any:
        """The PeerAgent that will talk to the service: the caller's, this client's, or a new one on the control plane
        the service itself is registered with."""
        for candidate in (given, self.peer_agent):
            if candidate is not None and callable(getattr(candidate, "connect_to", None)):
                return candidate
        where = ctrl or info.get("nanoctrl_url")
        if not where:
            raise RuntimeError("no control-plane address: the service published none and none was passed (ctrl=...)")
        from ..peer_agent import PeerAgent

        return PeerAgent(nanoctrl_url=where, alias=alias, device=device, scope=info.get("scope") if scope is None else scope)

    def connect_to_server(self, *, peer_agent: Any | None = None, alias: str | None = None, ctrl: str | None = None,
                          scope: str | None = None, local_device: str | None = None, peer_device: str | None = None,
                          ib_port: int = 1, qp_num: int = 1, timeout_sec: float = 60.0, link_type: str | None = None) -> dict[str, Any]:
        """Connect a PeerAgent to the service's; returns the service's description. Idempotent per client."""
        info = self.server_peer_agent()
        self.peer_agent = self._agent_for(info, peer_agent, alias=alias, ctrl=ctrl, scope=scope, device=local_device)
        if peer_device is None and str(link_type or "").lower() == "nvlink" and str(info.get("device") or "").startswith("cuda"):
            peer_device = info["device"]  # the GPU that holds the slabs, not just any GPU the service's host lists
        link = self.peer_agent.connect_to(str(info["peer_agent_id"]), local_device=local_device, peer_device=peer_device,
                                          ib_port=ib_port, qp_num=qp_num, link_type=link_type)
        link.wait(timeout=timeout_sec)
        self._server_info = info
        return info

    # -- identity ------------------------------------------------------------------------------------
    @staticmethod
    def peer_agent_id(peer_agent: Any | None) -> str:
        alias = getattr(peer_agent, "alias", None) if peer_agent is not None else None
        if alias:
            return str(alias)
        raise ValueError("no owner for this request: pass peer_agent_id=..., or a PeerAgent that has an alias")

    def default_peer_agent_id(self) -> str:
        return self.peer_agent_id(self.peer_agent)

    # -- directory -----------------------------------------------------------------------------------
    def store(self, assignments: Iterable[Assignment], *, peer_agent: Any | None = None, peer_agent_id: str | None = None) -> dict[str, Any]:
        owner = peer_agent_id if peer_agent_id else self.peer_agent_id(self.peer_agent if peer_agent is None else peer_agent)
        request = {"peer_agent_id": owner, "assignments": list(map(assignment_to_json, assignments))}
        return self._http.call("/store", request)

    def _versioned(self, path: str, owner: str, version: int) -> dict[str, Any]:
        return self._http.call(path, {"peer_agent_id": owner, "version": int(version)})

    def query(self, peer_agent_id: str, version: int) -> dict[str, Any]:
        return self._versioned("/query", peer_agent_id, version)

    load = query  # the reference offers both names for the same lookup

    def delete(self, peer_agent_id: str, version: int) -> bool:
        return bool(self._versioned("/delete", peer_agent_id, version).get("deleted"))

    def stats(self) -> dict[str, Any]:
        return self._http.call("/stats")

    # -- data movement -----------------------------------------------------------------------
    def _server(self) -> dict:
        if self._server_info is None:
            self.connect_to_server()
        return self._server_info

    def _tuples(self, local_region: str, manifest: dict) -> list[tuple]:
        cache_mr = (self._server_info or self.server_peer_agent())["cache_mr_name"]
        return [(local_region, cache_mr, int(a["target_offset"]), int(a["source_offset"]), int(a["length"]))
                for a in manifest["assignments"]]

    def _move(self, verb: str, local_region: str, manifest: dict, timeout: float) -> dict[str, Any]:
        server = self._server()
        op = self.peer_agent.write if verb == "put" else self.peer_agent.read
        status = op(server["peer_agent_id"], self._tuples(local_region, manifest)).wait(timeout)
        if status != 0:
            raise RuntimeError(f"cache {verb} failed with status {status}")
        return manifest

    def put(self, local_region: str, extents: list[tuple[int, int]], timeout: float = 30.0) -> dict[str, Any]:
        """Store ``[(local_offset, length), ...]`` of ``local_region`` in the cache; returns the manifest."""
        self._server()
        manifest = self.store([Assignment(0, 0, int(off), 0, int(n)) for off, n in extents])
        return self._move("put", local_region, manifest, timeout)

    def get(self, local_region: str, peer_agent_id: str, version: int, timeout: float = 30.0) -> dict[str, Any]:
        """Read a stored batch back into the offsets of ``local_region`` it came from."""
        self._server()
        return self._move("get", local_region, self.query(peer_agent_id, version), timeout)
