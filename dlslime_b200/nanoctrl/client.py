"""HTTP client of the NanoCtrl control plane.

Same methods and bodies as the reference's ``NanoCtrlClient``
(``NanoCtrl/nanoctrl/client.py:39-427`` in the reference): entity registration with
heartbeats, peer-agent registration / cleanup / query, desired topology. Built on
``urllib`` with proxies disabled, so it has no third-party dependency. The ``scope`` given
at construction is injected into every request body.
"""

from __future__ import annotations

import json
import threading
import urllib.error
import urllib.request
from typing import Any, Callable

from ..logging import get_logger

log = get_logger("nanoctrl.client")
_OPENER = urllib.request.build_opener(urllib.request.ProxyHandler({}))


class NanoCtrlError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"NanoCtrl returned {status}: {message}")
        self.status, self.message = status, message


class NanoCtrlClient:
    def __init__(self, address: str = "http://127.0.0.1:3000", scope: str | None = None, timeout: float = 10.0):
        self.address = address.rstrip("/")
        if "://" not in self.address:
            self.address = "http://" + self.address
        self.scope = scope or None
        self.timeout = timeout
        self._hb_thread: threading.Thread | None = None
        self._hb_stop = threading.Event()

    # -- plumbing ----------------------------------------------------------------------
    def _post(self, path: str, body: dict | None = None) -> Any:
        payload = dict(body or {})
        if self.scope and "scope" not in payload:
            payload["scope"] = self.scope
        req = urllib.request.Request(self.address + path, data=json.dumps(payload).encode(),
                                     headers={"Content-Type": "application/json"}, method="POST")
        try:
            with _OPENER.open(req, timeout=self.timeout) as rsp:
                return json.loads(rsp.read() or b"null")
        except urllib.error.HTTPError as e:
            text = e.read().decode(errors="replace")
            try:
                msg = json.loads(text).get("message", text)
            except Exception:
                msg = text
            raise NanoCtrlError(e.code, msg) from None

    def check_connection(self) -> bool:
        try:
            with _OPENER.open(self.address + "/", timeout=self.timeout) as rsp:
                return rsp.status == 200
        except Exception:
            return False

    # -- entities ------------------------------------------------------------------------
    def register(self, entity_id: str, kind: str, endpoint: dict | None = None, metadata: dict | None = None,
                 resource: dict | None = None, entity_type: str = "service") -> dict:
        return self._post("/register", {"entity_type": entity_type, "entity_id": entity_id, "kind": kind,
                                        "endpoint": endpoint, "metadata": metadata or {}, "resource": resource})

    def unregister(self, entity_id: str, entity_type: str = "service") -> dict:
        return self._post("/unregister", {"entity_type": entity_type, "entity_id": entity_id})

    def heartbeat(self, entity_id: str, entity_type: str = "service") -> str:
        """Returns ``"ok"`` or ``"not_found"``."""
        return self._post("/heartbeat", {"entity_type": entity_type, "entity_id": entity_id}).get("status", "error")

    def get_entity_info(self, entity_id: str, entity_type: str = "service") -> dict | None:
        rsp = self._post("/get_entity_info", {"entity_type": entity_type, "entity_id": entity_id})
        return rsp.get("entity_info") if rsp.get("status") == "ok" else None

    def list_entities(self, entity_type: str | None = None, kind: str | None = None) -> list[dict]:
        body: dict = {}
        if entity_type:
            body["entity_type"] = entity_type
        if kind:
            body["kind"] = kind
        return self._post("/list_entities", body).get("entities", [])

    def get_redis_url(self) -> str:
        return self._post("/get_redis_address").get("redis_address", "")

    def start_heartbeat(self, entity_id: str, entity_type: str = "service", interval: float = 15.0,
                        on_not_found: Callable[[], None] | None = None) -> None:
        """Background heartbeat; ``on_not_found`` runs when the registration expired (re-register there)."""
        self.stop_heartbeat()
        self._hb_stop.clear()

        def loop():
            while not self._hb_stop.wait(interval):
                try:
                    if self.heartbeat(entity_id, entity_type) == "not_found" and on_not_found is not None:
                        on_not_found()
                except Exception as e:  # the control plane may be restarting
                    log.warning("heartbeat for %s failed: %s", entity_id, e)

        self._hb_thread = threading.Thread(target=loop, name=f"nanoctrl-hb-{entity_id}", daemon=True)
        self._hb_thread.start()

    def stop_heartbeat(self) -> None:
        self._hb_stop.set()
        if self._hb_thread is not None and self._hb_thread is not threading.current_thread():
            self._hb_thread.join(timeout=2.0)
        self._hb_thread = None

    def stop(self) -> None:
        self.stop_heartbeat()

    # -- peer agents -----------------------------------------------------------------------
    def register_peer(self, address: str, alias: str | None = None, device: str | None = None, ib_port: int | None = None,
                      link_type: str | None = None, resource: dict | None = None, name_prefix: str = "agent") -> dict:
        body: dict = {"address": address, "name_prefix": name_prefix}
        for k, v in (("alias", alias), ("device", device), ("ib_port", ib_port), ("link_type", link_type), ("resource", resource)):
            if v is not None:
                body[k] = v
        return self._post("/start_peer_agent", body)

    def cleanup_peer(self, agent_name: str) -> dict:
        return self._post("/cleanup", {"agent_name": agent_name})

    def heartbeat_peer(self, agent_name: str) -> str:
        return self.heartbeat(agent_name, entity_type="agent")

    def set_desired_topology(self, alias: str, target_peers: list[str], min_bw: str | None = None, symmetric: bool = False) -> dict:
        body: dict = {"target_peers": list(target_peers), "symmetric": bool(symmetric)}
        if min_bw is not None:
            body["min_bw"] = min_bw
        return self._post(f"/v1/desired_topology/{alias}", body)

    def query_peers(self) -> list[dict]:
        return self._post("/query", {})

    def register_mr(self, agent_name: str, mr_name: str, addr: int, length: int, rkey: int, lkey: int = 0) -> dict:
        return self._post("/register_mr", {"agent_name": agent_name, "mr_name": mr_name, "addr": addr, "length": length,
                                           "rkey": rkey, "lkey": lkey})

    def get_mr_info(self, src: str, dst: str, mr_name: str) -> dict | None:
        return self._post("/get_mr_info", {"src": src, "dst": dst, "mr_name": mr_name}).get("mr_info")
