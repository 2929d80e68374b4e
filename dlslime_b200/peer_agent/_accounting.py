"""ObsReporter: periodic publication of transfer counters for ``nanoctrl obs``.

Every ``DLSLIME_OBS_TIME_STEP_MS`` (default 1000) the reporter takes the C++ counter
snapshot, derives exponentially weighted bandwidth (alpha 0.3, bits/s) for the peer and for
each link, lists the agent's connections and stores the JSON at ``{scope:}obs:peer:{alias}``
with a TTL of ``max(3 * step, 180 s)``. On a clean stop it writes ``status: "stopped"`` with a
short TTL so that a stopped agent can be told from a crashed one. Schema version 1, as the
reference's reporter (``dlslime/peer_agent/_accounting.py:162-259`` in the reference) with an
extra ``kind`` per link.
"""

from __future__ import annotations

import json
import os
import socket
import threading
import time

from .. import _slime_c
from ..logging import get_logger

log = get_logger("peer_agent.obs")
SCHEMA_VERSION = 1
ALPHA = 0.3


class ObsReporter:
    def __init__(self, agent, step_ms: int | None = None, publish: bool | None = None):
        self.agent = agent
        self.step_ms = int(step_ms if step_ms is not None else os.environ.get("DLSLIME_OBS_TIME_STEP_MS", "1000"))
        self.publish = publish if publish is not None else os.environ.get("DLSLIME_OBS_REDIS", "1") != "0"
        self.session_id = f"{agent.alias}:{os.getpid()}:{int(time.time() * 1000)}"
        self._stop = threading.Event()
        self._thread: threading.Thread | None = None
        self._prev_bytes: dict[str, int] = {}
        self._prev_t: float | None = None
        self._ewma: dict[str, float] = {}
        self.last_snapshot: dict | None = None

    # -- snapshot ------------------------------------------------------------------------
    def _bandwidth(self, name: str, completed_bytes: int, now: float) -> float:
        prev = self._prev_bytes.get(name)
        self._prev_bytes[name] = completed_bytes
        if prev is None or self._prev_t is None or now <= self._prev_t:
            return self._ewma.get(name, 0.0)
        inst = max(0, completed_bytes - prev) * 8.0 / (now - self._prev_t)
        cur = self._ewma.get(name)
        self._ewma[name] = inst if cur is None else ALPHA * inst + (1 - ALPHA) * cur
        return self._ewma[name]

    def build_snapshot(self, status: str | None = None) -> dict:
        raw = _slime_c.obs_snapshot()
        now = time.monotonic()
        summary = raw.get("summary", {})
        links = raw.get("nics", [])
        for link in links:
            link["ewma_bandwidth_bps"] = self._bandwidth("link:" + link["nic"], link.get("completed_bytes_total", 0), now)
        peer_bw = self._bandwidth("peer", summary.get("completed_bytes_total", 0), now)
        self._prev_t = now
        snap = {
            "schema_version": SCHEMA_VERSION, "session_id": self.session_id, "peer_id": self.agent.alias,
            "host": socket.gethostname(), "pid": os.getpid(), "reported_at_ms": int(time.time() * 1000),
            "enabled": bool(raw.get("enabled")), "summary": summary, "nics": links, "ewma_bandwidth_bps": peer_bw,
            "connections": self.agent._connection_records(),
        }
        if status:
            snap["status"] = status
        self.last_snapshot = snap
        return snap

    def report_once(self, status: str | None = None) -> dict:
        snap = self.build_snapshot(status)
        if self.publish:
            key = self.agent._key(f"obs:peer:{self.agent.alias}")
            ttl = max(3 * self.step_ms, 10_000 if status == "stopped" else 180_000)
            try:
                self.agent._store.set(key, json.dumps(snap), px=ttl)
            except Exception as e:
                log.warning("obs publish failed: %s", e)
        return snap

    # -- lifecycle -------------------------------------------------------------------------
    def start(self) -> None:
        def loop():
            while not self._stop.wait(self.step_ms / 1000.0):
                self.report_once()

        self._thread = threading.Thread(target=loop, name=f"obs-{self.agent.alias}", daemon=True)
        self._thread.start()

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2.0)
        self.report_once(status="stopped")
