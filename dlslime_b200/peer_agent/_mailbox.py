"""Stream mailbox: the handshake channel of a PeerAgent.

Every agent reads the stream ``{scope:}stream:{alias}`` from id ``0-0`` (so messages that
arrived before it started are not lost). Two message types travel on it, as in the reference
(``dlslime/peer_agent/_mailbox.py:149-386`` in the reference):

* ``connect_peer`` -- written by NanoCtrl when the desired topology names a peer;
* ``qp_ready``     -- written by a peer: its ``endpoint_info`` JSON plus the link metadata.

Peers that only speak the older handshake publish their endpoint description under
``exchange:{peer}:{me}`` instead of sending ``qp_ready``; links that stay unanswered are completed from
that key (``PeerAgent._poll_exchange_keys``), and this side always writes its own ``exchange:`` keys too.

The rendezvous is symmetric and idempotent: whichever side learns of the link first creates
its endpoint and announces it once; the other side answers with its own announcement and both
call ``endpoint.connect`` with what they received.
"""

from __future__ import annotations

import json
import threading
import time

from ..logging import get_logger
from ._obs import tlog

log = get_logger("peer_agent.mailbox")


class StreamMailbox:
    def __init__(self, agent, block_ms: int = 50, start_id: str = "0-0"):
        self.agent = agent
        self.block_ms = block_ms
        self._stop = threading.Event()
        self._thread: threading.Thread | None = None
        self._last_id = start_id  # entries up to this id belong to an earlier incarnation of the alias
        # fault-injection hook for tests: called with the message dict, returns False to drop it
        self.message_filter = None

    def start(self) -> None:
        self._thread = threading.Thread(target=self._loop, name=f"mailbox-{self.agent.alias}", daemon=True)
        self._thread.start()

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None and self._thread is not threading.current_thread():
            self._thread.join(timeout=2.0)

    def _loop(self) -> None:
        store = self.agent._store.clone()
        key = self.agent._key(f"stream:{self.agent.alias}")
        while not self._stop.is_set():
            try:
                res = store.xread({key: self._last_id}, count=64, block=self.block_ms)
            except Exception as e:
                if self._stop.is_set():
                    break
                log.warning("%s: mailbox read failed: %s", self.agent.alias, e)
                time.sleep(0.2)
                continue
            for _, entries in res:
                for eid, fields in entries:
                    self._last_id = eid
                    if self.message_filter is not None and not self.message_filter(fields):
                        continue
                    try:
                        self._dispatch(fields)
                    except Exception:
                        log.exception("%s: mailbox message %s failed", self.agent.alias, fields.get("type"))
            # links that were announced but never answered on the stream: the peer may speak only the older
            # exchange-key handshake (dlslime/peer_agent/_mailbox.py:342-363 in the reference)
            try:
                self.agent._poll_exchange_keys(store)
            except Exception:
                log.exception("%s: exchange-key poll failed", self.agent.alias)
        store.close()

    def _dispatch(self, msg: dict) -> None:
        kind = msg.get("type")
        peer = msg.get("peer", "")
        if kind == "connect_peer":
            tlog(f"{self.agent.alias}: connect_peer({peer})")
            for conn in self.agent._connections_to(peer):
                self.agent._announce(conn)
        elif kind == "qp_ready":
            tlog(f"{self.agent.alias}: qp_ready from {peer}")
            meta = json.loads(msg.get("conn_meta") or "{}")
            info = json.loads(msg.get("qp_info") or "{}")
            self.agent._on_peer_ready(peer, meta, info)
        else:
            log.debug("%s: ignoring mailbox message of type %r", self.agent.alias, kind)
