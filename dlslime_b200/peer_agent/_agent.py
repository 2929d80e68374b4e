"""PeerAgent: control-plane client and named I/O facade of one process.

An agent registers with NanoCtrl, publishes its topology and memory regions in the
control-plane store, connects to peers through a symmetric stream handshake and then offers
``read / write / write_with_imm / send / recv / imm_recv`` addressed by peer alias and region
name. The public surface, key schema and handshake messages follow the reference
(``dlslime/peer_agent/_agent.py`` in the reference: lifecycle ``:181-310``, registration
``:403-464``, handshake ``:975-1088``, regions ``:1093-1380``, named I/O ``:1487-1626``,
shutdown ``:1631-1733``). What differs: endpoints are transport-agnostic (TCP everywhere,
NVLink between GPUs of a node, RDMA where verbs exist), the store is the embedded one reached
over RESP, and every wait has a timeout.
"""

from __future__ import annotations

import hashlib
import json
import os
import socket
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from typing import Any, Dict, List, Optional

from .. import _slime_c
from ..logging import get_logger
from ..nanoctrl.client import NanoCtrlClient, NanoCtrlError
from ..nanoctrl.resp import RespClient
from ._accounting import ObsReporter
from ._mailbox import StreamMailbox
from ._obs import tlog
from ._types import (DirectedConnection, LogicalMemoryRegion, MaterializedMemoryRegion, PeerConnection, ResourceKey)

log = get_logger("peer_agent")

LINK_ALIASES = {"tcp": "TCP", "nvlink": "NVLink", "roce": "RoCE", "ethernet": "RoCE", "ib": "IB", "infiniband": "IB"}


def _norm_link(link: Optional[str]) -> Optional[str]:
    if not link:
        return None
    return LINK_ALIASES.get(link.lower(), link)


class _NVLinkAdapter:
    """Gives the kernel-driven NVLink endpoint the method names the agent uses for every transport.

    Every call runs with the agent's GPU as the current CUDA device: the agent creates and connects endpoints from its
    own threads (executor, mailbox), where the current device is whatever the process default is, and an endpoint whose
    mailbox, IPC export or copy kernels end up on another GPU than its regions does not work.
    """

    def __init__(self, device_index: int | None = None):
        import torch

        from ..ops.nvlink import NVLinkEndpoint

        self._torch = torch
        self.device_index = torch.cuda.current_device() if device_index is None else int(device_index)
        with torch.cuda.device(self.device_index):
            self.ep = NVLinkEndpoint()

    def _on_device(self):
        return self._torch.cuda.device(self.device_index)

    def kind(self):
        return "nvlink"

    def register_memory_region(self, name, ptr, offset, length):
        with self._on_device():
            return self.ep.register_memory_region(ptr, offset, length, name)

    def register_remote_memory_region(self, name, info):
        with self._on_device():
            return self.ep.register_remote_memory_region(info, name)

    def get_mr_handle(self, name):
        return self.ep.get_mr_handle(name)

    def get_remote_mr_handle(self, name):
        return self.ep.get_remote_mr_handle(name)

    def mr_info(self):
        with self._on_device():
            return self.ep.mr_info()

    def endpoint_info(self):
        with self._on_device():
            info = self.ep.endpoint_info()
        info["kind"] = "nvlink"
        return info

    def connect(self, info):
        with self._on_device():
            return self.ep.connect(info)

    def read(self, assign, stream=None):
        with self._on_device():
            return self.ep.read(assign, stream)

    def write(self, assign, stream=None):
        with self._on_device():
            return self.ep.write(assign, stream)

    def write_with_imm(self, assign, imm_data=0, stream=None):
        with self._on_device():
            return self.ep.write_with_imm(assign, imm_data, stream)

    def imm_recv(self, stream=None):
        with self._on_device():
            return self.ep.imm_recv()

    def send(self, chunk, stream=None):
        raise NotImplementedError("two-sided send over NVLink: use write_with_imm / imm_recv")

    recv = send

    def shutdown(self):
        with self._on_device():
            self.ep.close()

    def cancel_all(self):
        pass


class PeerAgent:
    """Manages connections to peers by declaring the desired topology to NanoCtrl."""

    HEARTBEAT_INTERVAL = 15.0

    def __init__(self, nanoctrl_url: str = "http://127.0.0.1:3000", alias: Optional[str] = None,
                 device: Optional[str] = None, scope: Optional[str] = None, link_type: Optional[str] = None,
                 bind_host: str = "127.0.0.1", enable_obs: Optional[bool] = None):
        self.nanoctrl_url = nanoctrl_url
        self.alias: str = alias or ""
        self._preferred_device = device
        self._preferred_link = _norm_link(link_type) or ("NVLink" if (device or "").startswith("cuda") else None)
        self._scope = scope or os.environ.get("NANOCTRL_SCOPE", "") or ""
        self._bind_host = bind_host
        self._client = NanoCtrlClient(nanoctrl_url, scope=self._scope or None)
        self._local_resource = self._discover_local_resource(device)
        self._connections: Dict[str, DirectedConnection] = {}
        self._connections_lock = threading.RLock()
        self._connected_cond = threading.Condition(self._connections_lock)
        self._notified: set[str] = set()
        self._announced_at: dict[str, float] = {}  # conn_id -> time of our announcement (exchange-key fallback)
        self._desired_peers: set[str] = set()  # every peer connect_to was called for (the posted topology)
        self._logical_regions: Dict[str, LogicalMemoryRegion] = {}
        self._materialized: Dict[tuple, MaterializedMemoryRegion] = {}
        self._pools: Dict[ResourceKey, Any] = {}
        self._regions_lock = threading.RLock()
        self._resource_cache: Dict[str, dict] = {}
        self._executor = ThreadPoolExecutor(max_workers=16, thread_name_prefix="peer-agent-ep")
        self._stop = threading.Event()
        self._shutdown_done = False
        self._rpc_buffer_size = 32 << 20
        self._rpc_max_inflight = int(os.environ.get("SLIME_RPC_MAX_INFLIGHT", "16"))
        self._rpc_channels: Dict[str, Any] = {}

        self._register()
        self._store = RespClient.from_address(self._redis_address)
        # Whatever sits in this alias's stream now was addressed to an earlier incarnation (one that crashed: a clean exit
        # deletes the stream). Its endpoint descriptions are dead, so the mailbox starts behind the last of them; what peers
        # send from now on has a larger id. Taken before the resource record is published, which is what peers need to
        # address us at all.
        start_id = "0-0"
        try:
            old = self._store.execute("XRANGE", self._key(f"stream:{self.alias}"), "-", "+")
            if old:
                start_id = old[-1][0] if isinstance(old[-1][0], str) else old[-1][0].decode()
        except Exception:
            pass
        self._publish_resource_record()
        self._purge_stale_keys()
        self._mailbox = StreamMailbox(self, start_id=start_id)
        self._mailbox.start()
        self._inbox_thread = threading.Thread(target=self._inbox_loop, name=f"inbox-{self.alias}", daemon=True)
        self._inbox_thread.start()
        self._hb_thread = threading.Thread(target=self._heartbeat_loop, name=f"hb-{self.alias}", daemon=True)
        self._hb_thread.start()
        want_obs = _slime_c.obs_enabled() if enable_obs is None else enable_obs
        self._obs = ObsReporter(self) if want_obs else None
        if self._obs:
            self._obs.start()

    # ------------------------------------------------------------------ keys / topology
    EXCHANGE_TTL = 600  # seconds an exchange key lives
    EXCHANGE_GRACE = 0.3  # seconds a link waits for qp_ready before the exchange key of its peer is looked up

    def _key(self, suffix: str) -> str:
        return f"{self._scope}:{suffix}" if self._scope else suffix

    def _agent_key(self, alias: str) -> str:
        return self._key(f"agent:{alias}")

    def _local_address(self) -> str:
        try:
            return self._local_resource["host"]["address"]
        except Exception:
            return socket.gethostbyname(socket.gethostname())

    def _discover_local_resource(self, preferred_device: Optional[str]) -> dict:
        nic_pref = preferred_device if preferred_device and not preferred_device.startswith(("cuda", "tcp")) else None
        res = _slime_c.discover_topology(preferred_device=nic_pref, ib_port=1, preferred_link_type=None,
                                         allow_software_links=True)
        nics = res["nics"]
        if not any(p["link_type"] == "TCP" for n in nics for p in n["ports"]):
            nics.append({"name": "tcp0", "health": "AVAILABLE", "numa_node": -1, "pci_bus_id": "",
                         "ports": [{"port": 1, "state": "ACTIVE", "link_type": "TCP"}]})
        try:
            import torch

            n_gpu = torch.cuda.device_count() if torch.cuda.is_available() else 0
        except Exception:
            n_gpu = 0
        for i in range(n_gpu):
            nics.append({"name": f"cuda:{i}", "health": "AVAILABLE", "numa_node": -1, "pci_bus_id": "",
                         "ports": [{"port": 1, "state": "ACTIVE", "link_type": "NVLink"}]})
        # devices of a verbs provider that sysfs does not list (the software loopback fabric)
        known = {n["name"] for n in nics}
        if _slime_c.rdma_provider()[0] == "loopback":
            for dev in _slime_c.rdma_devices():
                if dev not in known:
                    link = _slime_c.RDMAContext.acquire(dev, 1, "").link_type()
                    nics.append({"name": dev, "health": "AVAILABLE", "numa_node": -1, "pci_bus_id": "",
                                 "ports": [{"port": 1, "state": "ACTIVE", "link_type": link}]})
        return res

    @staticmethod
    def _resource_keys(resource: dict) -> List[ResourceKey]:
        keys = []
        for nic in resource.get("nics", []):
            if nic.get("health", "AVAILABLE") != "AVAILABLE":
                continue
            for p in nic.get("ports", []):
                if p.get("state", "ACTIVE") == "ACTIVE":
                    keys.append(ResourceKey(nic["name"], int(p.get("port", 1)), p.get("link_type", "UNKNOWN")))
        return keys

    def _first_usable_resource_key(self, resource: dict, device: Optional[str] = None, ib_port: Optional[int] = None,
                                   link_type: Optional[str] = None) -> ResourceKey:
        link_type = _norm_link(link_type)
        usable = {"TCP"}
        if _slime_c._BUILD_RDMA:
            usable |= {"RoCE", "IB"}
        usable.add("NVLink")
        for k in self._resource_keys(resource):
            if device and k.device != device:
                continue
            if ib_port and k.ib_port != ib_port:
                continue
            if link_type and k.link_type != link_type:
                continue
            if k.link_type not in usable:
                continue
            if not device and not link_type and k.link_type == "NVLink":
                continue  # NVLink only when asked for: its regions must be device memory
            return k
        raise RuntimeError(f"no usable resource (device={device}, port={ib_port}, link_type={link_type})")

    def _default_local_resource_key(self) -> ResourceKey:
        return self._first_usable_resource_key(self._local_resource, device=self._preferred_device if self._preferred_link else None,
                                               link_type=self._preferred_link)

    # ------------------------------------------------------------------ registration / liveness
    def _register(self) -> None:
        key = self._default_local_resource_key()
        delay = 0.1
        last: Exception | None = None
        for attempt in range(5):
            try:
                rsp = self._client.register_peer(self._local_address(), alias=self.alias or None, device=key.device,
                                                 ib_port=key.ib_port, link_type=key.link_type, resource=self._local_resource)
                self.alias = rsp["name"]
                self._redis_address = rsp["redis_address"]
                return
            except NanoCtrlError as e:
                if e.status == 409:
                    raise RuntimeError(f"peer agent alias {self.alias!r} is already registered in scope {self._scope!r}") from e
                last = e
            except Exception as e:  # control plane not reachable yet
                last = e
            time.sleep(delay)
            delay *= 2
        raise RuntimeError(f"could not register with NanoCtrl at {self.nanoctrl_url}: {last}")

    def _publish_resource_record(self) -> None:
        res = json.dumps(self._local_resource)
        self._store.hset(self._agent_key(self.alias), mapping={
            "addr": self._local_address(), "resource": res, "topology": res,
            "memory_keys": json.dumps(sorted(self._logical_regions)), "updated_at": str(int(time.time()))})
        self._store.expire(self._agent_key(self.alias), 60)

    def _purge_stale_keys(self) -> None:
        """Keys of a previous, crashed run under the same alias would poison the handshake."""
        stale = []
        for pattern in (f"exchange:{self.alias}:*", f"exchange:*:{self.alias}", f"exchange:*:{self.alias}:*", f"mr:{self.alias}:*"):
            stale += list(self._store.scan_iter(self._key(pattern)))
        if stale:
            self._store.delete(*stale)

    def _heartbeat_loop(self) -> None:
        while not self._stop.wait(self.HEARTBEAT_INTERVAL):
            self._heartbeat_once()

    def _heartbeat_once(self) -> None:
        try:
            if self._client.heartbeat_peer(self.alias) == "not_found":
                log.warning("%s: registration expired, registering again", self.alias)
                self._register()
                self._publish_resource_record()
                self._publish_memory_keys()
        except Exception as e:
            log.warning("%s: heartbeat failed: %s", self.alias, e)

    def _inbox_loop(self) -> None:
        store = self._store.clone()
        key = self._key(f"inbox:{self.alias}")
        while not self._stop.is_set():
            try:
                item = store.blpop([key], timeout=0.2)
            except Exception:
                if self._stop.is_set():
                    break
                time.sleep(0.2)
                continue
            if not item:
                continue
            try:
                ev = json.loads(item[1])
            except Exception:
                continue
            if ev.get("type") == "cleanup":
                self._drop_peer(ev.get("peer", ""))
        store.close()

    def _drop_peer(self, peer: str) -> None:
        with self._connections_lock:
            victims = [c for c in self._connections.values() if c.peer_alias == peer]
            for c in victims:
                self._connections.pop(c.conn_id, None)
                self._notified.discard(c.conn_id)
                c.state = "closed"
            self._connected_cond.notify_all()
        for c in victims:
            if c.endpoint is not None:
                try:
                    c.endpoint.shutdown()  # fails every future in flight with 403 so that no waiter hangs
                except Exception:
                    pass
        self._rpc_channels.pop(peer, None)
        self._resource_cache.pop(peer, None)
        with self._connections_lock:
            self._desired_peers.discard(peer)  # connect_to() asks for it again if the peer returns

    # ------------------------------------------------------------------ discovery
    def list_agents(self) -> List[str]:
        prefix = self._key("agent:")
        return sorted(k[len(prefix):] for k in self._store.scan_iter(prefix + "*"))

    def get_resource(self, peer_alias: Optional[str] = None, refresh: bool = False) -> dict:
        if peer_alias in (None, self.alias):
            return self._local_resource
        if not refresh and peer_alias in self._resource_cache:
            return self._resource_cache[peer_alias]
        raw = self._store.hget(self._agent_key(peer_alias), "resource")
        if not raw:
            raise KeyError(f"peer agent {peer_alias!r} is not registered")
        res = json.loads(raw)
        self._resource_cache[peer_alias] = res
        return res

    def list_mem_keys(self, peer_alias: Optional[str] = None) -> List[str]:
        if peer_alias in (None, self.alias):
            return sorted(self._logical_regions)
        raw = self._store.hget(self._agent_key(peer_alias), "memory_keys")
        return json.loads(raw) if raw else []

    # ------------------------------------------------------------------ connections
    def _connections_to(self, peer: str) -> List[DirectedConnection]:
        with self._connections_lock:
            return [c for c in self._connections.values() if c.peer_alias == peer]

    def _connection_records(self) -> List[dict]:
        with self._connections_lock:
            return [{"conn_id": c.conn_id, "peer": c.peer_alias, "local_nic": c.local_key.device,
                     "remote_nic": c.peer_key.device, "state": c.state, "connected": c.state == "connected"}
                    for c in self._connections.values()]

    def get_connections(self) -> Dict[str, Dict[str, PeerConnection]]:
        out: Dict[str, Dict[str, PeerConnection]] = {}
        with self._connections_lock:
            for cid, c in self._connections.items():
                out.setdefault(c.peer_alias, {})[cid] = PeerConnection(self, cid)
        return out

    def query_connection(self, peer_alias: str, local_device: Optional[str] = None, peer_device: Optional[str] = None) -> Optional[PeerConnection]:
        try:
            return PeerConnection(self, self._get_connection(peer_alias, local_device, peer_device).conn_id)
        except KeyError:
            return None

    def _create_endpoint(self, conn: DirectedConnection):
        """Builds the transport endpoint of one link and registers every known region on it."""
        link = conn.local_key.link_type
        if link == "TCP":
            ep = _slime_c.TcpEndpoint(self._bind_host, 0, conn.qp_num)
            ep.set_pool(self._pool_for(conn.local_key))
        elif link == "NVLink":
            dev = conn.local_key.device or self._preferred_device or ""
            ep = _NVLinkAdapter(int(dev.split(":")[1]) if dev.startswith("cuda:") else None)
            with self._regions_lock:
                for r in self._logical_regions.values():
                    ep.register_memory_region(r.name, r.ptr, r.offset, r.length)
        elif link in ("RoCE", "IB") and _slime_c._BUILD_RDMA:
            ep = _slime_c.RDMAEndpoint(conn.local_key.device, conn.local_key.ib_port, link, conn.qp_num)
            with self._regions_lock:
                for r in self._logical_regions.values():
                    ep.register_memory_region(r.name, r.ptr, r.offset, r.length)
        else:
            raise RuntimeError(f"no transport for link type {link!r} in this build")
        if link != "TCP":
            # the keys peers need exist only now: publish them for this resource
            with self._regions_lock:
                names = list(self._logical_regions)
            for name in names:
                self._materialize_region(name, conn.local_key, endpoint=ep)
        return ep

    def _ensure_endpoint(self, conn: DirectedConnection):
        with conn.lock:
            if conn.endpoint is None:
                t0 = time.perf_counter()
                conn.endpoint = self._create_endpoint(conn)
                tlog(f"{self.alias}: endpoint for {conn.conn_id} created in {(time.perf_counter() - t0) * 1e3:.2f} ms")
            return conn.endpoint

    def _announce(self, conn: DirectedConnection) -> None:
        """Publish this side's endpoint info to the peer, once per connection."""
        with self._connections_lock:
            if conn.conn_id in self._notified:
                return
            self._notified.add(conn.conn_id)
        ep = self._ensure_endpoint(conn)
        info_json = json.dumps(ep.endpoint_info())
        self._store.xadd(self._key(f"stream:{conn.peer_alias}"),
                         {"type": "qp_ready", "peer": self.alias, "qp_info": info_json,
                          "conn_meta": json.dumps(conn.meta()), "timestamp": str(int(time.time()))}, maxlen=1000)
        # Interoperation with peers that only speak the older exchange-key handshake
        # (dlslime/peer_agent/_mailbox.py:342-363 in the reference): the same description under
        # exchange:{me}:{peer}:{conn_id}, which such a peer GETs, and without the connection id, which is the form it
        # reads. Its own description is looked for by _poll_exchange_keys.
        try:
            self._store.set(self._key(f"exchange:{self.alias}:{conn.peer_alias}:{conn.conn_id}"), info_json, ex=self.EXCHANGE_TTL)
            self._store.set(self._key(f"exchange:{self.alias}:{conn.peer_alias}"), info_json, ex=self.EXCHANGE_TTL)
        except Exception as e:
            log.debug("%s: exchange keys for %s not written: %s", self.alias, conn.peer_alias, e)
        with self._connections_lock:
            self._announced_at[conn.conn_id] = time.monotonic()

    def _poll_exchange_keys(self, store=None) -> int:
        """Connect links whose peer never sent ``qp_ready`` but published ``exchange:{peer}:{me}``.

        Called from the mailbox thread between reads. A link qualifies once it has been announced for
        ``EXCHANGE_GRACE`` seconds without an answer on the stream. Returns the number of links connected.
        """
        store = store or self._store
        now = time.monotonic()
        with self._connections_lock:
            waiting = [c for c in self._connections.values() if c.state in ("pending", "connecting")
                       and now - self._announced_at.get(c.conn_id, now) >= self.EXCHANGE_GRACE]
        done = 0
        for conn in waiting:
            try:
                raw = store.get(self._key(f"exchange:{conn.peer_alias}:{self.alias}"))
            except Exception:
                return done
            if not raw:
                continue
            try:
                info = json.loads(raw)
            except (TypeError, ValueError):
                log.warning("%s: exchange key of %s does not hold JSON", self.alias, conn.peer_alias)
                continue
            with self._connections_lock:
                if conn.state == "connected":
                    continue
                conn.state = "connecting"
            try:
                self._ensure_endpoint(conn).connect(info)
            except Exception as e:
                log.warning("%s: connect to %s from its exchange key failed: %s", self.alias, conn.peer_alias, e)
                continue
            conn.peer_digest = hashlib.sha1(json.dumps(info, sort_keys=True).encode()).hexdigest()
            with self._connections_lock:
                conn.state = "connected"
                self._connected_cond.notify_all()
            tlog(f"{self.alias}: {conn.conn_id} connected through exchange keys")
            done += 1
        return done

    def _on_peer_ready(self, peer: str, meta: dict, info: dict) -> None:
        """The peer announced its endpoint: mirror the link locally, answer, connect."""
        link = _norm_link(meta.get("link_type")) or "TCP"
        local_key = ResourceKey(meta.get("dst_device", ""), int(meta.get("ib_port", 1)), link)
        peer_key = ResourceKey(meta.get("src_device", ""), int(meta.get("ib_port", 1)), link)
        probe = DirectedConnection(self.alias, peer, local_key, peer_key, int(meta.get("qp_num", 1)), meta.get("profile", "default"))
        digest = hashlib.sha1(json.dumps(info, sort_keys=True).encode()).hexdigest()
        stale = None
        with self._connections_lock:
            conn = self._connections.get(probe.conn_id)
            if conn is not None and conn.state == "connected":
                if conn.peer_digest == digest:
                    return  # the announcement this link was built from, seen again
                # The peer announces other endpoints than the ones this link is connected to: it went away and came back
                # under the same alias (its cleanup notice may never have reached us, e.g. after a crash). The old link is
                # dead; drop it and shake hands again with a fresh endpoint.
                stale = conn
                self._connections.pop(conn.conn_id, None)
                self._notified.discard(conn.conn_id)
                stale.state = "closed"
                conn = None
            if conn is None:
                conn = self._connections[probe.conn_id] = probe
            conn.state = "connecting"
        if stale is not None:
            log.info("%s: %s restarted; replacing link %s", self.alias, peer, stale.conn_id)
            if stale.endpoint is not None:
                try:
                    stale.endpoint.shutdown()  # fails what was still in flight on the dead link with 403
                except Exception:
                    pass
            self._rpc_channels.pop(peer, None)
            self._resource_cache.pop(peer, None)
        try:
            ep = self._ensure_endpoint(conn)
            self._announce(conn)
            ep.connect(info)
            conn.peer_digest = digest
        except Exception:
            with self._connections_lock:
                conn.state = "failed"
                self._connected_cond.notify_all()
            raise
        with self._connections_lock:
            conn.state = "connected"
            self._connected_cond.notify_all()
        tlog(f"{self.alias}: {conn.conn_id} connected")

    def connect_to(self, peer_alias: str, local_device: Optional[str] = None, peer_device: Optional[str] = None,
                   ib_port: Optional[int] = 1, qp_num: Optional[int] = 1, min_bw: Optional[str] = None,
                   link_type: Optional[str] = None) -> PeerConnection:
        """Start connecting to a peer and return a handle; call ``.wait()`` before I/O."""
        if not isinstance(peer_alias, str) or not peer_alias:
            raise TypeError("connect_to() requires a non-empty peer alias string")
        if peer_alias == self.alias:
            raise ValueError(f"connect_to() cannot target this agent's own alias {peer_alias!r}. "
                             "Start peer agents with distinct aliases.")
        tlog(f"{self.alias}: connect_to({peer_alias}) ENTER")
        link = _norm_link(link_type) or self._preferred_link
        local_key = self._first_usable_resource_key(self._local_resource, device=local_device or (self._preferred_device if link == "NVLink" else None),
                                                    ib_port=ib_port, link_type=link)
        peer_res = self.get_resource(peer_alias, refresh=True)
        peer_key = self._first_usable_resource_key(peer_res, device=peer_device, ib_port=ib_port, link_type=local_key.link_type)
        conn = DirectedConnection(self.alias, peer_alias, local_key, peer_key, int(qp_num or 1))
        with self._connections_lock:
            conn = self._connections.setdefault(conn.conn_id, conn)
        fut = self._executor.submit(self._ensure_endpoint, conn)  # endpoint construction off the caller's thread

        def _mark_failed(f):
            if f.exception() is not None:
                with self._connections_lock:
                    conn.state = "failed"
                    self._connected_cond.notify_all()

        fut.add_done_callback(_mark_failed)
        # The stored specification is this agent's whole desired topology (the control plane replaces it on every post and
        # uses it to find whom to notify when this agent leaves), so every peer asked for so far is posted again.
        with self._connections_lock:
            self._desired_peers.add(peer_alias)
            targets = sorted(self._desired_peers)
        self._client.set_desired_topology(self.alias, targets, min_bw=min_bw)
        return PeerConnection(self, conn.conn_id)

    def _wait_connected(self, conn_id: str, timeout_sec: float = 60.0) -> None:
        deadline = time.monotonic() + timeout_sec
        with self._connected_cond:
            while True:
                conn = self._connections.get(conn_id)
                if conn is None:
                    raise RuntimeError(f"connection {conn_id} was dropped")
                if conn.state == "connected":
                    return
                if conn.state == "failed":
                    raise RuntimeError(f"connection {conn_id} failed")
                left = deadline - time.monotonic()
                if left <= 0:
                    raise TimeoutError(f"connection {conn_id} not established within {timeout_sec} s")
                self._connected_cond.wait(min(left, 0.5))

    def _get_connection(self, peer_alias: str, local_device: Optional[str] = None, peer_device: Optional[str] = None) -> DirectedConnection:
        with self._connections_lock:
            cands = [c for c in self._connections.values() if c.peer_alias == peer_alias
                     and (local_device is None or c.local_key.device == local_device)
                     and (peer_device is None or c.peer_key.device == peer_device)]
        if not cands:
            raise KeyError(f"no connection to {peer_alias!r}; call connect_to({peer_alias!r}).wait() first")
        cands.sort(key=lambda c: (c.state != "connected", c.conn_id))
        return cands[0]

    def _get_endpoint(self, peer_alias: str, local_device: Optional[str] = None, peer_device: Optional[str] = None):
        conn = self._get_connection(peer_alias, local_device, peer_device)
        if conn.state != "connected" or conn.endpoint is None:
            raise RuntimeError(f"connection to {peer_alias!r} is {conn.state}; call .wait() on the handle first")
        return conn.endpoint

    # ------------------------------------------------------------------ memory regions
    def _pool_for(self, key: ResourceKey):
        with self._regions_lock:
            pool = self._pools.get(key)
            if pool is None:
                pool = self._pools[key] = _slime_c.MemoryPool()
            return pool

    def register_memory_region(self, mr_name: str, ptr: int, offset: int, length: int) -> int:
        """Register a logical region and publish it; returns the handle on the default resource."""
        with self._regions_lock:
            self._logical_regions[mr_name] = LogicalMemoryRegion(mr_name, int(ptr), int(offset), int(length))
        # links that keep per-endpoint registries learn about the region right away
        for c in list(self._connections.values()):
            if c.endpoint is not None and c.local_key.link_type != "TCP":
                c.endpoint.register_memory_region(mr_name, int(ptr), int(offset), int(length))
                self._materialize_region(mr_name, c.local_key, endpoint=c.endpoint)
        m = self._materialize_region(mr_name, self._default_local_resource_key())
        self._publish_memory_keys()
        return m.handler

    def _materialize_region(self, mr_name: str, key: ResourceKey, endpoint=None) -> MaterializedMemoryRegion:
        with self._regions_lock:
            r = self._logical_regions.get(mr_name)
            if r is None:
                raise KeyError(f"memory region {mr_name!r} is not registered")
            if key.link_type == "TCP":
                pool = self._pool_for(key)
                handle = pool.register_memory_region(r.ptr + r.offset, r.length, mr_name)
                info = dict(pool.mr_info()[mr_name])
            else:
                ep = endpoint
                if ep is None:
                    for c in self._connections.values():
                        if c.local_key == key and c.endpoint is not None:
                            ep = c.endpoint
                            break
                if ep is None:
                    # nothing to materialise on yet: the link's endpoint registers it when it is created
                    handle, info = -1, {"addr": r.ptr + r.offset, "length": r.length, "rkey": 0}
                else:
                    handle = ep.get_mr_handle(mr_name)
                    if handle < 0:
                        handle = ep.register_memory_region(mr_name, r.ptr, r.offset, r.length)
                    info = dict(ep.mr_info()[mr_name])
            info.update({"agent_name": self.alias, "mr_name": mr_name, "device": key.device, "ib_port": key.ib_port,
                         "link_type": key.link_type, "lkey": 0, "handle": handle})
            m = MaterializedMemoryRegion(mr_name, key, handle, info)
            self._materialized[(mr_name, key)] = m
        payload = json.dumps(info)
        self._store.set(self._key(f"mr:{self.alias}:{mr_name}"), payload)
        self._store.set(self._key(f"mr:{self.alias}:{mr_name}:{key.redis_suffix()}"), payload)
        return m

    def _publish_memory_keys(self) -> None:
        self._store.hset(self._agent_key(self.alias), mapping={"memory_keys": json.dumps(sorted(self._logical_regions)),
                                                               "updated_at": str(int(time.time()))})

    def unregister_memory_region(self, mr_name: str) -> bool:
        with self._regions_lock:
            if mr_name not in self._logical_regions:
                return False
            keys = [k for (n, k) in self._materialized if n == mr_name]
            # all-or-nothing: registries first, bookkeeping only once they all succeeded
            for k in keys:
                if k.link_type == "TCP" and self._pool_for(k).unregister_memory_region(mr_name) != 0:
                    return False
            for k in keys:
                self._materialized.pop((mr_name, k), None)
            del self._logical_regions[mr_name]
        doomed = [self._key(f"mr:{self.alias}:{mr_name}")] + [self._key(f"mr:{self.alias}:{mr_name}:{k.redis_suffix()}") for k in keys]
        self._store.delete(*doomed)
        self._publish_memory_keys()
        return True

    def get_mr_info(self, peer_alias: str, mr_name: str, key: Optional[ResourceKey] = None) -> Optional[dict]:
        names = [f"mr:{peer_alias}:{mr_name}:{key.redis_suffix()}"] if key else []
        names.append(f"mr:{peer_alias}:{mr_name}")
        for n in names:
            raw = self._store.get(self._key(n))
            if raw:
                return json.loads(raw)
        return None

    def get_handle(self, conn: DirectedConnection, mr_name: str, remote: bool = False, validate_cache: bool = True) -> int:
        """Handle of a region on one connection: local (materialising it there if needed) or remote."""
        if not remote:
            m = self._materialized.get((mr_name, conn.local_key))
            if m is None or m.handler < 0:
                m = self._materialize_region(mr_name, conn.local_key, endpoint=conn.endpoint)
            return m.handler
        cached = conn.remote_handles.get(mr_name)
        if cached is not None and not validate_cache:
            return cached[0]
        info = self.get_mr_info(conn.peer_alias, mr_name, conn.peer_key)
        if info is None:
            raise KeyError(f"peer {conn.peer_alias!r} has no memory region {mr_name!r} on {conn.peer_key.redis_suffix()}")
        if cached is not None and cached[1] == info:
            return cached[0]
        handle = conn.endpoint.register_remote_memory_region(mr_name, info)
        conn.remote_handles[mr_name] = (handle, info)
        return handle

    # ------------------------------------------------------------------ named I/O
    @staticmethod
    def _is_named(a: Any) -> bool:
        return isinstance(a, (tuple, list)) and len(a) in (4, 5) and isinstance(a[0], str)

    def _endpoint_assign(self, conn: DirectedConnection, a, local_handles: Optional[dict] = None,
                         remote_handles: Optional[dict] = None) -> tuple:
        """``(region, local_off, remote_off, len)`` or ``(local_region, remote_region, local_off, remote_off, len)``
        -> the endpoint tuple ``(local_handle, remote_handle, remote_off, local_off, len)``. The two dicts memoise the
        handles of one call: a region is resolved (and a remote one checked against the directory) once per call, not
        once per piece."""
        if len(a) == 4:
            local_name = remote_name = a[0]
            local_off, remote_off, length = a[1], a[2], a[3]
        else:
            local_name, remote_name, local_off, remote_off, length = a
        local_handles = {} if local_handles is None else local_handles
        remote_handles = {} if remote_handles is None else remote_handles
        lh = local_handles.get(local_name)
        if lh is None:
            lh = local_handles[local_name] = self.get_handle(conn, local_name)
        rh = remote_handles.get(remote_name)
        if rh is None:
            rh = remote_handles[remote_name] = self.get_handle(conn, remote_name, remote=True)
        return (lh, rh, int(remote_off), int(local_off), int(length))

    def _maybe_endpoint_assign(self, conn: DirectedConnection, assign):
        if self._is_named(assign):
            return [self._endpoint_assign(conn, assign)]
        if isinstance(assign, (list, tuple)) and assign and self._is_named(assign[0]):
            local_handles, remote_handles = {}, {}
            return [self._endpoint_assign(conn, a, local_handles, remote_handles) for a in assign]
        return assign

    def _io(self, op: str, peer_alias: str, assign, stream, local_nic, remote_nic, **kw):
        conn = self._get_connection(peer_alias, local_nic, remote_nic)
        ep = self._get_endpoint(peer_alias, local_nic, remote_nic)
        args = self._maybe_endpoint_assign(conn, assign)
        if conn.local_key.link_type == "NVLink":
            return getattr(ep, op)(args, stream=stream, **kw)
        return getattr(ep, op)(args, stream=int(stream or 0), **kw)

    def read(self, peer_alias: str, assign, stream=None, *, local_nic: Optional[str] = None, remote_nic: Optional[str] = None):
        return self._io("read", peer_alias, assign, stream, local_nic, remote_nic)

    def write(self, peer_alias: str, assign, stream=None, *, local_nic: Optional[str] = None, remote_nic: Optional[str] = None):
        return self._io("write", peer_alias, assign, stream, local_nic, remote_nic)

    def write_with_imm(self, peer_alias: str, assign, imm_data: int = 0, stream=None, *, local_nic: Optional[str] = None,
                       remote_nic: Optional[str] = None):
        return self._io("write_with_imm", peer_alias, assign, stream, local_nic, remote_nic, imm_data=imm_data)

    def send(self, peer_alias: str, chunk, stream=None, *, local_nic: Optional[str] = None, remote_nic: Optional[str] = None):
        return self._get_endpoint(peer_alias, local_nic, remote_nic).send(tuple(chunk), int(stream or 0))

    def recv(self, peer_alias: str, chunk, stream=None, *, local_nic: Optional[str] = None, remote_nic: Optional[str] = None):
        return self._get_endpoint(peer_alias, local_nic, remote_nic).recv(tuple(chunk), int(stream or 0))

    def imm_recv(self, peer_alias: str, stream=None, *, local_nic: Optional[str] = None, remote_nic: Optional[str] = None):
        ep = self._get_endpoint(peer_alias, local_nic, remote_nic)
        return ep.imm_recv() if isinstance(ep, _NVLinkAdapter) else ep.imm_recv(int(stream or 0))

    # ------------------------------------------------------------------ shutdown
    def shutdown(self) -> None:
        if self._shutdown_done:
            return
        self._shutdown_done = True
        self._stop.set()
        for ch in list(self._rpc_channels.values()):
            try:
                ch.close()
            except Exception:
                pass
        if self._obs:
            try:
                self._obs.stop()
            except Exception:
                pass
        self._mailbox.stop()
        with self._connections_lock:
            conns = list(self._connections.values())
            self._connections.clear()
            self._connected_cond.notify_all()
        for c in conns:
            if c.endpoint is not None:
                try:
                    c.endpoint.shutdown()
                except Exception:
                    pass
        try:
            # NanoCtrl reads this agent's topology spec to find the peers it must notify, so it goes first
            self._client.cleanup_peer(self.alias)
            doomed = [self._key(f"stream:{self.alias}"), self._key(f"spec:topology:{self.alias}"),
                      self._key(f"obs:peer:{self.alias}")] if not self._obs else [self._key(f"stream:{self.alias}")]
            for pattern in (f"exchange:{self.alias}:*", f"mr:{self.alias}:*"):
                doomed += list(self._store.scan_iter(self._key(pattern)))
            self._store.delete(*doomed)
        except Exception as e:
            log.warning("%s: cleanup during shutdown failed: %s", self.alias, e)
        self._executor.shutdown(wait=False)
        for t in (self._inbox_thread, self._hb_thread):
            if t is not threading.current_thread():
                t.join(timeout=1.0)
        self._store.close()

    def __enter__(self) -> "PeerAgent":
        return self

    def __exit__(self, exc_type, exc_val, exc_tb) -> bool:
        self.shutdown()
        return False


def start_peer_agent(nanoctrl_url: str = "http://127.0.0.1:3000", alias: Optional[str] = None,
                     device: Optional[str] = None, scope: Optional[str] = None, **kw) -> PeerAgent:
    """Convenience constructor; use ``connect_to(peer).wait()`` before data-plane I/O."""
    return PeerAgent(nanoctrl_url=nanoctrl_url, alias=alias, device=device, scope=scope, **kw)
