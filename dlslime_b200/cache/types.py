"""JSON shapes of the DLSlimeCache HTTP API and conversions to / from the C++ types."""

from __future__ import annotations

from typing import Any

from .._slime_c import Assignment

DEFAULT_SLAB_SIZE = 256 * 1024
DEFAULT_MEMORY_SIZE = 0
DEFAULT_CACHE_MR_NAME = "cache"
DEFAULT_SERVICE_ID = "cache:0"
DEFAULT_AGENT_ALIAS = "cache-agent:0"


def assignment_to_json(a: Assignment) -> dict[str, int]:
    return {"mr_key": int(a.mr_key), "remote_mr_key": int(a.remote_mr_key), "target_offset": int(a.target_offset),
            "source_offset": int(a.source_offset), "length": int(a.length)}


def assignment_from_json(d: dict[str, Any]) -> Assignment:
    return Assignment(int(d["mr_key"]), int(d.get("remote_mr_key", d["mr_key"])), int(d["target_offset"]),
                      int(d["source_offset"]), int(d["length"]))


def assignment_to_tuple(a: Assignment) -> tuple[int, int, int, int, int]:
    """``(mr_key, remote_mr_key, target_offset, source_offset, length)``, the order the endpoints take."""
    return tuple(int(getattr(a, k)) for k in ("mr_key", "remote_mr_key", "target_offset", "source_offset", "length"))


def manifest_to_json(m) -> dict[str, Any]:
    return {"peer_agent_id": m.peer_agent_id, "version": int(m.version), "total_bytes": int(m.total_bytes()),
            "slab_ids": [int(s) for s in m.slab_ids], "assignments": [assignment_to_json(a) for a in m.assignments]}


def stats_to_json(s) -> dict[str, int]:
    return {k: int(getattr(s, k)) for k in ("slab_size", "memory_size", "num_slabs", "used_slabs", "free_slabs",
                                            "num_assignment_peers", "num_assignment_entries", "num_assignments", "assignment_bytes")}
