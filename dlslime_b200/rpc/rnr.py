"""SoftRnrMonitor: watches the ``out_of_buffer`` hardware counters of RDMA ports.

A rising counter means a peer sent before a receive was posted (receiver-not-ready), the
symptom of an undersized mailbox. Reads ``{sysfs}/class/infiniband/*/ports/*/hw_counters/out_of_buffer``
and reports deltas; with no RDMA device present it reports nothing. Same role as the reference's
monitor (``dlslime/rpc/rnr.py:30-92`` in the reference); the sysfs root can be injected for tests.
"""

from __future__ import annotations

import glob
import os


class SoftRnrMonitor:
    def __init__(self, sysfs_root: str = "/sys"):
        self.sysfs_root = sysfs_root
        self._last = self._read()

    def _read(self) -> dict[str, int]:
        out = {}
        pattern = os.path.join(self.sysfs_root, "class", "infiniband", "*", "ports", "*", "hw_counters", "out_of_buffer")
        for path in glob.glob(pattern):
            parts = path.split(os.sep)
            key = f"{parts[-5]}:{parts[-3]}"
            try:
                with open(path) as f:
                    out[key] = int(f.read().strip())
            except (OSError, ValueError):
                continue
        return out

    def poll(self) -> dict[str, int]:
        """Counter increases since the previous call, per ``device:port`` (only non-zero ones)."""
        now = self._read()
        delta = {k: v - self._last.get(k, 0) for k, v in now.items() if v - self._last.get(k, 0) > 0}
        self._last = now
        return delta

    def total(self) -> int:
        return sum(self._read().values())
