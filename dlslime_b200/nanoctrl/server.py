"""In-process NanoCtrl: the C++ server running on threads of the current Python process.

Used by tests, single-node jobs and the CPU plumbing benchmark, where starting a separate
control-plane daemon would be overkill. ``url`` is what ``PeerAgent(nanoctrl_url=...)`` takes.
For a long-lived deployment use the stand-alone binary (``python -m dlslime_b200.nanoctrl``).
"""

from __future__ import annotations

from .. import _slime_c


class LocalNanoCtrl:
    def __init__(self, host: str = "127.0.0.1", http_port: int = 0, resp_port: int = 0):
        self._srv = _slime_c.ctrl.NanoCtrl()
        self._srv.start(host, http_port, resp_port)
        self.host = host

    @property
    def http_port(self) -> int:
        return self._srv.http_port

    @property
    def resp_port(self) -> int:
        return self._srv.resp_port

    @property
    def url(self) -> str:
        return f"http://{self.host}:{self.http_port}"

    @property
    def store(self):
        """Direct (in-process) handle of the key-value store."""
        return self._srv.store

    def stop(self) -> None:
        self._srv.stop()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.stop()
        return False


def start_local_nanoctrl(host: str = "127.0.0.1", http_port: int = 0, resp_port: int = 0) -> LocalNanoCtrl:
    return LocalNanoCtrl(host, http_port, resp_port)
