"""Handshake timing probe: ``DLSLIME_TIMING=1`` prints ``[TLOG <ms>] message`` lines to stderr."""

import os
import sys
import time

_ENABLED = os.environ.get("DLSLIME_TIMING", "0") == "1"
_T0 = time.perf_counter()


def tlog(message: str) -> None:
    if _ENABLED:
        print(f"[TLOG {(time.perf_counter() - _T0) * 1e3:10.3f}] {message}", file=sys.stderr, flush=True)
