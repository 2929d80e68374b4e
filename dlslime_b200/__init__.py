"""B200-native communication runtime with the capabilities of DLSlime.

Layers (top to bottom): ``rpc`` and ``cache`` (services) · ``peer_agent`` (named I/O, handshake) ·
``nanoctrl`` (control plane: C++ server, HTTP and store clients) · ``_slime_c`` (C++ host runtime: endpoints,
futures, pools, counters, topology) · ``ops`` / ``models`` / ``parallel`` (sm_100a kernels over NVLink peer
memory and what is built from them). ``import dlslime_b200 as dlslime`` gives the names a user of the
reference's top-level package expects.
"""

from . import _build as _build_mod

__version__ = "0.1.0"


def _ensure_built() -> None:
    if not _build_mod.host_ext_path().exists():
        _build_mod.build_host()


_ensure_built()

from . import _slime_c  # noqa: E402
from ._slime_c import *  # noqa: E402,F401,F403
from ._slime_c import (Assignment, OpCode, TcpEndpoint, available_nic, discover_topology, obs_enabled,  # noqa: E402,F401
                       obs_snapshot, socket_id)
from .logging import get_logger, set_log_level  # noqa: E402,F401
from .peer_agent import PeerAgent, start_peer_agent  # noqa: E402,F401


def NVLinkEndpoint(*args, **kwargs):
    """The kernel-driven NVLink endpoint (needs CUDA); see :mod:`dlslime_b200.ops.nvlink`."""
    from .ops.nvlink import NVLinkEndpoint as _Ep

    return _Ep(*args, **kwargs)


def get_cmake_dir() -> str:
    """Directory with the C headers of the native libraries (``slime_cuda.h``, ``slime_noalloc.h``)."""
    import os

    return os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc", "include")


_LAZY_OPS = {
    # names of the reference's collective buffers (bound in its `_slime_c` when the ops are built); they need CUDA,
    # so they are imported on first use
    "AllGatherInterLLBuffer": ("ops.allgather", "AllGatherLLBuffer"),
    "AllGatherLLBuffer": ("ops.allgather", "AllGatherLLBuffer"),
    "AllToAllIntraLLBuffer": ("ops.alltoall", "AllToAllLLBuffer"),
    "AllToAllLLBuffer": ("ops.alltoall", "AllToAllLLBuffer"),
}


def __getattr__(name: str):
    target = _LAZY_OPS.get(name)
    if target is None:
        raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
    import importlib

    return getattr(importlib.import_module(f"{__name__}.{target[0]}"), target[1])
