"""NanoCtrl: control-plane server (C++, embedded or stand-alone), HTTP client and store client."""

from .client import NanoCtrlClient, NanoCtrlError
from .resp import RespClient, RespError
from .server import LocalNanoCtrl, start_local_nanoctrl

__all__ = ["NanoCtrlClient", "NanoCtrlError", "RespClient", "RespError", "LocalNanoCtrl", "start_local_nanoctrl"]
