"""Exception types of SlimeRPC."""


class RpcError(RuntimeError):
    """Base class: transport or protocol failure of an RPC."""


class RpcTimeoutError(RpcError, TimeoutError):
    """No reply within the caller's timeout; the request was detached so a late reply only frees its slot."""


class RemoteRpcError(RpcError):
    """The handler raised on the server; carries the remote type name, message and traceback text."""

    def __init__(self, remote_type: str, message: str, remote_traceback: str = ""):
        super().__init__(f"{remote_type}: {message}")
        self.remote_type, self.remote_message, self.remote_traceback = remote_type, message, remote_traceback
