"""``torch.distributed`` backend ``"dlslime"``: point-to-point send / recv over this runtime's endpoints.

    import dlslime_b200.torch_backend  # registers the backend
    dist.init_process_group("dlslime", rank=r, world_size=n)
    dist.send(t, dst=1); dist.recv(t, src=0); dist.batch_isend_irecv([...])

Two forms with one contract: a C++ ``c10d::Backend`` (``csrc/torch/slime_backend.cpp``, built against the installed
torch; the default when it loads) and the Python ``ProcessGroup`` below (``SLIME_TORCH_BACKEND=python``, or when the
extension is not built).

Like the reference's backend (``dlslime/csrc/torch/slime_backend.h:105-208`` in the reference) it builds one
endpoint per peer at construction, exchanges their ``endpoint_info()`` through the c10d store (keys
``SLIME_ENDPOINT_<rank>_<peer>``), connects the full mesh, and implements ``send`` / ``recv`` only; every
collective raises "not supported" (use NCCL or gloo for those, as pipeline-parallel users do). Differences:
every tensor of the list is transferred (not just the first) and ``wait(timeout)`` honours its timeout. CUDA tensors
between GPUs of one host go device to device over NVLink (``torch_direct.py``: the receiver exports its tensor, the
sender copies into it; no host bounce); other CUDA tensors are staged through pinned host memory.
"""

from __future__ import annotations

import json
import os
from datetime import timedelta

import torch
import torch.distributed as dist

from . import _slime_c

_WORK_BASE = getattr(dist, "_Work", None) or dist.Work


class SlimeWork(_WORK_BASE):
    """Handle of one send or recv; ``wait`` returns once the bytes moved (and, for CUDA, reached the device)."""

    def __init__(self, futures, finish=None, default_timeout: float = 300.0):
        super().__init__()
        self._futures, self._finish, self._default = list(futures), finish, default_timeout
        self._done = False
        self._fut = torch.futures.Future()

    def wait(self, timeout: timedelta | None = None) -> bool:
        if self._done:
            return True
        secs = timeout.total_seconds() if isinstance(timeout, timedelta) and timeout.total_seconds() > 0 else self._default
        for f in self._futures:
            status = f.wait(secs)
            if status != 0:
                raise RuntimeError(f"dlslime backend: transfer ended with status {status}" + (" (timeout)" if status == 402 else ""))
        if self._finish is not None:
            self._finish()
        self._done = True
        if not self._fut.done():
            self._fut.set_result(None)
        return True

    def is_completed(self) -> bool:
        return self._done or all(f.done() for f in self._futures)

    def is_success(self) -> bool:
        return self._done

    def get_future(self):
        return self._fut


class SlimeProcessGroup(dist.ProcessGroup):
    def __init__(self, store, rank: int, size: int, timeout: timedelta | None = None, bind_host: str = "127.0.0.1"):
        super().__init__(rank, size)
        self._rank, self._size = rank, size
        self._timeout = (timeout or timedelta(seconds=300)).total_seconds()
        self._eps = {}
        self._keep = []  # staging buffers of operations in flight
        for peer in range(size):
            if peer == rank:
                continue
            ep = self._make_endpoint(bind_host, peer)
            self._eps[peer] = ep
            store.set(f"SLIME_ENDPOINT_{rank}_{peer}", json.dumps(ep.endpoint_info()))
        for peer, ep in self._eps.items():
            info = json.loads(store.get(f"SLIME_ENDPOINT_{peer}_{rank}"))  # blocks until the peer published it
            ep.connect(info)

    def _make_endpoint(self, bind_host: str, peer: int):
        """RDMA when a verbs provider with a device exists (NIC picked round robin by rank, as the reference
        backend does), else TCP. ``SLIME_BACKEND_TRANSPORT=tcp|rdma`` forces one."""
        want = os.environ.get("SLIME_BACKEND_TRANSPORT", "")
        devices = _slime_c.rdma_devices() if want != "tcp" else []
        if want == "rdma" and not devices:
            raise RuntimeError(f"SLIME_BACKEND_TRANSPORT=rdma but no RDMA provider: {_slime_c.rdma_provider()[1]}")
        if devices and (want == "rdma" or _slime_c.rdma_provider()[0] == "ibverbs"):
            return _slime_c.RDMAEndpoint(devices[self._rank % len(devices)], 1, "", 0)
        return _slime_c.TcpEndpoint(bind_host, 0, 1)

    def getBackendName(self) -> str:
        return "dlslime"

    # -- point to point --------------------------------------------------------------------------
    def _chunks(self, tensors):
        for t in tensors:
            if not t.is_contiguous():
                raise ValueError("dlslime backend: tensors must be contiguous")
            yield t, t.numel() * t.element_size()

    def send(self, tensors, dst: int, tag: int = 0):
        futs = []
        for t, nbytes in self._chunks(tensors):
            host = t if not t.is_cuda else t.to("cpu", non_blocking=False)  # device -> host staging completes before the send is posted
            self._keep.append(host)
            futs.append(self._eps[dst].send((host.data_ptr(), 0, nbytes)))
        return SlimeWork(futs, finish=self._gc, default_timeout=self._timeout)

    def recv(self, tensors, src: int, tag: int = 0):
        futs, copies = [], []
        for t, nbytes in self._chunks(tensors):
            if t.is_cuda:
                host = torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
                copies.append((t, host))
            else:
                host = t
            self._keep.append(host)
            futs.append(self._eps[src].recv((host.data_ptr(), 0, nbytes)))

        def finish():
            for dev, host in copies:
                dev.copy_(host, non_blocking=False)
            self._gc()

        return SlimeWork(futs, finish=finish, default_timeout=self._timeout)

    def _gc(self):
        if len(self._keep) > 256:
            del self._keep[:128]

    def recv_anysource(self, tensors, tag: int = 0):
        raise NotImplementedError("dlslime backend: recv from any source is not supported")

    # -- collectives: not supported, by design -------------------------------------------------------
    def _unsupported(self, name):
        raise NotImplementedError(f"dlslime backend: {name} is not supported; it provides send / recv only")

    def broadcast(self, *a, **k):
        self._unsupported("broadcast")

    def allreduce(self, *a, **k):
        self._unsupported("allreduce")

    def allgather(self, *a, **k):
        self._unsupported("allgather")

    def _allgather_base(self, *a, **k):
        self._unsupported("all_gather_into_tensor")

    def reduce_scatter(self, *a, **k):
        self._unsupported("reduce_scatter")

    def alltoall(self, *a, **k):
        self._unsupported("alltoall")

    def alltoall_base(self, *a, **k):
        self._unsupported("all_to_all_single")

    def gather(self, *a, **k):
        self._unsupported("gather")

    def scatter(self, *a, **k):
        self._unsupported("scatter")

    def reduce(self, *a, **k):
        self._unsupported("reduce")

    def barrier(self, *a, **k):
        self._unsupported("barrier")

    def shutdown(self):
        for ep in self._eps.values():
            ep.shutdown()
        self._eps.clear()

    def __del__(self):
        try:
            self.shutdown()
        except Exception:
            pass


def _load_cpp():
    """The C++ backend (``csrc/torch/slime_backend.cpp``, a ``c10d::Backend``), or None with the reason."""
    try:
        from . import _slime_torch  # built by dlslime_b200/_build.py against the installed torch

        return _slime_torch, ""
    except ImportError as e:
        return None, str(e)


def implementation() -> str:
    """``"cpp"`` or ``"python"``: which form ``init_process_group("dlslime")`` creates. ``SLIME_TORCH_BACKEND`` forces one;
    by default the C++ backend is used when its extension is built and loads."""
    want = os.environ.get("SLIME_TORCH_BACKEND", "")
    if want == "python":
        return "python"
    mod, why = _load_cpp()
    if mod is None:
        if want == "cpp":
            raise RuntimeError(f"SLIME_TORCH_BACKEND=cpp but the extension does not load: {why}")
        return "python"
    return "cpp"


def _create(store, rank, size, timeout):
    if implementation() == "cpp":
        mod, _ = _load_cpp()
        ms = int(timeout.total_seconds() * 1000) if isinstance(timeout, timedelta) else 300_000
        inner = mod.create_backend(store, rank, size, ms, _slime_c.bridge_table(), os.environ.get("SLIME_BACKEND_TRANSPORT", ""),
                                   "127.0.0.1")
    else:
        inner = SlimeProcessGroup(store, rank, size, timeout)
    # CUDA tensors between GPUs of one host go device to device over NVLink (torch_direct.py); SLIME_BACKEND_DIRECT=off
    # keeps every tensor on the staged path of the backend above
    mode = os.environ.get("SLIME_BACKEND_DIRECT", "auto")
    if mode == "off" or (mode == "auto" and not torch.cuda.is_available()):
        return inner
    from .torch_direct import DirectGroup

    return DirectGroup(inner, store, rank, size, timeout if isinstance(timeout, timedelta) else None, mode=mode)


def register() -> None:
    if "DLSLIME" not in dist.Backend.backend_list and "dlslime" not in getattr(dist.Backend, "backend_list", []):
        dist.Backend.register_backend("dlslime", _create, devices=["cpu", "cuda"])


register()
