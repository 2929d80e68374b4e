"""ctypes binding of ``libslime_cuda.so`` (the sm_100a kernels and CUDA plumbing).

The library is built in-tree by :mod:`dlslime_b200._build`. On a machine with a
GPU a missing library is an error: there is no PyTorch fallback for the kernels.
"""

from __future__ import annotations

import ctypes
import threading
from ctypes import c_char_p, c_float, c_int, c_longlong, c_ulonglong, c_void_p, POINTER
from pathlib import Path

_LIB = None
_LOCK = threading.Lock()

c_ubyte_p = POINTER(ctypes.c_ubyte)

# name -> argtypes (every function returns int unless listed in _RESTYPES)
_SIGNATURES = {
    "slime_cuda_version": [],
    "slime_status_alloc": [POINTER(c_void_p), POINTER(c_void_p)],
    "slime_status_free": [c_void_p],
    "slime_host_flags_alloc": [c_ulonglong, POINTER(c_void_p), POINTER(c_void_p)],
    "slime_host_flags_free": [c_void_p],
    "slime_wait_flag_kernel": [c_void_p, c_ulonglong, c_ulonglong, c_void_p, c_void_p],
    "slime_signal_flag_kernel": [c_void_p, c_ulonglong, c_int, c_void_p],
    "slime_symm_alloc": [c_ulonglong, POINTER(c_void_p), c_ubyte_p],
    "slime_symm_free": [c_void_p],
    "slime_ipc_get_handle": [c_void_p, c_ubyte_p, POINTER(c_ulonglong), POINTER(c_ulonglong)],
    "slime_ipc_open": [c_ubyte_p, POINTER(c_void_p)],
    "slime_ipc_close": [c_void_p],
    "slime_enable_peer_access": [c_int],
    "slime_memset_async": [c_void_p, c_int, c_ulonglong, c_void_p],
    "slime_memcpy_async": [c_void_p, c_void_p, c_ulonglong, c_void_p],
    "slime_fp8_quant_1x128": [c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_longlong, c_longlong, c_void_p],
    "slime_fp8_dequant_1x128": [c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_longlong, c_longlong, c_void_p],
    "slime_fp8_quant_128x128": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_longlong, c_longlong, c_void_p],
    "slime_gemm_bf16": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong, c_void_p, c_void_p],
    "slime_gemm_bf16_pair": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong, c_void_p, c_void_p],
    "slime_gemm_fp8_blockscaled": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong,
                                   c_longlong, c_void_p, c_void_p],
    "slime_grouped_gemm_fp8a": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_longlong, c_longlong,
                                c_longlong, c_int, c_void_p, c_void_p],
    "slime_gemm_bf16_gated": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong,
                              c_void_p, c_int, c_ulonglong, c_int, c_void_p, c_void_p],
    "slime_grouped_gemm_bf16_gated": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_longlong,
                                      c_longlong, c_longlong, c_int, c_void_p, c_ulonglong, c_void_p, c_void_p, c_void_p],
    "slime_grouped_gemm_bf16_gated_traced": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_longlong,
                                             c_longlong, c_longlong, c_int, c_void_p, c_ulonglong, c_void_p, c_void_p, c_void_p,
                                             c_void_p, c_void_p],
    "slime_grouped_gemm_bf16": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_longlong,
                                c_longlong, c_longlong, c_int, c_void_p, c_void_p, c_ulonglong, c_ulonglong, c_void_p,
                                c_void_p, c_void_p],
}
_SIGNATURES["slime_grouped_gemm_bf16_pair"] = _SIGNATURES["slime_grouped_gemm_bf16"]
_SIGNATURES["slime_grouped_gemm_bf16_wide"] = _SIGNATURES["slime_grouped_gemm_bf16"]
_SIGNATURES["slime_grouped_gemm_bf16_swapped"] = _SIGNATURES["slime_grouped_gemm_bf16"]
_SIGNATURES["slime_gemm_bf16_wide"] = _SIGNATURES["slime_gemm_bf16_pair"]
_SIGNATURES["slime_grouped_gemm_bf16_tile"] = [*_SIGNATURES["slime_grouped_gemm_bf16"][:-2], c_int, c_int, c_int, c_void_p, c_void_p]


class SlimeCudaError(RuntimeError):
    """A launcher or CUDA call inside libslime_cuda.so reported an error."""


def lib_path() -> Path:
    return Path(__file__).resolve().parent / "_C" / "libslime_cuda.so"


def load(build_if_missing: bool = True) -> ctypes.CDLL:
    """Load (building first if needed) the kernel library and declare prototypes."""
    global _LIB
    if _LIB is not None:
        return _LIB
    with _LOCK:
        if _LIB is not None:
            return _LIB
        path = lib_path()
        if not path.exists():
            if not build_if_missing:
                raise SlimeCudaError(f"{path} is missing; run `python -m dlslime_b200._build`")
            from . import _build

            _build.build_cuda()
        lib = ctypes.CDLL(str(path), mode=ctypes.RTLD_GLOBAL)
        lib.slime_last_error.restype = c_char_p
        lib.slime_last_error.argtypes = []
        for name, argtypes in _SIGNATURES.items():
            fn = getattr(lib, name, None)
            if fn is None:
                continue
            fn.argtypes = argtypes
            fn.restype = c_int
        _LIB = lib
        _install_stream_hooks(lib)
    return _LIB


def _install_stream_hooks(lib) -> None:
    """Give the host runtime the addresses of the four functions behind its stream-ordered signals."""
    try:
        from . import _slime_c

        addr = lambda name: ctypes.cast(getattr(lib, name), ctypes.c_void_p).value  # noqa: E731
        _slime_c.install_stream_hooks(addr("slime_host_flags_alloc"), addr("slime_host_flags_free"),
                                      addr("slime_hook_record_value"), addr("slime_hook_wait_mask"))
    except Exception:  # the host module is optional for pure kernel users
        pass


def declare(name: str, argtypes) -> None:
    """Register the prototype of one more exported function (used by ops modules)."""
    _SIGNATURES[name] = argtypes
    if _LIB is not None:
        fn = getattr(_LIB, name)
        fn.argtypes = argtypes
        fn.restype = c_int


def call(name: str, *args) -> int:
    """Call ``name`` and raise :class:`SlimeCudaError` on a negative return code."""
    lib = load()
    rc = getattr(lib, name)(*args)
    if rc < 0:
        msg = lib.slime_last_error()
        raise SlimeCudaError(f"{name}: {msg.decode(errors='replace') if msg else 'unknown error'}")
    return rc


def available() -> bool:
    return lib_path().exists()
