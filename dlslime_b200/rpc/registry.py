"""``@method`` decorator and the per-class method registry.

Tags are the indices of the decorated methods in sorted-name order, so both sides derive the
same table from the same class (as in the reference, ``dlslime/rpc/registry.py:135-166``).
Arguments and results are pickled (highest protocol) unless the method is ``raw``, in which
case one ``bytes`` argument and a ``bytes``-like result pass through untouched.
"""

from __future__ import annotations

import inspect
import pickle
from dataclasses import dataclass
from typing import Any, Callable

_MARK = "__slime_rpc__"


def method(fn: Callable | None = None, *, streaming: bool = False, raw: bool = False, parallel: bool = False, inplace: bool = False):
    """Mark a service method as remotely callable.

    ``raw``: takes and returns bytes, no pickling. ``parallel``: may run concurrently with other
    calls on the same service object (no per-service lock). ``inplace``: the handler receives
    ``(payload_view, reply_ptr, reply_capacity)`` and returns the number of reply bytes it wrote.
    """

    def mark(f):
        setattr(f, _MARK, {"streaming": streaming, "raw": raw, "parallel": parallel, "inplace": inplace})
        return f

    return mark(fn) if fn is not None else mark


@dataclass
class MethodInfo:
    tag: int
    name: str
    fn: Callable
    streaming: bool = False
    raw: bool = False
    parallel: bool = False
    inplace: bool = False

    def dumps_args(self, args: tuple, kwargs: dict) -> bytes:
        if self.raw:
            if len(args) != 1 or kwargs or not isinstance(args[0], (bytes, bytearray, memoryview)):
                raise TypeError(f"raw RPC {self.name!r} takes exactly one bytes-like argument")
            return bytes(args[0])
        return pickle.dumps((args, kwargs), protocol=pickle.HIGHEST_PROTOCOL)

    def loads_args(self, data: bytes):
        if self.raw:
            return (data,), {}
        return pickle.loads(data)

    def dumps_result(self, result: Any) -> bytes:
        if self.raw:
            return b"" if result is None else bytes(result)
        return b"" if result is None else pickle.dumps(result, protocol=pickle.HIGHEST_PROTOCOL)

    def loads_result(self, data: bytes) -> Any:
        if self.raw:
            return data
        return None if not data else pickle.loads(data)


class MethodRegistry:
    def __init__(self, service_cls: type):
        members = sorted((name, fn) for name, fn in inspect.getmembers(service_cls, predicate=inspect.isfunction) if hasattr(fn, _MARK))
        self.by_tag: dict[int, MethodInfo] = {}
        self.by_name: dict[str, MethodInfo] = {}
        for tag, (name, fn) in enumerate(members):
            info = MethodInfo(tag=tag, name=name, fn=fn, **getattr(fn, _MARK))
            self.by_tag[tag] = self.by_name[name] = info
        if not self.by_tag:
            raise ValueError(f"{service_cls.__name__} has no @method functions")
