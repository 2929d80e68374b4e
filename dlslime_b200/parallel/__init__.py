"""Symmetric device memory shared by the ranks of one node (see :mod:`dlslime_b200.parallel.symm`)."""

from .symm import SymmetricHeap, tensor_from_ptr  # noqa: F401

__all__ = ["SymmetricHeap", "tensor_from_ptr"]
