"""mimir_b200 -- B200 (sm_100a) kernels behind MimIR's `tensor` plugin operators.

`mimir_b200.tensor` mirrors the operator names of the reference's tensor plugin (product_2d, bmm, reduce,
softmax, binary_ax, ...) on CUDA torch tensors; every call goes through the C ABI in include/mimk.h.
"""
from . import _lib  # noqa: F401
from ._lib import MimkError  # noqa: F401

__all__ = ["tensor", "MimkError"]
