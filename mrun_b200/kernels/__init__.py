"""Python bindings of the hand-written CUDA kernels (``csrc/``)."""
from .lib import KernelError

__all__ = ["KernelError"]
