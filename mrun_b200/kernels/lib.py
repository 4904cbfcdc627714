"""Loads the compiled kernel libraries through their C ABI.

There is no other implementation behind these calls: if a library cannot be built or opened the
import fails with the reason, and every entry point raises :class:`KernelError` with the
library's own message when it refuses its arguments.
"""
from __future__ import annotations

import ctypes
from typing import Dict

from . import build


class KernelError(RuntimeError):
    pass


class Library:
    """A loaded ``.so``: ``lib.call("mrun_x", args...)`` raises on a non-zero return."""

    def __init__(self, path: str, error_symbol: str = "mrun_last_error"):
        self.path = path
        try:
            self._dll = ctypes.CDLL(path, mode=ctypes.RTLD_LOCAL)
        except OSError as error:
            raise KernelError(f"cannot open the kernel library {path}: {error}") from None
        self._last_error = getattr(self._dll, error_symbol)
        self._last_error.restype = ctypes.c_char_p
        self._functions: Dict[str, ctypes._CFuncPtr] = {}

    def function(self, name: str):
        fn = self._functions.get(name)
        if fn is None:
            try:
                fn = getattr(self._dll, name)
            except AttributeError:
                raise KernelError(f"{self.path} exports no {name}") from None
            fn.restype = ctypes.c_int
            self._functions[name] = fn
        return fn

    def call(self, name: str, *args) -> None:
        global _calls
        _calls += 1
        if self.function(name)(*args) != 0:
            raise KernelError(self._last_error().decode("utf-8", "replace"))


_calls = 0


def call_count() -> int:
    """How many kernel entry points were called so far (each launches this library's kernels)."""
    return _calls


_core: Library | None = None
_attention: Dict[int, Library] = {}


def core() -> Library:
    global _core
    if _core is None:
        lib = Library(build.build_core())
        arch = lib._dll.mrun_target_arch
        arch.restype = ctypes.c_int
        if arch() != 100:
            raise KernelError(f"{lib.path} was not built for sm_100a")
        _core = lib
    return _core


def attention(head_dim: int) -> Library:
    """The tensor-core attention library for ``head_dim`` (built at first use)."""
    lib = _attention.get(head_dim)
    if lib is None:
        lib = Library(build.build_attention(head_dim))
        query = lib._dll.mrun_attn_head_dim
        query.restype = ctypes.c_int
        if query() != head_dim:
            raise KernelError(f"{lib.path} was built for head_dim={query()}, not {head_dim}")
        _attention[head_dim] = lib
    return lib
