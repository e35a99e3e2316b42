"""Loads the kernel library and checks that it is the one these bindings were written for.

There is no fallback: if the library cannot be built or loaded, or no CUDA device is present when a
kernel is asked for, the call fails with a message that says so.
"""
from __future__ import annotations

import ctypes
import threading
from typing import Optional

from . import build

ABI_VERSION = 1

_lock = threading.Lock()
_lib: Optional[ctypes.CDLL] = None


class KernelError(RuntimeError):
    """A kernel entry point refused its arguments or its launch failed."""


def load(verbose: bool = True) -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        path = build.library_path(create=True, verbose=verbose)
        try:
            lib = ctypes.CDLL(path)
        except OSError as e:
            raise KernelError(f"the kernel library {path} could not be loaded: {e}") from None
        lib.gi_last_error.restype = ctypes.c_char_p
        lib.gi_abi_version.restype = ctypes.c_int
        got = lib.gi_abi_version()
        if got != ABI_VERSION:
            raise KernelError(f"{path} has ABI version {got}, these bindings want {ABI_VERSION}: rebuild it")
        _lib = lib
        return lib


def last_error(lib: ctypes.CDLL) -> str:
    msg = lib.gi_last_error()
    return msg.decode("utf-8", "replace") if msg else ""
