"""Locates (and, when missing, builds) the in-tree native libraries."""
from __future__ import annotations

import ctypes
import importlib
import os
from pathlib import Path

_PKG = Path(__file__).resolve().parent
_device_lib = None


def device_library_path() -> Path:
    return _PKG / "lib" / "libcatch_b200_device.so"


def load_device_library() -> ctypes.CDLL:
    """ctypes handle of the kernel library (C ABI, see csrc/device/*.h)."""
    global _device_lib
    if _device_lib is None:
        path = device_library_path()
        if not path.exists():
            from . import _build

            _build.build()
        _device_lib = ctypes.CDLL(str(path))
    return _device_lib


def load_native():
    try:
        load_device_library()
        return importlib.import_module("catch_b200._C")
    except (ImportError, OSError):
        if os.environ.get("CATCH_B200_NO_AUTOBUILD") == "1":
            raise
        from . import _build

        _build.build()
        load_device_library()
        return importlib.import_module("catch_b200._C")
