"""tilert_b200 -- B200-native batch-1 FP8 decode path behind the TileRT operator interface.

Mirrors the reference package entry points (tilert/__init__.py:51-80, tilert/tilert_init.py):
``load_backend(model_type)`` loads the in-tree CUDA library once per process and
``tilert_init()`` creates the per-device context.  There is no CPU fallback: without the
compiled library, or without a CUDA device, these raise.
"""

from __future__ import annotations

import ctypes
import logging
from pathlib import Path

__version__ = "0.1.0"
logger = logging.getLogger(__name__)

_BACKENDS = {"deepseek_v3_2": "libtilert_b200.so"}
_lib: ctypes.CDLL | None = None
_contexts: dict[int, int] = {}


class TilertError(RuntimeError):
    """An error reported by the native library (mirrors the RuntimeError of a failed torch op)."""


def library_path() -> Path:
    """The in-tree library; ``TILERT_B200_LIB`` names another build of the same sources (tuning)."""
    import os

    override = os.environ.get("TILERT_B200_LIB")
    return Path(override) if override else Path(__file__).resolve().parent / "libtilert_b200.so"


def load_backend(model_type: str = "deepseek_v3_2") -> ctypes.CDLL:
    """Load the native library for ``model_type`` (tilert/__init__.py:51-80)."""
    global _lib
    if model_type not in _BACKENDS:
        raise ValueError(f"Unknown model_type {model_type!r}. Supported: {sorted(_BACKENDS)}")
    if _lib is not None:
        return _lib
    path = library_path()
    if not path.exists():
        raise RuntimeError(
            f"Backend library not found: {path}. Build it with `python -m tilert_b200.build` "
            "(needs nvcc; compiles for sm_100a).")
    from ._cabi import bind

    _lib = bind(path)
    logger.info("Loaded tilert_b200 backend %s", path.name)
    return _lib


def lib() -> ctypes.CDLL:
    return load_backend()


def check(rc: int) -> None:
    """Raise ``TilertError`` for a negative return code of a C-ABI call."""
    if rc != 0:
        msg = lib().tilert_b200_last_error()
        raise TilertError(f"tilert_b200 call failed ({rc}): {msg.decode() if msg else ''}")


def tilert_init(device: int | None = None) -> int:
    """Create (once) the context of ``device`` and return its handle (tilert/tilert_init.py:11-13)."""
    import torch

    if not torch.cuda.is_available():
        raise RuntimeError("tilert_b200 needs a CUDA device (sm_100a); there is no CPU path")
    dev = torch.cuda.current_device() if device is None else device
    if dev not in _contexts:
        ctx = ctypes.c_void_p()
        check(lib().tilert_b200_default_context(dev, ctypes.byref(ctx)))
        _contexts[dev] = ctx.value
    return _contexts[dev]


def device_status(device: int | None = None) -> int:
    """Synchronise and return the device status word (0 = every kernel ran to completion)."""
    st = ctypes.c_int(0)
    check(lib().tilert_b200_status(tilert_init(device), ctypes.byref(st)))
    return st.value


def set_wait_budget(cycles: int, device: int | None = None) -> None:
    """Upper bound (SM clock cycles) of every bounded wait in the library's kernels; ``cycles <= 0`` restores
    the default of about half a second."""
    check(lib().tilert_b200_set_wait_budget(ctypes.c_void_p(tilert_init(device)), int(cycles)))


__all__ = ["set_wait_budget", "load_backend", "tilert_init", "device_status", "lib", "check", "TilertError", "__version__"]
