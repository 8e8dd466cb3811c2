"""Loading of the native extension (`_C.so`, built in-tree by `build.py`)."""
from __future__ import annotations

import importlib
import os
from pathlib import Path

_PKG = Path(__file__).resolve().parent
_C = None


class NativeExtensionMissing(ImportError):
    pass


def load():
    """Returns the `_C` module (and registers the `torch.ops.b200ipc` operators).

    Never falls back to a Python implementation: if the extension cannot be
    imported the error says how to build it.
    """
    global _C
    if _C is not None:
        return _C
    import torch  # noqa: F401  (libtorch must be loaded before the extension)

    so = _PKG / "_C.so"
    if not so.exists() and os.environ.get("B200IPC_NO_AUTOBUILD", "0") != "1":
        from . import build as _build

        _build.build()
    try:
        _C = importlib.import_module("gpu_ipc_example_b200._C")
    except ImportError as e:  # pragma: no cover - depends on the machine
        raise NativeExtensionMissing(
            f"gpu_ipc_example_b200._C could not be imported ({e}). Build it with "
            f"`python -m gpu_ipc_example_b200.build` (needs nvcc with sm_100a support)."
        ) from e
    return _C


def emulator_path() -> Path:
    so = _PKG / "libb200ipc_emu.so"
    if not so.exists():
        from . import build as _build

        _build.build(with_torch=False)
    return so
