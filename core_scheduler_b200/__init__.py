# SPDX-License-Identifier: Apache-2.0
"""core_scheduler_b200: a B200-native training framework with the capabilities of CoreScheduler.

The runtime (future-tensor handles, the three-stream task scheduler, ops, modules, optimizers,
collectives, data loaders, checkpoints, GPT-2) is C++/CUDA in ``csrc/``; this package loads the
in-tree build and exposes it. ``core_scheduler_b200._C`` is the pybind11 module; the
sub-packages add configuration presets and process launch helpers only.
"""
from __future__ import annotations

import os as _os

import torch as _torch  # noqa: F401  (libtorch must be loaded before the extension)

from . import build as _build

if not _build.is_built():
    if _os.environ.get("CS_NO_AUTOBUILD") == "1":
        raise ImportError("core_scheduler_b200 native library is not built; run `python -m core_scheduler_b200.build`")
    _build.build()

import pyarrow as _pyarrow  # noqa: F401,E402  (provides libarrow/libparquet for checkpoints and datasets)

if _os.environ.get("CS_BOUNDS_CHECK") == "1":
    # Diagnostic run: load the library whose kernels check every derived index (same soname, so the
    # extension binds to it instead of lib/libcs_b200.so). Never falls back silently.
    import ctypes as _ctypes

    if not _build.is_checked_built():
        if _os.environ.get("CS_NO_AUTOBUILD") == "1":
            raise ImportError("CS_BOUNDS_CHECK=1 needs lib_checked/libcs_b200.so; run `python -m core_scheduler_b200.build checked`")
        _build.build(checked=True)
    _ctypes.CDLL(str(_build.CHECKED_LIBDIR / "libcs_b200.so"), mode=_ctypes.RTLD_GLOBAL)

from . import _C  # noqa: E402

if _os.environ.get("CS_BOUNDS_CHECK") == "1" and not _C.bounds_check_enabled():
    raise ImportError("CS_BOUNDS_CHECK=1 but the extension bound to the unchecked library")
from ._C import (  # noqa: E402,F401
    AdamW,
    AllReduceBucket,
    DynamicScheduler,
    Error,
    GPT2,
    GPT2Config,
    GradientSync,
    Tensor,
    autocast,
    from_torch,
    library_fallbacks,
    manual_seed,
    to_torch,
)

__all__ = [
    "_C",
    "AdamW",
    "AllReduceBucket",
    "DynamicScheduler",
    "Error",
    "GPT2",
    "GPT2Config",
    "GradientSync",
    "Tensor",
    "autocast",
    "from_torch",
    "library_fallbacks",
    "manual_seed",
    "to_torch",
]
