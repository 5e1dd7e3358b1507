"""B200 (sm_100a) operator backend for the `mops` library that nano-vLLM's layers call.

* `nano_vllm_ninetoothed_b200.mops`   -- the drop-in operator surface (same names/signatures
  as the reference's `mops` package), each op one hand-written CUDA kernel behind the C ABI
  declared in `include/b200mops.h`.
* `nano_vllm_ninetoothed_b200.build`  -- nvcc recipe for `lib/libb200mops.so`.
* `nano_vllm_ninetoothed_b200.workloads` -- seeded synthetic inputs of the benchmark shapes.

The compiled library is required: importing `.mops` without it raises ImportError.
"""
from __future__ import annotations

import importlib
import sys

__version__ = "0.1.0"

_LAZY = ("mops", "workloads", "_cabi", "build")


def __getattr__(name: str):
    if name in _LAZY:
        return importlib.import_module(f"{__name__}.{name}")
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


def install_as_mops() -> None:
    """Make `import mops` / `from mops import ...` resolve to this backend.

    Call it before the first import of `nanovllm.layers`; the reference's layers bind the
    operator names at import time (nanovllm/layers/attention.py:5 and siblings).
    """
    mod = importlib.import_module(f"{__name__}.mops")
    existing = sys.modules.get("mops")
    if existing is not None and existing is not mod:
        raise RuntimeError("another `mops` module is already imported")
    sys.modules["mops"] = mod
