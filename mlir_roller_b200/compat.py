"""Lets scripts written against the reference's flat module layout run unchanged.

The reference is used from inside its `src/` directory with `from analyze import ...`,
`from arch import CUDA`, `from roller import Compiler, run_eval` (src/benchmark.py:5-7).
`install()` registers this package's modules under those top-level names.
"""
from __future__ import annotations

import importlib
import sys

_NAMES = ("arch", "utils", "analyze", "roller", "benchmark")


def install(names=_NAMES) -> None:
    for name in names:
        sys.modules.setdefault(name, importlib.import_module(f"{__package__}.{name}"))
