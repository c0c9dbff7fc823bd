"""Host backend of the B200 MegaMoE expert layer (heuristics, workspace, weights, staging, launch sequence).
Sub-modules are imported on first use so that importing the package needs neither torch nor a GPU."""

import importlib
from typing import Any

_SUBMODULES = ("heuristics", "workspace", "weights", "staging", "frontend", "locality", "_native")


def __getattr__(name: str) -> Any:
    if name in _SUBMODULES:
        return importlib.import_module(f"{__name__}.{name}")
    raise AttributeError(name)
