"""Optional dependencies of the adapters, and one error type that names the missing one.

Same role as the reference's python/nanochat_cpp_bridge/_extras.py: a feature asks for its package by name at the
point of use; a missing package becomes a `MissingExtra` that says which feature group it belongs to.
"""
from __future__ import annotations

import importlib
from typing import Any

# package -> feature group (the names a user would look for in an install command)
EXTRAS = {
    "huggingface_hub": "hub",
    "safetensors": "hub",
    "pyarrow": "hfdata",
    "filelock": "hfdata",
    "numpy": "hfdata",
    "tiktoken": "tiktoken",
    "torch": "torch",
}


class MissingExtra(RuntimeError):
    """An optional package is not installed; `.package` and `.extra` say which."""

    def __init__(self, package: str, detail: str = ""):
        self.package = package
        self.extra = EXTRAS.get(package, package)
        msg = f"this call needs the optional package '{package}' (feature group '{self.extra}')"
        super().__init__(msg + (": " + detail if detail else ""))


def need(package: str, detail: str = "") -> Any:
    """Import `package` or raise MissingExtra."""
    try:
        return importlib.import_module(package)
    except ImportError as e:
        raise MissingExtra(package, detail or str(e)) from e
