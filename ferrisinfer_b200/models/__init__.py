"""Architectures: one module each, which registers itself (``config.registry.register_architecture``) when imported.

Every module of this package is imported when the registry is first asked, so an architecture is added by
adding its file here (or, from outside the package, by calling ``register_architecture`` directly).
"""

from __future__ import annotations

import importlib
import pkgutil


def import_all() -> list:
    """Import every module of this package; returns their names."""
    names = []
    for info in pkgutil.iter_modules(__path__):
        importlib.import_module(f"{__name__}.{info.name}")
        names.append(info.name)
    return names
