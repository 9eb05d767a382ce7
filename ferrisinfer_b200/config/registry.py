"""One registry from an architecture's name to its configuration class and model plan.

The reference has no registry: it matches ``model_type`` in two places and
rejects everything but "qwen2" (crates/ferrisinfer-io/src/hf.rs:306-313,
371-378, 502-510).  Here ``architectures[0]`` of config.json selects an entry;
an entry gives the typed configuration class (``from_dict`` / ``to_dict``) and a
function from a configuration to a ``ModelPlan`` (the description of layers,
parts and run order that ``parts.model.build_model`` turns into a model).

Adding an architecture = writing its configuration class and its plan function
and calling ``register_architecture`` once; nothing else in the package names
an architecture.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable

from ..errors import ConfigError, UnsupportedError
from .json_file import read_config_json


@dataclass(frozen=True)
class Architecture:
    name: str
    config_cls: Any  # has from_dict(dict) -> config and config.to_dict() -> dict
    plan: Callable[[Any], Any]  # config -> parts.plan.ModelPlan


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(name: str, config_cls, plan: Callable, *, replace: bool = False) -> None:
    if name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture '{name}' is already registered")
    _ARCHITECTURES[name] = Architecture(name, config_cls, plan)


def registered_architectures() -> list[str]:
    _ensure_builtin()
    return sorted(_ARCHITECTURES)


def get_architecture(name: str) -> Architecture:
    _ensure_builtin()
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise UnsupportedError(
            f"architecture '{name}' is not registered (registered: {', '.join(sorted(_ARCHITECTURES))})"
        ) from None


def architecture_name_of(config_dict: dict) -> str:
    archs = config_dict.get("architectures")
    if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
        raise ConfigError("config.json: 'architectures' must be a non-empty list of strings")
    return archs[0]


def resolve_config(source) -> tuple[Architecture, Any]:
    """``source`` is a model folder, a config.json path, a dict, or a typed config."""
    if isinstance(source, (str, bytes)) or hasattr(source, "__fspath__"):
        source = read_config_json(source)
    if isinstance(source, dict):
        arch = get_architecture(architecture_name_of(source))
        return arch, arch.config_cls.from_dict(source)
    name = getattr(source, "architecture", None)
    if name is None:
        raise ConfigError(f"cannot tell the architecture of {type(source).__name__}")
    return get_architecture(name), source


def _ensure_builtin() -> None:
    # the architectures that come with the package register themselves on import
    from .. import models

    models.import_all()
