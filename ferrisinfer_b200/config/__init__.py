"""Typed configurations and the architecture registry."""

from .qwen2 import Qwen2Config, read_config_json
from .registry import (Architecture, get_architecture, register_architecture, registered_architectures,
                       resolve_config)
