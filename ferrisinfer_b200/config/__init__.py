"""Typed configurations and the architecture registry."""

from .json_file import read_config_json
from .qwen2 import Qwen2Config
from .registry import (Architecture, get_architecture, register_architecture, registered_architectures,
                       resolve_config)
