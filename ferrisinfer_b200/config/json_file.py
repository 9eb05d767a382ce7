"""Reading a config.json into a dict: shared by every architecture's typed configuration and by the registry.

The reference parses config.json with its own JSON reader and treats ``null`` as an absent key
(crates/ferrisinfer-io/src/hf.rs:315-369, 629-680); which keys mean what is the typed configuration's business,
not this file's.
"""

from __future__ import annotations

import json
import os

from ..errors import ConfigError


def read_config_json(path: str) -> dict:
    """Parse ``path`` (a config.json, or a folder holding one) into a dict."""
    if os.path.isdir(path):
        path = os.path.join(path, "config.json")
    try:
        with open(path, "r", encoding="utf-8") as f:
            d = json.load(f)
    except FileNotFoundError:
        raise ConfigError(f"no config.json at {path}") from None
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: top level must be a JSON object")
    return d
