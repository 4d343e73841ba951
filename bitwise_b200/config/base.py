"""What every architecture's configuration shares: the error type and the reader of
``config.json``.  An architecture's typed configuration lives in a file of its own
(``config/llama.py``) and is found through the registry (``config/registry.py``)."""
from __future__ import annotations

import json
import os


class ConfigError(ValueError):
    """A config.json that cannot describe a runnable model."""


def read_config_json(folder: str) -> dict:
    path = os.path.join(folder, "config.json")
    try:
        with open(path, "r", encoding="utf-8") as f:
            return json.load(f)
    except FileNotFoundError:
        raise ConfigError(f"no config.json in {folder}") from None
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path} is not valid JSON: {e}") from None
