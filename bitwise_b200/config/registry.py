"""One registry from the architecture's name to its configuration type and model.

The reference keeps this table in its converter (tools/convert.py:29,56-58:
``ARCHS = {"LlamaForCausalLM": "llama", ...}``, anything else is refused).  Here an
entry names the typed configuration and a function that assembles the model from
parts; the same lookup serves loading, random weights, replay and generation.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict

from .base import ConfigError, read_config_json


@dataclass(frozen=True)
class Architecture:
    name: str
    config_from_json: Callable[[dict], object]
    # build(config, dtype, device) -> models.decoder.DecoderModel (weights not yet loaded)
    build: Callable[..., object]


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, config_from_json, build) -> None:
    """Add (or replace) an architecture; ``name`` is config.json's ``architectures[0]``."""
    _ARCHITECTURES[name] = Architecture(name, config_from_json, build)


def known_architectures():
    _ensure_builtin()
    return sorted(_ARCHITECTURES)


def lookup_architecture(name: str) -> Architecture:
    _ensure_builtin()
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(
            f"unsupported architecture {name!r}; known: {', '.join(sorted(_ARCHITECTURES))}"
        ) from None


def architecture_of(config_json: dict) -> Architecture:
    archs = config_json.get("architectures")
    if not archs:
        raise ConfigError("config.json has no 'architectures' entry")
    return lookup_architecture(archs[0])


def config_from_folder(folder: str):
    """Read ``folder/config.json`` and return (Architecture, typed config)."""
    raw = read_config_json(folder)
    arch = architecture_of(raw)
    return arch, arch.config_from_json(raw)


def _ensure_builtin() -> None:
    if "LlamaForCausalLM" not in _ARCHITECTURES:
        from ..models import llama  # noqa: F401  (registers itself on import)
