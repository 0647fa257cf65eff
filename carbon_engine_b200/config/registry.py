"""The one registry from an architecture's name to its configuration class and model builder.

The reference picks the model by ``model_type`` (src/config.rs:457-467) and lists the supported
names in its error.  Here the first entry of ``architectures`` decides, ``model_type`` is the
fallback, and the error lists what is registered.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Iterable, List, Optional

from .base import ConfigError, ModelConfig, read_config_dict


@dataclass(frozen=True)
class Architecture:
    name: str
    parse_config: Callable[[Dict[str, Any]], ModelConfig]
    build_model: Callable[..., Any]          # (config, dtype) -> DecoderModel
    model_types: tuple = ()


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, parse_config: Callable[[Dict[str, Any]], ModelConfig],
                          build_model: Callable[..., Any], model_types: Iterable[str] = (),
                          replace: bool = False) -> None:
    if name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture '{name}' is already registered")
    _ARCHITECTURES[name] = Architecture(name, parse_config, build_model, tuple(model_types))


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def registered_architectures() -> List[str]:
    return sorted(_ARCHITECTURES)


def resolve_architecture(raw: Dict[str, Any]) -> Architecture:
    names = raw.get("architectures")
    if isinstance(names, list):
        for n in names:
            if n in _ARCHITECTURES:
                return _ARCHITECTURES[n]
    model_type = raw.get("model_type")
    for arch in _ARCHITECTURES.values():
        if model_type is not None and model_type in arch.model_types:
            return arch
    asked = names if names else model_type
    raise ConfigError(
        f"unsupported architecture {asked!r} (registered: {', '.join(registered_architectures())})")


def load_config(model_dir: str, overrides: Optional[Dict[str, Any]] = None):
    """(architecture entry, typed config) of a model folder."""
    raw = read_config_dict(model_dir, overrides)
    arch = resolve_architecture(raw)
    return arch, arch.parse_config(raw)
