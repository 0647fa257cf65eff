"""Reading a model folder's config.json, merging overrides, and the base class of typed configs.

Behaviour follows the reference's loader (src/config.rs:416-444): config.json is parsed, an
optional overrides object is merged in (src/config.rs:275-293: sections whose key ends in
``_config`` merge key by key, every other value is replaced whole), quantised checkpoints are
refused, and generation_config.json contributes further end-of-sequence ids.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field, fields
from typing import Any, Dict, List, Optional


class ConfigError(ValueError):
    """A config.json that cannot be turned into a model."""


def merge_overrides(config: Dict[str, Any], overrides: Optional[Dict[str, Any]]) -> Dict[str, Any]:
    """Return ``config`` with ``overrides`` applied (src/config.rs:275-293)."""
    if overrides is None:
        return dict(config)
    if not isinstance(overrides, dict):
        raise ConfigError("--hf-overrides must be a JSON object")
    out = dict(config)
    for key, value in overrides.items():
        section = out.get(key)
        if key.endswith("_config") and isinstance(section, dict) and isinstance(value, dict):
            out[key] = merge_overrides(section, value)
        else:
            out[key] = value
    return out


def token_id_list(value: Any) -> List[int]:
    """A token id given as a number or a list of numbers (src/config.rs:261-271)."""
    if isinstance(value, bool):
        return []
    if isinstance(value, int) and value >= 0:
        return [int(value)]
    if isinstance(value, list):
        return [int(v) for v in value if isinstance(v, int) and not isinstance(v, bool) and v >= 0]
    return []


def read_config_dict(model_dir: str, overrides: Optional[Dict[str, Any]] = None) -> Dict[str, Any]:
    """config.json of ``model_dir`` as a dict, overrides merged, EOS ids of generation_config.json
    appended under the private key ``_generation_eos_token_ids``."""
    path = os.path.join(model_dir, "config.json")
    try:
        with open(path, "r", encoding="utf-8") as fh:
            raw = json.load(fh)
    except FileNotFoundError:
        raise ConfigError(f"no config.json in {model_dir}") from None
    except json.JSONDecodeError as exc:
        raise ConfigError(f"{path}: not valid JSON ({exc})") from None
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: config.json is not an object")
    raw = merge_overrides(raw, overrides)
    gen_path = os.path.join(model_dir, "generation_config.json")
    extra: List[int] = []
    if os.path.exists(gen_path):
        try:
            with open(gen_path, "r", encoding="utf-8") as fh:
                gen = json.load(fh)
            extra = token_id_list(gen.get("eos_token_id")) if isinstance(gen, dict) else []
        except (OSError, json.JSONDecodeError):
            extra = []
    raw["_generation_eos_token_ids"] = extra
    return raw


@dataclass(frozen=True)
class ModelConfig:
    """What every architecture's typed config offers to the engine.

    Subclasses add the architecture's own keys. The engine itself reads only these.
    """

    architecture: str
    vocab_size: int
    max_position_embeddings: int
    eos_token_ids: tuple = field(default_factory=tuple)

    def to_json_dict(self) -> Dict[str, Any]:
        """The config.json this configuration would be read back from."""
        raise NotImplementedError

    def describe(self) -> Dict[str, Any]:
        return {f.name: getattr(self, f.name) for f in fields(self)}
