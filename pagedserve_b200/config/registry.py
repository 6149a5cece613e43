"""Architecture registry: config.json -> (typed config class, model spec builder).

The reference selects a model with a string switch over three names
(reference: main.py:22-25, 97-133).  Here one table maps the architecture
name found in ``config.json`` (``architectures[0]``, falling back to
``model_type``) to a typed configuration class and to a function that turns
that configuration into a :class:`pagedserve_b200.models.spec.ModelSpec`.
Adding an architecture is one ``register_architecture`` call; nothing else in
the engine names a model.
"""

from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Callable, Dict, Optional, Tuple


class ConfigError(ValueError):
    """A config.json that is missing, malformed or asks for unsupported math."""


@dataclass
class ModelConfig:
    """Base of every typed model configuration.

    Subclasses declare the architecture's own ``config.json`` keys as fields
    and implement :meth:`from_dict` / :meth:`to_dict`.  The engine itself only
    needs the three properties below.
    """

    @classmethod
    def from_dict(cls, values: dict) -> "ModelConfig":  # pragma: no cover - abstract
        raise NotImplementedError

    def to_dict(self) -> dict:  # pragma: no cover - abstract
        raise NotImplementedError

    @property
    def architecture(self) -> str:  # pragma: no cover - abstract
        raise NotImplementedError

    @property
    def vocabulary_size(self) -> int:  # pragma: no cover - abstract
        raise NotImplementedError

    @property
    def max_model_len(self) -> int:  # pragma: no cover - abstract
        """Longest sequence (prompt + generated) a request may reach."""
        raise NotImplementedError


# name -> (config class, builder(config) -> ModelSpec)
_ARCHITECTURES: Dict[str, Tuple[type, Callable]] = {}
# model_type -> architecture name (fallback when "architectures" is absent)
_MODEL_TYPES: Dict[str, str] = {}


def register_architecture(
    name: str,
    config_class: type,
    builder: Callable,
    model_type: Optional[str] = None,
    replace: bool = False,
) -> None:
    """Register ``name`` (as written in ``config.json``'s ``architectures``)."""
    if name in _ARCHITECTURES and not replace:
        raise ConfigError(f"architecture {name!r} is already registered")
    _ARCHITECTURES[name] = (config_class, builder)
    if model_type is not None:
        _MODEL_TYPES[model_type] = name


def architecture_names():
    _ensure_builtin()
    return sorted(_ARCHITECTURES)


def _ensure_builtin() -> None:
    # Importing the models package registers the built-in architecture(s).
    import pagedserve_b200.models  # noqa: F401


def resolve_architecture(values: dict) -> Tuple[str, type, Callable]:
    """Pick the registered architecture for a parsed ``config.json``."""
    _ensure_builtin()
    name = None
    architectures = values.get("architectures")
    if isinstance(architectures, (list, tuple)) and architectures:
        name = architectures[0]
    elif isinstance(architectures, str):
        name = architectures
    if name is None:
        model_type = values.get("model_type")
        if model_type in _MODEL_TYPES:
            name = _MODEL_TYPES[model_type]
    if name is None:
        raise ConfigError(
            "config.json names no architecture: expected \"architectures\": [name] "
            f"or a known \"model_type\"; registered: {sorted(_ARCHITECTURES)}"
        )
    if name not in _ARCHITECTURES:
        raise ConfigError(
            f"unknown architecture {name!r}; registered: {sorted(_ARCHITECTURES)}"
        )
    config_class, builder = _ARCHITECTURES[name]
    return name, config_class, builder


def load_config_dict(folder: str) -> dict:
    path = os.path.join(folder, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"no config.json in {folder!r}")
    with open(path, "r", encoding="utf-8") as handle:
        try:
            values = json.load(handle)
        except json.JSONDecodeError as error:
            raise ConfigError(f"{path}: not valid JSON ({error})") from error
    if not isinstance(values, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return values


def load_model_config(folder: str) -> ModelConfig:
    """Read ``folder/config.json`` into the typed config of its architecture."""
    values = load_config_dict(folder)
    _, config_class, _ = resolve_architecture(values)
    return config_class.from_dict(values)
