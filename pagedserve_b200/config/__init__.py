"""Typed configuration and the architecture registry."""

from pagedserve_b200.config.registry import (  # noqa: F401
    ConfigError,
    ModelConfig,
    architecture_names,
    load_config_dict,
    load_model_config,
    register_architecture,
    resolve_architecture,
)
from pagedserve_b200.config.engine_config import EngineConfig  # noqa: F401
from pagedserve_b200.config.gpt2 import GPT2Config  # noqa: F401
