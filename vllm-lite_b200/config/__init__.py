"""Typed configuration and the architecture registry."""
from .errors import ConfigError, InvalidField, MissingField, UnknownArchitecture  # noqa: F401
from .qwen3 import Qwen3Config, read_config_json  # noqa: F401
from .registry import (ArchitectureEntry, plan_from_config_json, register_architecture,  # noqa: F401
                       registered_architectures, resolve_architecture, unregister_architecture)
from . import qwen3_plan as _qwen3_plan  # noqa: F401  (registers Qwen3ForCausalLM)
