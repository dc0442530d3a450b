from .errors import ConfigError, MissingKey, InvalidValue, UnknownArchitecture
from .qwen3 import Qwen3Config
from .registry import (Architecture, register_architecture, unregister_architecture,
                       registered_architectures, resolve_architecture, architecture_name,
                       load_config, resolve_eos)

__all__ = ["ConfigError", "MissingKey", "InvalidValue", "UnknownArchitecture", "Qwen3Config",
           "Architecture", "register_architecture", "unregister_architecture",
           "registered_architectures", "resolve_architecture", "architecture_name",
           "load_config", "resolve_eos"]
