from .llama import ConfigError, LlamaConfig, read_config_json  # noqa: F401
from .registry import Architecture, architectures, register_architecture, resolve  # noqa: F401
