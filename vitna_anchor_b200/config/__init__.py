from .errors import ConfigError  # noqa: F401
from .llama import LlamaConfig, read_config_json  # noqa: F401
from .registry import Architecture, architectures, register_architecture, resolve  # noqa: F401
