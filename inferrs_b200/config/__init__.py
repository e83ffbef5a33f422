from .base import (Architecture, ConfigError, RawConfig, register_architecture, registered_architectures,
                   resolve_architecture)
from .qwen3 import Qwen3Config
