from .base import ConfigError, ModelConfig, read_config_json
from .qwen3 import Qwen3Config
from .resolorn import ResolornConfig

__all__ = ["ConfigError", "ModelConfig", "Qwen3Config", "ResolornConfig", "read_config_json"]
