from .base import ConfigError, ConfigReader, architecture_name, read_config_json
from .qwen3 import Qwen3Config

__all__ = ["ConfigError", "ConfigReader", "architecture_name", "read_config_json", "Qwen3Config"]
