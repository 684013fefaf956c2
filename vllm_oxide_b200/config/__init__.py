from .model_config import ConfigError, Qwen3Config, read_config_json, write_config_json
from .engine_options import EngineOptions

__all__ = ["ConfigError", "Qwen3Config", "EngineOptions", "read_config_json", "write_config_json"]
