from emberserve_b200.config.engine import EngineConfig, dtype_from_str
from emberserve_b200.config.model import ConfigError, ModelConfig, Qwen2Config, read_config_json

__all__ = ["ConfigError", "EngineConfig", "ModelConfig", "Qwen2Config", "dtype_from_str",
           "read_config_json"]
