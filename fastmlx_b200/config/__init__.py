from .base import ConfigError, ModelConfig, parse_config_json, read_config_json
from .llama import LlamaConfig, RopeScaling
from .medirax import MediraxConfig

__all__ = ["ConfigError", "ModelConfig", "LlamaConfig", "MediraxConfig", "RopeScaling",
           "parse_config_json", "read_config_json"]
