from .base import ConfigError, ModelConfig, parse_config_json, read_config_json
from .gekavik import GekavikConfig
from .llama import LlamaConfig, RopeScaling
from .medirax import MediraxConfig

__all__ = ["ConfigError", "ModelConfig", "LlamaConfig", "MediraxConfig", "GekavikConfig", "RopeScaling",
           "parse_config_json", "read_config_json"]
