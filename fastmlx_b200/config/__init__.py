from .base import ConfigError, ModelConfig, parse_config_json, read_config_json
from .gekavik import GekavikConfig
from .kafepel import KafepelConfig
from .llama import LlamaConfig, RopeScaling
from .medirax import MediraxConfig
from .sorupel import SorupelConfig

__all__ = ["ConfigError", "ModelConfig", "LlamaConfig", "MediraxConfig", "GekavikConfig", "SorupelConfig", "KafepelConfig", "RopeScaling",
           "parse_config_json", "read_config_json"]
