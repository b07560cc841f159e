from .engine_config import Config
from .model_config import ConfigError, ModelConfig, parse_dtype, read_config_json
from .registry import ARCHITECTURES, ArchitectureEntry, load_model_config, register_architecture

__all__ = ["Config", "ConfigError", "ModelConfig", "parse_dtype", "read_config_json",
           "ARCHITECTURES", "ArchitectureEntry", "load_model_config", "register_architecture"]
