from .model_config import ConfigError, Qwen2MoeConfig, read_config_json
from .engine_config import EngineConfig, SamplingParams
from .bizodra_config import BizodraConfig
from .kifunex_config import KifunexConfig
from .registry import (Architecture, register_architecture, get_architecture,
                       known_architectures, load_model_config, architecture_name)

__all__ = ["ConfigError", "Qwen2MoeConfig", "read_config_json", "EngineConfig", "SamplingParams",
           "Architecture", "register_architecture", "get_architecture", "known_architectures",
           "load_model_config", "architecture_name", "BizodraConfig", "KifunexConfig"]
