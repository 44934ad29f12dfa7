from .base import ConfigError, ModelConfig, load_config_dict
from .engine_config import EngineConfig
from .qwen3 import Qwen3Config
from .rimopel import RimopelConfig
from .nagavik import NagavikConfig
from .fifudra import FifudraConfig
from .mefupel import MefupelConfig

__all__ = ["ConfigError", "ModelConfig", "EngineConfig", "Qwen3Config", "RimopelConfig", "NagavikConfig", "FifudraConfig", "MefupelConfig", "load_config_dict"]
