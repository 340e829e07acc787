from .model_config import (ModelConfig, Qwen3Config, ConfigError, read_config_json, write_config_json,
                           FULL_ATTENTION, SLIDING_ATTENTION)
from .engine_config import EngineConfig
