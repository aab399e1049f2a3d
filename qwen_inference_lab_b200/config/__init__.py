from .model_config import ConfigError, GogotarConfig, LarolornConfig, Qwen3Config, VirulixConfig, read_config_json
from .registry import Architecture, known, lookup, read_model_config, register, unregister
