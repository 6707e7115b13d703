from .base import (ConfigError, ModelConfig, config_from_dict, known_architectures, load_config,
                   lookup_architecture, register_architecture, save_config, unregister_architecture)
from .lfm2 import Lfm2Config, adjusted_ff_dim
