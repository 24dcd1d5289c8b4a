from .base import ConfigError
from .lfm2 import Lfm2Config, adjusted_ffn_dim
from .registry import (Architecture, config_from_dict, get_architecture, load_config, register_architecture,
                       registered_architectures, unregister_architecture)

__all__ = ["ConfigError", "Lfm2Config", "adjusted_ffn_dim", "Architecture", "config_from_dict", "get_architecture",
           "load_config", "register_architecture", "registered_architectures", "unregister_architecture"]
