from .base import (ConfigError, ModelConfig, config_class, config_from_dict, known_architectures,
                   load_config, register_config, save_config)
from .opt import OptConfig, opt_preset

__all__ = ["ConfigError", "ModelConfig", "OptConfig", "config_class", "config_from_dict",
           "known_architectures", "load_config", "opt_preset", "register_config", "save_config"]
