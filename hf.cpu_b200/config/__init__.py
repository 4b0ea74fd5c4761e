from .base import (ConfigError, LayerSpec, ModelConfig, ModelPlan, PartSpec, ScheduleEntry,
                   UnsupportedError)
from .registry import (config_from_dict, config_from_gguf, known_architectures, load_config, register_architecture,
                       unregister_architecture)
from .qwen2 import Qwen2Config
from .manapel import ManapelConfig
from .peludra import PeludraConfig
from .mokisun import MokisunConfig
from .silupel import SilupelConfig

__all__ = ["ConfigError", "UnsupportedError", "ModelConfig", "ModelPlan", "PartSpec", "LayerSpec",
           "ScheduleEntry", "Qwen2Config", "ManapelConfig", "PeludraConfig", "MokisunConfig", "SilupelConfig", "config_from_dict", "config_from_gguf", "load_config",
           "register_architecture", "unregister_architecture", "known_architectures"]
