from .engine_config import EngineConfig
from .model_config import (ConfigError, LayerSpec, LlamaConfig, ModelSpec, PartSpec, RunEntry,
                           read_config_json)
from .registry import (architectures, config_class_for, load_config, load_preset, preset_names,
                       register_architecture)

__all__ = ["EngineConfig", "ConfigError", "LayerSpec", "LlamaConfig", "ModelSpec", "PartSpec", "RunEntry",
           "read_config_json", "architectures", "config_class_for", "load_config", "load_preset", "preset_names", "register_architecture"]
