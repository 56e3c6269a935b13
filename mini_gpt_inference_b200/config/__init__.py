from .engine_config import EngineConfig, SamplingParams, canonical_dtype
from .model_config import ConfigError, GPTConfig, read_config_json
from .registry import (MODEL_REGISTRY, ModelFamily, UnknownArchitectureError, architecture_name,
                       load_config, lookup, register_model)

__all__ = ["EngineConfig", "SamplingParams", "canonical_dtype", "ConfigError", "GPTConfig",
           "read_config_json", "MODEL_REGISTRY", "ModelFamily", "UnknownArchitectureError",
           "architecture_name", "load_config", "lookup", "register_model"]
