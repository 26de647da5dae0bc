from .model_config import ConfigError, LlamaConfig, RopeScaling
from .engine_config import EngineConfig, canonical_dtype
from .registry import (
    Architecture, architecture, architecture_of, known_architectures,
    part_class, register_architecture, register_part,
)
