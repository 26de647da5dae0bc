"""A small, whole, single-GPU inference engine for NVIDIA B200 (sm_100a).

Folders: ``config`` (typed model and engine configuration, registries), ``weights``
(safetensors by tensor name, random-weights mode), ``parts`` (mixer, feed-forward,
norm, position encoding, block; the model as a list of layers), ``models`` (the
architectures built from the parts), ``cache`` (paged keys and values, block
tables, state slots), ``engine`` (step function, scheduler, generation, trace
replay), ``sampling``, ``csrc`` (CUDA kernels and the native host library).
"""
__version__ = "0.1.0"

from .config import ConfigError, EngineConfig, LlamaConfig  # noqa: F401
from . import models  # noqa: F401,E402  (registers the architectures)
