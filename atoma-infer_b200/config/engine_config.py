"""Engine options, named as the reference's TOML tables name them.

The reference reads one TOML with the tables ``[inference]`` (dtype, device_ids,
model_name, ... backends/vllm/src/config.rs:17-43), ``[cache]`` (block_size,
cache_dtype, gpu_memory_utilization, swap_space_fraction,
num_gpu_blocks_override, :137-159), ``[scheduler]`` (max_num_batched_tokens,
max_num_sequences, max_model_len, delay_factor, enable_chunked_prefill,
:349-365) and ``[validation]`` (:462-473).  The same file is accepted here
(``EngineConfig.from_toml``); options that belong to parts this engine does not
have (swap space, tokenizer workers, the hub) are read and ignored.
"""
from __future__ import annotations

import tomllib
from dataclasses import dataclass, field
from typing import Optional

from .model_config import ConfigError

_DTYPES = {
    "bf16": "bfloat16", "bfloat16": "bfloat16",
    "f32": "float32", "fp32": "float32", "float32": "float32",
}


def canonical_dtype(name: str) -> str:
    try:
        return _DTYPES[name.lower()]
    except KeyError:
        raise ConfigError(f"dtype {name!r} is not supported (known: bfloat16/bf16, float32/f32)") from None


@dataclass
class EngineConfig:
    # [inference]
    dtype: str = "bfloat16"
    device_id: int = 0
    # [cache]
    block_size: int = 16
    gpu_memory_utilization: float = 0.9
    num_gpu_blocks_override: Optional[int] = None
    # [scheduler]
    max_num_batched_tokens: int = 2048
    max_num_sequences: int = 64
    max_model_len: Optional[int] = None  # None: the model's max_position_embeddings
    enable_chunked_prefill: bool = True
    # [validation]
    max_input_length: Optional[int] = None
    max_total_tokens: Optional[int] = None
    # decode steps replay a captured CUDA graph per padded batch size
    cuda_graphs: bool = True
    # random-weights mode: the model folder needs only config.json, tensors are drawn on the device
    random_weights_seed: Optional[int] = None
    random_weights_std: float = 0.02

    def __post_init__(self):
        self.dtype = canonical_dtype(self.dtype)
        self.validate()

    def validate(self) -> None:
        if self.block_size <= 0:
            raise ConfigError("block_size must be positive")
        if not (0.0 < self.gpu_memory_utilization <= 1.0):
            raise ConfigError("gpu_memory_utilization must be in (0, 1]")
        if self.num_gpu_blocks_override is not None and self.num_gpu_blocks_override <= 0:
            raise ConfigError("num_gpu_blocks_override must be positive")
        if self.max_num_sequences <= 0 or self.max_num_batched_tokens <= 0:
            raise ConfigError("max_num_sequences and max_num_batched_tokens must be positive")
        # backends/vllm/src/config.rs:388-405
        if self.max_num_batched_tokens < self.max_num_sequences:
            raise ConfigError(
                f"max_num_batched_tokens ({self.max_num_batched_tokens}) must be at least "
                f"max_num_sequences ({self.max_num_sequences})"
            )
        if (not self.enable_chunked_prefill and self.max_model_len is not None
                and self.max_num_batched_tokens < self.max_model_len):
            raise ConfigError(
                f"max_num_batched_tokens ({self.max_num_batched_tokens}) is smaller than max_model_len "
                f"({self.max_model_len}); without chunked prefill a whole prompt must fit in one step"
            )

    @staticmethod
    def from_toml(path: str) -> "EngineConfig":
        with open(path, "rb") as f:
            doc = tomllib.load(f)
        inf, cache = doc.get("inference", {}), doc.get("cache", {})
        sch, val = doc.get("scheduler", {}), doc.get("validation", {})
        if "block_size" in sch and "block_size" in cache and sch["block_size"] != cache["block_size"]:
            raise ConfigError("[scheduler].block_size and [cache].block_size differ")
        kw = {}
        if "dtype" in inf:
            kw["dtype"] = inf["dtype"]
        if inf.get("device_ids"):
            if len(inf["device_ids"]) != 1:
                raise ConfigError("this engine runs on one GPU; device_ids must name exactly one")
            kw["device_id"] = int(inf["device_ids"][0])
        if "cache_dtype" in cache and "dtype" in inf:
            if canonical_dtype(cache["cache_dtype"]) != canonical_dtype(inf["dtype"]):
                raise ConfigError("cache_dtype must equal the inference dtype (no quantised cache)")
        for src, keys in (
            (cache, ("block_size", "gpu_memory_utilization", "num_gpu_blocks_override")),
            (sch, ("max_num_batched_tokens", "max_num_sequences", "max_model_len", "enable_chunked_prefill")),
            (val, ("max_input_length", "max_total_tokens")),
        ):
            for k in keys:
                if k in src:
                    kw[k] = src[k]
        return EngineConfig(**kw)
