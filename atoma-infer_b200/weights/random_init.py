"""Random-weights mode: writes a model folder from a configuration and a seed.

The reference has no such mode (its tests download checkpoints,
models/src/llama.rs:529-549).  Every tensor is drawn from its own generator,
seeded by the seed and the tensor's name, so a tensor's values do not depend on
which other tensors exist.  Matrices are N(0, std); norm weights are 1 plus
N(0, norm_jitter) (jitter 0 gives exactly 1); integer tables are a fixed pattern.
"""
from __future__ import annotations

import json
import os
import zlib
from typing import Dict, Mapping, Optional, Sequence

import torch

from .loader import TensorDecl
from .safetensors_io import write_safetensors


def _generator(seed: int, name: str, device="cpu") -> torch.Generator:
    g = torch.Generator(device=device)
    # both halves depend on seed and name (the CPU generator seeds from the low 32 bits alone)
    key = f"{seed}:{name}".encode()
    g.manual_seed((zlib.crc32(key[::-1]) << 32) | zlib.crc32(key))
    return g


def random_tensor(decl: TensorDecl, seed: int, *, std: float, norm_jitter: float,
                  dtype: torch.dtype, scale: float = 1.0, device="cpu") -> torch.Tensor:
    g = _generator(seed, decl.name, device)
    if decl.integer or decl.init == "index":
        n = 1
        for s in decl.shape:
            n *= s
        t = torch.arange(n, dtype=torch.int64, device=device)
        if decl.index_mod:
            t = (t * 7 + 3) % decl.index_mod
        return t.reshape(decl.shape).to(torch.int32)
    if decl.init == "normal":
        t = torch.randn(decl.shape, generator=g, dtype=torch.float32, device=device) * (std * scale)
    elif decl.init == "ones":
        t = torch.ones(decl.shape, dtype=torch.float32, device=device)
        if norm_jitter:
            t = t + torch.randn(decl.shape, generator=g, dtype=torch.float32, device=device) * norm_jitter
    elif decl.init == "zeros":
        t = torch.zeros(decl.shape, dtype=torch.float32, device=device)
    else:
        raise ValueError(f"unknown init {decl.init!r} for {decl.name}")
    return t.to(dtype)


def random_tensors(decls: Sequence[TensorDecl], seed: int, *, std: float = 0.02, norm_jitter: float = 0.0,
                   dtype: torch.dtype = torch.bfloat16, scales: Optional[Mapping[str, float]] = None,
                   device="cpu") -> Dict[str, torch.Tensor]:
    """``scales``: substring of a tensor name -> factor on its std (to make a part stand out)."""
    out = {}
    for d in decls:
        s = 1.0
        for key, f in (scales or {}).items():
            if key in d.name:
                s *= f
        out[d.name] = random_tensor(d, seed, std=std, norm_jitter=norm_jitter, dtype=dtype, scale=s, device=device)
    return out


def write_random_model(model_dir: str, config: dict, seed: int, *, std: float = 0.02,
                       norm_jitter: float = 0.0, dtype: torch.dtype = torch.bfloat16,
                       scales: Optional[Mapping[str, float]] = None, device="cpu") -> str:
    """Writes ``config.json`` and ``model.safetensors`` for the architecture ``config`` names."""
    from ..config.registry import architecture
    from ..parts.model import declared_tensors

    archs = config.get("architectures")
    if not archs:
        raise ValueError("the configuration needs an 'architectures' list to choose the model")
    arch = architecture(archs[0])
    spec = arch.build_spec(arch.parse_config(config))
    decls = declared_tensors(spec)
    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w") as f:
        json.dump(config, f, indent=1)
    tensors = random_tensors(decls, seed, std=std, norm_jitter=norm_jitter, dtype=dtype, scales=scales, device=device)
    write_safetensors(os.path.join(model_dir, "model.safetensors"), tensors,
                      {"format": "pt", "seed": str(seed), "std": str(std)})
    return model_dir
