"""Putting a model on the device: configuration, weights, cache, step function.

Start-up order as in the reference (backends/vllm/src/llm_service.rs:102-260): read
the configuration, load the weights, then size the cache from the memory that is
left (backends/vllm/src/config.rs:626-641) unless a page count is given, then build
the worker's cache and the block manager over the same geometry.
"""
from __future__ import annotations

import sys
from dataclasses import dataclass
from typing import Optional

import torch

from ..cache.kv_cache import KVCache, pages_for_memory, state_bytes_total
from ..cache.manager import CacheManager
from ..config.engine_config import canonical_dtype
from ..config.registry import architecture_of
from ..csrc.ops import CudaOps
from ..parts.base import Runtime
from ..parts.model import DecoderModel
from ..weights.loader import load_tensors
from ..weights.random_init import random_tensors
from .step import StepFunction

_TORCH_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


@dataclass
class LoadedModel:
    config: object
    model: DecoderModel
    rt: Runtime
    manager: CacheManager
    cache: KVCache
    step: StepFunction
    page_size: int
    num_pages: int  # usable pages per pool
    memory: Optional[dict] = None  # how the pools were sized from free memory (None: a page count was given)


def make_runtime(dtype: str, device=None, ops=None) -> Runtime:
    tdtype = _TORCH_DTYPES[canonical_dtype(dtype)]
    device = torch.device(device if device is not None else "cuda:0")
    if tdtype == torch.float32:
        # the 32-bit path is true float32 wherever a library product is used
        torch.backends.cuda.matmul.allow_tf32 = False
        torch.backends.cudnn.allow_tf32 = False
    return Runtime(device=device, dtype=tdtype, ops=ops if ops is not None else CudaOps(device))


def step_workspace_bytes(model: DecoderModel, dtype: torch.dtype, max_batched_tokens: int, max_seqs: int) -> int:
    """An upper estimate of what a step allocates besides the cache: per token the float32 residual stream and
    some ten rows of the widest activation any part says it makes (intermediate results live one or two at a
    time), and the float32 logits of one row per request; twice over, because captured decode graphs keep a
    pool of their own."""
    elem = torch.empty((), dtype=dtype).element_size()
    spec = model.spec
    widest = max([spec.hidden_size] + [blk.activation_width() for blk in model.blocks])
    per_token = 4 * spec.hidden_size + 10 * widest * elem
    return 2 * (max_batched_tokens * per_token + max(max_seqs, 1) * spec.vocab_size * 4)


def load_model(model_dir: str, *, dtype: str = "bfloat16", device=None, page_size: int = 16,
               num_pages: Optional[int] = None, max_seqs: int = 64, gpu_memory_utilization: float = 0.9,
               poison_cache: bool = False, ops=None, cuda_graphs: bool = False,
               max_model_len: Optional[int] = None, max_batched_tokens: int = 2048,
               random_weights_seed: Optional[int] = None, random_weights_std: float = 0.02) -> LoadedModel:
    """``num_pages``: usable pages per pool; None sizes the pools from free device memory, leaving room for
    the state slots of ``max_seqs`` requests and for the working memory of a step of ``max_batched_tokens``.
    ``random_weights_seed``: the folder needs only its config.json; every tensor the model declares is drawn on
    the device from that seed (what ``write_random_model`` draws on the same device with it)."""
    arch, config = architecture_of(model_dir)
    spec = arch.build_spec(config)
    model = DecoderModel(spec)
    rt = make_runtime(dtype, device, ops)
    if random_weights_seed is None:
        tensors = load_tensors(model_dir, model.declare(), dtype=rt.dtype, device=rt.device, ignore=spec.ignored_tensors)
    else:
        tensors = random_tensors(model.declare(), random_weights_seed, std=random_weights_std, dtype=rt.dtype,
                                 device=rt.device)
    model.bind(tensors, rt)
    del tensors
    groups = model.groups
    memory = None
    if num_pages is None:
        free, total = torch.cuda.mem_get_info(rt.device)
        state = state_bytes_total(model, max_seqs)
        work = step_workspace_bytes(model, rt.dtype, max_batched_tokens, max_seqs)
        pages, budget = pages_for_memory(groups, page_size, rt.dtype, free, gpu_memory_utilization, state, work)
        num_pages = pages - 1  # page 0 of a pool is never handed out
        memory = {"free": free, "total": total, "utilization": gpu_memory_utilization, "state_bytes": state,
                  "workspace_bytes": work, "budget": budget, "pages": num_pages}
        if num_pages <= 0:
            raise RuntimeError(f"no device memory is left for the cache after loading the weights ({memory})")
    for g in groups:
        g.num_pages = num_pages + 1  # page 0 is never handed out
    manager = CacheManager(page_size, groups, max_seqs)
    cache = KVCache(model, groups, page_size, max_seqs, rt, poison=poison_cache)
    limit = min(max_model_len or spec.max_position or 1 << 30, num_pages * page_size)
    step = StepFunction(model, cache, manager, rt, cuda_graphs=cuda_graphs, max_model_len=limit)
    return LoadedModel(config, model, rt, manager, cache, step, page_size, num_pages, memory)
