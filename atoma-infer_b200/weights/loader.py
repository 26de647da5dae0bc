"""Loading a model's tensors by name, with one error for everything that is wrong.

Each part of a model declares the checkpoint tensors it needs (``TensorDecl``:
name, shape, how to fill it in random mode).  ``load_tensors`` matches the
declarations against the files of a model folder and raises a single
``WeightError`` that lists every missing tensor, every tensor nobody asked for and
every wrong shape or dtype class; the reference surfaces these one at a time, or
panics inside the per-layer ``unwrap`` (models/src/llama.rs:488-490).

Stored dtypes: floating tensors stored in 16 bits are kept as bfloat16 and tensors
stored in 32 bits stay 32-bit when the engine runs in bfloat16; in float32 mode
every floating tensor is widened (exactly) to float32.  Integer tables become int32.
"""
from __future__ import annotations

import fnmatch
from dataclasses import dataclass
from typing import Callable, Dict, Iterable, List, Sequence, Tuple

import torch

from .safetensors_io import SafetensorsFile, open_model_files


class WeightError(ValueError):
    """Lists missing, unexpected and ill-shaped tensors of a checkpoint."""

    def __init__(self, model_dir, missing, unexpected, wrong):
        self.missing, self.unexpected, self.wrong = list(missing), list(unexpected), list(wrong)
        lines = [f"checkpoint {model_dir!r} does not fit the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}):")
            lines += [f"    {n}  expected shape {list(s)}" for n, s in self.missing]
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}):")
            lines += [f"    {n}  shape {list(s)}" for n, s in self.unexpected]
        if self.wrong:
            lines.append(f"  wrong shape or dtype ({len(self.wrong)}):")
            lines += [f"    {n}  {why}" for n, why in self.wrong]
        super().__init__("\n".join(lines))


@dataclass(frozen=True)
class TensorDecl:
    """One checkpoint tensor a part needs.

    init: 'normal' (N(0, std)), 'ones' (1 + N(0, jitter)), 'zeros', or 'index'
    (an integer table filled with arange modulo ``index_mod``).
    """

    name: str
    shape: Tuple[int, ...]
    init: str = "normal"
    integer: bool = False
    index_mod: int = 0


def _target_dtype(stored: torch.dtype, mode: torch.dtype, integer: bool) -> torch.dtype:
    if integer:
        return torch.int32
    if mode == torch.float32:
        return torch.float32
    if stored in (torch.float32, torch.float64):
        return torch.float32
    return torch.bfloat16


def load_tensors(
    model_dir: str,
    decls: Sequence[TensorDecl],
    *,
    dtype: torch.dtype,
    device,
    ignore: Iterable[str] = (),
) -> Dict[str, torch.Tensor]:
    """Returns name -> device tensor for every declaration, or raises ``WeightError``.

    ``ignore``: glob patterns of tensor names a checkpoint may carry without use
    (a stored ``lm_head.weight`` beside tied embeddings, rotary frequency buffers).
    """
    files = open_model_files(model_dir)
    where: Dict[str, SafetensorsFile] = {}
    for f in files:
        for n in f.names():
            where[n] = f
    wanted = {d.name: d for d in decls}
    if len(wanted) != len(decls):
        seen, dup = set(), []
        for d in decls:
            if d.name in seen:
                dup.append(d.name)
            seen.add(d.name)
        raise ValueError(f"parts declare the same tensor twice: {dup}")
    missing = [(d.name, d.shape) for d in decls if d.name not in where]
    unexpected = [
        (n, where[n].shape(n)) for n in sorted(where)
        if n not in wanted and not any(fnmatch.fnmatch(n, pat) for pat in ignore)
    ]
    wrong = []
    for d in decls:
        f = where.get(d.name)
        if f is None:
            continue
        if tuple(f.shape(d.name)) != tuple(d.shape):
            wrong.append((d.name, f"expected shape {list(d.shape)}, found {list(f.shape(d.name))}"))
        elif d.integer == f.dtype(d.name).is_floating_point:
            kind = "an integer table" if d.integer else "a floating tensor"
            wrong.append((d.name, f"expected {kind}, found dtype {f.dtype(d.name)}"))
    if missing or unexpected or wrong:
        raise WeightError(model_dir, missing, unexpected, wrong)
    out = {}
    for d in decls:
        f = where[d.name]
        t = f.tensor(d.name)
        out[d.name] = t.to(device=device, dtype=_target_dtype(t.dtype, dtype, d.integer)).contiguous()
    return out
