"""Rotary position encoding with optional llama3 frequency scaling.

Frequencies as the reference computes them, in float32: 1 / theta^(i/d) for even i
(models/src/llama.rs:146-152); llama3 scaling per frequency by wavelength bands
(:163-185).  The reference tabulates cos and sin for every position in the model
dtype, per layer (:189-198, :348); here the angle position * inv_freq and its cos
and sin are computed in float32 inside the kernel that also writes keys and values
to their pages, so no table exists.  Pairs are (x[i], x[i + rot/2]) (:250).

Parameters: ``head_dim``, ``theta``, ``scaling`` (dict or None), ``rotary_dim``
(defaults to head_dim).  ``kind: "none"`` is the same kernel with zero frequencies.
"""
from __future__ import annotations

import math

import torch

from ..config.registry import register_part
from .base import PositionEncoding


def rotary_inv_freq(head_dim: int, theta: float, scaling=None, rotary_dim=None) -> torch.Tensor:
    rot = rotary_dim or head_dim
    idx = torch.arange(0, rot, 2, dtype=torch.float32)
    freq = 1.0 / torch.pow(torch.tensor(theta, dtype=torch.float32), idx / rot)
    if not scaling or scaling.get("rope_type", "default") == "default":
        return freq
    f32 = lambda v: torch.tensor(float(v), dtype=torch.float32)  # noqa: E731
    factor, low, high = f32(scaling["factor"]), f32(scaling["low_freq_factor"]), f32(scaling["high_freq_factor"])
    orig = f32(scaling["original_max_position_embeddings"])
    wavelen = 2.0 * f32(math.pi) / freq
    smooth = (orig / wavelen - low) / (high - low)
    mid = (1.0 - smooth) * freq / factor + smooth * freq
    out = torch.where(wavelen < orig / high, freq, torch.where(wavelen > orig / low, freq / factor, mid))
    return out.to(torch.float32)


class RotaryEncoding(PositionEncoding):
    def __init__(self, params, prefix):
        super().__init__(params, prefix)
        self.head_dim = int(params["head_dim"])
        self.rotary_dim = int(params.get("rotary_dim") or self.head_dim)
        if self.rotary_dim % 2 or self.rotary_dim > self.head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and at most head_dim {self.head_dim}")
        self.theta = float(params.get("theta", 10000.0))
        self.scaling = params.get("scaling")

    def _frequencies(self):
        return rotary_inv_freq(self.head_dim, self.theta, self.scaling, self.rotary_dim)

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.inv_freq = self._frequencies().to(rt.device).contiguous()

    def rotary(self):
        return self.inv_freq, self.rotary_dim

    def encode_and_store(self, qkv, ctx, cache, *, num_heads, num_kv_heads, head_dim):
        self.rt.ops.rope_kv_store(qkv, ctx.positions, ctx.token_entry, ctx.meta, max(cache.group, 0), self.inv_freq,
                                  cache.pages, cache.num_pages, ctx.T, num_heads, num_kv_heads, head_dim,
                                  self.rotary_dim, cache.page_size, cache.writes and cache.pages is not None)


class NoPositionEncoding(RotaryEncoding):
    """Keys and queries as they are: a rotation by angle zero."""

    def _frequencies(self):
        return torch.zeros(self.rotary_dim // 2, dtype=torch.float32)


register_part("position", "rope", RotaryEncoding)
register_part("position", "none", NoPositionEncoding)
