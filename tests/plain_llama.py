"""A plain, slow Llama: whole sequences, no cache, no batching, one function a part.

It rests on the reference's formulas (AtomaAI/atoma-infer, file:line beside each
function), not on its code being run: the reference is Rust on candle with CUDA-only
attention (csrc/src/lib.rs:350-360) and there is no Rust toolchain or GPU where
these tests are written, so no output of the reference could be recorded.  Two
literal vectors that the reference's own tests carry are checked in
test_plain.py instead.

It shares no code with the engine: configuration is a plain dict (the keys of
config.json), weights a dict of tensors by checkpoint name, everything is done in
the dtype of ``compute`` (float64 by default, so it serves as the truth for both
the 32-bit and the bfloat16 engine).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import torch


def head_dim_of(cfg: dict) -> int:
    # models/src/llama.rs:147, :326 — hidden_size / num_attention_heads
    return cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"]


def rope_inv_freq(cfg: dict) -> torch.Tensor:
    """Rotation frequencies in float32, as the reference computes them.

    Default: 1 / theta^(i/d) for even i (models/src/llama.rs:146-152).  llama3
    scaling per frequency (:163-185): wavelengths shorter than orig/high stay,
    longer than orig/low are divided by factor, between them interpolated.
    """
    d = head_dim_of(cfg)
    theta = torch.tensor(float(cfg.get("rope_theta") or 10000.0), dtype=torch.float32)
    idx = torch.arange(0, d, 2, dtype=torch.float32)
    freq = 1.0 / torch.pow(theta, idx / d)  # f32 powf, f32 divide
    sc = cfg.get("rope_scaling")
    if not sc or sc.get("rope_type", sc.get("type")) == "default":
        return freq
    f32 = lambda v: torch.tensor(float(v), dtype=torch.float32)  # noqa: E731
    factor, low, high = f32(sc["factor"]), f32(sc["low_freq_factor"]), f32(sc["high_freq_factor"])
    orig = f32(sc["original_max_position_embeddings"])
    low_wavelen, high_wavelen = orig / low, orig / high
    out = []
    for f in freq:
        wavelen = 2.0 * f32(math.pi) / f
        if wavelen < high_wavelen:
            out.append(f)
        elif wavelen > low_wavelen:
            out.append(f / factor)
        else:
            smooth = (orig / wavelen - low) / (high - low)
            out.append((1.0 - smooth) * f / factor + smooth * f)
    return torch.stack(out)


def rope(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """Half-split rotation of x [T, heads, d] (models/src/llama.rs:189-198, :250).

    angle[p, i] = p * inv_freq[i] in float32 (:189-194, a float32 matmul); pairs are
    (x[i], x[i + d/2]) — candle's non-interleaved ``rope``.
    """
    d = x.shape[-1]
    ang = positions.to(torch.float32)[:, None] * inv_freq.to(torch.float32)[None, :]  # f32 product
    cos, sin = ang.cos().to(x.dtype)[:, None, :], ang.sin().to(x.dtype)[:, None, :]
    x1, x2 = x[..., : d // 2], x[..., d // 2:]
    return torch.cat([x1 * cos - x2 * sin, x1 * sin + x2 * cos], dim=-1)


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x * rsqrt(mean(x^2) + eps) * w  (candle RmsNorm, used at models/src/llama.rs:402, 408, 474)."""
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                     window: Optional[int] = None) -> torch.Tensor:
    """q [T, nq, d], k/v [T, nkv, d] -> [T, nq, d].

    Query head h reads key/value head h // (nq/nkv) (csrc/kernels/flash_fwd_kernel.h:153,
    159).  Scores scale*q.k for keys at or before the query (csrc/kernels/mask.h:172-173),
    softmax, weighted sum of values (csrc/kernels/softmax.h:136-166).  ``window`` keeps
    the last ``window`` keys, the query's own included (not used by Llama).
    """
    T, nq, d = q.shape
    nkv = k.shape[1]
    g = nq // nkv
    kk = k.repeat_interleave(g, dim=1)
    vv = v.repeat_interleave(g, dim=1)
    s = torch.einsum("thd,shd->hts", q, kk) * scale
    i = torch.arange(T)
    mask = i[None, :] > i[:, None]
    if window is not None:
        mask = mask | (i[:, None] - i[None, :] >= window)
    s = s.masked_fill(mask[None], float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.einsum("hts,shd->thd", p, vv)


def attention_block(x, positions, w: Dict[str, torch.Tensor], prefix: str, cfg: dict) -> torch.Tensor:
    """q,k,v projections, rotation of q and k, attention, output projection
    (models/src/llama.rs:269-311); no biases (:3)."""
    nq, nkv, d = cfg["num_attention_heads"], cfg.get("num_key_value_heads") or cfg["num_attention_heads"], head_dim_of(cfg)
    T = x.shape[0]
    q = (x @ w[prefix + "q_proj.weight"].T).reshape(T, nq, d)
    k = (x @ w[prefix + "k_proj.weight"].T).reshape(T, nkv, d)
    v = (x @ w[prefix + "v_proj.weight"].T).reshape(T, nkv, d)
    inv_freq = rope_inv_freq(cfg)
    q, k = rope(q, positions, inv_freq), rope(k, positions, inv_freq)
    o = causal_attention(q, k, v, 1.0 / math.sqrt(d))  # scale: models/src/llama.rs:342
    return o.reshape(T, nq * d) @ w[prefix + "o_proj.weight"].T


def swiglu(x, w: Dict[str, torch.Tensor], prefix: str) -> torch.Tensor:
    """down(silu(gate(x)) * up(x))  (models/src/llama.rs:362-366)."""
    g = x @ w[prefix + "gate_proj.weight"].T
    u = x @ w[prefix + "up_proj.weight"].T
    return (g * torch.sigmoid(g) * u) @ w[prefix + "down_proj.weight"].T


def decoder_block(x, positions, w, i: int, cfg: dict) -> torch.Tensor:
    """h = x + attn(norm1(x)); out = h + mlp(norm2(h))  (models/src/llama.rs:393-410)."""
    p = f"model.layers.{i}."
    eps = cfg["rms_norm_eps"]
    h = x + attention_block(rms_norm(x, w[p + "input_layernorm.weight"], eps), positions, w, p + "self_attn.", cfg)
    return h + swiglu(rms_norm(h, w[p + "post_attention_layernorm.weight"], eps), w, p + "mlp.")


def forward(w: Dict[str, torch.Tensor], cfg: dict, tokens: Sequence[int], compute=torch.float64) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence (models/src/llama.rs:456-478):
    embedding, the blocks, final norm, output head (the embedding matrix when tied, :482-486)."""
    w = {k: v.to(compute) for k, v in w.items()}
    ids = torch.as_tensor(list(tokens), dtype=torch.long)
    positions = torch.arange(len(ids))
    x = w["model.embed_tokens.weight"][ids]
    for i in range(cfg["num_hidden_layers"]):
        x = decoder_block(x, positions, w, i, cfg)
    x = rms_norm(x, w["model.norm.weight"], cfg["rms_norm_eps"])
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings") else w["lm_head.weight"]
    return x @ head.T


# --------------------------------------------------------------------------- sampling

def greedy(logits: torch.Tensor) -> int:
    """Highest logit; the lowest index among equals (candle's ArgMax sampling, chosen at
    backends/vllm/src/llm_service.rs:346-349)."""
    return int(torch.argmax(logits.to(torch.float32)))


def _mulhilo(a: int, b: int):
    p = a * b
    return (p >> 32) & 0xFFFFFFFF, p & 0xFFFFFFFF


def philox4x32(counter: Sequence[int], key: Sequence[int], rounds: int = 10) -> List[int]:
    """Philox-4x32-10 (Salmon et al. 2011), the counter-based generator of the engine's sampler."""
    c = list(counter)
    k = list(key)
    for _ in range(rounds):
        hi0, lo0 = _mulhilo(0xD2511F53, c[0])
        hi1, lo1 = _mulhilo(0xCD9E8D57, c[2])
        c = [hi1 ^ c[1] ^ k[0], lo1, hi0 ^ c[3] ^ k[1], lo0]
        k = [(k[0] + 0x9E3779B9) & 0xFFFFFFFF, (k[1] + 0xBB67AE85) & 0xFFFFFFFF]
    return c


def uniform(seed: int, step: int) -> float:
    """The request's random number for its ``step``-th sampled token, in [0, 1):
    the top 24 bits of the first Philox word, keyed by the 64-bit seed."""
    r = philox4x32([step & 0xFFFFFFFF, (step >> 32) & 0xFFFFFFFF, 0, 0], [seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF])
    return (r[0] >> 8) * (1.0 / 16777216.0)


def apply_repeat_penalty(logits: torch.Tensor, penalty: float, context: Sequence[int]) -> torch.Tensor:
    """Each token id of ``context`` once: a positive logit is divided by the penalty, a negative
    one multiplied (candle_transformers::utils::apply_repeat_penalty, called at
    backends/vllm/src/model_executor.rs:211-225 with the last ``repeat_last_n`` ids)."""
    out = logits.clone()
    for t in set(int(c) for c in context):
        if 0 <= t < out.numel():
            out[t] = out[t] / penalty if out[t] >= 0 else out[t] * penalty
    return out


def sample(logits: torch.Tensor, *, temperature: float, seed: int, step: int,
           top_k: int = 0, top_p: float = 1.0) -> int:
    """Sampling from softmax(logits / T), optionally cut to the k most likely tokens and then
    to the smallest set of most likely tokens whose mass reaches top_p (the reference picks
    All / TopK / TopP / TopKThenTopP by these parameters, backends/vllm/src/llm_service.rs:346-369).
    The token is the first, in index order, at which the running sum of kept probabilities
    exceeds u times their total."""
    p = torch.softmax(logits.to(torch.float64) / temperature, dim=-1)
    keep = torch.ones_like(p, dtype=torch.bool)
    if top_k and top_k < p.numel():
        kth = torch.sort(p, descending=True).values[top_k - 1]
        keep &= p >= kth
    if top_p < 1.0:
        q = torch.where(keep, p, torch.zeros_like(p))
        q = q / q.sum()
        sp, order = torch.sort(q, descending=True, stable=True)
        csum = torch.cumsum(sp, 0)
        n = int((csum < top_p).sum()) + 1  # smallest prefix whose mass reaches top_p
        cut = sp[min(n, sp.numel()) - 1]
        keep &= q >= cut
    q = torch.where(keep, p, torch.zeros_like(p))
    u = uniform(seed, step) * float(q.sum())
    c = torch.cumsum(q, 0)
    idx = int((c <= u).sum())
    idx = min(idx, p.numel() - 1)
    while not keep[idx]:  # u fell on the rounding edge of a dropped token
        idx -= 1
    return idx


def generate_greedy(w, cfg, prompt: Sequence[int], n: int, compute=torch.float64) -> List[int]:
    """n greedy tokens, recomputing the whole sequence each time (no cache)."""
    toks = list(prompt)
    out = []
    for _ in range(n):
        t = greedy(forward(w, cfg, toks, compute)[-1])
        out.append(t)
        toks.append(t)
    return out
