"""Shared test material: three tiny configurations that differ in every size and option,
model folders with random weights, trace builders for the replay program, comparison."""
from __future__ import annotations

import json
import os
import subprocess
import sys
from typing import Dict, List, Sequence

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import atoma_infer_b200  # noqa: E402,F401
from atoma_infer_b200.weights import write_random_model  # noqa: E402
from atoma_infer_b200.weights.safetensors_io import SafetensorsFile  # noqa: E402

# A: grouped-query 2:1, head 16, tied head, no frequency scaling, page 4
CONFIG_A = {
    "architectures": ["LlamaForCausalLM"], "hidden_size": 64, "intermediate_size": 176, "vocab_size": 256,
    "num_hidden_layers": 2, "num_attention_heads": 4, "num_key_value_heads": 2, "rms_norm_eps": 1e-5,
    "rope_theta": 10000.0, "max_position_embeddings": 1024, "tie_word_embeddings": True, "eos_token_id": 255,
}
# B: one key/value head for three query heads, head 64, untied head, llama3 scaling whose
# original length (64) puts frequencies in all three bands, page 8, sizes that are no power of two
CONFIG_B = {
    "architectures": ["LlamaForCausalLM"], "hidden_size": 192, "intermediate_size": 320, "vocab_size": 1000,
    "num_hidden_layers": 3, "num_attention_heads": 3, "num_key_value_heads": 1, "rms_norm_eps": 1e-6,
    "rope_theta": 500000.0,
    "rope_scaling": {"factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 64, "rope_type": "llama3"},
    "max_position_embeddings": 1024, "tie_word_embeddings": False, "eos_token_id": [998, 999],
}
# C: the head size (128) and group size (3 query heads per key/value head) of the larger Llama 3 models, page 16
CONFIG_C = {
    "architectures": ["LlamaForCausalLM"], "hidden_size": 768, "intermediate_size": 1024, "vocab_size": 777,
    "num_hidden_layers": 2, "num_attention_heads": 6, "num_key_value_heads": 2, "rms_norm_eps": 1e-5,
    "rope_theta": 500000.0,
    "rope_scaling": {"factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 128, "rope_type": "llama3"},
    "max_position_embeddings": 2048, "tie_word_embeddings": False, "eos_token_id": 776,
}
TINY = {"A": (CONFIG_A, 4), "B": (CONFIG_B, 8), "C": (CONFIG_C, 16)}  # name -> (config, page size)



def _cfg(hidden, inter, vocab, layers, nq, nkv, eps, theta, tie, scaling=None, eos=0):
    c = {"architectures": ["LlamaForCausalLM"], "hidden_size": hidden, "intermediate_size": inter, "vocab_size": vocab,
         "num_hidden_layers": layers, "num_attention_heads": nq, "num_key_value_heads": nkv, "rms_norm_eps": eps,
         "rope_theta": theta, "max_position_embeddings": 2048, "tie_word_embeddings": tie, "eos_token_id": eos}
    if scaling:
        c["rope_scaling"] = {"factor": scaling[0], "low_freq_factor": 1.0, "high_freq_factor": scaling[1],
                             "original_max_position_embeddings": scaling[2], "rope_type": "llama3"}
    return c


# Further geometries, one replay each: other head sizes (32 .. 256 in steps of 16), group sizes 1 .. 16, odd
# intermediate sizes and vocabularies, an intermediate size below the width, page sizes 4 .. 64.
# name -> (config, page size)
MORE = {
    "d32g2": (_cfg(192, 301, 511, 1, 6, 3, 1e-3, 1e6, True), 32),
    "d48g1": (_cfg(240, 336, 99, 2, 5, 5, 1e-5, 10000.0, False, scaling=(4.0, 2.0, 32)), 4),
    "d80g4": (_cfg(640, 1000, 1201, 1, 8, 2, 1e-5, 500000.0, True, scaling=(32.0, 4.0, 64)), 16),
    "d96g5": (_cfg(960, 520, 300, 2, 10, 2, 1e-6, 500000.0, False), 8),
    "d256g2": (_cfg(512, 777, 1000, 1, 2, 1, 1e-5, 10000.0, False), 64),
    "d112g8": (_cfg(896, 1024, 333, 1, 8, 1, 1e-5, 500000.0, True, scaling=(8.0, 4.0, 128)), 16),
    "d16g16": (_cfg(256, 384, 128, 2, 16, 1, 1e-5, 10000.0, False), 16),
    # a head size that is no multiple of 16: the plain attention kernel serves bfloat16 too
    "d24g2": (_cfg(96, 200, 150, 1, 4, 2, 1e-5, 10000.0, True), 8),
}

FP32_TOL = 2e-5   # times the largest |logit| of the sequence
BF16_TOL = 3e-2


def make_model(path: str, config: dict, seed: int = 0, **kw) -> str:
    """Random weights large enough that attention and norms matter (std 0.05, norm weights 1 +- 0.1)."""
    kw.setdefault("std", 0.05)
    kw.setdefault("norm_jitter", 0.1)
    return write_random_model(path, config, seed, **kw)


def read_weights(model_dir: str) -> Dict[str, torch.Tensor]:
    f = SafetensorsFile(os.path.join(model_dir, "model.safetensors"))
    return {n: f.tensor(n).to(torch.float32) for n in f.names()}


def random_tokens(vocab: int, lengths: Sequence[int], seed: int) -> Dict[str, List[int]]:
    g = torch.Generator().manual_seed(seed)
    return {f"r{i}": torch.randint(0, vocab, (n,), generator=g).tolist() for i, n in enumerate(lengths)}


# ------------------------------------------------------------------ traces
def trace_whole(seqs, tag="w"):
    return [{"entries": [{"id": f"{tag}{k}", "tokens": v, "want": list(range(len(v)))}], "end": [f"{tag}{k}"]}
            for k, v in seqs.items()]


def trace_tail(seqs, tail=32, tag="t"):
    """Most of a request in one step, its last ``tail`` tokens one by one."""
    steps = []
    for k, v in seqs.items():
        head = max(len(v) - tail, 0)
        if head:
            steps.append({"entries": [{"id": f"{tag}{k}", "tokens": v[:head], "want": list(range(head))}], "end": []})
        for i in range(head, len(v)):
            steps.append({"entries": [{"id": f"{tag}{k}", "tokens": [v[i]], "want": [0]}],
                          "end": [f"{tag}{k}"] if i == len(v) - 1 else []})
    return steps


def trace_chunks(seqs, sizes=(5, 2, 7, 3, 2, 11, 1, 4), tag="c"):
    """Portions of changing size, down to two tokens (and one)."""
    steps, si = [], 0
    for k, v in seqs.items():
        pos = 0
        while pos < len(v):
            n = min(sizes[si % len(sizes)], len(v) - pos)
            si += 1
            steps.append({"entries": [{"id": f"{tag}{k}", "tokens": v[pos:pos + n], "want": list(range(n))}],
                          "end": [f"{tag}{k}"] if pos + n == len(v) else []})
            pos += n
    return steps


def trace_mixed(seqs, max_live=4, sizes=(6, 2, 9, 3, 5), tag="m", seed=0):
    """Up to ``max_live`` requests at a time; each either runs a portion of its prompt, a
    single token (as a decode step would) or sits a step out; new requests take the
    pages of ended ones."""
    rng = np.random.RandomState(seed)
    pending = list(seqs)
    live, pos, steps, si = [], {k: 0 for k in seqs}, [], 0
    single = {k: i % 2 == 1 for i, k in enumerate(seqs)}  # every other request: one token at a time after a start
    while pending or live:
        while pending and len(live) < max_live:
            live.append(pending.pop(0))
        entries, end = [], []
        for k in list(live):
            if len(live) > 1 and rng.rand() < 0.2:
                continue  # left out of this step, goes on later
            v = seqs[k]
            if single[k] and pos[k] >= min(len(v) // 2, 8):
                n = 1
            else:
                n = sizes[si % len(sizes)]
                si += 1
            n = min(n, len(v) - pos[k])
            entries.append({"id": f"{tag}{k}", "tokens": v[pos[k]:pos[k] + n], "want": list(range(n))})
            pos[k] += n
            if pos[k] == len(v):
                end.append(f"{tag}{k}")
                live.remove(k)
        if entries:
            steps.append({"entries": entries, "end": end})
    return steps


def number(steps):
    return [dict(s, step=i) for i, s in enumerate(steps)]


def run_trace(model_dir: str, dtype: str, steps, out_dir: str, max_tokens: int, page_size: int, timeout=600, env=None):
    """Runs bin/trace_run as a user would; returns the list of per-step arrays (None where nothing was wanted)."""
    steps = number(steps)
    text = "\n".join(json.dumps(s) for s in steps) + "\n"
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype,
           "--out", out_dir, "--max-tokens", str(max_tokens), "--page-size", str(page_size)]
    p = subprocess.run(cmd, input=text, capture_output=True, text=True, timeout=timeout,
                       env=dict(os.environ, **env) if env else None)
    assert p.returncode == 0, f"trace_run failed ({p.returncode}):\n{p.stdout[-2000:]}\n{p.stderr[-4000:]}"
    done = [l for l in p.stdout.splitlines() if l.startswith("done ")]
    assert [int(l.split()[1]) for l in done] == [s["step"] for s in steps], "a 'done <step>' line is missing"
    return steps, out_dir


def compare_trace(steps, out_dir: str, vocab: int, ref_logits: Dict[str, torch.Tensor], strip=1, bound=2 * BF16_TOL):
    """Largest |difference| / largest |logit| over every wanted place, the place where it is reached (for
    messages), the share of places whose top-1 equals the plain one, and that share among the places where the
    plain top-1 leads the runner-up by more than ``bound`` times the logit scale (there a reduced-precision
    engine has no excuse).  Request ids carry a ``strip``-letter tag."""
    pos: Dict[str, int] = {}
    worst, where = 0.0, None
    agree = total = clear = clear_agree = 0
    for s in steps:
        wanted = sum(len(e["want"]) for e in s["entries"])
        if not wanted:
            for e in s["entries"]:
                pos[e["id"]] = pos.get(e["id"], 0) + len(e["tokens"])
            continue
        got = np.fromfile(os.path.join(out_dir, f"{s['step']}.f32"), dtype="<f4").reshape(-1, vocab)
        assert got.shape[0] == wanted, f"step {s['step']}: {got.shape[0]} rows written, {wanted} wanted"
        r = 0
        for e in s["entries"]:
            key = e["id"][strip:]
            start = pos.get(e["id"], 0)
            ref = ref_logits[key]
            scale = float(ref.abs().max())
            for w in e["want"]:
                exp = ref[start + w].to(torch.float32).numpy()
                err = float(np.abs(got[r] - exp).max()) / scale
                if not np.isfinite(got[r]).all():
                    err = float("inf")
                if err > worst:
                    worst, where = err, (s["step"], e["id"], start + w)
                same = int(got[r].argmax() == exp.argmax())
                agree += same
                total += 1
                top = np.partition(exp, -2)[-2:]
                if vocab > 1 and float(top[1] - top[0]) > bound * scale:
                    clear += 1
                    clear_agree += same
                r += 1
            pos[e["id"]] = start + len(e["tokens"])
    return worst, where, agree / max(total, 1), clear_agree / max(clear, 1)


def greedy_agreement(w, cfg, prompt, got: Sequence[int], bound: float = 2 * BF16_TOL):
    """Policy for greedy tokens of a reduced-precision engine.  Every generated token is judged against the
    plain implementation run on the engine's own history (the prompt and the tokens generated before it), so
    no token is lost to an earlier, permitted difference: it must be the plain top-1, or its plain logit must
    lie within ``bound`` times the largest |logit| of that position below the top-1 (twice the tolerance the
    logits themselves are held to, since both candidates may move).  Returns (tokens equal to the plain
    top-1, tokens generated)."""
    import plain_llama as P

    logits = P.forward(w, cfg, list(prompt) + list(got))
    same = 0
    for i, tok in enumerate(got):
        row = logits[len(prompt) - 1 + i]
        best = int(torch.argmax(row))
        if tok == best:
            same += 1
            continue
        lead = float(row[best] - row[tok]) / float(row.abs().max())
        assert lead <= bound, (f"token {i}: engine {tok}, plain {best}, although the plain top-1 leads it by "
                               f"{lead:.3g} of the logit scale (bound {bound:.3g})")
    return same, len(got)


def plain_sampled(w, cfg, prompt, n, sp):
    """The plain loop: whole sequence each time, penalty over the last ids, then the seeded draw."""
    import plain_llama as P

    p = sp.validated()
    toks, out = list(prompt), []
    for step in range(n):
        logits = P.forward(w, cfg, toks)[-1]
        if p.repetition_penalty != 1.0:
            logits = P.apply_repeat_penalty(logits, p.repetition_penalty, toks[-p.repeat_last_n:])
        t = P.greedy(logits) if p.greedy else P.sample(logits, temperature=p.temperature, seed=p.seed, step=step,
                                                       top_k=p.top_k, top_p=p.top_p)
        out.append(t)
        toks.append(t)
    return out
