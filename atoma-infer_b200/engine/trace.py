"""Trace replay: feeds given token ids through the model step by step, writes logits.

Nothing is sampled and nothing is scheduled: each input line names the requests of
one step with their next tokens, and the step function that generation uses runs
them.  The reference has no such program; its nearest precedents are the hand-made
per-step loops of its model tests (models/src/llama.rs:597-690, 993-1138).

Input, one JSON object a line:
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
Output: ``<out>/<step>.f32`` (little-endian float32 [wanted, vocab]) for steps that
want something, and a line ``done <step>`` on standard output after every step.
"""
from __future__ import annotations

import json
import os
import sys
from typing import Dict, IO

import torch

from .runtime import load_model
from .step import StepEntry

ROUND_TOKENS = 64  # a request's token count is rounded up to this when the pool is sized


def replay(model_dir: str, dtype: str, out_dir: str, max_tokens: int, stream: IO[str] = sys.stdin,
           page_size: int = 16, max_live: int = 4, out: IO[str] = sys.stdout, device=None, ops=None) -> int:
    os.makedirs(out_dir, exist_ok=True)
    if ROUND_TOKENS % page_size and page_size % ROUND_TOKENS:
        raise ValueError(f"page size {page_size} neither divides nor is a multiple of {ROUND_TOKENS}")
    unit = max(ROUND_TOKENS, page_size)
    num_pages = ((max_tokens + unit - 1) // unit) * unit // page_size
    # A replayed request may be as long as the pool is large: rotation angles are computed from the position,
    # not looked up, so nothing ends at the configuration's max_position_embeddings (generation stops there).
    lm = load_model(model_dir, dtype=dtype, device=device, page_size=page_size, num_pages=num_pages,
                    max_seqs=max_live, poison_cache=True, ops=ops, cuda_graphs=True,
                    max_model_len=num_pages * page_size)
    ids: Dict[str, int] = {}
    next_id = 0
    steps = 0
    for line in stream:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        entries = []
        for e in rec.get("entries", []):
            key = str(e["id"])
            if key not in ids:
                ids[key] = next_id
                next_id += 1
            entries.append(StepEntry(ids[key], list(e["tokens"]), list(e.get("want", []))))
        logits = lm.step.run(entries)
        if logits.shape[0]:
            path = os.path.join(out_dir, f"{rec['step']}.f32")
            logits.to("cpu", torch.float32).contiguous().numpy().astype("<f4").tofile(path)
        else:
            torch.cuda.synchronize() if torch.cuda.is_available() else None
        if hasattr(lm.rt.ops, "check_status"):
            lm.rt.ops.check_status()
        for key in rec.get("end", []):
            key = str(key)
            if key in ids:
                lm.step.finish(ids.pop(key))
        out.write(f"done {rec['step']}\n")
        out.flush()
        steps += 1
    return steps


def main(argv=None) -> int:
    import argparse

    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for the <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to 64); sizes the page pool")
    ap.add_argument("--page-size", type=int, default=16)
    args = ap.parse_args(argv)
    replay(args.model, args.dtype, args.out, args.max_tokens, page_size=args.page_size)
    return 0
