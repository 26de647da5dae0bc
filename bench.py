"""Benchmark: decode and prefill throughput of Llama 3.2 1B (random weights) on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference] [--layers L]

A "step" is one decode step of a batch of 8 requests, each with a 2,048-token prompt
in the cache (context up to 4,096).  ``value`` is decoded tokens a second over exactly
K steps, timed on the device; ``e2e`` is the same through ``Engine.step()``, with the
step's inputs copied from pinned host memory and the sampled tokens read back every
step.  Also: prefill of 2,048 tokens, decode at batch 1 and 64, and the decode step's
fraction of the measured HBM bandwidth.  Prints ONE JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

MODEL = {  # Llama 3.2 1B
    "architectures": ["LlamaForCausalLM"], "hidden_size": 2048, "intermediate_size": 8192, "vocab_size": 128256,
    "num_hidden_layers": 16, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64,
    "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
    "rope_scaling": {"factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192, "rope_type": "llama3"},
    "max_position_embeddings": 131072, "tie_word_embeddings": True, "bos_token_id": 128000, "eos_token_id": 128001,
}
PROMPT_LEN, PREFILL_TOKENS, DECODE_TOKENS, PAGE = 2048, 2048, 256, 16


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(p):
        with open(p) as f:
            d = json.load(f)
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        self.proc.terminate()
        self.thread.join(timeout=2)
        sm = [float(r[0]) for r in self.rows if len(r) >= 6 and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) >= 6 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 6 for n, v in zip(names, r[2:6]) if v == "Active"})
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=MODEL["num_hidden_layers"],
                    help="fewer layers than the model has (both numbers are reported)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--skip-points", action="store_true", help="skip the batch 1 / 64 points")
    ap.add_argument("--phase", default="all", choices=["all", "prefill", "decode"],
                    help="measure only one phase (for profiling); the JSON line then lacks the other")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is Rust (candle, cudarc) with no toolchain or vendored crates here, its "
                          "CUTLASS submodule is empty and its kernels reject sm_100 (csrc/src/lib.rs:2216-2231)"}))
        return 0
    if args.gpus != 1 or int(os.environ.get("WORLD_SIZE", "1")) != 1:
        if int(os.environ.get("RANK", "0")) == 0:
            print(f"bench.py measures a one-GPU engine; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(args.warmup, 3)

    import torch

    import atoma_infer_b200  # noqa: F401
    from atoma_infer_b200.engine import Engine, StepEntry
    from atoma_infer_b200.sampling import SamplingParams
    from atoma_infer_b200.weights import write_random_model

    hbm_gbs, bf16_tflops, peak_kind = peaks()
    cfg = dict(MODEL, num_hidden_layers=args.layers)
    import atexit
    import shutil

    tmp = tempfile.mkdtemp(prefix="bench_model_")
    atexit.register(shutil.rmtree, tmp, ignore_errors=True)  # 2.5 GB of random weights: do not leave them behind
    write_random_model(tmp, cfg, seed=0, std=0.02, device="cuda")
    L, H, I, V = args.layers, cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nq, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    lin_params = L * (H * (nq + 2 * nkv) * d + nq * d * H + 3 * H * I)
    weight_bytes = 2 * (lin_params + V * H)  # every weight once; the tied embedding matrix is the head
    kv_bytes_per_token = 2 * L * nkv * d * 2

    max_batch = 64 if not args.skip_points else args.batch
    tokens_per_req = PROMPT_LEN + DECODE_TOKENS + args.steps + args.warmup + 64
    pages = max_batch * (-(-tokens_per_req // PAGE)) + 256
    eng = Engine(tmp, dtype="bfloat16", block_size=PAGE, num_gpu_blocks_override=pages,
                 max_num_sequences=max(max_batch, 8), max_num_batched_tokens=max(PREFILL_TOKENS, max_batch))
    lm, ops = eng.lm, eng.lm.rt.ops
    g = torch.Generator().manual_seed(2)
    greedy = SamplingParams(do_sample=False, max_new_tokens=10 ** 6, ignore_eos_token=True)

    def prompt():
        return torch.randint(0, V, (PROMPT_LEN,), generator=g).tolist()

    def event_ms(fn):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b)

    # ------------------------------------------------------------------ prefill of 2,048 tokens
    toks = prompt()
    times = []
    for i in range(3 + 5 if args.phase != "decode" else 0):
        req = 10 ** 6 + i
        ms = event_ms(lambda: lm.step.run([StepEntry(req, toks, [PREFILL_TOKENS - 1])]))
        lm.step.finish(req)
        if i >= 3:
            times.append(ms)
    prefill_ms = statistics.median(times) if times else float("nan")
    prefill_flops = 2 * PREFILL_TOKENS * lin_params + 4 * (PREFILL_TOKENS ** 2 // 2) * d * nq * L + 2 * V * H
    prefill = {"value": PREFILL_TOKENS / prefill_ms * 1e3, "tokens": PREFILL_TOKENS, "ms": prefill_ms,
               "frac": prefill_flops / (prefill_ms * 1e-3) / (bf16_tflops * 1e12), "peak": f"{peak_kind} bf16 burst"}

    # ------------------------------------------------------------------ decode
    def decode_run(batch, steps, warmup, through_engine):
        """Prefills ``batch`` requests, then times ``steps`` decode steps after ``warmup``."""
        ids = [eng.add_request(prompt(), greedy) for _ in range(batch)]
        while any(eng.scheduler.num_computed(i) < PROMPT_LEN for i in ids):
            eng.step()  # prompts in portions under the token budget; the last portion samples
        for _ in range(warmup):
            eng.step()
        launches0 = ops.launches
        if through_engine:
            ms = event_ms(lambda: [eng.step() for _ in range(steps)])
        else:
            # device-timed: the same decode step with the tokens already on the host side
            # (synthetic ids), no read-back between steps
            fake = torch.randint(0, V, (steps, batch), generator=g).tolist()
            out = torch.empty(batch, dtype=torch.int32, device=lm.rt.device)

            def loop():
                for s in range(steps):
                    logits = lm.step.run([StepEntry(i, [fake[s][k]], [0]) for k, i in enumerate(ids)])
                    ops.sample(logits, None, None, None, None, None, out)
            ms = event_ms(loop)
        launches = ops.launches - launches0
        ctx_mid = PROMPT_LEN + warmup + steps / 2
        for i in ids:
            eng.abort_request(i)
        return ms, launches, ctx_mid

    if args.phase == "prefill":
        print(json.dumps({"impl": "ours", "phase": "prefill", "prefill": prefill}))
        return 0
    clocks = ClockSampler()
    clocks.start()
    ms, launches, ctx_mid = decode_run(args.batch, args.steps, args.warmup, through_engine=False)
    clock_rec = clocks.stop()
    ms_step = ms / args.steps
    value = args.batch * args.steps / ms * 1e3
    step_bytes = weight_bytes + args.batch * ctx_mid * kv_bytes_per_token
    achieved = step_bytes / (ms_step * 1e-3) / 1e9
    e2e_ms = float("nan")
    if args.phase == "all":
        e2e_ms, _, _ = decode_run(args.batch, args.steps, args.warmup, through_engine=True)
    meta_ints = 20 + 3 * args.batch + (args.batch + 1) + 2 * args.batch + args.batch \
        + args.batch * (-(-(PROMPT_LEN + DECODE_TOKENS) // PAGE))
    points = {}
    if not args.skip_points and args.phase == "all":
        for b in (1, 64):
            pms, _, _ = decode_run(b, 32, 3, through_engine=False)
            points[f"decode_b{b}"] = b * 32 / pms * 1e3

    rec = {
        "metric": "decode tok/s (Llama 3.2 1B, batch 8, 2,048-token prompts)", "value": value, "unit": "tok/s",
        "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "config": {
            "model": "Llama-3.2-1B (random weights N(0,0.02), seed 0)", "layers": L,
            "layers_full": MODEL["num_hidden_layers"], "hidden": H, "heads": nq, "kv_heads": nkv, "head_dim": d,
            "intermediate": I, "vocab": V, "global_batch": args.batch, "seq_len": PROMPT_LEN, "context": 4096,
            "decode_tokens": DECODE_TOKENS, "page_size": PAGE, "parallelism": "1 GPU",
            "l2": "inputs larger than L2 (2.47 GB of weights read every step)", "prompt_ids": "uniform, seed 2",
        },
        "e2e": {"value": args.batch * args.steps / e2e_ms * 1e3, "unit": "tok/s",
                "h2d_bytes_per_step": 4 * meta_ints + 28 * args.batch, "d2h_bytes_per_step": 4 * args.batch},
        "gpu_launches": launches,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_gbs, "unit": "GB/s",
                     "frac": achieved / hbm_gbs, "of": peak_kind},
        "points": points,
        "clocks": clock_rec,
    }
    print(json.dumps(rec))
    return 0


if __name__ == "__main__":
    sys.exit(main())
