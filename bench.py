"""Benchmark: decode and prefill throughput of Llama 3.2 1B (random weights) on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference] [--layers L]

A "step" is one decode step of a batch of 8 requests, each with a 2,048-token prompt
in the cache (context up to 4,096).  ``value`` is decoded tokens a second over exactly
K steps, timed on the device; ``e2e`` is the same through ``Engine.step()``, with the
step's inputs copied from pinned host memory and the sampled tokens read back every
step.  Also: prefill of 2,048 tokens, decode at batch 1 and 64, and the decode step's
fraction of the measured HBM bandwidth.  Prints ONE JSON line.

Tables for profiles/ instead of the JSON line: ``--linears [--model 1b|3b|8b]`` (the two few-row linear
kernels on the four matrices of a layer) and ``--layer-kernel-phases`` (the persistent layer kernel's time
per phase); ``--model 3b|8b`` alone runs that configuration's serving workload through ``Engine.generate``.
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
PROMPT_LEN, PREFILL_TOKENS, PAGE = 2048, 2048, 16

_LLAMA3 = {"architectures": ["LlamaForCausalLM"], "vocab_size": 128256, "num_key_value_heads": 8, "head_dim": 128,
           "rms_norm_eps": 1e-5, "rope_theta": 500000.0, "max_position_embeddings": 131072, "bos_token_id": 128000,
           "eos_token_id": 128001}
# The larger configurations with their serving workloads: requests, prompt lengths and new tokens (uniform, both
# ends included), seed, temperature, token budget of a step.
WORKLOADS = {
    "3b": {"config": dict(_LLAMA3, hidden_size=3072, intermediate_size=8192, num_hidden_layers=28, num_attention_heads=24,
                          tie_word_embeddings=True,
                          rope_scaling={"factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                                        "original_max_position_embeddings": 8192, "rope_type": "llama3"}),
           "name": "Llama-3.2-3B", "requests": 16, "prompt": (256, 2048), "new": (256, 256), "seed": 3,
           "temperature": None, "budget": 2048},
    "8b": {"config": dict(_LLAMA3, hidden_size=4096, intermediate_size=14336, num_hidden_layers=32, num_attention_heads=32,
                          tie_word_embeddings=False,
                          rope_scaling={"factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                                        "original_max_position_embeddings": 8192, "rope_type": "llama3"}),
           "name": "Llama-3.1-8B", "requests": 64, "prompt": (128, 4096), "new": (128, 512), "seed": 4,
           "temperature": 0.7, "budget": 2048},
}


def serving_workload(which: str) -> int:
    """A larger configuration with its serving workload through ``Engine.generate`` (random weights drawn on the
    device; scheduler, chunked prefill, mixed steps, decode graphs).  Run twice: once as a user would, for the
    end-to-end rate; once with a synchronisation after every step, to split the time into decode-only steps
    (bytes they must read against the copy bandwidth) and steps that carry prompt tokens (flops against the
    tensor peak).  Prints one JSON line."""
    import tempfile
    import time

    import torch

    import atoma_infer_b200  # noqa: F401
    from atoma_infer_b200.engine import Engine
    from atoma_infer_b200.sampling import SamplingParams

    wl = WORKLOADS[which]
    cfg = wl["config"]
    hbm_gbs, bf16_tflops, peak_kind = peaks()
    g = torch.Generator().manual_seed(wl["seed"])
    n = wl["requests"]
    plens = torch.randint(wl["prompt"][0], wl["prompt"][1] + 1, (n,), generator=g).tolist()
    news = torch.randint(wl["new"][0], wl["new"][1] + 1, (n,), generator=g).tolist()
    prompts = [torch.randint(0, cfg["vocab_size"], (p,), generator=g).tolist() for p in plens]
    params = [SamplingParams(do_sample=wl["temperature"] is not None, temperature=wl["temperature"], random_seed=100 + i,
                             max_new_tokens=m, ignore_eos_token=True) for i, m in enumerate(news)]
    L, H, I, V = cfg["num_hidden_layers"], cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nq, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    lin_params = L * (H * (nq + 2 * nkv) * d + nq * d * H + 3 * H * I)
    head_params = V * H
    weight_bytes = 2 * (lin_params + head_params)  # decode reads every linear once and the head; no embedding rows to speak of
    kv_bytes_per_token = 2 * L * nkv * d * 2
    pages = sum(-(-(p + m) // PAGE) for p, m in zip(plens, news)) + 64
    with tempfile.TemporaryDirectory() as tmp:
        with open(os.path.join(tmp, "config.json"), "w") as f:
            json.dump(cfg, f)
        eng = Engine(tmp, dtype="bfloat16", block_size=PAGE, num_gpu_blocks_override=pages, max_num_sequences=n,
                     max_num_batched_tokens=wl["budget"], random_weights_seed=0)
    lm = eng.lm
    eng.generate([prompts[0][:64]], SamplingParams(do_sample=False, max_new_tokens=4, ignore_eos_token=True))  # libraries load
    clocks = ClockSampler()
    clocks.start()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    outs = eng.generate(prompts, params)
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    steps_e2e, launches = eng.num_steps, lm.rt.ops.launches
    generated = sum(len(o.token_ids) for o in outs)
    assert [len(o.token_ids) for o in outs] == news
    # second run, a synchronisation after every step
    rec = {"decode": [0, 0.0, 0.0, 0], "mixed": [0, 0.0, 0.0, 0]}  # steps, seconds, bytes or flops, tokens
    run = lm.step.run

    def timed(entries):
        ctx = [lm.manager.num_tokens(e.req) if lm.manager.has_request(e.req) else 0 for e in entries]
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        out = run(entries)
        b.record()
        torch.cuda.synchronize()
        dt = a.elapsed_time(b) * 1e-3  # device time of the step, launch gaps of prompt steps included
        toks = sum(len(e.tokens) for e in entries)
        if all(len(e.tokens) == 1 for e in entries):
            r = rec["decode"]
            r[2] += weight_bytes + kv_bytes_per_token * sum(c + 1 for c in ctx)
        else:
            r = rec["mixed"]
            attn = sum(4 * d * nq * L * (len(e.tokens) * c + len(e.tokens) * (len(e.tokens) + 1) // 2) for e, c in zip(entries, ctx))
            r[2] += 2 * toks * lin_params + attn + 2 * head_params * sum(1 for e in entries if e.want)
        r[0] += 1
        r[1] += dt
        r[3] += toks
        return out

    lm.step.run = timed
    eng.generate(prompts, params)
    lm.step.run = run
    clock_rec = clocks.stop()
    dec, mix = rec["decode"], rec["mixed"]
    out = {
        "metric": f"generated tok/s through Engine.generate ({wl['name']} sizes, {n} requests)", "value": generated / wall,
        "unit": "tok/s", "n_gpus": 1, "higher_is_better": True, "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "vs_baseline": None, "seconds": wall, "total_tok_s": (generated + sum(plens)) / wall, "steps": steps_e2e,
        "prompt_tokens": sum(plens), "generated_tokens": generated, "preemptions": eng.scheduler.num_preemptions,
        "gpu_launches": launches,
        "config": {"model": f"{wl['name']} (random weights N(0,0.02), seed 0)", "layers": L, "hidden": H, "heads": nq,
                   "kv_heads": nkv, "head_dim": d, "intermediate": I, "vocab": V, "requests": n,
                   "prompt_lengths": f"uniform {wl['prompt']}, seed {wl['seed']}", "new_tokens": f"uniform {wl['new']}",
                   "temperature": wl["temperature"], "token_budget": wl["budget"], "page_size": PAGE, "parallelism": "1 GPU"},
        "decode_steps": {"steps": dec[0], "ms_per_step": dec[1] / max(dec[0], 1) * 1e3, "tokens_per_step": dec[3] / max(dec[0], 1),
                         "achieved": dec[2] / max(dec[1], 1e-9) / 1e9, "peak": hbm_gbs, "unit": "GB/s",
                         "frac": dec[2] / max(dec[1], 1e-9) / 1e9 / hbm_gbs, "of": peak_kind},
        "prompt_steps": {"steps": mix[0], "ms_per_step": mix[1] / max(mix[0], 1) * 1e3, "tokens_per_step": mix[3] / max(mix[0], 1),
                         "achieved": mix[2] / max(mix[1], 1e-9) / 1e12, "peak": bf16_tflops, "unit": "TFLOP/s",
                         "frac": mix[2] / max(mix[1], 1e-9) / 1e12 / bf16_tflops, "of": f"{peak_kind} bf16 burst"},
        "clocks": clock_rec,
    }
    print(json.dumps(out))
    return 0


def few_row_linears(which: str) -> int:
    """Times the two few-row linear kernels on the four matrices of a layer: 32 calls in one CUDA graph that cycle
    through as many weight sets as fit 2.5 GB (so no weight is found in L2), CUDA events around three replays."""
    import torch

    import atoma_infer_b200  # noqa: F401
    from atoma_infer_b200.engine.runtime import make_runtime

    H, I, nq, nkv, d = {"1b": (2048, 8192, 32, 8, 64), "3b": (3072, 8192, 24, 8, 128), "8b": (4096, 14336, 32, 8, 128)}[which]
    shapes = {"q/k/v": ((nq + 2 * nkv) * d, H, False), "output": (H, nq * d, False), "gate/up + SwiGLU": (2 * I, H, True),
              "down": (H, I, False)}
    rt = make_runtime("bfloat16", "cuda:0")
    ops, dev = rt.ops, rt.device
    hbm = peaks()[0]

    def graph_us(fn, n=32):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(n):
                fn()
        g.replay()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        for _ in range(3):
            g.replay()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / (3 * n) * 1e3

    print(f"few-row linears, Llama sizes {which}: us a call, direct | streamed (at the copy bandwidth {hbm:.0f} GB/s: ideal)")
    for name, (N, K, silu) in shapes.items():
        sets = max(2, min(16, int(2.5e9 // (N * K * 2))))
        ws = [torch.randn(N, K, device=dev, dtype=torch.bfloat16) * 0.02 for _ in range(sets)]
        row = []
        for M in (1, 8, 16):
            x = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
            cell = []
            for streamed in (False, True):
                ops.stream_linear = streamed
                if streamed and not ops._stream_linear(2, N, K):
                    cell.append(float("nan"))
                    continue
                calls = [0]

                def call():
                    if streamed:  # whatever the policy for this row count says
                        ops.linear_streamed(x, ws[calls[0] % sets], silu_mul=silu)
                    else:
                        ops.linear(x, ws[calls[0] % sets], silu_mul=silu)
                    calls[0] += 1
                cell.append(graph_us(call))
            row.append(f"{M:2d} rows {cell[0]:6.1f} | {cell[1]:6.1f}")
        print(f"  {name:18s} {N:6d} x {K:5d} ({N * K * 2 / 1e6:6.1f} MB, ideal {N * K * 2 / hbm / 1e3:5.1f}):  " + "   ".join(row))
        del ws
    ops.check_status()
    return 0


def layer_kernel_phases(eng, args, prompt, greedy, cfg) -> int:
    """Decode steps through the persistent layer kernel (csrc/kernels/decode_stack.cu), eagerly, with every block
    writing the global clock after each phase and each barrier of each layer; prints the mean, the slowest and the
    fastest block per slot.  The clock reads themselves cost about 0.3 us a slot."""
    import torch

    lm, ops = eng.lm, eng.lm.rt.ops
    ops.fused_layers = True
    lm.step.cuda_graphs = False
    d, H, L = cfg["head_dim"], cfg["hidden_size"], cfg["num_hidden_layers"]
    ids = [eng.add_request(prompt(), greedy) for _ in range(args.batch)]
    while any(eng.scheduler.num_computed(i) < args.context for i in ids):
        eng.step()
    for _ in range(max(args.warmup, 3)):
        eng.step()
    blocks = ops.decode_stack_blocks(d, args.batch, max(H, cfg["num_attention_heads"] * d))
    if not blocks:
        print("the layer kernel does not take this geometry")
        return 1
    clocks = torch.zeros((blocks, L, 10), dtype=torch.int64, device=lm.rt.device)
    ops.decode_stack_record_clocks(d, clocks)
    for _ in range(3):
        eng.step()
    torch.cuda.synchronize()
    ops.decode_stack_record_clocks(d, None)
    t = clocks.cpu().double()
    begin = torch.cat([t[:, :-1, 9:10], t[:, 1:, :9]], dim=2)  # a slot begins where the one before it ended
    dur = (t[:, 1:, :] - begin) / 1000.0                      # us; layers 1 .. L-1
    names = ["norm scales + q/k/v", "barrier", "attention", "barrier", "output projection", "barrier",
             "norm scales + gate/up", "barrier", "down projection", "barrier"]
    print(f"layer kernel, batch {args.batch}, context {args.context}, {L} layers, {blocks} blocks: us per slot "
          f"(mean over blocks and layers | slowest block | fastest block)")
    for j, name in enumerate(names):
        per_block = dur[:, :, j].mean(1)
        print(f"  {name:24s} {dur[:, :, j].mean().item():6.2f} | {per_block.max().item():6.2f} | {per_block.min().item():6.2f}")
    print(f"  a layer (block 0): {((t[0, -1, 9] - t[0, 0, 9]) / 1000.0 / (L - 1)).item():.2f} us")
    return 0


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
                                          "--format=csv,noheader,nounits", "-lms", "50"],
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
    ap.add_argument("--model", default="1b", choices=["1b", "3b", "8b"],
                    help="1b: the headline benchmark; 3b / 8b: the larger configurations with their serving workloads")
    ap.add_argument("--context", type=int, default=PROMPT_LEN,
                    help="prompt length of the decode measurements (default 2,048; 8,192 and 32,768 for long contexts)")
    ap.add_argument("--skip-points", action="store_true", help="skip the batch 1 / 64 points")
    ap.add_argument("--layer-kernel-phases", action="store_true",
                    help="instead of the benchmark: decode steps with the persistent layer kernel switched on, and the "
                         "time its blocks spend in every phase and at every barrier of a layer (a table, for profiles/)")
    ap.add_argument("--linears", action="store_true",
                    help="instead of the benchmark: the four linears of a layer (sizes of --model) at 1, 8 and 16 rows on the "
                         "direct and on the streamed few-row kernel, weights cold (a table, for profiles/)")
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
    if args.linears:
        return few_row_linears(args.model)
    if args.model != "1b":
        return serving_workload(args.model)

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
    prompt_len = args.context
    tokens_per_req = prompt_len + 5 * args.steps + args.warmup + 64
    pages = max_batch * (-(-tokens_per_req // PAGE)) + 256
    eng = Engine(tmp, dtype="bfloat16", block_size=PAGE, num_gpu_blocks_override=pages,
                 max_num_sequences=max(max_batch, 8), max_num_batched_tokens=max(PREFILL_TOKENS, max_batch))
    lm, ops = eng.lm, eng.lm.rt.ops
    g = torch.Generator().manual_seed(2)
    greedy = SamplingParams(do_sample=False, max_new_tokens=10 ** 6, ignore_eos_token=True)

    def prompt():
        return torch.randint(0, V, (prompt_len,), generator=g).tolist()

    def event_ms(fn):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b)

    if args.layer_kernel_phases:
        return layer_kernel_phases(eng, args, prompt, greedy, cfg)

    # ------------------------------------------------------------------ prefill of 2,048 tokens
    toks = torch.randint(0, V, (PREFILL_TOKENS,), generator=g).tolist()
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
    REPEATS = 5

    def decode_run(batch, steps, warmup, through_engine):
        """Prefills ``batch`` requests, warms up, then times ``steps`` decode steps REPEATS times over (the
        context grows from one repeat to the next).  Returns a record of the median repeat."""
        ids = [eng.add_request(prompt(), greedy) for _ in range(batch)]
        while any(eng.scheduler.num_computed(i) < prompt_len for i in ids):
            eng.step()  # prompts in portions under the token budget; the last portion samples
        for _ in range(warmup):
            eng.step()
        runs = []
        for rep in range(REPEATS):
            launches0 = ops.launches
            h2d0, d2h0 = lm.step.h2d_bytes + eng.sampler.h2d_bytes, eng.sampler.d2h_bytes
            ctx0 = lm.manager.num_tokens(ids[0])  # tokens in the cache when the region starts
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
            ctx_mid = ctx0 + steps / 2
            nbytes = weight_bytes + batch * ctx_mid * kv_bytes_per_token
            runs.append({"ms": ms, "launches": ops.launches - launches0, "ctx_mid": ctx_mid, "bytes": nbytes,
                         "h2d": (lm.step.h2d_bytes + eng.sampler.h2d_bytes - h2d0) / steps,
                         "d2h": (eng.sampler.d2h_bytes - d2h0) / steps})
        for i in ids:
            eng.abort_request(i)
        runs.sort(key=lambda r: r["ms"])
        med = dict(runs[len(runs) // 2])
        med["ms_min"], med["ms_max"] = runs[0]["ms"], runs[-1]["ms"]
        return med

    def roofline_of(run, batch, steps):
        ms_step = run["ms"] / steps
        achieved = run["bytes"] / (ms_step * 1e-3) / 1e9
        return {"bound": "hbm", "achieved": achieved, "peak": hbm_gbs, "unit": "GB/s", "frac": achieved / hbm_gbs,
                "of": peak_kind, "ms_per_step": ms_step, "ms_per_step_min": run["ms_min"] / steps,
                "ms_per_step_max": run["ms_max"] / steps, "bytes": run["bytes"], "context": run["ctx_mid"],
                "tok_s": batch * steps / run["ms"] * 1e3}

    if args.phase == "prefill":
        print(json.dumps({"impl": "ours", "phase": "prefill", "prefill": prefill}))
        return 0
    clocks = ClockSampler()
    clocks.start()
    run = decode_run(args.batch, args.steps, args.warmup, through_engine=False)
    roofline = roofline_of(run, args.batch, args.steps)
    e2e = None
    if args.phase == "all":
        e2e = decode_run(args.batch, args.steps, args.warmup, through_engine=True)
    points, points_roofline = {}, {f"decode_b{args.batch}": roofline}
    if not args.skip_points and args.phase == "all":
        for b in (1, 64):
            r = roofline_of(decode_run(b, args.steps, args.warmup, through_engine=False), b, args.steps)
            points[f"decode_b{b}"] = r["tok_s"]
            points_roofline[f"decode_b{b}"] = r
    clock_rec = clocks.stop()

    rec = {
        "metric": f"decode tok/s (Llama 3.2 1B, batch {args.batch}, {prompt_len:,}-token prompts)", "value": roofline["tok_s"],
        "unit": "tok/s",
        "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": roofline["ms_per_step"],
        "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "config": {
            "model": "Llama-3.2-1B (random weights N(0,0.02), seed 0)", "layers": L,
            "layers_full": MODEL["num_hidden_layers"], "hidden": H, "heads": nq, "kv_heads": nkv, "head_dim": d,
            "intermediate": I, "vocab": V, "global_batch": args.batch, "seq_len": prompt_len,
            "context": 4096 if prompt_len == PROMPT_LEN else prompt_len + 5 * args.steps + args.warmup,
            "page_size": PAGE, "parallelism": "1 GPU", "repeats": f"median of {REPEATS} regions of --steps steps each",
            "l2": "inputs larger than L2 (2.47 GB of weights read every step)", "prompt_ids": "uniform, seed 2",
        },
        "e2e": None if e2e is None else {
            "value": args.batch * args.steps / e2e["ms"] * 1e3, "unit": "tok/s",
            "h2d_bytes_per_step": e2e["h2d"], "d2h_bytes_per_step": e2e["d2h"],
            "bytes_counted": "from the pinned buffers copied each step (metadata, sampler parameters; tokens back)"},
        "gpu_launches": run["launches"],
        "prefill": prefill,
        "roofline": {k: roofline[k] for k in ("bound", "achieved", "peak", "unit", "frac", "of")},
        "points": points,
        "points_roofline": points_roofline,
        "clocks": clock_rec,
    }
    print(json.dumps(rec))
    return 0


if __name__ == "__main__":
    sys.exit(main())
