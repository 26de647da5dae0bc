"""Command line: generate from token ids, write a random-weights model folder, replay a trace.

The reference's binary takes one option, ``--config-path <toml>`` (server/src/main.rs:22-27),
whose tables ``[inference] [cache] [scheduler] [validation]`` carry everything else
(backends/vllm/src/tests/test_config.toml).  That file is accepted here as it is; every
key of it can also be given as a flag of the same name, and the request parameters are
flags named like GenerateParameters (backends/vllm/src/types.rs:32-95).  Prompts are
token ids (the tokenizer is outside this engine).

    atoma-infer generate --model DIR --prompt-ids 1,2,3 --max-new-tokens 16
    atoma-infer random-model --config config.json --seed 0 --out DIR
    atoma-infer replay --model DIR --dtype float32 --out DIR --max-tokens 256 < trace.jsonl
"""
from __future__ import annotations

import argparse
import json
import sys
import time


def _engine_flags(ap):
    ap.add_argument("--config-path", help="TOML with [inference] [cache] [scheduler] [validation] tables")
    ap.add_argument("--dtype", help="bf16 | f32 (default bf16)")
    ap.add_argument("--block-size", type=int, help="tokens per cache page")
    ap.add_argument("--gpu-memory-utilization", type=float)
    ap.add_argument("--num-gpu-blocks-override", type=int, help="cache pages per pool instead of sizing from memory")
    ap.add_argument("--max-num-batched-tokens", type=int, help="token budget of a step")
    ap.add_argument("--max-num-sequences", type=int)
    ap.add_argument("--max-model-len", type=int)
    ap.add_argument("--enable-chunked-prefill", dest="enable_chunked_prefill", action="store_true", default=None)
    ap.add_argument("--no-enable-chunked-prefill", dest="enable_chunked_prefill", action="store_false")
    ap.add_argument("--no-cuda-graphs", dest="cuda_graphs", action="store_false", default=None)
    ap.add_argument("--random-weights", dest="random_weights_seed", type=int, metavar="SEED",
                    help="the model folder holds only config.json: draw every tensor on the device from this seed")


def _engine_config(args):
    from .config import EngineConfig

    cfg = EngineConfig.from_toml(args.config_path) if args.config_path else EngineConfig()
    for k in ("dtype", "block_size", "gpu_memory_utilization", "num_gpu_blocks_override", "max_num_batched_tokens",
              "max_num_sequences", "max_model_len", "enable_chunked_prefill", "cuda_graphs", "random_weights_seed"):
        v = getattr(args, k, None)
        if v is not None:
            setattr(cfg, k, v)
    cfg.__post_init__()
    return cfg


def _cmd_generate(args) -> int:
    from .engine import Engine
    from .sampling import SamplingParams

    prompts = [[int(t) for t in p.replace(" ", "").split(",") if t] for p in (args.prompt_ids or [])]
    if args.prompt_file:
        with open(args.prompt_file) as f:
            prompts += [json.loads(line) for line in f if line.strip()]
    if not prompts:
        print("no prompt given (--prompt-ids 1,2,3 or --prompt-file FILE with one JSON list a line)", file=sys.stderr)
        return 2
    params = SamplingParams(
        temperature=args.temperature, top_k=args.top_k, top_p=args.top_p, repetition_penalty=args.repetition_penalty,
        repeat_last_n=args.repeat_last_n, do_sample=args.do_sample, max_new_tokens=args.max_new_tokens,
        random_seed=args.random_seed, ignore_eos_token=args.ignore_eos_token)
    eng = Engine(args.model, _engine_config(args))
    t0 = time.time()
    outs = eng.generate(prompts, params)
    dt = time.time() - t0
    for o in outs:
        m = o.metrics
        print(json.dumps({
            "request_id": o.request_id, "token_ids": o.token_ids, "finish_reason": o.finish_reason,
            "prompt_tokens": len(o.prompt_token_ids),
            "time_to_first_token": None if m.first_token_time is None else round(m.first_token_time - m.arrival_time, 6),
            "preemptions": m.num_preemptions,
        }))
    n = sum(len(o.token_ids) for o in outs)
    st = eng.stats()
    print(f"{n} tokens generated ({n / dt:.1f} token/s), {st['steps']} steps ({st['graph_replays']} as graph replays), "
          f"{st['preemptions']} preemptions, {st['kernel_launches']} kernel launches", file=sys.stderr)
    return 0


def _cmd_random_model(args) -> int:
    import torch

    from .weights import write_random_model

    with open(args.config) as f:
        config = json.load(f)
    dtype = {"bf16": torch.bfloat16, "bfloat16": torch.bfloat16, "f32": torch.float32, "float32": torch.float32}[args.dtype]
    write_random_model(args.out, config, args.seed, std=args.std, norm_jitter=args.norm_jitter, dtype=dtype)
    print(args.out)
    return 0


def _cmd_replay(args) -> int:
    from .engine.trace import replay

    replay(args.model, args.dtype, args.out, args.max_tokens, page_size=args.page_size)
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="atoma-infer", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)
    g = sub.add_parser("generate", help="generate tokens for prompts given as token ids")
    g.add_argument("--model", required=True, help="folder with config.json and *.safetensors")
    g.add_argument("--prompt-ids", action="append", help="comma-separated token ids; may be given several times")
    g.add_argument("--prompt-file", help="file with one JSON list of token ids a line")
    _engine_flags(g)
    g.add_argument("--temperature", type=float)
    g.add_argument("--top-k", type=int)
    g.add_argument("--top-p", type=float)
    g.add_argument("--repetition-penalty", type=float)
    g.add_argument("--repeat-last-n", type=int)
    g.add_argument("--do-sample", dest="do_sample", action="store_true", default=True)
    g.add_argument("--no-do-sample", dest="do_sample", action="store_false")
    g.add_argument("--max-new-tokens", type=int, default=100)
    g.add_argument("--random-seed", type=int)
    g.add_argument("--ignore-eos-token", action="store_true")
    g.set_defaults(fn=_cmd_generate)
    r = sub.add_parser("random-model", help="write config.json and model.safetensors from a configuration and a seed")
    r.add_argument("--config", required=True, help="a config.json to take the sizes from")
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("--out", required=True)
    r.add_argument("--dtype", default="bf16")
    r.add_argument("--std", type=float, default=0.02)
    r.add_argument("--norm-jitter", type=float, default=0.0)
    r.set_defaults(fn=_cmd_random_model)
    t = sub.add_parser("replay", help="feed given token ids step by step, write logits (same as bin/trace_run)")
    t.add_argument("--model", required=True)
    t.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    t.add_argument("--out", required=True)
    t.add_argument("--max-tokens", type=int, required=True)
    t.add_argument("--page-size", type=int, default=16)
    t.set_defaults(fn=_cmd_replay)
    args = ap.parse_args(argv)
    return args.fn(args)


if __name__ == "__main__":
    sys.exit(main())
