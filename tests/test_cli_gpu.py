"""The command line as a user runs it: ``bin/atoma-infer random-model`` writes a model folder from a
configuration and a seed, ``bin/atoma-infer generate`` turns prompts (token ids) into token ids, with its
options as flags or in a TOML file of the reference's shape (``--config-path``, server/src/main.rs:22-27;
backends/vllm/src/tests/test_config.toml).  Both run as child processes; the printed tokens are compared
with the plain implementation."""
import json
import os
import subprocess
import sys

import pytest

import helpers
import plain_llama as P

pytestmark = pytest.mark.gpu

CLI = os.path.join(helpers.ROOT, "bin", "atoma-infer")

TOML = """
[inference]
api_key = ""
cache_dir = "./cache/"
flush_storage = true
model_name = "a-local-folder"
device_ids = [0]
dtype = "{dtype}"
num_tokenizer_workers = 4
revision = "main"

[cache]
block_size = 8
cache_dtype = "{dtype}"
gpu_memory_utilization = 0.5
swap_space_fraction = 0.1
num_gpu_blocks_override = 64

[scheduler]
max_num_batched_tokens = 128
max_num_sequences = 4
max_model_len = 128
delay_factor = 0.8
enable_chunked_prefill = false
block_size = 8

[validation]
best_of = 1
max_stop_sequences = 1
max_top_n_tokens = 1
max_input_length = 100
max_total_tokens = 128
"""


def _run(args, **kw):
    p = subprocess.run([sys.executable, CLI, *args], capture_output=True, text=True, timeout=900, **kw)
    assert p.returncode == 0, f"atoma-infer {' '.join(args)} failed ({p.returncode}):\n{p.stdout[-2000:]}\n{p.stderr[-4000:]}"
    return p


@pytest.fixture(scope="module")
def cli_model(tmp_path_factory):
    """A model folder written by the command line itself."""
    d = tmp_path_factory.mktemp("cli")
    cfg_path = d / "config_in.json"
    cfg_path.write_text(json.dumps(helpers.CONFIG_B))
    out = d / "model"
    p = _run(["random-model", "--config", str(cfg_path), "--seed", "5", "--out", str(out), "--std", "0.05",
              "--norm-jitter", "0.1"])
    assert p.stdout.strip() == str(out)
    assert (out / "config.json").is_file() and (out / "model.safetensors").is_file()
    assert json.loads((out / "config.json").read_text())["hidden_size"] == helpers.CONFIG_B["hidden_size"]
    return str(out), helpers.read_weights(str(out))


def _tokens(p):
    recs = [json.loads(line) for line in p.stdout.splitlines() if line.startswith("{")]
    return [r["token_ids"] for r in recs], recs


PROMPTS = [[3, 14, 15, 92, 65, 35, 89, 79], [2, 718, 281, 828, 459, 45, 235, 360, 287, 471, 352, 662, 497]]


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_generate_from_flags(dtype, cli_model):
    d, w = cli_model
    args = ["generate", "--model", d, "--dtype", dtype, "--block-size", "8", "--num-gpu-blocks-override", "32",
            "--max-num-batched-tokens", "16", "--max-num-sequences", "4", "--no-do-sample", "--max-new-tokens", "10",
            "--ignore-eos-token"]
    for p in PROMPTS:
        args += ["--prompt-ids", ",".join(map(str, p))]
    out = _run(args)
    got, recs = _tokens(out)
    assert len(got) == 2 and all(r["finish_reason"] == "length" for r in recs)
    assert "tokens generated" in out.stderr
    for p, g in zip(PROMPTS, got):
        if dtype == "f32":
            assert g == P.generate_greedy(w, helpers.CONFIG_B, p, 10)
        else:
            assert len(g) == 10
            helpers.greedy_agreement(w, helpers.CONFIG_B, p, g)


def test_generate_from_a_config_file_and_a_prompt_file(cli_model, tmp_path):
    """Every engine option from the reference's TOML tables (keys this engine has no use for are accepted and
    ignored), prompts from a file, sampling options as flags."""
    from atoma_infer_b200.sampling import SamplingParams

    d, w = cli_model
    toml = tmp_path / "engine.toml"
    toml.write_text(TOML.format(dtype="f32"))
    prompts = tmp_path / "prompts.jsonl"
    prompts.write_text("\n".join(json.dumps(p) for p in PROMPTS) + "\n")
    out = _run(["generate", "--model", d, "--config-path", str(toml), "--prompt-file", str(prompts),
                "--temperature", "0.8", "--top-k", "7", "--random-seed", "42", "--max-new-tokens", "8",
                "--ignore-eos-token"])
    got, _ = _tokens(out)
    sp = SamplingParams(temperature=0.8, top_k=7, random_seed=42, max_new_tokens=8, ignore_eos_token=True)
    assert got == [helpers.plain_sampled(w, helpers.CONFIG_B, p, 8, sp) for p in PROMPTS]
    # a flag wins over the file; a prompt beyond [validation].max_input_length is refused with a message
    long_prompt = ",".join(["1"] * 101)
    p = subprocess.run([sys.executable, CLI, "generate", "--model", d, "--config-path", str(toml), "--prompt-ids",
                        long_prompt], capture_output=True, text=True, timeout=900)
    assert p.returncode != 0 and "max_input_length" in p.stderr
