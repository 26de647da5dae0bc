"""The engine at Llama 3.2 1B's layer sizes (hidden 2048, 32/8 heads of 64, intermediate 8192, vocabulary
128256, llama3 frequency scaling, tied head) with two layers, against the plain implementation:
the kernels that the benchmark runs (tensor-core attention for prompts and decode, the few-row and
the library linears, the 525 MB output head) at the sizes they run there."""
import pytest
import torch

import helpers
import plain_llama as P

pytestmark = pytest.mark.gpu

CONFIG_1B_2L = {
    "architectures": ["LlamaForCausalLM"], "hidden_size": 2048, "intermediate_size": 8192, "vocab_size": 128256,
    "num_hidden_layers": 2, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64,
    "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
    "rope_scaling": {"factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192, "rope_type": "llama3"},
    "max_position_embeddings": 131072, "tie_word_embeddings": True, "eos_token_id": 128001,
}


@pytest.fixture(scope="module")
def model(tmp_path_factory):
    d = str(tmp_path_factory.mktemp("llama1b2l"))
    helpers.make_model(d, CONFIG_1B_2L, seed=7, std=0.02, norm_jitter=0.05, scales={"q_proj": 1.5, "k_proj": 1.5})  # attention that is not uniform, without amplifying bfloat16 rounding of the scores
    w = helpers.read_weights(d)
    seqs = helpers.random_tokens(CONFIG_1B_2L["vocab_size"], (150, 40), seed=21)
    # float32 is enough for the truth here (the sums are short) and keeps the test quick
    ref = {k: P.forward(w, CONFIG_1B_2L, v, compute=torch.float32) for k, v in seqs.items()}
    return d, seqs, ref


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_llama_1b_layer_sizes(dtype, model, tmp_path):
    d, seqs, ref = model
    steps = []
    # whole prompts with a few wanted rows; then a prompt in portions beside another's decoded tokens
    for k, v in seqs.items():
        steps.append({"entries": [{"id": f"w{k}", "tokens": v, "want": [0, len(v) // 2, len(v) - 1]}], "end": [f"w{k}"]})
    a, b = seqs["r0"], seqs["r1"]
    steps.append({"entries": [{"id": "ma", "tokens": a[:100], "want": [99]}, {"id": "mb", "tokens": b[:30], "want": [29]}], "end": []})
    steps.append({"entries": [{"id": "ma", "tokens": a[100:131], "want": [30]}, {"id": "mb", "tokens": b[30:31], "want": [0]}], "end": []})
    for i in range(131, 150):
        e = [{"id": "ma", "tokens": [a[i]], "want": [0]}]
        if i - 100 < len(b):
            e.append({"id": "mb", "tokens": [b[i - 100]], "want": [0]})
        steps.append({"entries": e, "end": (["ma"] if i == 149 else []) + (["mb"] if i - 100 == len(b) - 1 else [])})
    steps, out = helpers.run_trace(d, dtype, steps, str(tmp_path), 320, 16, timeout=900)
    refs = dict(ref, a=ref["r0"], b=ref["r1"])  # ids "wr0", "wr1", "ma", "mb" lose their first letter
    worst, where, agree, clear = helpers.compare_trace(steps, out, CONFIG_1B_2L["vocab_size"], refs, strip=1)
    assert worst <= (5e-5 if dtype == "float32" else helpers.BF16_TOL), (worst, where)
    if dtype == "float32":
        assert agree == 1.0
