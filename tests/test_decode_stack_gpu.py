"""The decode step's layers as one persistent kernel (csrc/kernels/decode_stack.cu) against the plain
implementation and against the same step run part by part: few and many rows (one and two n-tiles), contexts whose
newest position falls on page and tile edges, keys and values brought by the stream warp (pages of 16, head size
64) and fetched by the attention itself (other page sizes, head size 128), widths that are no multiple of 512 (the
last stage of a row is part zeros), a captured graph, and the refusal of widths the tensor maps cannot describe."""
import pytest
import torch

import helpers
import plain_llama as P

pytestmark = pytest.mark.gpu


def _load(model_dir, page):
    from atoma_infer_b200.engine.runtime import load_model

    lm = load_model(model_dir, dtype="bfloat16", page_size=page, num_pages=900, max_seqs=64)
    return lm


MODES = {  # name -> (one launch for all layers, norms folded into streamed linears)
    "fused": (True, False),
    "chain": (False, True),
    "parts": (False, False),
}


def _decode_and_compare(lm, cfg, w, lengths, steps, seed, one_launch=True):
    """Triplet requests: one set decodes through the layer kernel, one through the chain of streamed linears with the
    norms folded in, one part by part; all against the plain implementation on the whole sequences."""
    from atoma_infer_b200.engine import StepEntry

    ops, step = lm.rt.ops, lm.step
    vocab = cfg["vocab_size"]
    g = torch.Generator().manual_seed(seed)
    seqs = [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lengths]
    n = len(seqs)
    for k in range(len(MODES)):
        for i, s in enumerate(seqs):
            step.run([StepEntry(1000 * k + i, s, [])])
    worst = {name: 0.0 for name in MODES}
    launches = {}
    was = ops.fused_layers, ops.fold_norms
    try:
        for _ in range(steps):
            nxt = torch.randint(0, vocab, (n,), generator=g).tolist()
            for i in range(n):
                seqs[i].append(nxt[i])
            ref = torch.stack([P.forward(w, cfg, s, compute=torch.float32)[-1] for s in seqs])
            for k, (name, (fused, fold)) in enumerate(MODES.items()):
                ops.fused_layers, ops.fold_norms = fused, fold
                before = ops.launches
                got = step.run([StepEntry(1000 * k + i, [nxt[i]], [0]) for i in range(n)]).float().cpu()
                launches[name] = ops.launches - before
                ops.check_status()
                err = ((got - ref).abs().max() / ref.abs().max()).item()
                worst[name] = max(worst[name], err)
    finally:
        ops.fused_layers, ops.fold_norms = was
    if one_launch:
        assert launches["fused"] <= 6, "the layers did not run as one launch"
    for k in range(len(MODES)):
        for i in range(n):
            step.finish(1000 * k + i)
    assert lm.manager.audit() == ""
    worst["launches"] = launches
    return worst


@pytest.mark.parametrize("name,page,lengths", [
    ("B", 16, [1, 15, 16, 17, 31, 32, 33, 200]),           # 8 rows; the stream warp brings keys and values
    ("B", 16, [63]),                                        # one row: every pair cut into many parts
    ("B", 16, [5, 64, 65, 127, 128, 129, 300, 2, 47, 48, 49]),  # 11 rows: two n-tiles
    ("B", 16, [30 + 7 * i for i in range(16)]),             # 16 rows
    ("B", 8, [1, 7, 8, 9, 33, 150]),                        # pages of 8: the attention fetches keys and values itself
    ("C", 16, [3, 16, 100, 130, 17]),                       # head size 128: four arithmetic warps, one tile a stage
    ("C", 16, [20 + 9 * i for i in range(16)]),             # head size 128, two n-tiles
])
def test_layer_kernel_against_plain_and_parts(tiny_models, name, page, lengths):
    d, cfg, _ = tiny_models[name]
    lm = _load(d, page)
    if not lm.model.stacks:
        pytest.fail("the model planned no stack of layers")
    stack = next(iter(lm.model.stacks.values()))
    assert stack.supports(len(lengths)) and stack.end - stack.first == cfg["num_hidden_layers"]
    worst = _decode_and_compare(lm, cfg, helpers.read_weights(d), lengths, steps=5, seed=len(lengths))
    assert worst["fused"] <= helpers.BF16_TOL, worst
    assert worst["chain"] <= helpers.BF16_TOL, worst
    assert worst["parts"] <= helpers.BF16_TOL, worst
    if 2 <= len(lengths) <= 8:  # the chain has no norm kernels but the first: fewer launches than part by part
        assert worst["launches"]["chain"] < worst["launches"]["parts"], worst


def test_layer_kernel_refuses_widths_that_are_no_multiple_of_64(tiny_models):
    d, cfg, page = tiny_models["A"]  # intermediate 176
    lm = _load(d, page)
    assert all(not s.supports(4) for s in lm.model.stacks.values())
    lm.rt.ops.fused_layers = True
    worst = _decode_and_compare(lm, cfg, helpers.read_weights(d), [5, 9, 30], steps=2, seed=1, one_launch=False)  # runs part by part
    assert max(worst[k] for k in MODES) <= helpers.BF16_TOL


def test_layer_kernel_in_captured_graphs_generates_what_the_plain_model_would(tiny_models):
    from atoma_infer_b200.engine import Engine
    from atoma_infer_b200.sampling import SamplingParams

    d, cfg, _ = tiny_models["B"]
    w = helpers.read_weights(d)
    eng = Engine(d, dtype="bfloat16", block_size=16, num_gpu_blocks_override=400, max_num_sequences=8, cuda_graphs=True)
    eng.lm.rt.ops.fused_layers = True
    prompts = [[1, 2, 3, 4, 5], list(range(10, 60)), [7] * 17, list(range(100, 133))]
    before = eng.lm.step.graph_replays
    outs = eng.generate(prompts, SamplingParams(do_sample=False, max_new_tokens=24, ignore_eos_token=True))
    assert eng.lm.step.graph_replays > before
    for pr, o in zip(prompts, outs):
        assert o.finish_reason == "length" and len(o.token_ids) == 24
        agree, clear = helpers.greedy_agreement(w, cfg, pr, o.token_ids)
        assert clear, "a token differs where the plain logits leave no doubt"
