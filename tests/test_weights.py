"""Safetensors reading and writing, loader errors, random-weights mode (no GPU)."""
import json
import os

import pytest
import torch

import helpers
from atoma_infer_b200.config import architecture_of
from atoma_infer_b200.parts import declared_tensors
from atoma_infer_b200.weights import (SafetensorsError, SafetensorsFile, WeightError, load_tensors,
                                      write_random_model, write_safetensors)


def _load(d, dtype=torch.float32):
    arch, cfg = architecture_of(d)
    spec = arch.build_spec(cfg)
    return load_tensors(d, declared_tensors(spec), dtype=dtype, device="cpu", ignore=spec.ignored_tensors)


def test_safetensors_round_trip(tmp_path):
    t = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int32).reshape(2, 3)}
    p = str(tmp_path / "x.safetensors")
    write_safetensors(p, t, {"k": "v"})
    f = SafetensorsFile(p)
    assert sorted(f.names()) == ["a", "b", "c"] and f.metadata == {"k": "v"}
    for n in t:
        assert f.dtype(n) == t[n].dtype and torch.equal(f.tensor(n), t[n])
    (tmp_path / "bad.safetensors").write_bytes(b"\x05\x00")
    with pytest.raises(SafetensorsError):
        SafetensorsFile(str(tmp_path / "bad.safetensors"))


def test_safetensors_files_agree_with_the_format_library_both_ways(tmp_path):
    """Files written here are read by the ``safetensors`` package (the format's own library) and files it
    writes are read here, tensor for tensor: the round trip above alone would also pass with a private
    format.  Skipped where the package is not installed."""
    st = pytest.importorskip("safetensors.torch")
    t = {"w.a": torch.randn(4, 6), "w.b": torch.randn(5, 3).to(torch.bfloat16), "n": torch.randn(9).to(torch.float16),
         "i": torch.arange(12, dtype=torch.int32).reshape(3, 4), "s": torch.tensor(2.5)}
    ours, theirs = str(tmp_path / "ours.safetensors"), str(tmp_path / "theirs.safetensors")
    write_safetensors(ours, t, {"format": "pt"})
    back = st.load_file(ours)
    assert sorted(back) == sorted(t)
    for n in t:
        assert back[n].dtype == t[n].dtype and back[n].shape == t[n].shape and torch.equal(back[n], t[n])
    st.save_file(t, theirs, metadata={"format": "pt"})
    f = SafetensorsFile(theirs)
    assert sorted(f.names()) == sorted(t) and f.metadata == {"format": "pt"}
    for n in t:
        assert f.dtype(n) == t[n].dtype and tuple(f.shape(n)) == tuple(t[n].shape) and torch.equal(f.tensor(n), t[n])


def test_random_model_is_seeded_and_loads(tmp_path):
    a, b, c = (str(tmp_path / n) for n in "abc")
    write_random_model(a, helpers.CONFIG_A, 0)
    write_random_model(b, helpers.CONFIG_A, 0)
    write_random_model(c, helpers.CONFIG_A, 1)
    wa, wb, wc = _load(a), _load(b), _load(c)
    assert sorted(os.listdir(a)) == ["config.json", "model.safetensors"]
    assert all(torch.equal(wa[n], wb[n]) for n in wa)
    assert not torch.equal(wa["model.embed_tokens.weight"], wc["model.embed_tokens.weight"])
    assert torch.all(wa["model.norm.weight"] == 1)
    assert abs(float(wa["model.layers.0.mlp.up_proj.weight"].std()) - 0.02) < 2e-3
    assert "lm_head.weight" not in wa  # tied


def test_dtypes_kept(tmp_path):
    d = str(tmp_path / "m")
    write_random_model(d, helpers.CONFIG_B, 0, dtype=torch.bfloat16)
    w16 = _load(d, torch.bfloat16)
    assert all(t.dtype == torch.bfloat16 for t in w16.values())
    w32 = _load(d, torch.float32)
    assert all(t.dtype == torch.float32 for t in w32.values())
    assert torch.equal(w32["lm_head.weight"], w16["lm_head.weight"].float())  # widened exactly
    d32 = str(tmp_path / "m32")
    write_random_model(d32, helpers.CONFIG_B, 0, dtype=torch.float32)
    assert all(t.dtype == torch.float32 for t in _load(d32, torch.bfloat16).values())  # stored in 32 bits: stays so


def test_one_error_lists_missing_unexpected_and_wrong(tmp_path):
    d = str(tmp_path / "m")
    write_random_model(d, helpers.CONFIG_B, 0)
    f = SafetensorsFile(os.path.join(d, "model.safetensors"))
    t = {n: f.tensor(n).clone() for n in f.names()}
    del t["model.layers.1.self_attn.k_proj.weight"], t["model.norm.weight"]
    t["model.layers.2.mlp.down_proj.weight"] = torch.zeros(5, 5, dtype=torch.bfloat16)
    t["model.layers.7.extra.weight"] = torch.zeros(2)
    t["model.layers.0.input_layernorm.weight"] = torch.zeros(192, dtype=torch.int32)
    write_safetensors(os.path.join(d, "model.safetensors"), t)
    with pytest.raises(WeightError) as e:
        _load(d)
    err = e.value
    assert [n for n, _ in err.missing] == ["model.layers.1.self_attn.k_proj.weight", "model.norm.weight"]
    assert [n for n, _ in err.unexpected] == ["model.layers.7.extra.weight"]
    assert sorted(n for n, _ in err.wrong) == ["model.layers.0.input_layernorm.weight", "model.layers.2.mlp.down_proj.weight"]
    msg = str(err)
    for word in ("k_proj", "extra", "down_proj", "[192, 320]", "[5, 5]", "torch.int32"):
        assert word in msg


def test_tied_checkpoint_may_store_the_head_and_untied_must(tmp_path):
    d = str(tmp_path / "m")
    write_random_model(d, helpers.CONFIG_A, 0)
    f = SafetensorsFile(os.path.join(d, "model.safetensors"))
    t = {n: f.tensor(n).clone() for n in f.names()}
    t["lm_head.weight"] = t["model.embed_tokens.weight"].clone()
    write_safetensors(os.path.join(d, "model.safetensors"), t)
    _load(d)  # ignored, no error
    cfg = dict(helpers.CONFIG_A, tie_word_embeddings=False)
    del t["lm_head.weight"]
    write_safetensors(os.path.join(d, "model.safetensors"), t)
    with open(os.path.join(d, "config.json"), "w") as fh:
        json.dump(cfg, fh)
    with pytest.raises(WeightError) as e:
        _load(d)
    assert "lm_head.weight" in str(e.value)


def test_sharded_folder_with_index(tmp_path):
    d = str(tmp_path / "m")
    write_random_model(d, helpers.CONFIG_A, 0)
    whole = _load(d)
    f = SafetensorsFile(os.path.join(d, "model.safetensors"))
    names = sorted(f.names())
    half = len(names) // 2
    parts = {"model-00001-of-00002.safetensors": names[:half], "model-00002-of-00002.safetensors": names[half:]}
    for fn, ns in parts.items():
        write_safetensors(os.path.join(d, fn), {n: f.tensor(n).clone() for n in ns})
    with open(os.path.join(d, "model.safetensors.index.json"), "w") as fh:
        json.dump({"weight_map": {n: fn for fn, ns in parts.items() for n in ns}}, fh)
    del f
    os.remove(os.path.join(d, "model.safetensors"))
    again = _load(d)
    assert all(torch.equal(whole[n], again[n]) for n in whole)
