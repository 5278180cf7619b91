"""Weights: safetensors reading and writing, the loader's errors, the random-weights mode (no GPU)."""
import json
import os
import struct

import pytest
import torch

import trapetum_b200 as tb
from conftest import TINY_A, TINY_B
from trapetum_b200.engine.model import tensor_specs_for_config
from trapetum_b200.weights import (SafetensorsFile, TensorSpec, WeightError, WeightFileError, load_tensors,
                                   write_safetensors)
from trapetum_b200.weights.loader import storage_dtype


def test_written_file_reads_back_with_the_safetensors_library(tmp_path):
    from safetensors.torch import load_file
    tensors = [("a", torch.randn(3, 5).bfloat16()), ("b", torch.randn(7)), ("c", torch.arange(6, dtype=torch.int32).view(2, 3)),
               ("d", torch.randn(2, 2).half())]
    p = str(tmp_path / "x.safetensors")
    write_safetensors(p, tensors, metadata={"format": "pt"})
    lib = load_file(p)
    ours = SafetensorsFile(p)
    assert sorted(ours.names()) == sorted(lib)
    for name, t in tensors:
        assert torch.equal(lib[name], t) and torch.equal(ours.tensor(name), t)
        assert ours.shape(name) == tuple(t.shape) and ours.dtype(name) == t.dtype


def test_library_written_file_reads(tmp_path):
    from safetensors.torch import save_file
    t = {"w": torch.randn(4, 4).bfloat16(), "n": torch.randn(4)}
    p = str(tmp_path / "y.safetensors")
    save_file(t, p)
    f = SafetensorsFile(p)
    assert torch.equal(f.tensor("w"), t["w"]) and torch.equal(f.tensor("n"), t["n"])


def test_truncated_and_garbled_files(tmp_path):
    p = str(tmp_path / "t.safetensors")
    write_safetensors(p, [("a", torch.randn(64, 64))])
    data = open(p, "rb").read()
    open(p, "wb").write(data[:-100])
    with pytest.raises(WeightFileError, match="truncated"):
        SafetensorsFile(p)
    open(p, "wb").write(data[:4])
    with pytest.raises(WeightFileError, match="too short"):
        SafetensorsFile(p)
    open(p, "wb").write(struct.pack("<Q", 10) + b"not json!!" + b"\0" * 16)
    with pytest.raises(WeightFileError, match="JSON"):
        SafetensorsFile(p)
    with pytest.raises(WeightFileError, match="neither"):
        load_tensors(str(tmp_path / "empty"), {}, torch.bfloat16, "cpu")


def test_storage_rules():
    bf, f32 = torch.bfloat16, torch.float32
    assert storage_dtype(torch.bfloat16, "matrix", bf) == bf
    assert storage_dtype(torch.float16, "matrix", bf) == f32          # never rounded in silence: widened, exact
    assert storage_dtype(torch.float16, "matrix", bf, fp16="round") == bf
    assert storage_dtype(torch.float16, "matrix", f32, fp16="round") == f32
    assert storage_dtype(torch.float32, "norm", bf) == f32            # stored in 32 bits: stays so
    assert storage_dtype(torch.int64, "table", bf) == torch.int32      # integer tables become int32
    assert storage_dtype(torch.bfloat16, "matrix", f32) == f32         # the 32-bit engine up-casts


def test_random_model_is_reproducible_and_complete(tmp_path):
    a, b, c = (str(tmp_path / n) for n in "abc")
    tb.write_random_model(a, TINY_A, 0, 0.02, 0.1)
    tb.write_random_model(b, TINY_A, 0, 0.02, 0.1)
    tb.write_random_model(c, TINY_A, 1, 0.02, 0.1)
    fa, fb, fc = (SafetensorsFile(os.path.join(d, "model.safetensors")) for d in (a, b, c))
    wanted = tensor_specs_for_config(TINY_A)
    assert sorted(fa.names()) == sorted(n for n, s in wanted.items() if not s.optional)
    assert json.load(open(os.path.join(a, "config.json"))) == TINY_A
    diff = 0
    for n in fa.names():
        assert fa.dtype(n) == torch.bfloat16 and fa.shape(n) == wanted[n].shape
        assert torch.equal(fa.tensor(n), fb.tensor(n))
        diff += int(not torch.equal(fa.tensor(n), fc.tensor(n)))
    assert diff == len(fa.names())
    e = fa.tensor("model.embed_tokens.weight").float()
    nw = fa.tensor("model.layers.0.input_layernorm.weight").float()
    assert 0.015 < float(e.std()) < 0.025 and 0.05 < float(nw.std()) < 0.15


def test_loading_dtypes(tmp_path):
    d = str(tmp_path / "m")
    tb.write_random_model(d, TINY_A, 0, norm_dtype=torch.float32)
    wanted = tensor_specs_for_config(TINY_A)
    t = load_tensors(d, wanted, torch.bfloat16, "cpu")
    assert t["model.embed_tokens.weight"].dtype == torch.bfloat16
    assert t["model.norm.weight"].dtype == torch.float32
    assert "lm_head.weight" not in t
    t32 = load_tensors(d, wanted, torch.float32, "cpu")
    assert all(v.dtype == torch.float32 for v in t32.values())
    assert torch.equal(t32["model.embed_tokens.weight"], t["model.embed_tokens.weight"].float())


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    from safetensors.torch import load_file, save_file
    d = str(tmp_path / "m")
    tb.write_random_model(d, TINY_A, 0)
    p = os.path.join(d, "model.safetensors")
    w = load_file(p)
    del w["model.layers.1.mlp.up_proj.weight"]
    del w["model.norm.weight"]
    w["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(64, dtype=torch.bfloat16)
    w["model.layers.0.mlp.down_proj.weight"] = torch.zeros(64, 127, dtype=torch.bfloat16)
    w["model.layers.0.input_layernorm.weight"] = torch.zeros(64, dtype=torch.int32)
    save_file(w, p)
    with pytest.raises(WeightError) as ei:
        load_tensors(d, tensor_specs_for_config(TINY_A), torch.bfloat16, "cpu")
    e = ei.value
    assert e.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert e.unexpected == ["model.layers.0.self_attn.q_proj.bias"]
    assert [(n, tuple(g), tuple(x)) for n, g, x in e.wrong_shape] == \
        [("model.layers.0.mlp.down_proj.weight", (64, 127), (64, 128))]
    assert [n for n, _, _ in e.wrong_kind] == ["model.layers.0.input_layernorm.weight"]
    msg = str(e)
    for part in ("missing (2)", "unexpected (1)", "wrong shape (1)", "q_proj.bias", "[64, 127]", "[64, 128]"):
        assert part in msg


def test_weights_of_another_config_do_not_fit(tmp_path):
    d = str(tmp_path / "m")
    tb.write_random_model(d, TINY_A, 0)
    with pytest.raises(WeightError, match="wrong shape"):
        load_tensors(d, tensor_specs_for_config(TINY_B), torch.bfloat16, "cpu")


def test_untied_head_is_required_when_not_tied(tmp_path):
    cfg = dict(TINY_A, tie_word_embeddings=False)
    specs = tensor_specs_for_config(cfg)
    assert not specs["lm_head.weight"].optional
    d = str(tmp_path / "m")
    tb.write_random_model(d, cfg, 0)
    assert "lm_head.weight" in load_tensors(d, specs, torch.bfloat16, "cpu")


def test_sharded_folder(tmp_path):
    from safetensors.torch import load_file, save_file
    d = str(tmp_path / "m")
    tb.write_random_model(d, TINY_A, 0)
    w = load_file(os.path.join(d, "model.safetensors"))
    os.unlink(os.path.join(d, "model.safetensors"))
    names = sorted(w)
    half = len(names) // 2
    save_file({n: w[n] for n in names[:half]}, os.path.join(d, "model-00001-of-00002.safetensors"))
    save_file({n: w[n] for n in names[half:]}, os.path.join(d, "model-00002-of-00002.safetensors"))
    wm = {n: ("model-00001-of-00002.safetensors" if i < half else "model-00002-of-00002.safetensors")
          for i, n in enumerate(names)}
    json.dump({"weight_map": wm}, open(os.path.join(d, "model.safetensors.index.json"), "w"))
    t = load_tensors(d, tensor_specs_for_config(TINY_A), torch.bfloat16, "cpu")
    assert all(torch.equal(t[n], w[n]) for n in names)


def test_golden_reader_of_the_reference(tmp_path):
    """tests/golden/safetensors_reader.json holds what neuralboot/trapetum's own pure-numpy reader
    (model/export_safetensors.py:24-48) returned for the folder that write_random_model makes for
    Tiny A, seed 0 (made once by tests/golden/make_safetensors_golden.py).  Our reader must see the same."""
    golden = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "safetensors_reader.json")))
    d = str(tmp_path / "m")
    tb.write_random_model(d, TINY_A, 0, 0.02, 0.1)
    f = SafetensorsFile(os.path.join(d, "model.safetensors"))
    assert sorted(f.names()) == sorted(golden)
    for name, g in golden.items():
        t = f.tensor(name).float()
        assert list(t.shape) == g["shape"]
        assert float(t.double().sum()) == pytest.approx(g["sum"], rel=1e-12, abs=1e-12)
        assert float(t.double().abs().sum()) == pytest.approx(g["abs_sum"], rel=1e-12)
        assert [float(x) for x in t.reshape(-1)[:4]] == g["first"]


def test_float16_tensors_are_widened_rounded_or_refused_never_rounded_in_silence(tmp_path):
    from trapetum_b200.weights import WeightError, load_tensors, write_safetensors
    d = str(tmp_path)
    x = torch.tensor([[1.0 + 2.0 ** -10, 3.0]], dtype=torch.float16)          # the first value does not fit bfloat16
    write_safetensors(d + "/model.safetensors", [("w", x), ("n", torch.ones(2, dtype=torch.bfloat16))])
    wanted = {"w": TensorSpec((1, 2)), "n": TensorSpec((2,), "norm")}
    t = load_tensors(d, wanted, torch.bfloat16, "cpu")
    assert t["w"].dtype == torch.float32 and torch.equal(t["w"], x.float()) and t["n"].dtype == torch.bfloat16
    t = load_tensors(d, wanted, torch.bfloat16, "cpu", fp16="round")
    assert t["w"].dtype == torch.bfloat16 and float(t["w"][0, 0]) == 1.0
    with pytest.raises(WeightError, match="float16"):
        load_tensors(d, wanted, torch.bfloat16, "cpu", fp16="refuse")
    assert load_tensors(d, wanted, torch.float32, "cpu", fp16="refuse")["w"].dtype == torch.float32
    with pytest.raises(ValueError, match="fp16"):
        load_tensors(d, wanted, torch.bfloat16, "cpu", fp16="maybe")
