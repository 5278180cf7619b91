"""The counter-based random weights: the library's host version (numpy) and device version (CUDA) against
the plain one-element-at-a-time statement in tests/plain_random.py, bit for bit."""
import json
import os

import numpy as np
import pytest
import torch

import plain_random
from conftest import TINY_A, TINY_B


def bits(x) -> int:
    return int(np.asarray(x, dtype=np.float32).view(np.uint32))


def sample_indices(n: int, seed: int):
    """The first and last elements, the ends of a 4-element generator block, and a few random places."""
    rng = np.random.default_rng(seed)
    fixed = [0, 1, 2, 3, 4, 5, n - 1, n - 2, n // 2, n // 2 + 1]
    return sorted({i for i in fixed + rng.integers(0, n, 12).tolist() if 0 <= i < n})


def test_host_version_equals_the_plain_one_on_every_tensor():
    from trapetum_b200.engine import tensor_specs_for_config
    from trapetum_b200.weights.random_init import name_key, normal_host
    for cfg, seed, std in ((TINY_A, 0, 0.02), (TINY_B, 123456789012345, 0.3)):
        for name, spec in tensor_specs_for_config(cfg).items():
            n = int(np.prod(spec.shape))
            assert name_key(seed, name) == plain_random.key_of(seed, name)
            got = normal_host(n, name_key(seed, name), std)
            for i in sample_indices(n, len(name)):
                assert bits(got[i]) == bits(plain_random.element(seed, name, i, std)), (name, i)


def test_values_depend_on_name_seed_and_index_only_and_look_normal():
    from trapetum_b200.weights.random_init import name_key, normal_host
    a = normal_host(4096, name_key(3, "x.weight"), 1.0)
    assert np.array_equal(a[1024:2048], normal_host(1024, name_key(3, "x.weight"), 1.0, first=1024))   # any piece, any order
    assert not np.array_equal(a, normal_host(4096, name_key(4, "x.weight"), 1.0))
    assert not np.array_equal(a, normal_host(4096, name_key(3, "y.weight"), 1.0))
    far = 4 * ((1 << 33) // 4 + 7)                       # the counter's upper word
    w = normal_host(8, name_key(3, "x.weight"), 0.5, first=far)
    assert all(bits(w[j]) == bits(plain_random.element(3, "x.weight", far + j, 0.5)) for j in range(8))
    x = normal_host(1 << 20, name_key(1, "big"), 1.0).astype(np.float64)
    assert abs(x.mean()) < 5e-3 and abs(x.var() - 1.0) < 1e-2
    assert abs(((x - x.mean()) ** 4).mean() / x.var() ** 2 - 3.0) < 0.05          # a normal's fourth moment
    assert 4.0 < np.abs(x).max() < 6.5                                            # tails are there, nothing absurd
    assert np.all((x.astype(np.float32).view(np.uint32) & 0xFFFF) == 0)           # bfloat16 values


def test_folder_is_written_tensor_by_tensor_and_reads_back(tmp_path):
    import trapetum_b200 as tb
    from trapetum_b200.weights import open_model_files, write_safetensors
    from trapetum_b200.weights.random_init import name_key, normal_host
    d = str(tmp_path / "m")
    tb.write_random_model(d, TINY_B, 7, 0.03, 0.2, device="cpu")
    files = open_model_files(d)
    name = "model.layers.2.mlp.down_proj.weight"
    t = files[name].tensor(name)
    want = normal_host(t.numel(), name_key(7, name), 0.03).reshape(t.shape)
    assert t.dtype == torch.bfloat16 and np.array_equal(t.float().numpy(), want)
    norm = "model.norm.weight"
    assert np.array_equal(files[norm].tensor(norm).float().numpy(), normal_host(96, name_key(7, norm), 0.2))
    # a layout that the tensors do not follow is an error, not a corrupt file
    from trapetum_b200.weights import WeightFileError
    with pytest.raises(WeightFileError, match="expected 'b'"):
        write_safetensors(str(tmp_path / "x.safetensors"), iter([("a", torch.zeros(2)), ("c", torch.zeros(2))]),
                          layout=[("a", torch.float32, (2,)), ("b", torch.float32, (2,))])
    with pytest.raises(WeightFileError, match="end before"):
        write_safetensors(str(tmp_path / "y.safetensors"), iter([("a", torch.zeros(2))]),
                          layout=[("a", torch.float32, (2,)), ("b", torch.float32, (2,))])
    assert not os.path.exists(tmp_path / "x.safetensors")


def test_stop_ids_come_from_generation_config_and_config_together(tmp_path):
    import trapetum_b200 as tb
    d = str(tmp_path / "m")
    os.makedirs(d)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(dict(TINY_A, eos_token_id=1), f)
    assert tb.load_config(d)[1].stop_ids == (1,)
    with open(os.path.join(d, "generation_config.json"), "w") as f:
        json.dump({"eos_token_id": [107, 1]}, f)
    assert tb.load_config(d)[1].stop_ids == (1, 107)
    with open(os.path.join(d, "generation_config.json"), "w") as f:
        json.dump({"eos_token_id": "x"}, f)
    with pytest.raises(tb.ConfigError, match="generation_config.json"):
        tb.load_config(d)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_device_version_equals_the_plain_one_on_every_tensor(dtype):
    from trapetum_b200.engine import tensor_specs_for_config
    from trapetum_b200.weights.random_init import fill_normal, name_key, normal_host
    for cfg, seed, std in ((TINY_A, 0, 0.02), (TINY_B, 99, 0.3)):
        for name, spec in tensor_specs_for_config(cfg).items():
            t = fill_normal(torch.empty(spec.shape, dtype=dtype, device="cuda"), seed, name, std)
            flat = t.float().cpu().reshape(-1).numpy()
            for i in sample_indices(flat.size, len(name)):
                assert bits(flat[i]) == bits(plain_random.element(seed, name, i, std)), (name, i)
    # a tensor of a real model's size, every element against the host version
    n = 2304 * 9216 + 3
    t = fill_normal(torch.empty(n, dtype=dtype, device="cuda"), 2, "model.layers.0.mlp.down_proj.weight", 0.02)
    want = normal_host(n, name_key(2, "model.layers.0.mlp.down_proj.weight"), 0.02)
    assert np.array_equal(t.float().cpu().numpy(), want)


@pytest.mark.gpu
def test_model_made_on_the_device_is_the_model_of_the_folder(tmp_path):
    import trapetum_b200 as tb
    d = str(tmp_path / "m")
    tb.write_random_model(d, TINY_B, 11, 0.03, 0.2, device="cpu")
    prompts = [[5, 9, 200, 3, 77], [1]]
    for dtype in ("bfloat16", "float32"):
        a = tb.load_model(d, dtype)
        b = tb.random_model(TINY_B, 11, 0.03, 0.2, dtype)
        outs = []
        for m in (a, b):
            eng = tb.Engine(m, max_tokens=128)
            s = eng.start(2)
            outs.append(eng.step(s, prompts, [[0, 4], [0]]).cpu())
            eng.release(s)
        assert torch.equal(outs[0], outs[1])
