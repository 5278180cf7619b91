"""The native host's parts that need no GPU, through its C interface: the spec it builds from a config.json
against the Python side's, its one error for weights that do not fit, its cache bookkeeping (no slot or page
lost, held twice or freed twice) against the Python cache on the same random walk, and its batch planning."""
import ctypes
import json
import random

import pytest
import torch

from conftest import TINY_A, TINY_B, TINY_C


@pytest.fixture(scope="module")
def L():
    from trapetum_b200 import native
    lib = native.lib()
    lib.tb_spec_from_config.restype = ctypes.c_char_p
    lib.tb_sim_cache_new.restype = ctypes.c_void_p
    lib.tb_sim_cache_length.restype = ctypes.c_longlong
    lib.tb_sim_cache_epoch.restype = ctypes.c_longlong
    lib.tb_sim_cache_free.argtypes = [ctypes.c_void_p]
    return lib


def same(a, b, path=""):
    """Two JSON values are the same up to the last bit of a float."""
    if isinstance(a, dict) and isinstance(b, dict):
        assert set(a) == set(b), f"{path}: keys {sorted(set(a) ^ set(b))} differ"
        for k in a:
            same(a[k], b[k], f"{path}.{k}")
    elif isinstance(a, list) and isinstance(b, list):
        assert len(a) == len(b), path
        for i, (x, y) in enumerate(zip(a, b)):
            same(x, y, f"{path}[{i}]")
    elif isinstance(a, (int, float)) and isinstance(b, (int, float)) and not isinstance(a, bool) and not isinstance(b, bool):
        assert a == pytest.approx(b, rel=1e-15, abs=0), f"{path}: {a!r} != {b!r}"
    else:
        assert a == b, f"{path}: {a!r} != {b!r}"


REAL_27B = dict(TINY_A, num_hidden_layers=4, hidden_size=4608, num_attention_heads=32, num_key_value_heads=16, head_dim=128,
                intermediate_size=36864, vocab_size=256000, query_pre_attn_scalar=144, sliding_window=4096, eos_token_id=[1, 107],
                layer_types=["full_attention", "sliding_attention", "sliding_attention", "full_attention"])


@pytest.mark.parametrize("cfg", [TINY_A, TINY_B, TINY_C, REAL_27B, dict(TINY_B, sliding_window=None, tie_word_embeddings=False)])
def test_native_gemma2_spec_is_the_python_side_s(L, cfg):
    import trapetum_b200 as tb
    from trapetum_b200.config.base import spec_to_json
    text = L.tb_spec_from_config(json.dumps(cfg).encode())
    assert text, L.tb_last_error().decode()
    same(json.loads(text), json.loads(spec_to_json(tb.load_config(cfg)[1])))


def test_native_config_errors_name_the_key(L):
    for bad, key in ((dict(TINY_A, head_dim=15), "head_dim"), ({k: v for k, v in TINY_A.items() if k != "vocab_size"}, "vocab_size"),
                     (dict(TINY_A, num_key_value_heads=3), "num_key_value_heads"), (dict(TINY_A, hidden_activation="relu"), "hidden_activation"),
                     (dict(TINY_A, architectures=["NoSuchLM"]), "NoSuchLM"), (dict(TINY_A, sliding_window=0), "sliding_window")):
        assert L.tb_spec_from_config(json.dumps(bad).encode()) is None
        assert key in L.tb_last_error().decode()


def test_native_weight_check_lists_everything_that_does_not_fit(L, tmp_path):
    import trapetum_b200 as tb
    from safetensors.torch import load_file, save_file
    from trapetum_b200.config.base import spec_to_json
    d = str(tmp_path / "m")
    tb.write_random_model(d, TINY_A, 0, device="cpu")
    spec = spec_to_json(tb.load_config(d)[1]).encode()
    assert L.tb_check_weights(d.encode(), spec, b"bfloat16", None) == 0, L.tb_last_error().decode()
    w = load_file(d + "/model.safetensors")
    w["model.layers.1.mlp.up_proj.weight"] = torch.zeros(5, 7, dtype=torch.bfloat16)
    del w["model.layers.0.self_attn.k_proj.weight"]
    w["extra.tensor"] = torch.zeros(2)
    w["model.norm.weight"] = torch.zeros(64, dtype=torch.int32)
    w["model.layers.0.mlp.gate_proj.weight"] = w["model.layers.0.mlp.gate_proj.weight"].to(torch.float16)
    save_file(w, d + "/model.safetensors")
    assert L.tb_check_weights(d.encode(), spec, b"bfloat16", b"refuse") != 0
    msg = L.tb_last_error().decode()
    for piece in ("missing (1): model.layers.0.self_attn.k_proj.weight", "unexpected (1): extra.tensor",
                  "model.layers.1.mlp.up_proj.weight is [5, 7], expected [128, 64]", "model.norm.weight is I32",
                  "model.layers.0.mlp.gate_proj.weight is float16"):
        assert piece in msg, msg
    with open(d + "/model.safetensors", "r+b") as f:
        f.truncate(4000)
    assert L.tb_check_weights(d.encode(), spec, b"bfloat16", None) != 0 and "truncated" in L.tb_last_error().decode()
    assert L.tb_check_weights(str(tmp_path).encode(), spec, b"bfloat16", None) != 0 and "neither" in L.tb_last_error().decode()


def test_native_cache_walks_like_the_python_cache(L):
    """The same random sequence of claims, growths, shrinks and releases on both caches: same slots, same pages,
    same refusals, and the invariants hold after every move."""
    from trapetum_b200.cache import Cache, CacheError, CacheFull
    from trapetum_b200.parts import KVNeed
    needs = {0: KVNeed(2, 16, 100), 1: KVNeed(2, 16, None), 2: KVNeed(2, 16, 100), 3: KVNeed(4, 32, None)}
    py = Cache(needs, {}, 64 * 24, torch.bfloat16, "cpu", 6)
    spec = [{"entry": e, "n_kv_heads": n.n_kv_heads, "head_dim": n.head_dim, "window": n.window or 0} for e, n in needs.items()]
    nat = ctypes.c_void_p(L.tb_sim_cache_new(json.dumps(spec).encode(), ctypes.c_longlong(64 * 24), 6))
    assert nat, L.tb_last_error().decode()
    n_groups = L.tb_sim_cache_groups(nat)
    assert n_groups == len(py.groups) == 3
    # groups may be numbered differently: match them by the pages a first sequence gets
    I = ctypes.c_int
    rng = random.Random(3)
    live = []
    buf = (I * 64)()

    def pages_native(slot):
        out = []
        for g in range(n_groups):
            n = L.tb_sim_cache_pages(nat, slot, g, buf, 64)
            out.append(tuple(buf[:n]))
        return sorted(out)

    for move in range(600):
        kind = rng.choice(["claim", "grow", "grow", "grow", "release", "shrink", "bad"])
        if kind == "claim":
            try:
                s = py.claim()
            except CacheFull:
                assert L.tb_sim_cache_claim(nat) == -1
                continue
            assert L.tb_sim_cache_claim(nat) == s
            live.append(s)
        elif kind == "grow" and live:
            who = rng.sample(live, rng.randint(1, len(live)))
            by = [rng.choice([1, 1, 1, 30, 64, 200]) for _ in who]
            try:
                py.grow(dict(zip(who, by)))
                ok = True
            except CacheFull:
                ok = False
            st = L.tb_sim_cache_grow(nat, (I * len(who))(*who), (I * len(who))(*by), len(who))
            assert (st == 0) == ok, L.tb_last_error().decode()
            if not ok:
                assert st == 3 and "full" in L.tb_last_error().decode()
        elif kind == "shrink" and live:
            s = rng.choice(live)
            by = rng.randint(0, py.length(s))
            py.shrink({s: by})
            assert L.tb_sim_cache_shrink(nat, (I * 1)(s), (I * 1)(by), 1) == 0
        elif kind == "release" and live:
            s = live.pop(rng.randrange(len(live)))
            py.release(s)
            assert L.tb_sim_cache_release(nat, s) == 0
        elif kind == "bad":
            s = rng.choice([x for x in range(8) if x not in live])
            with pytest.raises(CacheError):
                py.release(s)
            assert L.tb_sim_cache_release(nat, s) != 0 and "not held" in L.tb_last_error().decode()
        py.check()
        assert L.tb_sim_cache_check(nat) == 0, L.tb_last_error().decode()
        for s in live:
            assert L.tb_sim_cache_length(nat, s) == py.length(s)
            assert pages_native(s) == sorted(tuple(py.pages(s, g)) for g in range(n_groups))
    assert L.tb_sim_cache_epoch(nat) == py.epoch
    L.tb_sim_cache_free(nat)


def test_native_batch_planning_is_the_python_side_s(L):
    from trapetum_b200.engine.generate import plan_batches
    rng = random.Random(1)
    I = ctypes.c_int
    for _ in range(50):
        lens = [rng.randint(1, 300) for _ in range(rng.randint(1, 12))]
        max_new, max_batch, max_tokens, max_pos = rng.randint(1, 100), rng.randint(1, 5), 64 * rng.randint(8, 40), rng.choice([256, 8192])
        out = (I * len(lens))()
        try:
            want = plan_batches(lens, max_new, max_batch, max_tokens, max_pos)
        except ValueError as e:
            assert L.tb_plan_batches((I * len(lens))(*lens), len(lens), max_new, max_batch, ctypes.c_longlong(max_tokens), max_pos, out) == -1
            assert str(e).split(":")[0] in L.tb_last_error().decode()
            continue
        n = L.tb_plan_batches((I * len(lens))(*lens), len(lens), max_new, max_batch, ctypes.c_longlong(max_tokens), max_pos, out)
        assert n == len(want) and [[i for i in range(len(lens)) if out[i] == b] for b in range(n)] == want


def test_native_decode_launch_shapes_are_the_python_side_s(L):
    """Bucket, unevenness, pieces and partition of a decode step: both hosts must choose alike, or their steps would
    not give the same bits."""
    from trapetum_b200.csrc.ops import PAGE_ROWS, choose_decode_splits, decode_partition_is_stream
    from trapetum_b200.engine.engine import len_bucket, unevenness
    rng = random.Random(2)
    I = ctypes.c_int
    for _ in range(300):
        n = rng.choice([1, 2, 3, 8, 17, 64])
        top = rng.choice([5, 70, 600, 3000, 8192])
        lens = [rng.randint(1, top) for _ in range(n)]
        if rng.random() < 0.3:
            lens = [top] * n
        n_kv, ring, sms = rng.choice([1, 2, 4, 8, 16]), rng.choice([0, 0, 128, 4096]), rng.choice([148, 132, 64])
        out = (I * 3)()
        stream = L.tb_decode_launch_shape((I * n)(*lens), n, n_kv, ring, sms, out)
        bucket = len_bucket(max(lens))
        rows = min(bucket, ring) if ring else bucket
        pages = max(1, (rows + PAGE_ROWS - 1) // PAGE_ROWS)
        splits = choose_decode_splits(n, n_kv, pages, sms)
        assert [out[0], out[1], out[2]] == [bucket, unevenness(lens), splits], (lens, n_kv, ring, sms)
        assert stream == int(decode_partition_is_stream(n, n_kv, pages, splits, unevenness(lens), sms))
