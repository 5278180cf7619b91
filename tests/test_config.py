"""Configuration and registry (no GPU)."""
import copy
import json

import pytest

import trapetum_b200  # noqa: F401
from conftest import TINY_A, TINY_B, TINY_C
from trapetum_b200.config import (ConfigError, Gemma2Config, ModelSpec, PartSpec, ScheduleEntry, known_architectures,
                                  load_config, register_architecture)
from trapetum_b200.models.gemma2 import gemma2_spec


def test_reads_every_key():
    cfg, spec = load_config(TINY_B)
    assert isinstance(cfg, Gemma2Config)
    assert (cfg.num_hidden_layers, cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads,
            cfg.head_dim, cfg.intermediate_size, cfg.vocab_size) == (3, 96, 6, 1, 32, 160, 384)
    assert cfg.rope_theta == 1000.0 and cfg.sliding_window == 16 and cfg.rms_norm_eps == 1e-5
    assert cfg.attn_logit_softcapping is None and cfg.final_logit_softcapping == 15.0
    assert cfg.attention_scale == pytest.approx(32 ** -0.5)
    assert len(spec.layers) == 3 and [e.layer for e in spec.schedule] == [0, 1, 2]


def test_scale_comes_from_query_pre_attn_scalar_not_head_dim():
    cfg, spec = load_config(TINY_C)
    assert cfg.head_dim == 48 and cfg.attention_scale == pytest.approx(24 ** -0.5)
    assert spec.layers[0].mixer.params["scale"] == pytest.approx(24 ** -0.5)


def test_even_layers_slide_odd_layers_do_not():
    _, spec = load_config(TINY_C)
    assert [l.mixer.params["window"] for l in spec.layers] == [70, None, 70, None]


def test_layer_types_in_config_win():
    d = dict(TINY_A, layer_types=["full_attention", "sliding_attention"])
    _, spec = load_config(d)
    assert [l.mixer.params["window"] for l in spec.layers] == [None, 8]


def test_defaults():
    d = {k: v for k, v in TINY_A.items() if k not in ("rope_theta", "query_pre_attn_scalar", "rms_norm_eps",
                                                      "attn_logit_softcapping", "final_logit_softcapping")}
    cfg, _ = load_config(d)
    assert cfg.rope_theta == 10000.0 and cfg.query_pre_attn_scalar == 16.0 and cfg.rms_norm_eps == 1e-6
    assert cfg.attn_logit_softcapping is None and cfg.final_logit_softcapping is None


def test_zero_cap_means_off():
    cfg, spec = load_config(dict(TINY_A, attn_logit_softcapping=0.0, final_logit_softcapping=0))
    assert cfg.attn_logit_softcapping is None and spec.head.params["softcap"] is None


@pytest.mark.parametrize("key", ["num_hidden_layers", "hidden_size", "num_attention_heads", "head_dim",
                                 "intermediate_size", "vocab_size"])
def test_missing_key_is_named(key):
    d = {k: v for k, v in TINY_A.items() if k != key}
    with pytest.raises(ConfigError, match=key):
        load_config(d)


@pytest.mark.parametrize("key,bad", [("hidden_size", "64"), ("num_hidden_layers", 0), ("head_dim", 15),
                                     ("rms_norm_eps", -1.0), ("vocab_size", 2.5), ("sliding_window", 0),
                                     ("hidden_activation", "relu"), ("rope_theta", 0)])
def test_bad_value_is_named(key, bad):
    with pytest.raises(ConfigError, match=key):
        load_config(dict(TINY_A, **{key: bad}))


def test_heads_must_divide():
    with pytest.raises(ConfigError, match="num_key_value_heads"):
        load_config(dict(TINY_A, num_attention_heads=4, num_key_value_heads=3))


def test_unknown_architecture_lists_known():
    with pytest.raises(ConfigError, match="Gemma2ForCausalLM"):
        load_config(dict(TINY_A, architectures=["NoSuchModel"]))
    assert "Gemma2ForCausalLM" in known_architectures()


def test_eos_number_or_list():
    assert load_config(dict(TINY_A, eos_token_id=1))[1].stop_ids == (1,)
    assert load_config(dict(TINY_A, eos_token_id=[1, 107]))[1].stop_ids == (1, 107)
    with pytest.raises(ConfigError, match="eos_token_id"):
        load_config(dict(TINY_A, eos_token_id="x"))


def test_to_dict_round_trip():
    cfg, _ = load_config(TINY_C)
    again, _ = load_config(json.loads(json.dumps(cfg.to_dict())))
    assert again == cfg


def test_config_json_from_folder(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    cfg, _ = load_config(str(tmp_path))
    assert cfg.hidden_size == 64
    with pytest.raises(ConfigError, match="config.json"):
        load_config(str(tmp_path / "nothing"))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="JSON"):
        load_config(str(tmp_path))


def test_schedule_is_validated():
    cfg, spec = load_config(TINY_A)
    def with_schedule(s):
        return ModelSpec(**{**spec.__dict__, "schedule": tuple(s)})
    with_schedule([ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0, cache_of=0)]).validate()
    with pytest.raises(ConfigError, match="layer 5"):
        with_schedule([ScheduleEntry(5)]).validate()
    with pytest.raises(ConfigError, match="earlier"):
        with_schedule([ScheduleEntry(0, cache_of=0)]).validate()
    with pytest.raises(ConfigError, match="does not own"):
        with_schedule([ScheduleEntry(0), ScheduleEntry(1, cache_of=0), ScheduleEntry(0, cache_of=1)]).validate()


def test_registering_an_architecture():
    class C(Gemma2Config):
        pass
    register_architecture("TestOnlyArch", C, gemma2_spec)
    cfg, spec = load_config(dict(TINY_A, architectures=["TestOnlyArch"]))
    assert isinstance(cfg, C) and len(spec.layers) == 2


def test_no_size_is_fixed_in_the_spec():
    """Every number of the spec traces back to config.json: change a key, the spec changes."""
    _, a = load_config(TINY_A)
    for key, val in (("hidden_size", 80), ("intermediate_size", 144), ("vocab_size", 300), ("head_dim", 32),
                     ("rope_theta", 123.0), ("rms_norm_eps", 1e-3), ("sliding_window", 5),
                     ("attn_logit_softcapping", 7.0), ("final_logit_softcapping", 9.0),
                     ("query_pre_attn_scalar", 99)):
        _, b = load_config(dict(TINY_A, **{key: val}))
        assert repr(a) != repr(b), key
