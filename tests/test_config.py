"""Configuration and registry (no GPU)."""
import json

import pytest

from conftest import TINY
from mimirmind_b200.config.engine_config import EngineConfigError, parse_engine_config
from mimirmind_b200.config.model_config import ConfigError, parse_qwen2_config
from mimirmind_b200.registry import RegistryError, get_architecture, is_supported_architecture


def test_parse_reads_every_size_from_the_file():
    c = parse_qwen2_config(TINY["B"])
    assert (c.num_hidden_layers, c.hidden_size, c.intermediate_size) == (3, 192, 352)
    assert (c.num_attention_heads, c.num_key_value_heads, c.head_dim) == (6, 1, 32)
    assert c.vocab_size == 384 and c.rope_theta == 1e6 and c.rms_norm_eps == 1e-5
    assert c.tie_word_embeddings is False
    assert c.layer_windows == (0, 72, 72)
    assert c.q_size == 192 and c.kv_size == 32


def test_defaults_follow_the_reference():
    d = dict(architectures=["Qwen2ForCausalLM"], vocab_size=10, hidden_size=12, intermediate_size=8,
             num_hidden_layers=1, num_attention_heads=3)
    c = parse_qwen2_config(d)
    assert c.num_key_value_heads == 3          # defaults to the head count
    assert c.head_dim == 4                     # hidden / heads
    assert c.rms_norm_eps == 1e-6 and c.rope_theta == 10000.0
    assert c.layer_windows == (0,)
    assert "rope_theta" in c.defaults_used


@pytest.mark.parametrize("key", ["num_hidden_layers", "hidden_size", "num_attention_heads", "intermediate_size", "vocab_size"])
def test_missing_required_key(key):
    d = dict(TINY["A"])
    del d[key]
    with pytest.raises(ConfigError, match=key):
        parse_qwen2_config(d)


def test_rejected_options():
    with pytest.raises(ConfigError, match="multiple"):
        parse_qwen2_config(dict(TINY["A"], num_key_value_heads=3))
    with pytest.raises(ConfigError, match="even"):
        parse_qwen2_config(dict(TINY["A"], head_dim=15))
    with pytest.raises(ConfigError, match="rope_scaling"):
        parse_qwen2_config(dict(TINY["A"], rope_scaling={"type": "yarn", "factor": 4.0}))
    with pytest.raises(ConfigError, match="hidden_act"):
        parse_qwen2_config(dict(TINY["A"], hidden_act="gelu"))
    with pytest.raises(ConfigError, match="sliding_window"):
        parse_qwen2_config(dict(TINY["A"], use_sliding_window=True))
    with pytest.raises(ConfigError, match="max_window_layers"):
        # windowed, but nothing says which layers: no boundary is guessed
        parse_qwen2_config(dict(TINY["A"], use_sliding_window=True, sliding_window=64))
    with pytest.raises(ConfigError, match="integer"):
        parse_qwen2_config(dict(TINY["A"], hidden_size="64"))


def test_layer_types_decide_the_windows():
    d = dict(TINY["B"], layer_types=["sliding_attention", "full_attention", "sliding_attention"])
    assert parse_qwen2_config(d).layer_windows == (72, 0, 72)
    with pytest.raises(ConfigError, match="layer_types"):
        parse_qwen2_config(dict(TINY["B"], layer_types=["full_attention"]))


def test_round_trip_through_json():
    c = parse_qwen2_config(TINY["B"])
    c2 = parse_qwen2_config(json.loads(json.dumps(c.to_json_dict())))
    assert c == c2


def test_text_config_nesting():
    inner = {k: v for k, v in TINY["A"].items() if k != "architectures"}
    c = parse_qwen2_config({"architectures": ["Qwen2ForCausalLM"], "text_config": inner})
    assert c.hidden_size == 64


def test_registry_names():
    assert is_supported_architecture("Qwen2ForCausalLM")
    assert not is_supported_architecture("NoSuchModel")
    with pytest.raises(RegistryError, match="Qwen2ForCausalLM"):
        get_architecture("NoSuchModel")


def test_spec_is_built_from_the_config_only():
    entry = get_architecture("Qwen2ForCausalLM")
    spec = entry.build_spec(entry.parse_config(TINY["B"], "t"))
    assert len(spec.layers) == 3 and [e.layer for e in spec.schedule] == [0, 1, 2]
    assert [l.mixer["window"] for l in spec.layers] == [0, 72, 72]
    assert spec.layers[0].mixer["position"]["theta"] == 1e6
    assert spec.head["tied_to"] is None
    specA = entry.build_spec(entry.parse_config(TINY["A"], "t"))
    assert specA.head["tied_to"] == "model.embed_tokens.weight"


# ---- engine (process) configuration -------------------------------------------------

def test_engine_config_defaults_and_ranges():
    cfg = parse_engine_config({"models": [{"id": "m", "path": "/x"}], "defaultModel": "m"})
    assert cfg.serving.tokenBudget == 512 and cfg.serving.maxActiveRequests == 32 and cfg.serving.blockSize == 16
    assert cfg.runtime.maxContextTokens == 8192
    for bad in ({"serving": {"tokenBudget": 0}}, {"serving": {"tokenBudget": 8193}},
                {"serving": {"maxActiveRequests": 257}}, {"serving": {"blockSize": 12}},
                {"runtime": {"dtype": "fp8"}}):
        with pytest.raises(EngineConfigError):
            parse_engine_config(bad)


def test_engine_config_diagnostics():
    cfg = parse_engine_config({"diagnostics": {"parityDump": "/tmp/p", "traceDecodeFile": "/tmp/t", "profile": True}})
    assert cfg.diagnostics.parityDump == "/tmp/p" and cfg.diagnostics.traceDecodeFile == "/tmp/t" and cfg.diagnostics.profile
    assert parse_engine_config({}).diagnostics.parityDump == ""
    with pytest.raises(EngineConfigError, match="diagnostics.traceBlock0"):
        parse_engine_config({"diagnostics": {"traceBlock0": True}})


def test_engine_config_rejects_unknown_keys():
    with pytest.raises(EngineConfigError, match="unknown key 'server'"):
        parse_engine_config({"server": {"port": 8080}})
    with pytest.raises(EngineConfigError, match="serving.tokenBudgett"):
        parse_engine_config({"serving": {"tokenBudgett": 5}})
    with pytest.raises(EngineConfigError, match="either 'path' or 'random'"):
        parse_engine_config({"models": [{"id": "m"}]})


def test_any_json_object_survives_the_library_reader_unchanged():
    """`models[].random` is an arbitrary JSON object that the C++ reader parses and hands back as text: what comes back
    must be what went in, for strings with escapes and other alphabets, nested lists and objects, integers up to 18 digits,
    fractions, exponents, true / false / null."""
    hypothesis = pytest.importorskip("hypothesis")
    from hypothesis import given, settings, strategies as st
    leaves = st.one_of(st.none(), st.booleans(), st.integers(min_value=-10 ** 17, max_value=10 ** 17),
                       st.floats(allow_nan=False, allow_infinity=False, width=64), st.text(max_size=12))
    values = st.recursive(leaves, lambda inner: st.one_of(st.lists(inner, max_size=4), st.dictionaries(st.text(max_size=6), inner, max_size=4)),
                          max_leaves=20)

    @settings(max_examples=150, deadline=None)
    @given(st.dictionaries(st.text(min_size=1, max_size=6), values, min_size=1, max_size=4))
    def check(obj):
        cfg = parse_engine_config({"models": [{"id": "m", "random": obj}]})
        assert cfg.models[0].random == obj

    check()


def test_half_a_surrogate_pair_is_refused_not_passed_on():
    with pytest.raises(EngineConfigError, match="surrogate"):
        parse_engine_config({"models": [{"id": "m", "random": {"a": "\ud800"}}]})
