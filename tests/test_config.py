"""Configuration and registry."""
import json

import pytest

from machserve_b200.config import ConfigError, Qwen2Config, config_from_json, known_architectures, load_config
from tests.helpers import TINY


def test_registry_knows_the_architecture():
    assert "Qwen2ForCausalLM" in known_architectures()
    cfg = config_from_json(TINY["A"]["config"])
    assert isinstance(cfg, Qwen2Config) and cfg.architecture == "Qwen2ForCausalLM"


def test_unknown_architecture_lists_known_ones():
    raw = dict(TINY["A"]["config"], architectures=["LlamaForCausalLM"])
    with pytest.raises(ConfigError, match="LlamaForCausalLM.*Qwen2ForCausalLM"):
        config_from_json(raw)


def test_defaults_follow_the_reference():
    raw = {"architectures": ["Qwen2ForCausalLM"], "vocab_size": 100, "hidden_size": 48, "num_hidden_layers": 2,
           "num_attention_heads": 6, "intermediate_size": 64}
    c = config_from_json(raw)
    assert (c.num_key_value_heads, c.head_dim) == (6, 8)
    assert (c.rms_norm_eps, c.rope_theta, c.max_position_embeddings) == (1e-6, 10000.0, 2048)
    assert c.tie_word_embeddings is False and c.use_sliding_window is False


def test_sizes_have_no_defaults():
    for key in ("vocab_size", "hidden_size", "num_hidden_layers", "num_attention_heads", "intermediate_size"):
        raw = dict(TINY["B"]["config"])
        del raw[key]
        with pytest.raises(ConfigError, match=key):
            config_from_json(raw)


def test_explicit_head_dim_may_differ_from_hidden_over_heads():
    c = config_from_json(TINY["C"]["config"])
    assert c.head_dim == 48 and c.hidden_size // c.num_attention_heads == 12
    m = c.model_spec().layers[0].mixer
    assert m["head_dim"] == 48 and m["num_heads"] == 6 and m["num_kv_heads"] == 2


@pytest.mark.parametrize("change,match", [
    ({"num_key_value_heads": 3}, "multiple"),
    ({"head_dim": 15}, "even"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"rope_scaling": {"type": "yarn", "factor": 4.0}}, "rope_scaling"),
    ({"rms_norm_eps": -1.0}, "rms_norm_eps"),
    ({"vocab_size": "big"}, "vocab_size"),
    ({"use_sliding_window": True, "sliding_window": None}, "sliding_window"),
    ({"eos_token_id": 100000}, "eos_token_id"),
])
def test_bad_values_are_refused(change, match):
    with pytest.raises(ConfigError, match=match):
        config_from_json(dict(TINY["A"]["config"], **change))


def test_round_trip_and_spec(tmp_path):
    c = config_from_json(TINY["C"]["config"])
    (tmp_path / "config.json").write_text(json.dumps(c.to_json()))
    assert load_config(tmp_path) == c
    spec = c.model_spec()
    assert len(spec.layers) == 3 and [r.layer for r in spec.run_order] == [0, 1, 2]
    # layers from max_window_layers on are windowed; the parts carry every constant as a parameter
    assert [l.mixer["window"] for l in spec.layers] == [None, 11, 11]
    assert spec.layers[1].mixer_norm["eps"] == 3e-5 and spec.layers[2].mixer["position"]["theta"] == 500000.0
    assert spec.head["tied_to"] is None and config_from_json(TINY["A"]["config"]).model_spec().head["tied_to"]


def test_run_order_is_checked():
    from machserve_b200.config.spec import ModelSpec, RunSpec
    import dataclasses

    spec = config_from_json(TINY["A"]["config"]).model_spec()
    dataclasses.replace(spec, run_order=(RunSpec(0), RunSpec(1), RunSpec(1), RunSpec(0, cache_of=0)))  # fine
    with pytest.raises(ValueError, match="earlier"):
        dataclasses.replace(spec, run_order=(RunSpec(0, cache_of=1), RunSpec(1)))
    with pytest.raises(ValueError, match="layer 5"):
        dataclasses.replace(spec, run_order=(RunSpec(5),))


def test_missing_config_file(tmp_path):
    with pytest.raises(ConfigError, match="no such file"):
        load_config(tmp_path)


def test_memory_estimate_before_allocation():
    """Weights once (a tied head costs nothing), pages of every layer, and the margin: the 0.5B sizes by hand."""
    import torch

    from machserve_b200.engine.runner import SCRATCH_MARGIN_BYTES, estimate_device_bytes
    from machserve_b200.parts import DecoderModel

    raw = {"architectures": ["Qwen2ForCausalLM"], "vocab_size": 151936, "hidden_size": 896, "num_hidden_layers": 24,
           "num_attention_heads": 14, "num_key_value_heads": 2, "intermediate_size": 4864, "tie_word_embeddings": True}
    model = DecoderModel(config_from_json(raw).model_spec())
    est = estimate_device_bytes(model, torch.bfloat16, page_size=64, num_pages=100, max_requests=8, max_seq_len=2048)
    d, i, qkv = 896, 4864, 896 + 2 * 128
    per_layer = 2 * (d * qkv + d * d + 3 * d * i) + 4 * (qkv + 2 * d)
    assert est["weights_bytes"] == 24 * per_layer + 2 * 151936 * d + 4 * d
    assert est["cache_bytes"] == 24 * 100 * 64 * (2 * 2 * 64) * 2
    assert est["table_bytes"] == 8 * 32 * 4 and est["state_bytes"] == 0
    assert est["total_bytes"] == est["weights_bytes"] + est["cache_bytes"] + est["table_bytes"] + SCRATCH_MARGIN_BYTES
    wide = estimate_device_bytes(model, torch.float32, page_size=64, num_pages=100, max_requests=8, max_seq_len=2048)
    assert wide["cache_bytes"] == 2 * est["cache_bytes"]
