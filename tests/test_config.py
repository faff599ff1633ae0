"""Configuration: every key the architecture's config.json gives, its defaults,
its errors, and the registry."""

import pytest

from paged_llm_b200.config import (ARCHITECTURES, ConfigError, EngineConfig, LlamaConfig, SamplingParams,
                                   parse_model_config, register_architecture)
from tests.tiny import TINY_A, TINY_B


def test_required_keys_and_defaults():
    cfg = LlamaConfig.from_hf_dict({"vocab_size": 10, "hidden_size": 64, "intermediate_size": 32,
                                    "num_hidden_layers": 1, "num_attention_heads": 4})
    assert cfg.num_key_value_heads == 4 and cfg.head_dim == 16
    assert cfg.rms_norm_eps == 1e-5 and cfg.rope_theta == 10000.0 and cfg.rope_scaling is None
    assert cfg.max_position_embeddings == 4096 and cfg.tie_word_embeddings is False
    with pytest.raises(ConfigError, match="intermediate_size"):
        LlamaConfig.from_hf_dict({"vocab_size": 10, "hidden_size": 64, "num_hidden_layers": 1,
                                  "num_attention_heads": 4})


def test_tiny_configs_differ_in_every_size_and_option():
    a, b = LlamaConfig.from_hf_dict(TINY_A), LlamaConfig.from_hf_dict(TINY_B)
    for f in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
              "head_dim", "rms_norm_eps", "rope_theta", "rope_scaling", "tie_word_embeddings",
              "max_position_embeddings"):
        assert getattr(a, f) != getattr(b, f), f
    assert a.num_attention_heads // a.num_key_value_heads != b.num_attention_heads // b.num_key_value_heads


@pytest.mark.parametrize("spelling", ["rope_scaling", "rope_parameters"])
@pytest.mark.parametrize("type_key", ["rope_type", "type"])
def test_rope_key_spellings(spelling, type_key):
    base = {k: v for k, v in TINY_B.items() if k not in ("rope_scaling", "rope_theta")}
    rope = {type_key: "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
            "original_max_position_embeddings": 64}
    if spelling == "rope_parameters":
        rope["rope_theta"] = 500000.0
        cfg = LlamaConfig.from_hf_dict({**base, "rope_parameters": rope})
    else:
        cfg = LlamaConfig.from_hf_dict({**base, "rope_scaling": rope, "rope_theta": 500000.0})
    assert cfg.rope_theta == 500000.0
    assert cfg.rope_scaling.factor == 8.0 and cfg.rope_scaling.original_max_position_embeddings == 64


def test_default_rope_type_means_no_scaling():
    cfg = LlamaConfig.from_hf_dict({**TINY_A, "rope_parameters": {"rope_type": "default", "rope_theta": 123.0}})
    assert cfg.rope_scaling is None and cfg.rope_theta == 123.0


@pytest.mark.parametrize("patch,match", [
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"attention_bias": True}, "attention_bias"),
    ({"mlp_bias": True}, "mlp_bias"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 2.0}}, "yarn"),
    ({"rope_scaling": {"rope_type": "llama3"}}, "factor"),
    ({"num_key_value_heads": 3}, "multiple"),
    ({"head_dim": 15}, "even"),
    ({"rms_norm_eps": 0.0}, "rms_norm_eps"),
])
def test_unsupported_values_are_errors(patch, match):
    with pytest.raises(ConfigError, match=match):
        LlamaConfig.from_hf_dict({**TINY_A, **patch})


def test_head_dim_null_and_dtype_spelling():
    cfg = LlamaConfig.from_hf_dict({**TINY_A, "head_dim": None, "torch_dtype": None, "dtype": "bfloat16"})
    assert cfg.head_dim == 16 and cfg.torch_dtype == "bfloat16"


def test_round_trip_through_config_json():
    for hf in (TINY_A, TINY_B):
        cfg = LlamaConfig.from_hf_dict(hf)
        assert LlamaConfig.from_hf_dict(cfg.to_hf_dict()) == cfg


def test_registry():
    arch, cfg = parse_model_config(TINY_A)
    assert arch.name == "LlamaForCausalLM" and isinstance(cfg, LlamaConfig)
    with pytest.raises(ConfigError, match="unsupported architecture"):
        parse_model_config({**TINY_A, "architectures": ["GPT2LMHeadModel"]})
    with pytest.raises(ValueError, match="already registered"):
        register_architecture("LlamaForCausalLM", LlamaConfig, lambda c: None)
    assert "LlamaForCausalLM" in ARCHITECTURES


def test_spec_has_no_constant_of_its_own():
    from paged_llm_b200.models.llama import llama_spec
    cfg = LlamaConfig.from_hf_dict(TINY_B)
    spec = llama_spec(cfg)
    assert len(spec.layers) == 3 and [e.layer for e in spec.schedule] == [0, 1, 2]
    m = spec.layers[0].mixer.params
    assert (m["num_heads"], m["num_kv_heads"], m["head_dim"]) == (3, 3, 32) and m["scale"] == 32 ** -0.5
    assert spec.layers[1].norms["input"].params["eps"] == 1e-6
    assert spec.positions["rotary"].params["theta"] == 500000.0
    assert spec.head.params["tied_to"] == "model.embed_tokens.weight"


def test_engine_config_validation():
    EngineConfig()
    for bad in (dict(block_size=12), dict(max_num_batched_tokens=8, block_size=16), dict(max_num_seqs=0),
                dict(gpu_memory_utilization=0.0), dict(attention_backend="triton"), dict(dtype="int8"),
                dict(num_gpu_blocks=0)):
        with pytest.raises(ValueError):
            EngineConfig(**bad)


def test_sampling_params():
    assert SamplingParams(temperature=0.0).greedy and not SamplingParams(temperature=0.7).greedy
    assert SamplingParams(stop_token_ids=[1, 2]).stop_token_ids == (1, 2)
    for bad in (dict(temperature=-1.0), dict(top_p=0.0), dict(top_p=1.5), dict(max_tokens=0)):
        with pytest.raises(ValueError):
            SamplingParams(**bad)
