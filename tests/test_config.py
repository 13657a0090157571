"""Configuration: typed engine options, the architecture's config.json keys, the registry."""
import json

import pytest

from helpers import CONFIGS, TINY_A, TINY_C
from vllm_cpp_b200 import ConfigError, EngineConfig, known_architectures, resolve_architecture
from vllm_cpp_b200.config.registry import read_config_json
from vllm_cpp_b200.models.qwen2 import Qwen2Config


def test_engine_defaults_follow_the_reference():
    c = EngineConfig()
    # include/vllm/core/config.hpp:34-66
    assert (c.gpu_memory_utilization, c.block_size, c.max_num_seqs, c.max_model_len) == (90, 16, 64, 8192)
    assert (c.max_num_batched_tokens, c.max_tokens_per_step) == (16384, 512)
    assert (c.temperature, c.top_p, c.top_k, c.repetition_penalty) == (1.0, 1.0, -1, 1.0)


@pytest.mark.parametrize("kw", [dict(block_size=0), dict(block_size=24), dict(gpu_memory_utilization=0),
                                dict(gpu_memory_utilization=101), dict(max_num_seqs=0), dict(dtype="float16"),
                                dict(quant_mode="fp8"), dict(top_p=0.0), dict(top_k=0), dict(load_format="gguf"),
                                dict(num_gpu_blocks=0), dict(repetition_penalty=0.0)])
def test_engine_config_refuses(kw):
    with pytest.raises(ConfigError):
        EngineConfig(**kw)


def test_registry_names_and_unknown():
    assert {"Qwen2ForCausalLM", "qwen"} <= set(known_architectures())
    with pytest.raises(ConfigError, match="Unknown model architecture"):
        resolve_architecture(dict(TINY_A, architectures=["LlamaForCausalLM"]))
    with pytest.raises(ConfigError, match="architectures"):
        resolve_architecture({k: v for k, v in TINY_A.items() if k != "architectures"})
    typed, spec = resolve_architecture({k: v for k, v in TINY_A.items() if k != "architectures"}, "qwen")
    assert spec.architecture == "Qwen2ForCausalLM" and len(spec.layers) == 2


def test_qwen2_sizes_come_from_config_json():
    for name, (cfg, _) in CONFIGS.items():
        typed, spec = resolve_architecture(cfg)
        assert spec.hidden_size == cfg["hidden_size"] and spec.vocab_size == cfg["vocab_size"]
        assert len(spec.layers) == cfg["num_hidden_layers"] == len(spec.run_order)
        m = spec.layers[0].mixer.params
        assert m["num_heads"] == cfg["num_attention_heads"] and m["num_kv_heads"] == cfg["num_key_value_heads"]
        assert m["head_dim"] == cfg.get("head_dim", cfg["hidden_size"] // cfg["num_attention_heads"])
        assert m["position"].params["theta"] == cfg["rope_theta"]
        assert spec.layers[0].mixer_norm.params["eps"] == cfg["rms_norm_eps"]
        assert spec.layers[0].feed_forward.params["intermediate_size"] == cfg["intermediate_size"]
        assert spec.tie_word_embeddings == cfg["tie_word_embeddings"]


def test_window_is_chosen_layer_by_layer():
    typed, spec = resolve_architecture(TINY_C)
    assert [l.mixer.params["window"] for l in spec.layers] == [0, 0, 24, 24]
    typed, spec = resolve_architecture(TINY_A)
    assert all(l.mixer.params["window"] == 0 for l in spec.layers)


@pytest.mark.parametrize("change, msg", [
    ({"hidden_size": None}, "hidden_size"), ({"rope_theta": None}, "rope_theta"),
    ({"num_key_value_heads": 3}, "multiple"), ({"hidden_act": "gelu"}, "hidden_act"),
    ({"rope_scaling": {"type": "yarn"}}, "rope_scaling"), ({"vocab_size": -5}, "positive"),
    ({"hidden_size": 70}, "head_dim"), ({"rms_norm_eps": 0}, "rms_norm_eps"),
    ({"use_sliding_window": True}, "sliding_window"), ({"tie_word_embeddings": "yes"}, "tie_word_embeddings"),
    ({"num_hidden_layers": 2.5}, "integer"), ({"eos_token_id": 99999}, "vocabulary")])
def test_qwen2_config_refuses(change, msg):
    cfg = dict(TINY_A)
    for k, v in change.items():
        if v is None:
            cfg.pop(k)
        else:
            cfg[k] = v
    with pytest.raises(ConfigError, match=msg):
        Qwen2Config.from_dict(cfg)


def test_eos_ids_and_defaults():
    c = Qwen2Config.from_dict(dict(TINY_A, eos_token_id=[3, 7]))
    assert c.eos_token_ids == [3, 7] and c.rms_norm_eps == 1e-6
    c = Qwen2Config.from_dict({k: v for k, v in TINY_A.items() if k not in ("rms_norm_eps", "tie_word_embeddings")})
    assert c.rms_norm_eps == 1e-6 and c.tie_word_embeddings is False and c.head_dim == 16
    assert Qwen2Config.from_dict(c.to_dict()) == c


def test_config_json_file_errors(tmp_path):
    with pytest.raises(ConfigError, match="Cannot open config"):
        read_config_json(str(tmp_path))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="not valid JSON"):
        read_config_json(str(tmp_path))
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    assert read_config_json(str(tmp_path))["hidden_size"] == 64
