"""Configuration and registry (CPU)."""

import json

import pytest

from mini_llm_stack_b200.config import (ConfigError, DenseLlamaConfig, build_model,
                                        config_from_dict, config_from_folder,
                                        lookup_architecture, register_architecture,
                                        unregister_architecture, write_config_json)
from tiny_configs import CONFIGS, TINY_A, TINY_C


def test_reference_keys_and_derived_sizes():
    # the reference's own keys alone (train/config.py:8-16): head_dim and the
    # feed-forward width are derived as there (train/config.py:27-35)
    cfg = config_from_dict(dict(architecture="llama_dense", vocab_size=256, d_model=64,
                                n_layers=2, n_heads=4, max_seq_len=128, ffn_mult=4.0,
                                rope_theta=10000.0, norm_eps=1e-5, tie_embeddings=True))
    assert cfg.head_dim == 16 and cfg.n_kv_heads == 4
    assert cfg.intermediate_size == 192          # round_up_32(int(2*4*64/3)) = 192
    assert cfg.layer_order == (0, 1) and cfg.cache_source == (None, None)
    assert cfg.attention_scale == 16 ** -0.5


@pytest.mark.parametrize("key", ["A", "B", "C"])
def test_round_trip(tmp_path, key):
    cfg = config_from_dict(CONFIGS[key])
    write_config_json(tmp_path, cfg)
    again = config_from_folder(tmp_path)
    assert again == cfg
    raw = json.loads((tmp_path / "config.json").read_text())
    assert raw["architecture"] == "llama_dense"


def test_aliases_of_common_llama_folders():
    cfg = config_from_dict(dict(architecture="llama_dense", vocab_size=300, hidden_size=96,
                                num_hidden_layers=3, num_attention_heads=6,
                                num_key_value_heads=2, intermediate_size=200,
                                rms_norm_eps=1e-6, max_position_embeddings=77,
                                tie_word_embeddings=False, torch_dtype="float32"))
    assert (cfg.d_model, cfg.n_layers, cfg.n_heads, cfg.n_kv_heads) == (96, 3, 6, 2)
    assert cfg.head_dim == 16 and cfg.norm_eps == 1e-6 and cfg.max_seq_len == 77
    assert cfg.dtype == "float32" and cfg.tie_embeddings is False


@pytest.mark.parametrize("patch, word", [
    (dict(n_kv_heads=3), "multiple of n_kv_heads"),
    (dict(head_dim=15), "even"),
    (dict(n_experts=4), "experts"),
    (dict(architecture="nope"), "unknown architecture"),
    (dict(dtype="float16"), "dtype"),
    (dict(layer_order=[0, 5]), "layer_order"),
    (dict(cache_source=[None, 1]), "earlier call"),
    (dict(layer_windows=[4]), "one entry per layer"),
    (dict(surprise=1), "does not know"),
    (dict(vocab_size=0), "positive"),
])
def test_rejections(patch, word):
    with pytest.raises(ConfigError, match=word):
        config_from_dict(dict(TINY_A, **patch))


def test_missing_required_key_and_head_dim():
    raw = dict(TINY_A)
    del raw["n_heads"]
    with pytest.raises(ConfigError, match="n_heads"):
        config_from_dict(raw)
    with pytest.raises(ConfigError, match="head_dim"):
        config_from_dict(dict(architecture="llama_dense", vocab_size=10, d_model=50,
                              n_layers=1, n_heads=4))


def test_no_config_file(tmp_path):
    with pytest.raises(ConfigError, match="no config.json"):
        config_from_folder(tmp_path)


def test_model_is_built_from_parts_by_the_config():
    m = build_model(config_from_dict(TINY_C))
    assert [c.layer for c in m.calls] == [0, 1, 2, 1, 3]
    assert [c.cache_slot for c in m.calls] == [0, 1, 2, 3, 2]
    assert [c.writes for c in m.calls] == [True, True, True, True, False]
    specs = m.cache_specs()
    assert len(specs) == 4 and specs[1].window == 40 and specs[0].window is None
    names = m.tensor_specs()
    assert names["blocks.2.attn.wk.weight"].shape == (5 * 48, 80)
    assert names["blocks.0.mlp.w_down.weight"].shape == (80, 200)
    assert "lm_head.weight" in names
    tied = build_model(config_from_dict(TINY_A))
    assert "lm_head.weight" not in tied.tensor_specs()
    assert tied.tied_names() == {"lm_head.weight": "embed.weight"}


def test_registry_takes_another_architecture():
    class ToyConfig:
        def __init__(self, raw):
            self.architecture, self.raw = raw["architecture"], raw

        @classmethod
        def from_dict(cls, raw):
            return cls(raw)

    register_architecture("toy_arch", ToyConfig, lambda cfg: ("built", cfg.raw["x"]))
    try:
        cfg = config_from_dict({"architecture": "toy_arch", "x": 7})
        assert build_model(cfg) == ("built", 7)
        assert lookup_architecture("toy_arch").config_class is ToyConfig
    finally:
        unregister_architecture("toy_arch")
    with pytest.raises(ConfigError):
        lookup_architecture("toy_arch")


def test_direct_construction_fills_the_arrangement():
    cfg = DenseLlamaConfig(n_layers=3, d_model=64, n_heads=4, n_kv_heads=2, head_dim=16)
    assert cfg.layer_order == (0, 1, 2) and cfg.layer_windows == (None, None, None)


LLAMA_FOLDER_CONFIG = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "attention_bias": False,
    "attention_dropout": 0.0, "bos_token_id": 128000, "eos_token_id": 128001,
    "hidden_act": "silu", "hidden_size": 2048, "initializer_range": 0.02,
    "intermediate_size": 8192, "max_position_embeddings": 8192, "mlp_bias": False,
    "num_attention_heads": 32, "num_hidden_layers": 16, "num_key_value_heads": 8,
    "pretraining_tp": 1, "rms_norm_eps": 1e-05, "rope_scaling": None, "rope_theta": 500000.0,
    "tie_word_embeddings": True, "torch_dtype": "bfloat16", "transformers_version": "4.45.0",
    "use_cache": True, "vocab_size": 128256, "head_dim": 64,
}


def test_a_llama_model_folders_config_is_read():
    """The spellings and the extra keys usual in Llama model folders: aliases are
    mapped, keys without meaning for the math are dropped, the architecture name is
    an alias of ``llama_dense``."""
    cfg = config_from_dict(LLAMA_FOLDER_CONFIG)
    assert isinstance(cfg, DenseLlamaConfig) and cfg.architecture == "llama_dense"
    assert (cfg.d_model, cfg.n_layers, cfg.n_heads, cfg.n_kv_heads, cfg.head_dim) == \
        (2048, 16, 32, 8, 64)
    assert cfg.intermediate_size == 8192 and cfg.vocab_size == 128256
    assert cfg.tie_embeddings and cfg.dtype == "bfloat16" and cfg.norm_eps == 1e-5
    assert lookup_architecture("LlamaForCausalLM") is lookup_architecture("llama_dense")
    assert build_model(cfg).tied_names() == {"lm_head.weight": "embed.weight"}


@pytest.mark.parametrize("key,value", [
    ("rope_scaling", {"rope_type": "llama3", "factor": 8.0}), ("attention_bias", True),
    ("mlp_bias", True), ("hidden_act", "gelu"), ("sliding_window", 4096),
    ("attention_dropout", 0.1)])
def test_keys_that_change_the_math_are_refused_by_name(key, value):
    with pytest.raises(ConfigError, match=key):
        config_from_dict(dict(LLAMA_FOLDER_CONFIG, **{key: value}))


def test_an_unknown_key_is_still_an_error():
    with pytest.raises(ConfigError, match="some_new_switch"):
        config_from_dict(dict(LLAMA_FOLDER_CONFIG, some_new_switch=1))


def test_engine_options_refuse_what_contradicts_the_loaded_model():
    from mini_llm_stack_b200.config import EngineOptions
    opts = EngineOptions(dtype="bf16", kv_dtype="bfloat16", device="cpu", seed=5)
    assert opts.dtype == "bfloat16" and opts.seed == 5
    opts.check_against("bfloat16", "cpu")
    with pytest.raises(ConfigError, match="kv_dtype"):
        EngineOptions(kv_dtype="float32", device="cpu").check_against("bfloat16", "cpu")
    with pytest.raises(ConfigError, match="dtype"):
        EngineOptions(dtype="float32", device="cpu").check_against("bfloat16", "cpu")
    with pytest.raises(ConfigError, match="device"):
        EngineOptions(device="cuda:1").check_against("bfloat16", "cuda:0")
