"""Configuration, registry and checkpoint errors (CPU)."""

from __future__ import annotations

import json

import pytest
import torch
from safetensors.torch import save_file

import plain_qwen3 as plain
from forge_engine_b200.config import (
    EngineConfig,
    Qwen3Config,
    SchedulerConfig,
    known_architectures,
    read_model_config,
)
from forge_engine_b200.errors import ConfigError, WeightsError
from forge_engine_b200.models import expected_tensors
from forge_engine_b200.sampling import SamplingParams
from forge_engine_b200.weights import load_checkpoint, random_tensors, write_model_folder


def test_reads_every_size_from_config_json() -> None:
    for raw in (plain.TINY_A, plain.TINY_B, plain.TINY_C, plain.TINY_D, plain.TINY_E):
        arch, cfg, spec = read_model_config(raw)
        assert arch.name == "Qwen3ForCausalLM"
        assert cfg.vocab_size == raw["vocab_size"] and cfg.head_dim == raw["head_dim"]
        assert cfg.q_size == raw["num_attention_heads"] * raw["head_dim"]
        assert spec.tie_embeddings == raw["tie_word_embeddings"]
        assert len(spec.layers) == len(spec.schedule) == raw["num_hidden_layers"]
        mixer = spec.layers[0].mixer
        assert mixer.scale == raw["head_dim"] ** -0.5
        assert mixer.position.theta == raw["rope_theta"]
        assert spec.layers[0].input_norm.eps == raw["rms_norm_eps"]
        assert mixer.bias == raw["attention_bias"]
        # names and shapes agree with the plain implementation's list
        mine = {k: tuple(v.shape) for k, v in expected_tensors(spec).items()}
        assert mine == plain.tensor_shapes(plain.PlainConfig.from_dict(raw))


def test_window_layers() -> None:
    _, cfg, spec = read_model_config(plain.TINY_D)
    assert [layer.mixer.window for layer in spec.layers] == [None, 11, 11]
    off = dict(plain.TINY_D, use_sliding_window=False)
    assert [l.mixer.window for l in read_model_config(off)[2].layers] == [None] * 3


def test_head_dim_defaults_and_eos_forms() -> None:
    raw = dict(plain.TINY_A)
    del raw["head_dim"]
    cfg = Qwen3Config.from_dict(raw)
    assert cfg.head_dim == 16 and cfg.eos_token_ids == (255,)
    assert Qwen3Config.from_dict(plain.TINY_B).eos_token_ids == (382, 383)
    again = Qwen3Config.from_dict(cfg.to_dict())
    assert again == cfg


@pytest.mark.parametrize(
    "change,fragment",
    [
        ({"architectures": ["LlamaForCausalLM"]}, "unknown architecture"),
        ({"architectures": []}, "architectures"),
        ({"model_type": "llama"}, "model_type"),
        ({"hidden_act": "gelu"}, "hidden_act"),
        ({"num_key_value_heads": 3}, "multiple"),
        ({"head_dim": 15}, "even"),
        ({"rope_scaling": {"rope_type": "yarn", "factor": 2.0}}, "rope_scaling"),
        ({"vocab_size": 0}, "vocab_size"),
        ({"rms_norm_eps": 0.0}, "rms_norm_eps"),
        ({"eos_token_id": 999}, "eos_token_id"),
    ],
)
def test_bad_configs_are_refused(change: dict, fragment: str) -> None:
    with pytest.raises(ConfigError, match=fragment):
        read_model_config(dict(plain.TINY_A, **change))


def test_missing_key_is_named() -> None:
    raw = dict(plain.TINY_A)
    del raw["rope_theta"]
    with pytest.raises(ConfigError, match="rope_theta"):
        read_model_config(raw)
    assert "Qwen3ForCausalLM" in known_architectures()


def test_settings_validate() -> None:
    with pytest.raises(ValueError):
        SamplingParams(temperature=-1.0)
    with pytest.raises(ValueError):
        SamplingParams(top_p=0.0)
    with pytest.raises(ValueError):
        SamplingParams(top_k=0)
    with pytest.raises(ValueError):
        SamplingParams(min_p=1.5)
    with pytest.raises(ValueError):
        SamplingParams(max_new_tokens=0)
    with pytest.raises(ValueError):
        SchedulerConfig(token_budget=0)
    with pytest.raises(ValueError):
        EngineConfig(dtype="float16")
    assert EngineConfig(temperature=0.7, top_k=5).sampling_params().top_k == 5
    assert SamplingParams().greedy


def test_random_folder_round_trip(tmp_path) -> None:
    _, _, spec = read_model_config(plain.TINY_B)
    expected = expected_tensors(spec)
    tensors = random_tensors(expected, seed=3)
    again = random_tensors(expected, seed=3)
    assert all(torch.equal(tensors[k], again[k]) for k in tensors)
    assert any(not torch.equal(tensors[k], v) for k, v in random_tensors(expected, seed=4).items())
    norm = tensors["model.norm.weight"].float()
    assert abs(float(norm.mean()) - 1.0) < 0.1
    assert float(tensors["model.embed_tokens.weight"].float().std()) == pytest.approx(0.02, rel=0.1)
    write_model_folder(tmp_path, plain.TINY_B, tensors)
    assert json.loads((tmp_path / "config.json").read_text())["vocab_size"] == 384
    loaded = load_checkpoint(tmp_path, expected, torch.bfloat16, "cpu")
    assert list(loaded) == list(expected)
    assert all(v.dtype == torch.bfloat16 for v in loaded.values())
    assert torch.equal(loaded["lm_head.weight"], tensors["lm_head.weight"])
    raised = load_checkpoint(tmp_path, expected, torch.float32, "cpu")
    assert all(v.dtype == torch.float32 for v in raised.values())


def test_stored_dtype_is_kept_in_bfloat16_engine(tmp_path) -> None:
    _, _, spec = read_model_config(plain.TINY_A)
    expected = expected_tensors(spec)
    tensors = random_tensors(expected, seed=0)
    tensors["model.norm.weight"] = tensors["model.norm.weight"].float()
    tensors["model.layers.0.mlp.down_proj.weight"] = tensors["model.layers.0.mlp.down_proj.weight"].half()
    write_model_folder(tmp_path, plain.TINY_A, tensors)
    loaded = load_checkpoint(tmp_path, expected, torch.bfloat16, "cpu")
    assert loaded["model.norm.weight"].dtype == torch.float32
    assert loaded["model.layers.0.mlp.down_proj.weight"].dtype == torch.bfloat16
    assert loaded["model.embed_tokens.weight"].dtype == torch.bfloat16


def test_one_error_lists_missing_unexpected_and_misshaped(tmp_path) -> None:
    _, _, spec = read_model_config(plain.TINY_A)
    expected = expected_tensors(spec)
    tensors = random_tensors(expected, seed=0)
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.rotary.inv_freq"] = torch.zeros(8)
    tensors["model.layers.0.self_attn.k_norm.weight"] = torch.zeros(17)
    (tmp_path / "config.json").write_text(json.dumps(plain.TINY_A))
    save_file(tensors, str(tmp_path / "model.safetensors"))
    with pytest.raises(WeightsError) as info:
        load_checkpoint(tmp_path, expected, torch.bfloat16, "cpu")
    text = str(info.value)
    assert "model.layers.1.mlp.up_proj.weight" in text and "model.norm.weight" in text
    assert "missing tensors (2)" in text
    assert "unexpected tensors (1)" in text and "rotary.inv_freq" in text
    assert "wrong shapes (1)" in text and "(17,)" in text and "(16,)" in text


def test_tied_model_may_carry_a_head_and_untied_needs_one(tmp_path) -> None:
    _, _, spec = read_model_config(plain.TINY_A)
    expected = expected_tensors(spec)
    tensors = random_tensors(expected, seed=0)
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    write_model_folder(tmp_path / "tied", plain.TINY_A, tensors)
    loaded = load_checkpoint(tmp_path / "tied", expected, torch.bfloat16, "cpu", optional=("lm_head.weight",))
    assert "lm_head.weight" not in loaded
    _, _, spec_b = read_model_config(plain.TINY_B)
    expected_b = expected_tensors(spec_b)
    tensors_b = random_tensors(expected_b, seed=0)
    del tensors_b["lm_head.weight"]
    write_model_folder(tmp_path / "untied", plain.TINY_B, tensors_b)
    with pytest.raises(WeightsError, match="lm_head.weight"):
        load_checkpoint(tmp_path / "untied", expected_b, torch.bfloat16, "cpu")


def test_sharded_checkpoint_with_index(tmp_path) -> None:
    _, _, spec = read_model_config(plain.TINY_A)
    expected = expected_tensors(spec)
    tensors = random_tensors(expected, seed=1)
    names = list(tensors)
    half = len(names) // 2
    shards = {"model-00001-of-00002.safetensors": names[:half], "model-00002-of-00002.safetensors": names[half:]}
    weight_map = {}
    for shard, members in shards.items():
        save_file({n: tensors[n] for n in members}, str(tmp_path / shard))
        weight_map.update({n: shard for n in members})
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": weight_map}))
    loaded = load_checkpoint(tmp_path, expected, torch.bfloat16, "cpu")
    assert all(torch.equal(loaded[n], tensors[n]) for n in names)
    with pytest.raises(WeightsError, match="no safetensors"):
        load_checkpoint(tmp_path / "nowhere", expected, torch.bfloat16, "cpu")


def test_values_that_are_not_finite_and_integer_matrices_are_refused(tmp_path) -> None:
    """NaN and infinities are found while loading, with the tensors' names (upstream:
    src/forge_engine/weights.py:238-241), and a matrix stored as integers is a wrong dtype."""
    from forge_engine_b200.weights import open_checkpoint

    _, _, spec = read_model_config(plain.TINY_A)
    expected = expected_tensors(spec)
    tensors = random_tensors(expected, seed=0)
    tensors["model.layers.1.mlp.down_proj.weight"][3, 5] = float("nan")
    tensors["model.layers.0.input_layernorm.weight"][2] = float("inf")
    write_model_folder(tmp_path / "nan", plain.TINY_A, tensors)
    with pytest.raises(WeightsError) as info:
        load_checkpoint(tmp_path / "nan", expected, torch.bfloat16, "cpu")
    text = str(info.value)
    assert "NaN or infinity (2)" in text
    assert "model.layers.1.mlp.down_proj.weight" in text and "model.layers.0.input_layernorm.weight" in text
    assert "model.layers.0.mlp.down_proj.weight" not in text
    # the lazy mapping reads on access, in any order, and keeps nothing
    lazy = open_checkpoint(tmp_path / "nan", expected, torch.float32, "cpu")
    names = list(lazy)
    assert names == list(expected) and len(lazy) == len(expected)
    last = lazy[names[-2]]
    assert last.dtype == torch.float32 and torch.equal(last, tensors[names[-2]].float())
    assert lazy[names[-2]] is not last
    lazy.close()                                   # nothing bad was read: no error
    with pytest.raises(KeyError):
        lazy["not.a.tensor"]
    good = random_tensors(expected, seed=0)
    good["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(expected["model.layers.0.self_attn.q_proj.weight"].shape,
                                                                 dtype=torch.int64)
    write_model_folder(tmp_path / "int", plain.TINY_A, good)
    with pytest.raises(WeightsError, match=r"wrong dtypes \(1\): model.layers.0.self_attn.q_proj.weight: stored as I64"):
        load_checkpoint(tmp_path / "int", expected, torch.bfloat16, "cpu")


def test_random_tensors_do_not_depend_on_the_order_they_are_drawn_in() -> None:
    from forge_engine_b200.weights import RandomTensors

    _, _, spec = read_model_config(plain.TINY_B)
    expected = expected_tensors(spec)
    eager = random_tensors(expected, seed=9, dtype=torch.float32)
    lazy = RandomTensors(expected, 9, dtype=torch.float32)
    for name in reversed(list(expected)):
        assert torch.equal(lazy[name], eager[name])
    a, b = "model.layers.0.mlp.gate_proj.weight", "model.layers.1.mlp.gate_proj.weight"
    assert not torch.equal(eager[a], eager[b])
