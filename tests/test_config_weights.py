"""Configuration parsing, the registry, safetensors and the loader's one-error report (CPU)."""

from __future__ import annotations

import json
import struct

import pytest
import torch

from cases import INIT_B, TINY_A, TINY_B, TINY_C
from ayaka_b200.config.engine import EngineConfig
from ayaka_b200.config.model import GPT2Config, read_config_json
from ayaka_b200.errors import ConfigError, ModelLoadError
from ayaka_b200.models import build_model, load_model
from ayaka_b200.models.registry import resolve_architecture, supported_architectures
from ayaka_b200.weights.random_init import random_state, write_random_model
from ayaka_b200.weights.safetensors import SafetensorsFile, write_safetensors


def test_gpt2_keys_and_defaults():
    config = GPT2Config.from_json_dict({
        "architectures": ["GPT2LMHeadModel"], "vocab_size": 50257, "n_embd": 1600, "n_layer": 48,
        "n_head": 25, "n_positions": 1024, "layer_norm_epsilon": 1e-5,
        "activation_function": "gelu_new", "eos_token_id": 50256})
    assert (config.n_inner, config.head_dim, config.tie_word_embeddings) == (6400, 64, True)
    assert config.scale_attn_by_inverse_layer_idx is False and config.eos_token_id == 50256
    other = GPT2Config.from_json_dict({
        "architectures": ["GPT2LMHeadModel"], "vocab_size": 11, "hidden_size": 32,
        "num_hidden_layers": 2, "num_attention_heads": 2, "intermediate_size": 48,
        "max_position_embeddings": 64, "layer_norm_eps": 1e-6, "hidden_act": "gelu"})
    assert (other.n_embd, other.n_inner, other.n_positions) == (32, 48, 64)
    assert GPT2Config.from_json_dict(config.to_json_dict()) == config


def test_every_missing_key_is_listed_at_once():
    with pytest.raises(ModelLoadError) as caught:
        GPT2Config.from_json_dict({"n_embd": 64})
    message = str(caught.value)
    for key in ("architecture", "vocab_size", "n_layer", "n_head", "n_positions",
                "activation_function", "layer_norm_epsilon"):
        assert key in message
    assert "n_inner" not in message  # defaults to 4 * n_embd


def test_bad_values_are_refused():
    base = dict(TINY_A)
    with pytest.raises(ConfigError):
        GPT2Config.from_json_dict({**base, "layer_norm_epsilon": 0.0})
    with pytest.raises(ConfigError):
        GPT2Config.from_json_dict({**base, "n_head": 5})  # 64 % 5
    with pytest.raises(ConfigError):
        GPT2Config.from_json_dict({**base, "n_layer": 0})
    with pytest.raises(ModelLoadError):
        GPT2Config.from_json_dict({**base, "reorder_and_upcast_attn": True})
    with pytest.raises(ModelLoadError):
        GPT2Config.from_json_dict({**base, "num_key_value_heads": 2})
    with pytest.raises(ModelLoadError):
        build_model({**base, "activation_function": "relu"}, "float32", "cpu")
    with pytest.raises(ModelLoadError):  # head size 12 is no multiple of 16
        build_model({**base, "n_embd": 48}, "float32", "cpu")


def test_registry_lists_what_it_supports():
    assert "GPT2LMHeadModel" in supported_architectures()
    with pytest.raises(ModelLoadError) as caught:
        resolve_architecture("LlamaForCausalLM")
    assert "GPT2LMHeadModel" in str(caught.value)
    with pytest.raises(ModelLoadError):
        build_model({"n_embd": 64}, "float32", "cpu")


def test_model_spec_follows_the_config():
    model, _, config = build_model(TINY_B, "float32", "cpu")
    spec = model.spec
    assert len(spec.layers) == 3 and [run.layer for run in spec.order] == [0, 1, 2]
    scales = [layer.mixer.scale for layer in spec.layers]
    assert scales == pytest.approx([32 ** -0.5 / (i + 1) for i in range(3)])
    assert spec.layers[0].feed_forward.activation == "gelu_erf"
    assert spec.layers[0].feed_forward.inner == 320 and spec.final_norm.eps == 1e-6
    names = dict(model.named_params())
    assert names["layers.2.mixer.qkv.weight"].tensor.shape == (288, 96)
    assert names["layers.0.feed_forward.down.weight"].tensor.shape == (96, 320)
    assert "head.weight" not in names  # tied
    untied, _, _ = build_model(TINY_C, "bfloat16", "cpu")
    params = dict(untied.named_params())
    assert params["head.weight"].tensor.dtype == torch.bfloat16
    assert params["final_norm.weight"].tensor.dtype == torch.float32  # vectors stay 32-bit


def test_engine_config_checks():
    EngineConfig(model="x", dtype="bf16")
    assert EngineConfig(model="x", dtype="fp32").dtype == "float32"
    for bad in (dict(dtype="fp16"), dict(device="cpu"), dict(num_blocks=1),
                dict(block_size=64, max_tokens_per_step=32), dict(num_blocks=4, max_running=8),
                dict(memory_ratio=0.0)):
        with pytest.raises(ConfigError):
            EngineConfig(model="x", **bad)


def test_strict_config_json(tmp_path):
    (tmp_path / "config.json").write_text('{"n_embd": 1, "n_embd": 2}')
    with pytest.raises(ModelLoadError):
        read_config_json(tmp_path)
    (tmp_path / "config.json").write_text("[1]")
    with pytest.raises(ModelLoadError):
        read_config_json(tmp_path)
    with pytest.raises(ModelLoadError):
        read_config_json(tmp_path / "nowhere")


# ---- safetensors -------------------------------------------------------------------------
def test_safetensors_round_trip(tmp_path):
    tensors = {"a": torch.arange(6, dtype=torch.float32).reshape(2, 3),
               "b": torch.tensor([1.5, -2.0], dtype=torch.bfloat16),
               "c": torch.tensor([[7]], dtype=torch.int32), "d": torch.zeros(0, 4)}
    write_safetensors(tmp_path / "m.safetensors", tensors, {"k": "v"})
    file = SafetensorsFile(tmp_path / "m.safetensors")
    assert set(file.names()) == set(tensors) and file.metadata == {"k": "v"}
    for name, value in tensors.items():
        got = file.tensor(name)
        assert got.dtype == value.dtype and torch.equal(got, value)


def _raw(path, header: dict, payload: bytes):
    raw = json.dumps(header).encode()
    path.write_bytes(struct.pack("<Q", len(raw)) + raw + payload)


def test_safetensors_header_is_validated(tmp_path):
    path = tmp_path / "bad.safetensors"
    good = {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}
    cases = [
        ({"x": {**good, "data_offsets": [0, 16]}}, b"\0" * 8),  # outside the payload
        ({"x": {**good, "shape": [3]}}, b"\0" * 8),  # size != shape
        ({"x": {**good, "dtype": "F8"}}, b"\0" * 8),  # unknown dtype
        ({"x": good, "y": {**good, "data_offsets": [4, 12]}}, b"\0" * 12),  # overlap
    ]
    for header, payload in cases:
        _raw(path, header, payload)
        with pytest.raises(ModelLoadError):
            SafetensorsFile(path)
    path.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(ModelLoadError):
        SafetensorsFile(path)
    path.write_bytes(struct.pack("<Q", 21) + b'{"x": 1, "x": 2}     ')
    with pytest.raises(ModelLoadError):
        SafetensorsFile(path)


# ---- loader -----------------------------------------------------------------------------
def test_random_model_folder_loads_and_is_reproducible(tmp_path):
    write_random_model(TINY_B, tmp_path / "m", seed=1, init=INIT_B, store_dtype="bfloat16")
    model, config = load_model(tmp_path / "m", "bfloat16", "cpu")
    state = random_state(TINY_B, 1, INIT_B, "bfloat16")
    params = dict(model.named_params())
    # Conv1D weights are transposed on load; vectors are widened to float32
    assert torch.equal(params["layers.1.mixer.qkv.weight"].tensor,
                       state["transformer.h.1.attn.c_attn.weight"].t())
    assert torch.equal(params["layers.1.feed_forward.down.bias"].tensor,
                       state["transformer.h.1.mlp.c_proj.bias"].float())
    assert torch.equal(params["embedding.weight"].tensor, state["transformer.wte.weight"])
    again = random_state(TINY_B, 1, INIT_B, "bfloat16")
    assert all(torch.equal(state[name], again[name]) for name in state)
    other = random_state(TINY_B, 2, INIT_B, "bfloat16")
    assert not torch.equal(state["transformer.wte.weight"], other["transformer.wte.weight"])
    assert float(state["transformer.h.0.attn.c_attn.bias"].float().std()) > 0.0
    assert config.n_inner == 320


def test_float32_storage_stays_float32_where_it_can(tmp_path):
    write_random_model(TINY_A, tmp_path / "m", seed=0, store_dtype="float32")
    model, _ = load_model(tmp_path / "m", "bfloat16", "cpu")
    params = dict(model.named_params())
    assert params["layers.0.mixer_norm.weight"].tensor.dtype == torch.float32
    assert params["layers.0.mixer.qkv.bias"].tensor.dtype == torch.float32
    assert params["layers.0.mixer.qkv.weight"].tensor.dtype == torch.bfloat16


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    state = random_state(TINY_A, 0)
    del state["transformer.h.1.ln_2.bias"]
    del state["transformer.wpe.weight"]
    state["transformer.h.0.attn.rotary.inv_freq"] = torch.zeros(4)
    state["transformer.h.0.attn.c_attn.weight"] = torch.zeros(192, 64)  # not transposed
    state["transformer.ln_f.weight"] = torch.zeros(64, dtype=torch.int32)
    state["transformer.h.0.attn.bias"] = torch.ones(1, 1, 8, 8)  # a stored mask: ignored
    state["lm_head.weight"] = state["transformer.wte.weight"].clone()  # tied: ignored
    folder = tmp_path / "m"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(TINY_A))
    write_safetensors(folder / "model.safetensors", state)
    with pytest.raises(ModelLoadError) as caught:
        load_model(folder, "float32", "cpu")
    error = caught.value
    assert set(error.context["missing"]) == {"h.1.ln_2.bias", "wpe.weight"}
    assert error.context["unexpected"] == ("transformer.h.0.attn.rotary.inv_freq",)
    assert len(error.context["wrong_shape"]) == 1 and "c_attn" in error.context["wrong_shape"][0]
    assert len(error.context["unsupported_dtype"]) == 1
    for word in ("missing", "unexpected", "wrong_shape", "unsupported_dtype"):
        assert word in str(error)


def test_names_without_the_transformer_prefix_load(tmp_path):
    state = {name.removeprefix("transformer."): tensor
             for name, tensor in random_state(TINY_A, 0).items()}
    folder = tmp_path / "m"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(TINY_A))
    write_safetensors(folder / "model.safetensors", state)
    load_model(folder, "float32", "cpu")


def test_sharded_folder_with_index(tmp_path):
    state = random_state(TINY_A, 0)
    names = sorted(state)
    folder = tmp_path / "m"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(TINY_A))
    halves = (names[: len(names) // 2], names[len(names) // 2:])
    weight_map = {}
    for index, part in enumerate(halves):
        shard = f"model-{index}.safetensors"
        write_safetensors(folder / shard, {name: state[name] for name in part})
        weight_map.update({name: shard for name in part})
    (folder / "model.safetensors.index.json").write_text(json.dumps({"weight_map": weight_map}))
    load_model(folder, "float32", "cpu")
    del weight_map[names[0]]
    (folder / "model.safetensors.index.json").write_text(json.dumps({"weight_map": weight_map}))
    with pytest.raises(ModelLoadError):
        load_model(folder, "float32", "cpu")
