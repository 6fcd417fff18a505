"""An architecture registered from the tests whose checkpoint needs stacking, slicing and one
stored tensor for two parameters (``tests/toy_architecture.py``): the loader on the CPU."""

from __future__ import annotations

import pytest
import torch

import toy_architecture as toy
from cases import INIT_B, TINY_C
from ayaka_b200.errors import ModelLoadError
from ayaka_b200.models import build_model
from ayaka_b200.models.registry import resolve_architecture
from ayaka_b200.weights.loader import TensorSource, load_into
from ayaka_b200.weights.rules import WeightRule, WeightRules

CONFIG = {**TINY_C, "architectures": [toy.NAME]}


def _built():
    toy.register()
    model, architecture, config = build_model(CONFIG, "float32", "cpu")
    gpt2 = resolve_architecture("GPT2LMHeadModel")
    state = dict(gpt2.random_tensors(config, 3, INIT_B))
    return model, architecture, config, state


def test_stacked_sliced_and_shared_tensors_fill_the_parameters():
    model, architecture, config, state = _built()
    stored = toy.gpt2_state_to_toy(state, config)
    load_into(model, architecture.weight_rules(config), TensorSource(tensors=stored))
    params = {name: param.tensor for name, param in model.named_params()}
    assert torch.equal(params["embedding.weight"], state["lm_head.weight"])
    assert torch.equal(params["head.weight"], state["lm_head.weight"])
    for i in range(config.n_layer):
        src, dst = f"transformer.h.{i}.", f"layers.{i}."
        assert torch.equal(params[f"{dst}mixer.qkv.weight"],
                           state[f"{src}attn.c_attn.weight"].t())
        assert torch.equal(params[f"{dst}mixer.qkv.bias"], state[f"{src}attn.c_attn.bias"])
        assert torch.equal(params[f"{dst}feed_forward.up.weight"],
                           state[f"{src}mlp.c_fc.weight"].t())
        assert torch.equal(params[f"{dst}feed_forward.down.weight"],
                           state[f"{src}mlp.c_proj.weight"].t())
        assert torch.equal(params[f"{dst}feed_forward.down.bias"], state[f"{src}mlp.c_proj.bias"])


def test_every_problem_of_a_stacked_checkpoint_is_reported_at_once():
    model, architecture, config, state = _built()
    stored = toy.gpt2_state_to_toy(state, config)
    del stored["model.blocks.1.k_proj.weight"]
    stored["model.blocks.0.v_proj.weight"] = torch.zeros(config.n_embd + 1, config.n_embd)
    stored["model.blocks.0.ff_in_b.bias"] = torch.zeros(3)
    stored["model.tok.weight"] = torch.zeros(config.vocab_size - 1, config.n_embd)  # too short
    stored["model.stray"] = torch.zeros(2)
    before = {name: param.tensor.clone() for name, param in model.named_params()}
    with pytest.raises(ModelLoadError) as caught:
        load_into(model, architecture.weight_rules(config), TensorSource(tensors=stored))
    context = caught.value.context
    assert context["missing"] == ("blocks.1.k_proj.weight",)
    assert context["unexpected"] == ("model.stray",)
    wrong = " ".join(context["wrong_shape"])
    for name in ("blocks.0.v_proj.weight", "tok.weight"):
        assert name in wrong
    # a piece of the wrong length leaves its parameter partly covered
    assert any("layers.0.feed_forward.up.bias" in line for line in context["badly_covered"])
    # nothing was copied
    for name, param in model.named_params():
        assert torch.equal(param.tensor, before[name]) or param.tensor.isnan().any()


def test_pieces_must_cover_a_parameter_exactly_once():
    model, _, config, state = _built()
    stored = toy.gpt2_state_to_toy(state, config)
    rules = toy.toy_weight_rules(config)
    d = config.n_embd
    for offset, what in ((d - 1, "overlap"), (d + 1, "gap")):
        bent = dict(rules.rules)
        bent["blocks.0.k_proj.bias"] = WeightRule("layers.0.mixer.qkv.bias", offset=offset)
        if offset == d + 1:  # keep the last piece inside: shorten nothing, expect the gap first
            bent["blocks.0.v_proj.bias"] = WeightRule("layers.0.mixer.qkv.bias", offset=2 * d)
        with pytest.raises(ModelLoadError) as caught:
            load_into(model, WeightRules(bent, rules.ignore, rules.optional_prefixes),
                      TensorSource(tensors=stored))
        assert what in " ".join(caught.value.context["badly_covered"]) or \
            "wrong_shape" in str(caught.value)
