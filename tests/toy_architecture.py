"""A toy architecture defined in the tests, to show what adding one takes.

``ToySplitLM`` is computed like GPT-2 (so the plain implementation can check it) but its
checkpoints are laid out the way many decoder checkpoints are: separate query, key and value
matrices stored ``[out, in]``, the feed-forward input stored as two halves, a token table
padded with rows the model does not use, and an untied head that the file stores as the same
tensor as the token table. Loading it needs stacking, slicing and one stored tensor feeding
two parameters; none of that touches the package: the architecture is registered from here.
"""

from __future__ import annotations

from collections.abc import Iterator, Mapping

import torch

from ayaka_b200.config.model import GPT2Config
from ayaka_b200.models.gpt2 import gpt2_model_spec
from ayaka_b200.models.registry import Architecture, register_architecture
from ayaka_b200.weights.rules import RandomInit, WeightRule, WeightRules

NAME = "ToySplitLM"
PADDED_ROWS = 8  # rows the stored token table has beyond the vocabulary


def _parse(config_json: Mapping[str, object]) -> GPT2Config:
    return GPT2Config.from_json_dict({**config_json, "architectures": ["GPT2LMHeadModel"],
                                      "tie_word_embeddings": False})


def toy_weight_rules(config: GPT2Config) -> WeightRules:
    d, inner, vocab = config.n_embd, config.n_inner, config.vocab_size
    half = inner // 2
    rules: dict[str, WeightRule | tuple[WeightRule, ...]] = {
        # one stored tensor, two parameters, each takes the rows below the padding
        "tok.weight": (WeightRule("embedding.weight", take=(0, vocab)),
                       WeightRule("head.weight", take=(0, vocab))),
        "pos.weight": WeightRule("position.weight"),
        "norm.weight": WeightRule("final_norm.weight"),
        "norm.bias": WeightRule("final_norm.bias"),
    }
    for i in range(config.n_layer):
        src, dst = f"blocks.{i}.", f"layers.{i}."
        for kind in ("weight", "bias"):
            rules[f"{src}norm_a.{kind}"] = WeightRule(f"{dst}mixer_norm.{kind}")
            rules[f"{src}norm_b.{kind}"] = WeightRule(f"{dst}feed_forward_norm.{kind}")
            for index, name in enumerate(("q", "k", "v")):  # stacked into the fused matrix
                rules[f"{src}{name}_proj.{kind}"] = WeightRule(f"{dst}mixer.qkv.{kind}",
                                                               offset=index * d)
            rules[f"{src}o_proj.{kind}"] = WeightRule(f"{dst}mixer.out.{kind}")
            rules[f"{src}ff_in_a.{kind}"] = WeightRule(f"{dst}feed_forward.up.{kind}", offset=0)
            rules[f"{src}ff_in_b.{kind}"] = WeightRule(f"{dst}feed_forward.up.{kind}",
                                                       offset=half)
            # stored [in, out] (transposed), and in two files' worth of columns: stacked
            # along the parameter's second dimension
            if kind == "weight":
                rules[f"{src}ff_out_a.weight"] = WeightRule(
                    f"{dst}feed_forward.down.weight", transposed=True, dim=1, offset=0)
                rules[f"{src}ff_out_b.weight"] = WeightRule(
                    f"{dst}feed_forward.down.weight", transposed=True, dim=1, offset=half)
            else:
                rules[f"{src}ff_out.bias"] = WeightRule(f"{dst}feed_forward.down.bias")
    return WeightRules(rules=rules, ignore=(r"blocks\.\d+\.rope\.inv_freq",),
                       optional_prefixes=("model.",))


def gpt2_state_to_toy(state: Mapping[str, torch.Tensor], config: GPT2Config
                      ) -> dict[str, torch.Tensor]:
    """The same weights as a GPT-2 checkpoint (Hugging Face names, Conv1D ``[in, out]``), in
    the toy layout; the plain GPT-2 implementation on ``state`` is then the oracle."""
    d, inner = config.n_embd, config.n_inner
    half = inner // 2
    pad = torch.full((PADDED_ROWS, d), 7.0)  # loud: a padded row that leaks in shows
    out = {"model.tok.weight": torch.cat([state["lm_head.weight"], pad]),
           "model.pos.weight": state["transformer.wpe.weight"],
           "model.norm.weight": state["transformer.ln_f.weight"],
           "model.norm.bias": state["transformer.ln_f.bias"]}
    for i in range(config.n_layer):
        src, dst = f"transformer.h.{i}.", f"model.blocks.{i}."
        for kind in ("weight", "bias"):
            out[f"{dst}norm_a.{kind}"] = state[f"{src}ln_1.{kind}"]
            out[f"{dst}norm_b.{kind}"] = state[f"{src}ln_2.{kind}"]
        qkv_w = state[f"{src}attn.c_attn.weight"].t().contiguous()  # [3d, d]
        qkv_b = state[f"{src}attn.c_attn.bias"]
        for index, name in enumerate(("q", "k", "v")):
            out[f"{dst}{name}_proj.weight"] = qkv_w[index * d:(index + 1) * d].clone()
            out[f"{dst}{name}_proj.bias"] = qkv_b[index * d:(index + 1) * d].clone()
        out[f"{dst}o_proj.weight"] = state[f"{src}attn.c_proj.weight"].t().contiguous()
        out[f"{dst}o_proj.bias"] = state[f"{src}attn.c_proj.bias"]
        up_w = state[f"{src}mlp.c_fc.weight"].t().contiguous()  # [inner, d]
        up_b = state[f"{src}mlp.c_fc.bias"]
        out[f"{dst}ff_in_a.weight"], out[f"{dst}ff_in_b.weight"] = \
            up_w[:half].clone(), up_w[half:].clone()
        out[f"{dst}ff_in_a.bias"], out[f"{dst}ff_in_b.bias"] = \
            up_b[:half].clone(), up_b[half:].clone()
        down = state[f"{src}mlp.c_proj.weight"]  # [inner, d] as Conv1D stores it
        out[f"{dst}ff_out_a.weight"] = down[:half].clone()
        out[f"{dst}ff_out_b.weight"] = down[half:].clone()
        out[f"{dst}ff_out.bias"] = state[f"{src}mlp.c_proj.bias"]
        out[f"{dst}rope.inv_freq"] = torch.zeros(4)  # something checkpoints carry along
    return out


def _random_tensors(config: GPT2Config, seed: int,
                    init: RandomInit) -> Iterator[tuple[str, torch.Tensor]]:
    from ayaka_b200.models.registry import resolve_architecture

    gpt2 = resolve_architecture("GPT2LMHeadModel")
    state = dict(gpt2.random_tensors(config, seed, init))
    yield from gpt2_state_to_toy(state, config).items()


def register() -> Architecture:
    return register_architecture(Architecture(
        name=NAME, parse_config=_parse, model_spec=gpt2_model_spec,  # type: ignore[arg-type]
        weight_rules=toy_weight_rules, random_tensors=_random_tensors,  # type: ignore[arg-type]
        config_json=lambda config: {**config.to_json_dict(),  # type: ignore[attr-defined]
                                    "architectures": [NAME]}))
