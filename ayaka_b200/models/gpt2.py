"""GPT-2 (``GPT2LMHeadModel``) as data: its parts, its checkpoint names, its random weights.

Block: ``x += attn(ln_1(x)); x += mlp(ln_2(x))``; ``hidden = ln_f(x)``; ``logits = hidden @
wte.T`` (``python/ayaka/models/gpt2.py:1-18, 99-101, 170-182`` in the reference). Checkpoints
store the four projections of a block as Conv1D weights ``[in, out]`` with ``c_attn`` already
fused (columns: queries, keys, values); parameters here are ``[out, in]``, so those four are
transposed on load (``python/ayaka/models/gpt2.py:124-129``). Names may carry the prefix
``transformer.``; the stored causal masks and, when tied, ``lm_head.weight`` are ignored
(``:51-61, 162``).
"""

from __future__ import annotations

import hashlib
import math
from collections.abc import Iterator, Mapping

import torch

from ayaka_b200.config.model import GPT2Config
from ayaka_b200.errors import ModelLoadError
from ayaka_b200.models.registry import Architecture, register_architecture
from ayaka_b200.parts.spec import LayerSpec, ModelSpec, PartSpec, Run
from ayaka_b200.weights.rules import RandomInit, WeightRule, WeightRules

__all__ = ["GPT2", "gpt2_model_spec", "gpt2_weight_rules"]

#: ``activation_function`` values and the activation kernel each names.
_ACTIVATIONS = {"gelu_new": "gelu_tanh", "gelu_pytorch_tanh": "gelu_tanh", "gelu": "gelu_erf"}


def _parse(config_json: Mapping[str, object]) -> GPT2Config:
    config = GPT2Config.from_json_dict(config_json)
    problems = []
    if config.n_head * config.head_dim != config.n_embd:
        problems.append(f"n_head * head_dim is {config.n_head * config.head_dim}, not n_embd "
                        f"{config.n_embd}")
    if config.activation_function not in _ACTIVATIONS:
        problems.append(f"activation_function {config.activation_function!r} is not one of "
                        f"{sorted(_ACTIVATIONS)}")
    if config.head_dim % 16 or config.head_dim > 256:
        problems.append(f"head_dim {config.head_dim} is not a multiple of 16 up to 256, which "
                        "the attention kernels need")
    if problems:
        raise ModelLoadError(f"cannot build {config.architecture} from this config: "
                             + "; ".join(problems))
    return config


def gpt2_model_spec(config: GPT2Config) -> ModelSpec:
    """The model as parts. Every size comes from ``config``."""
    width = config.n_embd
    norm = PartSpec("layer_norm", width=width, eps=config.layer_norm_epsilon, bias=True)
    layers = []
    for index in range(config.n_layer):
        scale = config.head_dim ** -0.5
        if config.scale_attn_by_inverse_layer_idx:
            scale /= index + 1
        layers.append(LayerSpec(
            block="pre_norm",
            mixer=PartSpec("attention", width=width, num_heads=config.n_head,
                           num_kv_heads=config.n_head, head_dim=config.head_dim, scale=scale,
                           window=0, bias=True),
            feed_forward=PartSpec("dense", width=width, inner=config.n_inner,
                                  activation=_ACTIVATIONS[config.activation_function],
                                  bias=True),
            mixer_norm=norm,
            feed_forward_norm=norm,
        ))
    return ModelSpec(
        hidden_size=width,
        vocab_size=config.vocab_size,
        max_positions=config.n_positions,
        embedding=PartSpec("token", vocab_size=config.vocab_size, width=width),
        position=PartSpec("learned", max_positions=config.n_positions, width=width),
        layers=tuple(layers),
        order=tuple(Run(layer=index) for index in range(config.n_layer)),
        final_norm=norm,
        head=PartSpec("linear", vocab_size=config.vocab_size, width=width,
                      tied=config.tie_word_embeddings),
        eos_token_id=config.eos_token_id,
    )


def gpt2_weight_rules(config: GPT2Config) -> WeightRules:
    rules: dict[str, WeightRule] = {
        "wte.weight": WeightRule("embedding.weight"),
        "wpe.weight": WeightRule("position.weight"),
        "ln_f.weight": WeightRule("final_norm.weight"),
        "ln_f.bias": WeightRule("final_norm.bias"),
    }
    for i in range(config.n_layer):
        src, dst = f"h.{i}.", f"layers.{i}."
        for kind in ("weight", "bias"):
            rules[f"{src}ln_1.{kind}"] = WeightRule(f"{dst}mixer_norm.{kind}")
            rules[f"{src}ln_2.{kind}"] = WeightRule(f"{dst}feed_forward_norm.{kind}")
            transposed = kind == "weight"
            rules[f"{src}attn.c_attn.{kind}"] = WeightRule(f"{dst}mixer.qkv.{kind}", transposed)
            rules[f"{src}attn.c_proj.{kind}"] = WeightRule(f"{dst}mixer.out.{kind}", transposed)
            rules[f"{src}mlp.c_fc.{kind}"] = WeightRule(f"{dst}feed_forward.up.{kind}",
                                                        transposed)
            rules[f"{src}mlp.c_proj.{kind}"] = WeightRule(f"{dst}feed_forward.down.{kind}",
                                                          transposed)
    ignore = [r"h\.\d+\.attn\.(?:bias|masked_bias)"]
    if config.tie_word_embeddings:
        ignore.append(r"lm_head\.weight")
    else:
        rules["lm_head.weight"] = WeightRule("head.weight")
    return WeightRules(rules=rules, ignore=tuple(ignore), optional_prefixes=("transformer.",))


def _generator(seed: int, name: str) -> torch.Generator:
    digest = hashlib.blake2b(f"{seed}:{name}".encode(), digest_size=8).digest()
    return torch.Generator().manual_seed(int.from_bytes(digest, "big") & ((1 << 63) - 1))


def _random_tensors(config: GPT2Config, seed: int,
                    init: RandomInit) -> Iterator[tuple[str, torch.Tensor]]:
    """Random float32 tensors under Hugging Face names in checkpoint layout (Conv1D
    ``[in, out]``). Each tensor has its own generator, seeded from ``seed`` and its name,
    so a tensor's values do not depend on which others were drawn."""
    d, inner = config.n_embd, config.n_inner

    def normal(name: str, shape: tuple[int, ...], std: float, mean: float = 0.0) -> torch.Tensor:
        if std == 0.0:
            return torch.full(shape, mean, dtype=torch.float32)
        values = torch.randn(shape, generator=_generator(seed, name), dtype=torch.float32)
        return values.mul_(std).add_(mean)

    proj_std = init.weight_std / math.sqrt(2 * config.n_layer) \
        if init.scale_residual_projections else init.weight_std
    p = "transformer."
    yield f"{p}wte.weight", normal("wte.weight", (config.vocab_size, d), init.weight_std)
    yield f"{p}wpe.weight", normal("wpe.weight", (config.n_positions, d), init.weight_std)
    for i in range(config.n_layer):
        b = f"h.{i}."
        for ln in ("ln_1", "ln_2"):
            yield f"{p}{b}{ln}.weight", normal(f"{b}{ln}.weight", (d,), init.norm_std, 1.0)
            yield f"{p}{b}{ln}.bias", normal(f"{b}{ln}.bias", (d,), init.norm_std)
        for name, shape, std in (
            ("attn.c_attn", (d, 3 * d), init.weight_std),
            ("attn.c_proj", (d, d), proj_std),
            ("mlp.c_fc", (d, inner), init.weight_std),
            ("mlp.c_proj", (inner, d), proj_std),
        ):
            yield f"{p}{b}{name}.weight", normal(f"{b}{name}.weight", shape, std)
            yield f"{p}{b}{name}.bias", normal(f"{b}{name}.bias", (shape[1],), init.bias_std)
    yield f"{p}ln_f.weight", normal("ln_f.weight", (d,), init.norm_std, 1.0)
    yield f"{p}ln_f.bias", normal("ln_f.bias", (d,), init.norm_std)
    if not config.tie_word_embeddings:
        yield "lm_head.weight", normal("lm_head.weight", (config.vocab_size, d), init.weight_std)


GPT2 = register_architecture(Architecture(
    name="GPT2LMHeadModel",
    parse_config=_parse,
    model_spec=gpt2_model_spec,  # type: ignore[arg-type]
    weight_rules=gpt2_weight_rules,  # type: ignore[arg-type]
    random_tensors=_random_tensors,  # type: ignore[arg-type]
    config_json=lambda config: config.to_json_dict(),  # type: ignore[attr-defined]
))
