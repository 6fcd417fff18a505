"""The typed model configuration, read from GPT-2's own ``config.json`` keys.

Key spellings and defaults follow the reference's parser
(``python/ayaka/configs/model.py:182-191, 310-396``): the first present, non-null
spelling of a key wins, ``n_inner`` defaults to ``4 * n_embd``, ``head_dim`` to
``n_embd // n_head``, ``tie_word_embeddings`` to true; every missing key is listed in
one error. Two things differ on purpose: ``scale_attn_by_inverse_layer_idx`` is read and
honoured (the reference ignores it), and an option that would change the arithmetic but
is not implemented (``reorder_and_upcast_attn``, ``add_cross_attention``) is refused
instead of being ignored.
"""

from __future__ import annotations

import json
import math
from collections.abc import Mapping
from dataclasses import dataclass, fields
from pathlib import Path

from ayaka_b200.errors import ConfigError, ModelLoadError

__all__ = ["GPT2Config", "read_config_json"]

#: field -> spellings in config.json, GPT-2's own first.
_KEYS: dict[str, tuple[str, ...]] = {
    "vocab_size": ("vocab_size",),
    "n_embd": ("n_embd", "hidden_size"),
    "n_layer": ("n_layer", "num_hidden_layers"),
    "n_head": ("n_head", "num_attention_heads"),
    "n_inner": ("n_inner", "intermediate_size"),
    "n_positions": ("n_positions", "max_position_embeddings"),
    "activation_function": ("activation_function", "hidden_act"),
    "layer_norm_epsilon": ("layer_norm_epsilon", "layer_norm_eps"),
}
_REFUSED_WHEN_TRUE = ("reorder_and_upcast_attn", "add_cross_attention")
_MAX_CONFIG_BYTES = 16 << 20


def _strict_object(pairs: list[tuple[str, object]]) -> dict[str, object]:
    seen: dict[str, object] = {}
    for key, value in pairs:
        if key in seen:
            raise ModelLoadError(f"config.json repeats the key {key!r}")
        seen[key] = value
    return seen


def read_config_json(model_dir: str | Path) -> dict[str, object]:
    """Parse ``model_dir/config.json`` strictly: an object, no repeated key, at most 16 MiB."""
    path = Path(model_dir) / "config.json"
    if not path.is_file():
        raise ModelLoadError(f"{path} does not exist", context={"path": str(path)})
    if path.stat().st_size > _MAX_CONFIG_BYTES:
        raise ModelLoadError(f"{path} is larger than {_MAX_CONFIG_BYTES} bytes")
    try:
        parsed = json.loads(path.read_text(encoding="utf-8"), object_pairs_hook=_strict_object)
    except json.JSONDecodeError as error:
        raise ModelLoadError(f"{path} is not valid JSON: {error}") from None
    if not isinstance(parsed, dict):
        raise ModelLoadError(f"{path} must hold a JSON object")
    return parsed


def _require_int(value: object, path: str, minimum: int = 1) -> int:
    if type(value) is not int:
        raise ConfigError(path, "WRONG_TYPE", f"must be an integer, got {value!r}")
    if value < minimum:
        raise ConfigError(path, "INVALID_RANGE", f"must be at least {minimum}, got {value}")
    return value


def _require_bool(value: object, path: str) -> bool:
    if type(value) is not bool:
        raise ConfigError(path, "WRONG_TYPE", f"must be true or false, got {value!r}")
    return value


@dataclass(frozen=True, slots=True)
class GPT2Config:
    """Sizes and options of one GPT-2 checkpoint; every number the model uses is here.

    Attributes:
        architecture: ``architectures[0]`` of ``config.json``; the registry key.
        vocab_size: rows of ``wte`` and width of the logits.
        n_embd: width of the residual stream.
        n_layer: number of blocks.
        n_head: attention heads (keys/values have as many).
        n_inner: width of the feed-forward hidden layer.
        n_positions: rows of ``wpe``; the longest sequence.
        activation_function: ``gelu_new`` / ``gelu_pytorch_tanh`` (tanh form) or ``gelu`` (erf).
        layer_norm_epsilon: eps of every LayerNorm.
        head_dim: width of a head; ``n_head * head_dim`` must equal ``n_embd``.
        scale_attn_by_inverse_layer_idx: divide layer ``i``'s attention scale by ``i + 1``.
        tie_word_embeddings: the output head is ``wte``.
        eos_token_id: token that ends a generation, or ``None``.
    """

    architecture: str
    vocab_size: int
    n_embd: int
    n_layer: int
    n_head: int
    n_inner: int
    n_positions: int
    activation_function: str
    layer_norm_epsilon: float
    head_dim: int
    scale_attn_by_inverse_layer_idx: bool = False
    tie_word_embeddings: bool = True
    eos_token_id: int | None = None

    def __post_init__(self) -> None:
        if not isinstance(self.architecture, str) or not self.architecture.strip():
            raise ConfigError("model.architecture", "WRONG_TYPE", "must be a non-empty string")
        if not isinstance(self.activation_function, str) or not self.activation_function:
            raise ConfigError("model.activation_function", "WRONG_TYPE", "must be a string")
        for name in ("vocab_size", "n_embd", "n_layer", "n_head", "n_inner", "n_positions",
                     "head_dim"):
            _require_int(getattr(self, name), f"model.{name}")
        eps = self.layer_norm_epsilon
        if isinstance(eps, bool) or not isinstance(eps, (int, float)):
            raise ConfigError("model.layer_norm_epsilon", "WRONG_TYPE", "must be a number")
        if not math.isfinite(eps) or eps <= 0:
            raise ConfigError("model.layer_norm_epsilon", "INVALID_RANGE",
                              "must be finite and positive")
        object.__setattr__(self, "layer_norm_epsilon", float(eps))
        _require_bool(self.scale_attn_by_inverse_layer_idx,
                      "model.scale_attn_by_inverse_layer_idx")
        _require_bool(self.tie_word_embeddings, "model.tie_word_embeddings")
        if self.eos_token_id is not None:
            _require_int(self.eos_token_id, "model.eos_token_id", minimum=0)

    @classmethod
    def from_json_dict(cls, config: Mapping[str, object]) -> GPT2Config:
        """Build the configuration from a parsed ``config.json``."""
        found: dict[str, object] = {}
        for name, spellings in _KEYS.items():
            for key in spellings:
                if config.get(key) is not None:
                    found[name] = config[key]
                    break
        architectures = config.get("architectures")
        if isinstance(architectures, (list, tuple)) and architectures:
            found["architecture"] = architectures[0]
        if "n_inner" not in found and type(found.get("n_embd")) is int:
            found["n_inner"] = 4 * found["n_embd"]  # type: ignore[operator]
        missing = [name for name in ("architecture", *_KEYS) if name not in found]
        if missing:
            raise ModelLoadError(
                "config.json lacks required keys for " + ", ".join(missing),
                context={"missing": tuple(missing)},
            )
        refused = [key for key in _REFUSED_WHEN_TRUE if config.get(key)]
        if refused:
            raise ModelLoadError(
                "config.json sets options that change the arithmetic and are not implemented: "
                + ", ".join(refused),
                context={"refused": tuple(refused)},
            )
        heads = _require_int(found["n_head"], "model.n_head")
        hidden = _require_int(found["n_embd"], "model.n_embd")
        head_dim = config.get("head_dim")
        if head_dim is None:
            if hidden % heads:
                raise ConfigError("model.head_dim", "HEAD_DIM_UNDEFINED",
                                  f"n_embd {hidden} is not a multiple of n_head {heads}")
            head_dim = hidden // heads
        kv_heads = config.get("num_key_value_heads")
        if kv_heads is not None and kv_heads != heads:
            raise ModelLoadError(
                f"GPT-2 uses multi-head attention, but num_key_value_heads is {kv_heads} "
                f"for {heads} heads")
        eos = config.get("eos_token_id")
        return cls(
            architecture=found["architecture"],  # type: ignore[arg-type]
            vocab_size=found["vocab_size"],  # type: ignore[arg-type]
            n_embd=hidden,
            n_layer=found["n_layer"],  # type: ignore[arg-type]
            n_head=heads,
            n_inner=found["n_inner"],  # type: ignore[arg-type]
            n_positions=found["n_positions"],  # type: ignore[arg-type]
            activation_function=found["activation_function"],  # type: ignore[arg-type]
            layer_norm_epsilon=found["layer_norm_epsilon"],  # type: ignore[arg-type]
            head_dim=head_dim,  # type: ignore[arg-type]
            scale_attn_by_inverse_layer_idx=config.get(  # type: ignore[arg-type]
                "scale_attn_by_inverse_layer_idx", False),
            tie_word_embeddings=config.get("tie_word_embeddings", True),  # type: ignore[arg-type]
            eos_token_id=eos if type(eos) is int else None,
        )

    def to_json_dict(self) -> dict[str, object]:
        """The ``config.json`` content that reads back as this configuration."""
        out: dict[str, object] = {"architectures": [self.architecture], "model_type": "gpt2"}
        for field in fields(self):
            if field.name == "architecture":
                continue
            value = getattr(self, field.name)
            if value is not None:
                out[field.name] = value
        return out
