"""What a caller may ask of generation, validated once.

Names, defaults and ranges follow the reference's ``SamplingParams``
(``python/ayaka/core/params.py:100-150, 180-320``): temperature in [0, 2] with values below
1e-5 meaning greedy, ``top_p`` in (0, 1], ``top_k`` -1 or 0 for off, ``min_p`` in [0, 1],
``seed`` a 63-bit integer or ``None``, ``max_tokens`` 128 by default (``None``: up to the
context), ``min_tokens``, ``stop_token_ids``, ``ignore_eos``, ``repetition_penalty`` > 0,
``frequency_penalty`` and ``presence_penalty`` in [-2, 2], ``logit_bias`` (token id to a bias
in [-100, 100], each id once), ``allowed_token_ids`` (``None`` or a non-empty set). The options
of the reference that belong to its text layer or its server (stop strings, logprobs,
structured output, ``n`` > 1) are not part of this engine.
"""

from __future__ import annotations

from collections.abc import Mapping
from dataclasses import dataclass

from ayaka_b200.errors import InvalidRequestError

__all__ = ["GREEDY_EPS", "LOGIT_BIAS_LIMIT", "MAX_PENALTY", "MAX_SEED", "SamplingParams",
           "TOP_K_DISABLED"]

TOP_K_DISABLED = -1
GREEDY_EPS = 1e-5
MAX_SEED = (1 << 63) - 1
MAX_PENALTY = 2.0
LOGIT_BIAS_LIMIT = 100.0


@dataclass(frozen=True, slots=True, kw_only=True)
class SamplingParams:
    """Generation intent of one request.

    Attributes:
        temperature: softmax temperature; below ``1e-5`` selects greedy decoding.
        top_p: nucleus cumulative probability in ``(0, 1]``.
        top_k: keep the ``k`` most likely tokens; ``-1`` or ``0`` disables.
        min_p: drop tokens less likely than ``min_p`` times the most likely one.
        seed: seed of the request's random numbers; ``None`` or ``-1`` derives one from the
            request id.
        max_tokens: most tokens to generate; ``None`` means up to the model's context.
        min_tokens: tokens generated before a stop token may end the request.
        stop_token_ids: token ids that end the request (the stop token is kept).
        ignore_eos: do not stop at the model's end-of-sequence token.
        repetition_penalty: logits of tokens in the prompt or the output are divided by it
            when positive and multiplied by it when negative.
        frequency_penalty: subtracted from a token's logit once per occurrence in the output.
        presence_penalty: subtracted from the logits of tokens that occur in the output.
        logit_bias: added to the raw logits of the given token ids (a mapping or pairs;
            stored as pairs sorted by id).
        allowed_token_ids: when set, only these ids can be chosen.

    While fewer than ``min_tokens`` tokens exist the stop ids (and the end-of-sequence token
    unless ``ignore_eos``) cannot be chosen at all (``python/ayaka/sampling/logits.py:5-12``).
    """

    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = TOP_K_DISABLED
    min_p: float = 0.0
    seed: int | None = None
    max_tokens: int | None = 128
    min_tokens: int = 0
    stop_token_ids: frozenset[int] = frozenset()
    ignore_eos: bool = False
    repetition_penalty: float = 1.0
    frequency_penalty: float = 0.0
    presence_penalty: float = 0.0
    logit_bias: Mapping[int, float] | tuple[tuple[int, float], ...] | None = None
    allowed_token_ids: frozenset[int] | None = None

    def __post_init__(self) -> None:
        def number(value: object, name: str) -> float:
            if isinstance(value, bool) or not isinstance(value, (int, float)):
                raise InvalidRequestError(f"{name} must be a number, got {value!r}")
            if value != value or value in (float("inf"), float("-inf")):
                raise InvalidRequestError(f"{name} must be finite")
            return float(value)

        def integer(value: object, name: str) -> int:
            if type(value) is not int:
                raise InvalidRequestError(f"{name} must be an integer, got {value!r}")
            return value

        temperature = number(self.temperature, "temperature")
        if not 0.0 <= temperature <= 2.0:
            raise InvalidRequestError(f"temperature must be in [0, 2], got {temperature}")
        top_p = number(self.top_p, "top_p")
        if not 0.0 < top_p <= 1.0:
            raise InvalidRequestError(f"top_p must be in (0, 1], got {top_p}")
        top_k = integer(self.top_k, "top_k")
        if top_k == 0:
            top_k = TOP_K_DISABLED
        if top_k < TOP_K_DISABLED:
            raise InvalidRequestError(f"top_k must be -1 (off) or positive, got {top_k}")
        min_p = number(self.min_p, "min_p")
        if not 0.0 <= min_p <= 1.0:
            raise InvalidRequestError(f"min_p must be in [0, 1], got {min_p}")
        seed = self.seed
        if seed is not None:
            seed = integer(seed, "seed")
            if seed == -1:
                seed = None
            elif not 0 <= seed <= MAX_SEED:
                raise InvalidRequestError(f"seed must be in [0, {MAX_SEED}], got {seed}")
        if self.max_tokens is not None and integer(self.max_tokens, "max_tokens") < 1:
            raise InvalidRequestError(f"max_tokens must be at least 1, got {self.max_tokens}")
        if integer(self.min_tokens, "min_tokens") < 0:
            raise InvalidRequestError("min_tokens must not be negative")
        if self.max_tokens is not None and self.min_tokens > self.max_tokens:
            raise InvalidRequestError("min_tokens exceeds max_tokens")
        stops = frozenset(integer(t, "stop_token_ids") for t in self.stop_token_ids)
        if any(t < 0 for t in stops):
            raise InvalidRequestError("stop_token_ids must not be negative")
        if not isinstance(self.ignore_eos, bool):
            raise InvalidRequestError("ignore_eos must be true or false")
        repetition = number(self.repetition_penalty, "repetition_penalty")
        if not repetition > 0.0:
            raise InvalidRequestError("repetition_penalty must be greater than 0")
        frequency = number(self.frequency_penalty, "frequency_penalty")
        presence = number(self.presence_penalty, "presence_penalty")
        for name, value in (("frequency_penalty", frequency), ("presence_penalty", presence)):
            if not -MAX_PENALTY <= value <= MAX_PENALTY:
                raise InvalidRequestError(
                    f"{name} must be in [-{MAX_PENALTY:g}, {MAX_PENALTY:g}], got {value}")
        bias: tuple[tuple[int, float], ...] | None = None
        if self.logit_bias is not None:
            raw = self.logit_bias
            if isinstance(raw, Mapping):
                items = list(raw.items())
            elif isinstance(raw, (tuple, list)):
                items = list(raw)
            else:
                raise InvalidRequestError(
                    "logit_bias must be a mapping of token ids to biases or a sequence of pairs")
            pairs = []
            for item in items:
                if not isinstance(item, tuple) or len(item) != 2:
                    raise InvalidRequestError("logit_bias entries must be (token id, bias) pairs")
                token = integer(item[0], "logit_bias token")
                if token < 0:
                    raise InvalidRequestError("logit_bias token ids must not be negative")
                value = number(item[1], "logit_bias value")
                if abs(value) > LOGIT_BIAS_LIMIT:
                    raise InvalidRequestError(
                        f"logit_bias values must be in [-{LOGIT_BIAS_LIMIT:g}, "
                        f"{LOGIT_BIAS_LIMIT:g}], got {value}")
                pairs.append((token, value))
            if len({token for token, _ in pairs}) != len(pairs):
                raise InvalidRequestError("logit_bias names a token id twice")
            bias = tuple(sorted(pairs)) or None
        allowed = self.allowed_token_ids
        if allowed is not None:
            allowed = frozenset(integer(t, "allowed_token_ids") for t in allowed)
            if not allowed or any(t < 0 for t in allowed):
                raise InvalidRequestError(
                    "allowed_token_ids must be a non-empty set of non-negative token ids")
        for name, value in (("temperature", temperature), ("top_p", top_p), ("top_k", top_k),
                            ("min_p", min_p), ("seed", seed), ("stop_token_ids", stops),
                            ("repetition_penalty", repetition), ("frequency_penalty", frequency),
                            ("presence_penalty", presence), ("logit_bias", bias),
                            ("allowed_token_ids", allowed)):
            object.__setattr__(self, name, value)

    @property
    def greedy(self) -> bool:
        return self.temperature < GREEDY_EPS or self.top_k == 1

    @property
    def penalises(self) -> bool:
        """Whether a penalty needs the request's own tokens."""
        return self.repetition_penalty != 1.0 or self.frequency_penalty != 0.0 or \
            self.presence_penalty != 0.0

    def banned_at(self, produced: int, eos: int | None) -> frozenset[int]:
        """The ids that cannot be chosen when ``produced`` tokens exist: the stop ids, and
        the end-of-sequence id unless ignored, until ``min_tokens`` tokens exist."""
        if produced >= self.min_tokens:
            return frozenset()
        if eos is not None and not self.ignore_eos:
            return self.stop_token_ids | {eos}
        return self.stop_token_ids

    def adjusts_logits(self, produced: int, eos: int | None) -> bool:
        """Whether the logits of the next token need anything besides temperature, the
        filters and the draw (``python/ayaka/sampling/logits.py:105-128``)."""
        return self.penalises or self.logit_bias is not None or \
            self.allowed_token_ids is not None or bool(self.banned_at(produced, eos))
