"""What a caller may ask of generation, validated once.

Names, defaults and ranges follow the reference's ``SamplingParams``
(``python/ayaka/core/params.py:100-150, 180-320``): temperature in [0, 2] with values below
1e-5 meaning greedy, ``top_p`` in (0, 1], ``top_k`` -1 or 0 for off, ``min_p`` in [0, 1],
``seed`` a 63-bit integer or ``None``, ``max_tokens`` 128 by default (``None``: up to the
context), ``min_tokens``, ``stop_token_ids``, ``ignore_eos``. The options of the reference
that belong to its text layer or its server (stop strings, penalties, logprobs, logit bias,
structured output, ``n`` > 1) are not part of this engine.
"""

from __future__ import annotations

from dataclasses import dataclass

from ayaka_b200.errors import InvalidRequestError

__all__ = ["GREEDY_EPS", "MAX_SEED", "SamplingParams", "TOP_K_DISABLED"]

TOP_K_DISABLED = -1
GREEDY_EPS = 1e-5
MAX_SEED = (1 << 63) - 1


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
        for name, value in (("temperature", temperature), ("top_p", top_p), ("top_k", top_k),
                            ("min_p", min_p), ("seed", seed), ("stop_token_ids", stops)):
            object.__setattr__(self, name, value)

    @property
    def greedy(self) -> bool:
        return self.temperature < GREEDY_EPS or self.top_k == 1
