"""One request's state between admission and its last token."""

from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum

import numpy as np

from ayaka_b200.engine.outputs import FinishReason
from ayaka_b200.errors import EngineError
from ayaka_b200.sampling.params import SamplingParams

__all__ = ["Request", "RequestEvent", "RequestStatus"]


class RequestStatus(str, Enum):
    WAITING = "waiting"
    RUNNING = "running"
    FINISHED = "finished"


_LEGAL = {
    RequestStatus.WAITING: {RequestStatus.RUNNING, RequestStatus.FINISHED},
    RequestStatus.RUNNING: {RequestStatus.FINISHED},
    RequestStatus.FINISHED: set(),
}


@dataclass(frozen=True, slots=True)
class RequestEvent:
    """What one step changed for a request: new tokens, and the end if it ended."""

    request_id: str
    tokens: tuple[int, ...]
    finish_reason: FinishReason | None = None
    stop_reason: int | None = None
    error: str | None = None


@dataclass(slots=True)
class Request:
    """A request the scheduler knows.

    ``computed`` counts the tokens whose keys and values are in the cache. The request is
    prefilling while ``computed < len(prompt)``; afterwards its last output token is the one
    not yet fed (``pending``), so ``computed == len(prompt) + len(output) - 1``.
    """

    request_id: str
    prompt: tuple[int, ...]
    #: the prompt once more as an array: a step takes its portions as views of it
    prompt_ids: np.ndarray
    params: SamplingParams
    seed: int
    arrival: int
    status: RequestStatus = RequestStatus.WAITING
    output: list[int] = field(default_factory=list)
    computed: int = 0
    finish_reason: FinishReason | None = None

    def move(self, status: RequestStatus) -> None:
        if status not in _LEGAL[self.status]:
            raise EngineError(f"request {self.request_id!r} cannot go from {self.status.value} "
                              f"to {status.value}")
        self.status = status

    @property
    def prefilling(self) -> bool:
        return self.computed < len(self.prompt)

    @property
    def pending(self) -> int | None:
        """The sampled token that has not been fed yet, if any."""
        if self.prefilling or not self.output:
            return None
        return self.output[-1]

    def tokens_left(self, max_positions: int) -> int:
        left = max_positions - len(self.prompt) - len(self.output)
        if self.params.max_tokens is not None:
            left = min(left, self.params.max_tokens - len(self.output))
        return left

    def accept(self, token: int, eos: int | None,
               max_positions: int) -> tuple[FinishReason | None, int | None]:
        """Take a sampled token; say whether it ends the request and why. A stop token is
        kept as the last token and counts only once more than ``min_tokens`` tokens exist
        (``python/ayaka/scheduler/request.py:217-251``)."""
        self.output.append(token)
        stops = set(self.params.stop_token_ids)
        if eos is not None and not self.params.ignore_eos:
            stops.add(eos)
        if token in stops and len(self.output) > self.params.min_tokens:
            return FinishReason.STOP, token
        if self.tokens_left(max_positions) <= 0:
            return FinishReason.LENGTH, None
        return None, None
