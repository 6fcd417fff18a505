"""What generation returns. Shapes follow the reference's ``RequestOutput`` /
``CompletionOutput`` / ``Usage`` (``python/ayaka/core/outputs.py:56-200``) without the text
fields: this engine takes and returns token ids."""

from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum

__all__ = ["CompletionOutput", "FinishReason", "RequestOutput", "Usage"]


class FinishReason(str, Enum):
    """Why a request ended (``python/ayaka/core/types.py:92-104``)."""

    STOP = "stop"
    LENGTH = "length"
    CANCELLED = "cancelled"
    ERROR = "error"


@dataclass(frozen=True, slots=True)
class Usage:
    prompt_tokens: int
    completion_tokens: int


@dataclass(frozen=True, slots=True)
class CompletionOutput:
    index: int
    token_ids: tuple[int, ...]
    finish_reason: FinishReason | None = None
    stop_reason: int | None = None  # the stop token that ended it


@dataclass(frozen=True, slots=True)
class RequestOutput:
    """One request's result (final, or the new tokens of one step when streaming)."""

    request_id: str
    prompt_token_ids: tuple[int, ...]
    outputs: tuple[CompletionOutput, ...]
    finished: bool
    usage: Usage | None = None
    error: str | None = None
    seed: int | None = None
    notes: tuple[str, ...] = field(default_factory=tuple)
