"""Typed errors of the engine.

One base class, one subclass per kind of failure, each with a stable ``code``. The
command line maps the kinds to exit codes; nothing prints a traceback for them.
Follows the split of the reference's ``python/ayaka/core/errors.py:41-196`` (base with
``code``/``context``, a configuration error with a path, load, capacity, request and
backend errors) without its serialisation machinery.
"""

from __future__ import annotations

from collections.abc import Mapping

__all__ = [
    "AyakaError",
    "BackendError",
    "CapacityError",
    "ConfigError",
    "EngineError",
    "InvalidRequestError",
    "ModelLoadError",
]


class AyakaError(Exception):
    """Base of every error the engine raises on purpose."""

    code: str = "ayaka_error"

    def __init__(self, message: str, *, context: Mapping[str, object] | None = None) -> None:
        self.message = message
        self.context: dict[str, object] = dict(context or {})
        super().__init__(message)


class ConfigError(AyakaError, ValueError):
    """A configuration value is missing, of the wrong type or out of range."""

    code = "config_error"

    def __init__(self, path: str, code: str, message: str) -> None:
        self.path = path
        super().__init__(f"{path}: {message} [{code}]", context={"path": path})
        self.code = code


class ModelLoadError(AyakaError):
    """A model folder cannot be read, or does not fit the model built from its config."""

    code = "model_load_error"


class CapacityError(AyakaError):
    """The cache or a buffer is too small for what was asked."""

    code = "capacity_error"


class InvalidRequestError(AyakaError, ValueError):
    """A request that can never be served (empty prompt, too long, bad parameters)."""

    code = "invalid_request"


class BackendError(AyakaError):
    """A kernel refused its arguments, the CUDA library is missing, or a launch failed."""

    code = "backend_error"


class EngineError(AyakaError):
    """The engine was used out of protocol (two steps in flight, use after close)."""

    code = "engine_error"
