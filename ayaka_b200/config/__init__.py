"""Typed configurations: the model's (from ``config.json``) and the engine's."""

from ayaka_b200.config.engine import EngineConfig
from ayaka_b200.config.model import GPT2Config, read_config_json

__all__ = ["EngineConfig", "GPT2Config", "read_config_json"]
