"""Weights: safetensors by tensor name, the binding rules, and the random-weights mode."""

from ayaka_b200.weights.loader import TensorSource, load_into, open_model_dir
from ayaka_b200.weights.rules import RandomInit, WeightRule, WeightRules
from ayaka_b200.weights.safetensors import SafetensorsFile, write_safetensors

__all__ = ["RandomInit", "SafetensorsFile", "TensorSource", "WeightRule", "WeightRules",
           "load_into", "open_model_dir", "write_safetensors"]
