"""The tiny configurations and workloads the tests share.

Two configurations that differ in every size and option (heads, head size, widths that are
no power of two, layers, vocabulary, eps, activation, the per-layer attention scale), plus
the two golden cases that the reference's own model code can run. Weights are random with
large deviations so that attention is peaked and a wrong key, page or position shows.
"""

from __future__ import annotations

import torch

from ayaka_b200.weights.random_init import random_state
from ayaka_b200.weights.rules import RandomInit

ARCH = ["GPT2LMHeadModel"]

TINY_A = {
    "architectures": ARCH, "n_layer": 2, "n_embd": 64, "n_head": 4, "n_inner": 256,
    "vocab_size": 256, "n_positions": 128, "layer_norm_epsilon": 1e-5,
    "activation_function": "gelu_new", "scale_attn_by_inverse_layer_idx": False,
    "tie_word_embeddings": True,
}
TINY_B = {
    "architectures": ARCH, "n_layer": 3, "n_embd": 96, "n_head": 3, "n_inner": 320,
    "vocab_size": 503, "n_positions": 256, "layer_norm_epsilon": 1e-6,
    "activation_function": "gelu", "scale_attn_by_inverse_layer_idx": True,
    "tie_word_embeddings": True,
}
# a third shape: head size 48 (a multiple of 16 that is no power of two), 5 heads, untied head
TINY_C = {
    "architectures": ARCH, "n_layer": 2, "n_embd": 240, "n_head": 5, "n_inner": 700,
    "vocab_size": 1021, "n_positions": 320, "layer_norm_epsilon": 3e-5,
    "activation_function": "gelu_pytorch_tanh", "scale_attn_by_inverse_layer_idx": True,
    "tie_word_embeddings": False,
}

# a fourth: head size 64 and a context long enough for prompt portions of 256 rows and more,
# which the tcgen05 attention kernel serves in bfloat16
TINY_D = {
    "architectures": ARCH, "n_layer": 2, "n_embd": 128, "n_head": 2, "n_inner": 272,
    "vocab_size": 300, "n_positions": 640, "layer_norm_epsilon": 2e-5,
    "activation_function": "gelu_new", "scale_attn_by_inverse_layer_idx": False,
    "tie_word_embeddings": True,
}

#: Initialisations with the small deviations a trained checkpoint has, and a "loud" one for sensitive tests.
INIT_A = RandomInit(weight_std=0.02, scale_residual_projections=True, bias_std=0.0, norm_std=0.0)
INIT_B = RandomInit(weight_std=0.02, scale_residual_projections=False, bias_std=0.02,
                    norm_std=0.02)
INIT_LOUD = RandomInit(weight_std=0.2, scale_residual_projections=False, bias_std=0.1,
                       norm_std=0.1)
# for TINY_D: twice as wide, so the same deviation is louder; at 0.2 the bfloat16 rounding of
# the activations alone (the same with either attention kernel) reaches the tolerance
INIT_LOUD_WIDE = RandomInit(weight_std=0.14, scale_residual_projections=False, bias_std=0.1,
                            norm_std=0.1)

CASES = {
    "golden_a": {"config": TINY_A, "seed": 0, "init": INIT_LOUD, "lengths": (5, 17, 32, 9),
                 "chunk": 7, "keep_every": 1},
    "golden_b": {"config": {**TINY_B, "scale_attn_by_inverse_layer_idx": False}, "seed": 1,
                 "init": INIT_LOUD, "lengths": (1, 64, 130), "chunk": 48, "keep_every": 8},
}


def case_config(case: dict) -> dict:
    return dict(case["config"])


def case_state(case: dict, dtype: str = "float32") -> dict[str, torch.Tensor]:
    return random_state(case["config"], case["seed"], case["init"], dtype)


def random_tokens(vocab: int, length: int, seed: int) -> list[int]:
    generator = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (length,), generator=generator).tolist()


def case_sequences(case: dict) -> list[list[int]]:
    vocab = case["config"]["vocab_size"]
    return [random_tokens(vocab, length, 1000 * case["seed"] + index)
            for index, length in enumerate(case["lengths"])]
