"""The plain implementation against the reference's own model code (golden files) and
against itself in float64."""

from __future__ import annotations

from pathlib import Path

import numpy as np
import pytest
import torch

import plain_gpt2 as plain
from cases import CASES, TINY_B, INIT_LOUD, case_config, case_sequences, case_state, random_tokens
from ayaka_b200.weights.random_init import random_state

GOLDEN = Path(__file__).resolve().parent / "golden"


@pytest.mark.parametrize("name", ["golden_a", "golden_b"])
def test_plain_matches_golden(name: str) -> None:
    case = CASES[name]
    golden = np.load(GOLDEN / f"{name}.npz")
    state, config = case_state(case), case_config(case)
    for index, tokens in enumerate(case_sequences(case)):
        assert golden[f"tokens_{index}"].tolist() == tokens
        ours = plain.logits(state, config, torch.tensor(tokens))
        rows = golden[f"rows_{index}"]
        expected = torch.from_numpy(golden[f"logits_{index}"])
        torch.testing.assert_close(ours[rows], expected, rtol=1e-4, atol=1e-4)


def test_float32_agrees_with_float64() -> None:
    state = random_state(TINY_B, 3, INIT_LOUD)
    tokens = torch.tensor(random_tokens(TINY_B["vocab_size"], 90, 5))
    single = plain.logits(state, TINY_B, tokens)
    double = plain.logits(plain.cast_state(state, torch.float64), TINY_B, tokens)
    torch.testing.assert_close(single.double(), double, rtol=1e-4, atol=1e-4)


def test_layer_scale_changes_the_result() -> None:
    state = random_state(TINY_B, 3, INIT_LOUD)
    tokens = torch.tensor(random_tokens(TINY_B["vocab_size"], 40, 6))
    with_scale = plain.logits(state, TINY_B, tokens)
    without = plain.logits(state, {**TINY_B, "scale_attn_by_inverse_layer_idx": False}, tokens)
    assert (with_scale - without).abs().max() > 1e-2
    # layer 0 divides by 1: a one-layer model is unchanged
    one = {**TINY_B, "n_layer": 1}
    state1 = random_state(one, 3, INIT_LOUD)
    a = plain.logits(state1, one, tokens)
    b = plain.logits(state1, {**one, "scale_attn_by_inverse_layer_idx": False}, tokens)
    torch.testing.assert_close(a, b)


def test_parts_against_torch() -> None:
    g = torch.Generator().manual_seed(0)
    x = torch.randn(7, 96, generator=g)
    w, b = torch.randn(96, generator=g), torch.randn(96, generator=g)
    torch.testing.assert_close(plain.layer_norm(x, w, b, 1e-6),
                               torch.nn.functional.layer_norm(x, (96,), w, b, 1e-6),
                               rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(plain.gelu(x, "gelu"), torch.nn.functional.gelu(x))
    torch.testing.assert_close(plain.gelu(x, "gelu_new"),
                               torch.nn.functional.gelu(x, approximate="tanh"))
    q, k, v = (torch.randn(11, 3, 32, generator=g) for _ in range(3))
    ours = plain.causal_attention(q, k, v, 0.3)
    ref = torch.nn.functional.scaled_dot_product_attention(
        q.transpose(0, 1), k.transpose(0, 1), v.transpose(0, 1), is_causal=True, scale=0.3)
    torch.testing.assert_close(ours, ref.transpose(0, 1), rtol=1e-5, atol=1e-5)
    # a window of 4: row 10 sees keys 7..10 only
    windowed = plain.causal_attention(q, k, v, 0.3, window=4)
    tail = plain.causal_attention(q[7:], k[7:], v[7:], 0.3)
    torch.testing.assert_close(windowed[10], tail[3], rtol=1e-5, atol=1e-5)


def test_philox_known_answers() -> None:
    # Random123 known-answer vectors for philox4x32_10
    assert plain.philox4x32_10((0, 0, 0, 0), (0, 0)) == (
        0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8)
    assert plain.philox4x32_10((0xFFFFFFFF,) * 4, (0xFFFFFFFF,) * 2) == (
        0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD)
    assert plain.philox4x32_10((0x243F6A88, 0x85A308D3, 0x13198A2E, 0x03707344),
                               (0xA4093822, 0x299F31D0)) == (
        0xD16CFE09, 0x94FDCCEB, 0x5001E420, 0x24126EA1)
    u = plain.draw_uniform(1234, 17)
    assert 0.0 <= u < 1.0 and u == plain.draw_uniform(1234, 17)
    assert u != plain.draw_uniform(1234, 18)


def test_sampling_oracle() -> None:
    row = torch.tensor([0.0, 2.0, 2.0, -1.0, 1.0])
    assert plain.argmax_smallest_id(row) == 1
    assert plain.sample_token(row, 0.0, 0.7) == 1
    # canonical order: ids 1, 2 (tie, smaller first), 4, 0, 3
    p = torch.softmax(row.double(), 0)
    assert plain.sample_token(row, 1.0, 0.0) == 1
    assert plain.sample_token(row, 1.0, float(p[1]) + 1e-9) == 2
    assert plain.sample_token(row, 1.0, float(p[1] + p[2]) + 1e-9) == 4
    assert plain.sample_token(row, 1.0, 0.999999) == 3
    assert plain.sample_token(row, 1.0, 0.999999, top_k=2) == 2
    assert plain.sample_token(row, 1.0, 0.999999, top_p=0.5) == 2
    assert plain.sample_token(row, 1.0, 0.999999, min_p=0.3) == 4


def test_bfloat16_attention_weights_alone_move_the_logits_by_this_much():
    """The noise floor of every bfloat16 comparison. A tensor-core attention kernel rounds
    its weights exp(s - reference) to bfloat16, and the reference is whatever running maximum
    the kernel holds at that block; two valid kernels therefore round every weight
    differently. Here the plain implementation with bfloat16 roundings runs twice, with the
    reference moved by a fraction of a bit: the logits of the loud tiny model A move by
    several thousandths of their scale at single places and by about a thousandth in a
    row's root-mean-square. The engine tests' limits against this oracle stand on these
    figures."""
    import plain_rounded

    case = CASES["golden_a"]
    state = plain.cast_state(case_state(case, "bfloat16"), torch.float64)
    config = case_config(case)
    tokens = torch.tensor(case_sequences({**case, "lengths": (128,)})[0])
    first = plain_rounded.logits(state, config, tokens, round_weights=True)
    second = plain_rounded.logits(state, config, tokens, round_weights=True, reference_shift=0.37)
    scale = float(first.abs().max())
    largest = float((first - second).abs().max()) / scale
    row_rms = float(((first - second) ** 2).mean(dim=1).sqrt().median()) / scale
    assert 2e-3 < largest < 1.2e-2, largest
    assert 3e-4 < row_rms < 3e-3, row_rms
