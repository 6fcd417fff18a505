"""The engine against the plain implementation under every way of cutting the work, in
float32 and in bfloat16, on three tiny configurations that differ in every size and option.

A difference that shows in only one way of cutting points at the cache or the batch; the
failure message names the first wrong position with its page and slot."""

from __future__ import annotations

import pytest

import engine_support as es
from cases import INIT_LOUD, INIT_LOUD_WIDE, TINY_A, TINY_B, TINY_C, TINY_D, random_tokens

pytestmark = pytest.mark.gpu

CONFIGS = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D}
LENGTHS = {"A": (5, 17, 32, 9, 100, 128), "B": (1, 64, 130, 200, 47), "C": (70, 33, 250, 2),
           "D": (600, 257, 40, 333)}
INITS = {"A": INIT_LOUD, "B": INIT_LOUD, "C": INIT_LOUD, "D": INIT_LOUD_WIDE}
DTYPES = ("float32", "bfloat16")


def sequences_of(name: str) -> dict[str, list[int]]:
    vocab = CONFIGS[name]["vocab_size"]
    return {f"{name.lower()}{index}": random_tokens(vocab, length, 100 * ord(name) + index)
            for index, length in enumerate(LENGTHS[name])}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """(model folder, float32 state for the plain side, config) per (config, dtype)."""
    made = {}
    for name, config in CONFIGS.items():
        for dtype in DTYPES:
            folder = tmp_path_factory.mktemp(f"tiny_{name}_{dtype}")
            made[name, dtype] = (*es.make_model(folder, config, seed=ord(name), init=INITS[name],
                                                dtype=dtype), config)
    return made


@pytest.fixture(scope="module")
def expected(models):
    return {key: es.plain_logits(state, config, sequences_of(key[0]))
            for key, (_, state, config) in models.items()}


@pytest.fixture(scope="module")
def expected_rounded(models):
    """The bfloat16 engine's second oracle: the plain implementation with bfloat16 roundings
    between its parts (attention weights left exact)."""
    return {key[0]: es.rounded_logits(state, config, sequences_of(key[0]))
            for key, (_, state, config) in models.items() if key[1] == "bfloat16"}


def check(got, models_expected, rounded, name, dtype, label, page=es.PAGE):
    """Against the float64 plain implementation, and in bfloat16 also, far more tightly,
    against the plain implementation that rounds where the engine does."""
    es.assert_logits_close(got, models_expected[name, dtype], dtype, f"{label}/{name}", page=page)
    if dtype == "bfloat16":
        es.assert_logits_close(got, rounded[name], dtype, f"{label}/{name}",
                               limits=es.ROUNDED_TOLERANCE, page=page,
                               row_rms=es.ROUNDED_ROW_RMS)


def _pages_for(sequences, extra=0):
    return sum(-(-len(t) // es.PAGE) for t in sequences.values()) + 1 + extra


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_requests(models, expected, expected_rounded, name, dtype):
    folder, _, _ = models[name, dtype]
    sequences = sequences_of(name)
    core = es.build_core(folder, dtype, num_blocks=_pages_for(sequences))
    got = es.replay(core, es.schedule_whole(sequences))
    check(got, expected, expected_rounded, name, dtype, "whole")
    assert core.manager.live_requests() == []


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_last_32_tokens_one_by_one(models, expected, expected_rounded, name, dtype):
    folder, _, _ = models[name, dtype]
    sequences = sequences_of(name)
    core = es.build_core(folder, dtype, num_blocks=_pages_for(sequences))
    got = es.replay(core, es.schedule_tail(sequences, 32))
    check(got, expected, expected_rounded, name, dtype, "tail")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_portions_of_changing_size(models, expected, expected_rounded, name, dtype):
    folder, _, _ = models[name, dtype]
    sequences = sequences_of(name)
    core = es.build_core(folder, dtype, num_blocks=_pages_for(sequences))
    got = es.replay(core, es.schedule_portions(sequences))
    check(got, expected, expected_rounded, name, dtype, "portions")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_mixed_batches_with_pages_used_again(models, expected, expected_rounded, name, dtype):
    folder, _, config = models[name, dtype]
    sequences = sequences_of(name)
    # every request twice (second copy under another id) so that later ones reuse pages
    doubled = {**sequences, **{rid + "x": tokens for rid, tokens in sequences.items()}}
    longest = max(len(t) for t in doubled.values())
    pool_tokens = 2 * (-(-longest // 64) * 64) + 64
    steps = es.schedule_mixed(doubled, pool_tokens)
    assert any(len(step["entries"]) > 1 for step in steps)
    assert any(len(e["tokens"]) > 1 for step in steps for e in step["entries"]
               if len(step["entries"]) > 1)
    peak = es.peak_tokens(steps, doubled)
    assert peak <= pool_tokens
    core = es.build_core(folder, dtype, num_blocks=peak // es.PAGE + 1)
    got = es.replay(core, steps)
    both = {**expected[name, dtype],
            **{rid + "x": value for rid, value in expected[name, dtype].items()}}
    es.assert_logits_close(got, both, dtype, f"mixed/{name}")
    if dtype == "bfloat16":
        rounded = expected_rounded[name]
        es.assert_logits_close(got, {**rounded, **{rid + "x": v for rid, v in rounded.items()}},
                               dtype, f"mixed/{name}", limits=es.ROUNDED_TOLERANCE,
                               row_rms=es.ROUNDED_ROW_RMS)
    # pages really were handed out more than once
    total_pages = sum(-(-len(t) // es.PAGE) for t in doubled.values())
    assert total_pages > core.manager.pools[0].num_usable
    assert core.manager.num_free_pages() == core.manager.pools[0].num_usable


@pytest.mark.parametrize("dtype", DTYPES)
def test_large_portions_side_by_side(models, expected, dtype):
    """Head size 64 and portions of 256 rows and more (in bfloat16 the tcgen05 attention
    kernel): two long prompts cut at 300 and 256 in the same steps beside a short one, then
    their rests beside single tokens."""
    folder, _, _ = models["D", dtype]
    sequences = sequences_of("D")
    a, b, c, d = (sequences[f"d{i}"] for i in range(4))

    def entry(rid, tokens, at, size):
        return {"id": rid, "tokens": tokens[at:at + size], "want": list(range(size))}

    steps = [
        {"entries": [entry("d0", a, 0, 300), entry("d1", b, 0, 256), entry("d2", c, 0, 39)],
         "end": []},
        {"entries": [entry("d0", a, 300, 299), entry("d1", b, 256, 1), entry("d2", c, 39, 1),
                     entry("d3", d, 0, 333)], "end": ["d1", "d2", "d3"]},
        {"entries": [entry("d0", a, 599, 1)], "end": ["d0"]},
    ]
    core = es.build_core(folder, dtype, num_blocks=_pages_for(sequences),
                         max_tokens_per_step=1024)
    got = es.replay(core, steps)
    es.assert_logits_close(got, expected["D", dtype], dtype, "large-portions/D")
    assert core.manager.live_requests() == []


@pytest.mark.parametrize("dtype", DTYPES)
def test_cutting_does_not_change_the_logits_beyond_rounding(models, dtype):
    """Whole, tail-decoded and chunked runs of the same request agree far more tightly with
    each other than bfloat16 agrees with the float64 oracle."""
    folder, _, _ = models["B", dtype]
    sequences = {"s": sequences_of("B")["b3"]}
    runs = []
    for schedule in (es.schedule_whole, es.schedule_tail, es.schedule_portions):
        core = es.build_core(folder, dtype, num_blocks=_pages_for(sequences))
        runs.append(es.replay(core, schedule(sequences))["s"])
    scale = float(runs[0].abs().max())
    limit = 1e-5 if dtype == "float32" else 1.5e-2
    for other in runs[1:]:
        worst = float((other - runs[0]).abs().max()) / scale
        es.log_error(f"cut-vs-whole/{dtype}", worst)
        assert worst <= limit


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_long_decoding_to_the_last_position(models, name, dtype):
    """Four prompt tokens, then one token a step until the context is full."""
    folder, state, config = models[name, dtype]
    length = config["n_positions"]
    sequences = {"long": random_tokens(config["vocab_size"], length, 7)}
    core = es.build_core(folder, dtype, num_blocks=_pages_for(sequences))
    got = es.replay(core, es.schedule_tail(sequences, length - 4))
    es.assert_logits_close(got, es.plain_logits(state, config, sequences), dtype,
                           f"long-decode/{name}")
    if dtype == "bfloat16":
        # decode rows keep their attention weights in float32, so here nothing is left
        # between the engine and the plain implementation with the same roundings but the
        # order of sums and the approximate tanh: the tightest bfloat16 comparison there is
        es.assert_logits_close(got, es.rounded_logits(state, config, sequences), dtype,
                               f"long-decode/{name}", limits=es.DECODE_ROUNDED_TOLERANCE,
                               row_rms=es.DECODE_ROUNDED_ROW_RMS)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_first_tokens_of_a_sequence(models, name, dtype):
    folder, state, config = models[name, dtype]
    sequences = {f"n{n}": random_tokens(config["vocab_size"], n, 11 + n) for n in (1, 2, 3)}
    core = es.build_core(folder, dtype, num_blocks=8)
    got = es.replay(core, es.schedule_tail(sequences, 2))
    es.assert_logits_close(got, es.plain_logits(state, config, sequences), dtype,
                           f"first-tokens/{name}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_trace_run_program(models, expected, tmp_path, dtype):
    """bin/trace_run as a child process, on the mixed schedule with pages used again."""
    folder, _, config = models["B", dtype]
    sequences = sequences_of("B")
    pool_tokens = 2 * 256 + 64
    steps = es.schedule_mixed(sequences, pool_tokens)
    peak = es.peak_tokens(steps, sequences)
    got = es.run_trace_program(folder, dtype, steps, peak, tmp_path / "out",
                               config["vocab_size"])
    es.assert_logits_close(got, expected["B", dtype], dtype, "trace_run/B")


def test_step_refuses_what_the_cache_cannot_hold(models):
    from ayaka_b200.engine.runner import StepEntry
    from ayaka_b200.errors import CapacityError, InvalidRequestError

    folder, _, config = models["A", "float32"]
    core = es.build_core(folder, "float32", num_blocks=3, max_running=2)  # two usable pages
    core.step([StepEntry("a", list(range(20)), [19])])
    with pytest.raises(CapacityError):
        core.step([StepEntry("b", list(range(20)), [])])
    core.manager.check_integrity()
    assert "b" not in core.manager
    with pytest.raises(InvalidRequestError):
        core.step([StepEntry("a", [config["vocab_size"]], [0])])
    core.release("a")
    core.step([StepEntry("b", list(range(20)), [])])
    core.release("b")
    core.manager.check_integrity()
    assert core.manager.num_free_pages() == 2
