"""Schedules and sizes beyond the tiny defaults, each against the plain implementation:
other page sizes (the cache layout's strides and the one-box-per-page loads change with the
page), two layers of GPT-2 XL's sizes through every way of cutting the work, and decode
steps of 24 and 48 live requests (the matrix-product kernel for 17 to 64 rows, the larger
graph buckets), eager and from CUDA graphs."""

from __future__ import annotations

import pytest
import torch

import engine_support as es
import plain_gpt2 as plain
from cases import INIT_LOUD, INIT_LOUD_WIDE, TINY_B, TINY_D, random_tokens
from ayaka_b200.weights.rules import RandomInit

pytestmark = pytest.mark.gpu

DTYPES = ("float32", "bfloat16")
CONFIGS = {"B": (TINY_B, INIT_LOUD, (1, 64, 130, 200, 47)),
           "D": (TINY_D, INIT_LOUD_WIDE, (600, 257, 40, 333))}


def sequences_of(name: str) -> dict[str, list[int]]:
    config, _, lengths = CONFIGS[name]
    return {f"{name.lower()}{index}": random_tokens(config["vocab_size"], length,
                                                    100 * ord(name) + index)
            for index, length in enumerate(lengths)}


def pages_for(sequences, page):
    return sum(-(-len(tokens) // page) for tokens in sequences.values()) + 1


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    made = {}
    for name, (config, init, _) in CONFIGS.items():
        for dtype in DTYPES:
            folder = tmp_path_factory.mktemp(f"pages_{name}_{dtype}")
            made[name, dtype] = (*es.make_model(folder, config, seed=ord(name), init=init,
                                                dtype=dtype), config)
    return made


@pytest.fixture(scope="module")
def expected(models):
    out = {}
    for (name, dtype), (_, state, config) in models.items():
        out[name, dtype] = es.plain_logits(state, config, sequences_of(name))
        if dtype == "bfloat16":
            out[name, "rounded"] = es.rounded_logits(state, config, sequences_of(name))
    return out


def compare(got, expected, name, dtype, label, page, doubled=False):
    def twice(values):
        return {**values, **{rid + "x": v for rid, v in values.items()}} if doubled else values

    es.assert_logits_close(got, twice(expected[name, dtype]), dtype, f"{label}/{name}/page{page}",
                           page=page)
    if dtype == "bfloat16":
        es.assert_logits_close(got, twice(expected[name, "rounded"]), dtype,
                               f"{label}/{name}/page{page}", limits=es.ROUNDED_TOLERANCE,
                               page=page, row_rms=es.ROUNDED_ROW_RMS)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("page", [8, 32, 64])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_other_page_sizes_under_every_cut(models, expected, name, page, dtype):
    """Whole, last 32 tokens one by one, portions of changing size, and mixed with pages used
    again, at pages of 8, 32 and 64 tokens (D's portions of 256 rows and more take the
    tcgen05 attention kernel, whose key and value loads are one box per page)."""
    folder, _, _ = models[name, dtype]
    sequences = sequences_of(name)
    for label, schedule in (("whole", es.schedule_whole), ("tail", es.schedule_tail),
                            ("portions", es.schedule_portions)):
        core = es.build_core(folder, dtype, num_blocks=pages_for(sequences, page),
                             block_size=page)
        got = es.replay(core, schedule(sequences))
        compare(got, expected, name, dtype, label, page)
        assert core.manager.live_requests() == []
    doubled = {**sequences, **{rid + "x": tokens for rid, tokens in sequences.items()}}
    longest = max(len(tokens) for tokens in doubled.values())
    pool_tokens = 2 * (-(-longest // 64) * 64) + 64
    steps = es.schedule_mixed(doubled, pool_tokens)
    peak = es.peak_tokens(steps, doubled)
    core = es.build_core(folder, dtype, num_blocks=peak // page + 1, block_size=page)
    got = es.replay(core, steps)
    compare(got, expected, name, dtype, "mixed", page, doubled=True)
    assert pages_for(doubled, page) - 1 > core.manager.pools[0].num_usable  # pages used again
    assert core.manager.num_free_pages() == core.manager.pools[0].num_usable


# ---- two layers of GPT-2 XL's sizes ----------------------------------------------------------
XL2 = {
    "architectures": ["GPT2LMHeadModel"], "n_layer": 2, "n_embd": 1600, "n_head": 25,
    "n_inner": 6400, "vocab_size": 50257, "n_positions": 1024, "layer_norm_epsilon": 1e-5,
    "activation_function": "gelu_new", "scale_attn_by_inverse_layer_idx": False,
    "tie_word_embeddings": True,
}
# as loud at width 1600 as INIT_LOUD is at width 64 (the same deviation of a projection's
# output), so that attention is peaked and a wrong key shows
XL_INIT = RandomInit(weight_std=0.04, scale_residual_projections=False, bias_std=0.1,
                     norm_std=0.1)
XL_LENGTHS = (200, 33, 257, 96)


def xl_sequences() -> dict[str, list[int]]:
    return {f"x{index}": random_tokens(XL2["vocab_size"], length, 4000 + index)
            for index, length in enumerate(XL_LENGTHS)}


def xl_decoders() -> dict[str, list[int]]:
    """24 short requests: prompts of 6 to 29 tokens and five more tokens each."""
    return {f"d{index}": random_tokens(XL2["vocab_size"], 6 + index + 5, 5000 + index)
            for index in range(24)}


@pytest.fixture(scope="module")
def xl(tmp_path_factory):
    """Per dtype: (config folder, checkpoint-named tensors for the engine, plain logits)."""
    import json

    from ayaka_b200.weights.random_init import random_state

    made = {}
    for dtype in DTYPES:
        folder = tmp_path_factory.mktemp(f"xl2_{dtype}")
        (folder / "config.json").write_text(json.dumps(XL2))
        stored = random_state(XL2, 48, XL_INIT, store_dtype=dtype)
        state = {name: tensor.float() for name, tensor in stored.items()}
        everything = {**xl_sequences(), **xl_decoders()}
        plain_logits = es.plain_logits(state, XL2, everything)
        rounded = es.rounded_logits(state, XL2, everything) if dtype == "bfloat16" else None
        made[dtype] = (folder, stored, plain_logits, rounded)
    return made


def xl_core(xl, dtype, num_blocks, max_running=4):
    from ayaka_b200.config.engine import EngineConfig
    from ayaka_b200.engine.core import EngineCore

    folder, stored, _, _ = xl[dtype]
    config = EngineConfig(model=str(folder), dtype=dtype, block_size=es.PAGE,
                          num_blocks=num_blocks, max_running=max_running,
                          max_tokens_per_step=1024)
    return EngineCore.from_config(config, tensors=stored, poison_cache=True)


def xl_compare(got, xl, dtype, label):
    _, _, plain_logits, rounded = xl[dtype]
    es.assert_logits_close(got, {rid: plain_logits[rid] for rid in got}, dtype, f"{label}/XL2")
    if rounded is not None:
        es.assert_logits_close(got, {rid: rounded[rid] for rid in got}, dtype, f"{label}/XL2",
                               limits=es.ROUNDED_TOLERANCE, row_rms=es.ROUNDED_ROW_RMS)


@pytest.mark.parametrize("dtype", DTYPES)
def test_gpt2_xl_layer_sizes_under_every_cut(xl, dtype):
    """Width 1600, 25 heads of 64, inner 6400, vocabulary 50257, 1024 positions, two layers:
    the sizes the benchmark times, through the four cuts, against the plain implementation."""
    sequences = xl_sequences()
    for label, schedule in (("whole", es.schedule_whole), ("tail", es.schedule_tail),
                            ("portions", es.schedule_portions)):
        core = xl_core(xl, dtype, pages_for(sequences, es.PAGE))
        xl_compare(es.replay(core, schedule(sequences)), xl, dtype, label)
        del core
    # every request twice, in a pool that holds two of the longest: pages are used again
    doubled = {**sequences, **{rid + "x": tokens for rid, tokens in sequences.items()}}
    pool_tokens = 2 * 320 + 64
    steps = es.schedule_mixed(doubled, pool_tokens)
    peak = es.peak_tokens(steps, doubled)
    core = xl_core(xl, dtype, peak // es.PAGE + 1)
    got = es.replay(core, steps)
    xl_compare({rid: value for rid, value in got.items() if not rid.endswith("x")}, xl, dtype,
               "mixed")
    xl_compare({rid[:-1]: value for rid, value in got.items() if rid.endswith("x")}, xl, dtype,
               "mixed")
    assert pages_for(doubled, es.PAGE) - 1 > core.manager.pools[0].num_usable
    assert core.manager.num_free_pages() == core.manager.pools[0].num_usable


def many_decoders_schedule(sequences: dict[str, list[int]], tail: int = 5) -> list[dict]:
    """All prompts as one step of portions, then ``tail`` steps of one token per request."""
    heads = {rid: len(tokens) - tail for rid, tokens in sequences.items()}
    steps = [{"entries": [{"id": rid, "tokens": tokens[:heads[rid]],
                           "want": list(range(heads[rid]))}
                          for rid, tokens in sequences.items()], "end": []}]
    for index in range(tail):
        steps.append({"entries": [{"id": rid, "tokens": [tokens[heads[rid] + index]],
                                   "want": [0]} for rid, tokens in sequences.items()],
                      "end": []})
    steps[-1]["end"] = list(sequences)
    return steps


@pytest.mark.parametrize("dtype", DTYPES)
def test_gpt2_xl_layer_sizes_with_24_requests_decoding(xl, dtype):
    """Decode steps of 24 rows at the benchmark's layer sizes: in bfloat16 the products take
    the tensor-core kernel for 17 to 64 rows."""
    sequences = xl_decoders()
    core = xl_core(xl, dtype, pages_for(sequences, es.PAGE), max_running=24)
    xl_compare(es.replay(core, many_decoders_schedule(sequences)), xl, dtype, "24-decoders")


# ---- 24 and 48 live requests on the tiny configurations, eager and from graphs ---------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("live", [24, 48])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_decode_steps_of_many_requests(models, name, live, dtype):
    folder, state, config = models[name, dtype]
    sequences = {f"m{index}": random_tokens(config["vocab_size"], 3 + (7 * index) % 40 + 6,
                                            6000 + index) for index in range(live)}
    core = es.build_core(folder, dtype, num_blocks=pages_for(sequences, es.PAGE),
                         max_running=live, max_tokens_per_step=2048)
    got = es.replay(core, many_decoders_schedule(sequences, tail=6))
    es.assert_logits_close(got, es.plain_logits(state, config, sequences), dtype,
                           f"{live}-decoders/{name}")
    if dtype == "bfloat16":
        es.assert_logits_close(got, es.rounded_logits(state, config, sequences), dtype,
                               f"{live}-decoders/{name}", limits=es.ROUNDED_TOLERANCE,
                               row_rms=es.ROUNDED_ROW_RMS)


@pytest.mark.parametrize("dtype,slack", [("float32", 1e-4), ("bfloat16", 3e-2)])
@pytest.mark.parametrize("live", [24, 48])
def test_graph_buckets_of_32_and_64_rows_against_plain(models, live, dtype, slack):
    """Greedy generation of many requests at once through ``LLM.generate`` with CUDA graphs:
    24 requests replay the 32-row bucket, 48 the 64-row bucket; every token is one the plain
    implementation allows at its position."""
    from ayaka_b200 import LLM, EngineConfig, SamplingParams

    folder, state, config = models["B", dtype]
    prompts = [tuple(random_tokens(config["vocab_size"], 2 + (5 * index) % 23, 7000 + index))
               for index in range(live)]
    params = SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True)
    engine = EngineConfig(model=str(folder), dtype=dtype, max_running=64, num_blocks=200,
                          max_tokens_per_step=2048, cuda_graph=True)
    with LLM.from_config(engine) as llm:
        outputs = llm.generate(prompts, params)
        assert llm.graphs.replays >= 9
        assert llm.graphs.bucket_for(live).size == (32 if live == 24 else 64)
        llm.core.manager.check_integrity()
    wide = plain.cast_state(state, torch.float64)
    for prompt, output in zip(prompts, outputs):
        got = output.outputs[0].token_ids
        assert len(got) == 10
        sequence = list(prompt) + list(got)
        logits = plain.logits(wide, config, torch.tensor(sequence))
        for index, token in enumerate(got):
            row = logits[len(prompt) + index - 1]
            assert float(row[token]) >= float(row.max()) - slack * float(row.abs().max()), \
                (index, token)


# ---- kernels that start before their predecessor has ended -------------------------------------
@pytest.mark.parametrize("name", list(CONFIGS))
def test_the_same_steps_give_the_same_bits_every_time(models, name):
    """Every kernel may start while the one ahead still runs and waits for it before it reads
    what that one writes. A load that slips ahead of the wait reads the layer before, or the
    step before, now and then: two layers launched from the C++ host code run close enough
    behind one another for that to show (it did: one run in three, when the compiler moved
    the query loads of the tensor-core decode attention above the wait), and nothing in the
    engine is allowed to depend on timing, so eight runs of the decode-heavy schedule must
    agree to the bit."""
    folder, _, _ = models[name, "bfloat16"]
    sequences = sequences_of(name)
    first = None
    for _ in range(8):
        core = es.build_core(folder, "bfloat16", num_blocks=pages_for(sequences, es.PAGE))
        got = es.replay(core, es.schedule_tail(sequences, 32))
        if first is None:
            first = got
            continue
        for rid, logits in got.items():
            assert torch.equal(logits, first[rid]), rid


# ---- the host far ahead of the device ----------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
def test_steps_that_return_nothing_queue_up_behind_a_busy_device(models, expected, dtype):
    """A step that wants no logits does not wait for the device, so a prompt cut into small
    portions is dozens of steps the host queues one behind the other. Here the device is
    kept busy first (a spin of some tens of milliseconds), every portion of two tokens is
    queued behind it, and only the last step wants logits: what each step copied to the
    device must still be what it wrote (the step's metadata goes through two pinned buffers
    in turn; a buffer filled again before its copy had run gave later steps' positions and
    slots to earlier ones: wrong tokens now and then, once an illegal address)."""
    from ayaka_b200.engine.runner import StepEntry

    folder, _, _ = models["B", dtype]
    rid, tokens = next((rid, tokens) for rid, tokens in sequences_of("B").items()
                       if len(tokens) >= 190)
    core = es.build_core(folder, dtype, num_blocks=pages_for({rid: tokens}, es.PAGE) + 1)
    torch.cuda._sleep(80_000_000)  # the device is busy while the host queues every step
    for at in range(0, len(tokens) - 2, 2):
        assert core.step([StepEntry(rid, tokens[at:at + 2], ())]) is None
    at = len(tokens) - 2 if len(tokens) % 2 == 0 else len(tokens) - 1
    last = core.step([StepEntry(rid, tokens[at:], (len(tokens) - at - 1,))])
    core.runner.check_device_flags()
    got = {rid: last.cpu()}
    want = {rid: expected["B", dtype][rid][-1:]}
    es.assert_logits_close(got, want, dtype, "queued-portions/B")


# ---- the C++ host path and the Python path launch the same kernels ----------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_host_library_and_python_forward_give_the_same_bits(models, name, dtype):
    """A step's layers run from the C++ host code (one call for the whole order) or kernel by
    kernel from Python: the same launches with the same arguments, so the same bits, under
    the mixed schedule (prompt portions beside single tokens, pages used again) and under
    decode steps of 24 requests."""
    from ayaka_b200.kernels import ops

    folder, _, config = models[name, dtype]
    sequences = sequences_of(name)
    doubled = {**sequences, **{rid + "x": tokens for rid, tokens in sequences.items()}}
    longest = max(len(tokens) for tokens in doubled.values())
    mixed = es.schedule_mixed(doubled, 2 * (-(-longest // 64) * 64) + 64)
    peak = es.peak_tokens(mixed, doubled)
    decoders = {f"m{index}": random_tokens(config["vocab_size"], 3 + (7 * index) % 40 + 6,
                                           6000 + index) for index in range(24)}
    results = {}
    for native in (True, False):
        ops.NATIVE_STEP = native
        try:
            launches = ops.launch_count()
            core = es.build_core(folder, dtype, num_blocks=peak // es.PAGE + 1)
            got = es.replay(core, mixed)
            core = es.build_core(folder, dtype, num_blocks=pages_for(decoders, es.PAGE),
                                 max_running=24, max_tokens_per_step=2048)
            got.update(es.replay(core, many_decoders_schedule(decoders, tail=6)))
            results[native] = (got, ops.launch_count() - launches)
        finally:
            ops.NATIVE_STEP = True
    (with_host, host_launches), (with_python, python_launches) = results[True], results[False]
    assert host_launches == python_launches  # the same number of kernels
    assert set(with_host) == set(with_python)
    for rid, logits in with_host.items():
        assert torch.equal(logits, with_python[rid]), rid


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_decoding_requests_ahead_of_prompt_portions(models, name, dtype):
    """Steps as the scheduler builds them: six requests that bring one token each, then
    portions of two long prompts (for D of 256 rows and more). In bfloat16 the single rows
    run through the decode attention kernel and the portions through a prompt kernel, in
    the same step."""
    folder, state, config = models[name, dtype]
    vocab, limit = config["vocab_size"], config["n_positions"]
    short = {f"s{i}": random_tokens(vocab, 9 + 5 * i + 8, 8000 + i) for i in range(6)}
    long = {"la": random_tokens(vocab, limit - 3, 8100), "lb": random_tokens(vocab, limit // 2, 8101)}
    sequences = {**short, **long}
    heads = {rid: len(tokens) - 8 for rid, tokens in short.items()}
    sizes = {"la": [(limit - 3) // 3 + 1, 2, (limit - 3) // 3, 5, 10 ** 6],
             "lb": [40, limit // 2 - 50, 3, 10 ** 6]}
    fed = dict.fromkeys(long, 0)

    def portion(rid, turn):
        tokens, at = long[rid], fed[rid]
        if at >= len(tokens) or turn >= len(sizes[rid]):
            return None
        size = min(sizes[rid][turn], len(tokens) - at)
        fed[rid] = at + size
        return {"id": rid, "tokens": tokens[at:at + size], "want": list(range(size))}

    steps = [{"entries": [{"id": rid, "tokens": tokens[:heads[rid]],
                           "want": list(range(heads[rid]))} for rid, tokens in short.items()],
              "end": []}]
    for turn in range(8):
        entries = [{"id": rid, "tokens": [tokens[heads[rid] + turn]], "want": [0]}
                   for rid, tokens in short.items()]
        entries += [entry for entry in (portion(rid, turn) for rid in long) if entry]
        steps.append({"entries": entries, "end": []})
    assert all(fed[rid] == len(long[rid]) for rid in long)
    steps[-1]["end"] = list(sequences)
    core = es.build_core(folder, dtype, num_blocks=pages_for(sequences, es.PAGE),
                         max_running=8, max_tokens_per_step=1024)
    got = es.replay(core, steps)
    es.assert_logits_close(got, es.plain_logits(state, config, sequences), dtype,
                           f"decoders-then-portions/{name}")
    if dtype == "bfloat16":
        es.assert_logits_close(got, es.rounded_logits(state, config, sequences), dtype,
                               f"decoders-then-portions/{name}", limits=es.ROUNDED_TOLERANCE,
                               row_rms=es.ROUNDED_ROW_RMS)
