"""Generation through the Python entry point and the command line, the sampling kernel, and
the scheduler on a real cache that is too small for the crowd."""

from __future__ import annotations

import subprocess
import sys
from pathlib import Path

import pytest
import torch

import engine_support as es
import plain_gpt2 as plain
from cases import INIT_A, INIT_B, INIT_LOUD, TINY_A, TINY_B, random_tokens

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def _llm(folder, dtype, **overrides):
    from ayaka_b200 import LLM, EngineConfig

    options = dict(model=str(folder), dtype=dtype, max_running=4, num_blocks=64,
                   max_tokens_per_step=256)
    options.update(overrides)
    return LLM.from_config(EngineConfig(**options))


def canonical_interval(row: torch.Tensor, temperature: float, token: int) -> tuple[float, float]:
    """[lo, hi) of ``token`` on the CDF over the canonical order (p descending, id ascending)."""
    p = torch.softmax(row.double() / temperature, 0)
    order = sorted(range(len(p)), key=lambda i: (-float(p[i]), i))
    cumulative = 0.0
    for index in order:
        if index == token:
            return cumulative, cumulative + float(p[index])
        cumulative += float(p[index])
    raise AssertionError("token not in the vocabulary")


def check_generation(state, config, prompt, got, params, seed, slack):
    """Every generated token is what the plain implementation allows at its position: the
    argmax within ``slack`` of the logit scale (greedy), or the token whose CDF interval
    holds this position's random number within ``slack`` (sampling)."""
    sequence = list(prompt) + list(got)
    logits = plain.logits(plain.cast_state(state, torch.float64), config, torch.tensor(sequence))
    for index, token in enumerate(got):
        position = len(prompt) + index
        row = logits[position - 1]
        if params.greedy:
            scale = float(row.abs().max())
            assert float(row[token]) >= float(row.max()) - slack * scale, (index, token)
        else:
            u = plain.draw_uniform(seed, position)
            lo, hi = canonical_interval(row, params.temperature, token)
            assert lo - slack <= u < hi + slack, (index, token, u, lo, hi)


@pytest.mark.parametrize("dtype,slack", [("float32", 1e-4), ("bfloat16", 3e-2)])
def test_greedy_generation_config_a(tmp_path, dtype, slack):
    """Tiny A as the benchmark file states it: four prompts of 5, 17, 32 and 9 tokens, 16
    greedy tokens each, weights N(0, 0.02)."""
    from ayaka_b200 import SamplingParams

    folder, state = es.make_model(tmp_path / "a", TINY_A, 0, INIT_A, dtype)
    prompts = [random_tokens(256, n, 300 + n) for n in (5, 17, 32, 9)]
    params = SamplingParams(temperature=0.0, max_tokens=16)
    with _llm(folder, dtype) as llm:
        outputs = llm.generate([tuple(p) for p in prompts], params)
        llm.core.manager.check_integrity()
        assert llm.core.manager.live_requests() == []
    for prompt, output in zip(prompts, outputs):
        got = output.outputs[0].token_ids
        assert len(got) == 16 and output.finished
        assert output.outputs[0].finish_reason.value == "length"
        assert output.usage.prompt_tokens == len(prompt) and output.usage.completion_tokens == 16
        check_generation(state, TINY_A, prompt, got, params, output.seed, slack)
    if dtype == "float32":  # with loud weights the margins are wide: tokens must be equal
        folder, state = es.make_model(tmp_path / "loud", TINY_A, 0, INIT_LOUD, dtype)
        with _llm(folder, dtype) as llm:
            outputs = llm.generate([tuple(p) for p in prompts], params)
        for prompt, output in zip(prompts, outputs):
            assert list(output.outputs[0].token_ids) == plain.greedy_generate(
                state, TINY_A, prompt, 16)


@pytest.mark.parametrize("dtype,slack", [("float32", 1e-4), ("bfloat16", 5e-2)])
def test_temperature_sampling_config_b(tmp_path, dtype, slack):
    """Tiny B as the benchmark file states it: prompts of 1, 64 and 130 tokens cut into
    portions of 48 beside decode steps, temperature 0.8, 24 tokens each, pages of 16."""
    from ayaka_b200 import SamplingParams

    folder, state = es.make_model(tmp_path / "b", TINY_B, 1, INIT_B, dtype)
    prompts = [random_tokens(503, n, 400 + n) for n in (1, 64, 130)]
    params = [SamplingParams(temperature=0.8, max_tokens=24, seed=1000 + i) for i in range(3)]
    with _llm(folder, dtype, max_tokens_per_step=48, block_size=16) as llm:
        outputs = llm.generate([tuple(p) for p in prompts], params)
        stats = llm.scheduler.stats
        assert stats.prefill_tokens == 195 and stats.decode_rows == 3 * 23
    for prompt, output, one in zip(prompts, outputs, params):
        got = output.outputs[0].token_ids
        assert len(got) == 24 and output.seed == one.seed
        check_generation(state, TINY_B, prompt, got, one, one.seed, slack)


def test_same_seed_same_tokens_in_any_company(tmp_path):
    from ayaka_b200 import SamplingParams

    folder, _ = es.make_model(tmp_path / "b", TINY_B, 1, INIT_LOUD, "float32")
    prompt = tuple(random_tokens(503, 37, 9))
    params = SamplingParams(temperature=1.0, top_k=40, top_p=0.9, max_tokens=20, seed=77)
    with _llm(folder, "float32") as llm:
        alone = llm.generate(prompt, params).outputs[0].token_ids
        again = llm.generate(prompt, params).outputs[0].token_ids
    others = [tuple(random_tokens(503, n, 50 + n)) for n in (3, 90, 12)]
    with _llm(folder, "float32", max_tokens_per_step=32, block_size=4, num_blocks=200) as llm:
        crowd = llm.generate([others[0], prompt, *others[1:]],
                             [SamplingParams(temperature=1.3, max_tokens=9, seed=1), params,
                              SamplingParams(temperature=0.0, max_tokens=30),
                              SamplingParams(temperature=0.7, max_tokens=15)])
    assert alone == again == crowd[1].outputs[0].token_ids
    other_seed = SamplingParams(temperature=1.0, top_k=40, top_p=0.9, max_tokens=20, seed=78)
    with _llm(folder, "float32") as llm:
        assert llm.generate(prompt, other_seed).outputs[0].token_ids != alone


def test_a_cache_smaller_than_the_crowd(tmp_path):
    """Twelve requests, four at a time, on 10 pages: some are cut short by the cache, none gets
    a wrong token, and every page comes back."""
    from ayaka_b200 import SamplingParams

    folder, state = es.make_model(tmp_path / "a", TINY_A, 0, INIT_LOUD, "float32")
    prompts = [random_tokens(256, 6 + 3 * (i % 4), 600 + i) for i in range(12)]
    params = SamplingParams(temperature=0.0, max_tokens=40)
    with _llm(folder, "float32", num_blocks=11, block_size=16, max_running=4) as llm:
        outputs = llm.generate([tuple(p) for p in prompts], params)
        manager = llm.core.manager
        manager.check_integrity()
        assert manager.live_requests() == []
        assert manager.num_free_pages() == manager.pools[0].num_usable
        assert llm.scheduler.stats.shed >= 1
    cut = 0
    for prompt, output in zip(prompts, outputs):
        got = list(output.outputs[0].token_ids)
        assert got == plain.greedy_generate(state, TINY_A, prompt, len(got))
        if len(got) < 40:
            cut += 1
            assert output.notes and "cache is full" in output.notes[0]
    assert cut >= 1


def test_stream_and_stop_token(tmp_path):
    from ayaka_b200 import SamplingParams

    folder, state = es.make_model(tmp_path / "a", TINY_A, 0, INIT_LOUD, "float32")
    prompt = random_tokens(256, 11, 5)
    expected = plain.greedy_generate(state, TINY_A, prompt, 12)
    with _llm(folder, "float32") as llm:
        pieces = list(llm.stream(tuple(prompt), SamplingParams(temperature=0.0, max_tokens=12)))
        assert [t for piece in pieces for t in piece.outputs[0].token_ids] == expected
        assert pieces[-1].finished and not any(piece.finished for piece in pieces[:-1])
        stop = expected[4]
        first = expected.index(stop)
        output = llm.generate(tuple(prompt), SamplingParams(
            temperature=0.0, max_tokens=12, stop_token_ids=frozenset({stop})))
        assert list(output.outputs[0].token_ids) == expected[:first + 1]
        assert output.outputs[0].finish_reason.value == "stop"
        assert output.outputs[0].stop_reason == stop
        generator = llm.stream(tuple(prompt), SamplingParams(temperature=0.0, max_tokens=12))
        next(generator)
        generator.close()  # cancels
        assert llm.core.manager.live_requests() == []
        from ayaka_b200.errors import InvalidRequestError
        with pytest.raises(InvalidRequestError):
            llm.generate("text", None)
        with pytest.raises(InvalidRequestError):
            llm.generate((1, 2, 256), None)


def test_command_line(tmp_path):
    folder, state = es.make_model(tmp_path / "a", TINY_A, 0, INIT_LOUD, "float32")
    prompt = random_tokens(256, 9, 8)
    done = subprocess.run(
        [sys.executable, "-m", "ayaka_b200", "run", str(folder), "-p",
         ",".join(map(str, prompt)), "--max-tokens", "10", "--dtype", "fp32"],
        capture_output=True, text=True, cwd=ROOT, timeout=600)
    assert done.returncode == 0, done.stderr
    assert [int(t) for t in done.stdout.split()] == plain.greedy_generate(state, TINY_A, prompt,
                                                                          10)
    assert "cache pages" in done.stderr
    bad = subprocess.run([sys.executable, "-m", "ayaka_b200", "run", str(folder), "-p", "hello"],
                         capture_output=True, text=True, cwd=ROOT, timeout=600)
    assert bad.returncode == 2 and "Traceback" not in bad.stderr
    missing = subprocess.run([sys.executable, "-m", "ayaka_b200", "run", str(tmp_path / "none"),
                              "-p", "1"], capture_output=True, text=True, cwd=ROOT, timeout=600)
    assert missing.returncode == 4


# ---- the sampling kernel alone ---------------------------------------------------------------
@pytest.mark.parametrize("vocab", [503, 50257])
def test_sample_kernel_against_the_float64_oracle(vocab):
    from ayaka_b200.kernels import ops

    g = torch.Generator().manual_seed(vocab)
    rows = 48
    logits = (torch.randn(rows, vocab, generator=g) * 3.0)
    logits[5, 10:20] = 7.0  # ties among the most likely tokens
    logits[6] = 0.25  # every token ties
    temperature = torch.tensor([0.8, 1.0, 1.7, 0.3] * 12)
    top_k = torch.tensor([0, 0, 5, 50, 0, 0, 0, 1000] * 6, dtype=torch.int32)
    top_p = torch.tensor([1.0, 0.9, 1.0, 0.5, 1.0, 0.95] * 8)
    min_p = torch.tensor([0.0, 0.0, 0.0, 0.0, 0.1, 0.02, 0.0, 0.3] * 6)
    temperature[7] = 0.0  # a greedy row inside a sampling batch
    seeds = torch.arange(rows, dtype=torch.int64) * 7919 + 3
    positions = torch.arange(rows, dtype=torch.int64) + 100
    out = torch.full((rows,), -1, dtype=torch.int32, device="cuda")
    ops.sample(logits.cuda(), temperature.cuda(), top_k.cuda(), top_p.cuda(), min_p.cuda(),
               seeds.cuda(), positions.cuda(), out)
    got = out.tolist()
    exact = 0
    for r in range(rows):
        u = plain.draw_uniform(int(seeds[r]), int(positions[r]))
        want = plain.sample_token(logits[r], float(temperature[r]), u, int(top_k[r]),
                                  float(top_p[r]), float(min_p[r]))
        if got[r] == want:
            exact += 1
            continue
        # fp32 exp against float64: only a u within rounding of a CDF boundary may differ
        assert float(temperature[r]) > 0
        nudged = {plain.sample_token(logits[r], float(temperature[r]), u + d, int(top_k[r]),
                                     float(top_p[r]), float(min_p[r]))
                  for d in (-1e-5, 1e-5)}
        assert got[r] in nudged, (r, got[r], want)
    assert exact >= rows - 2
    assert got[7] == plain.argmax_smallest_id(logits[7])


def test_sample_kernel_frequencies_follow_the_distribution():
    from ayaka_b200.kernels import ops

    probabilities = torch.tensor([0.5, 0.25, 0.125, 0.0625, 0.0625])
    draws = 4000
    logits = probabilities.log().repeat(draws, 1).cuda()
    seeds = torch.full((draws,), 12345, dtype=torch.int64, device="cuda")
    positions = torch.arange(draws, dtype=torch.int64, device="cuda")
    out = torch.zeros(draws, dtype=torch.int32, device="cuda")
    ops.sample(logits, torch.ones(draws, device="cuda"), None, None, None, seeds, positions, out)
    counts = torch.bincount(out.cpu().long(), minlength=5).double() / draws
    assert torch.allclose(counts, probabilities.double(), atol=0.03)
    expected = [plain.sample_token(probabilities.log(), 1.0, plain.draw_uniform(12345, p))
                for p in range(200)]
    assert out[:200].tolist() == expected


# ---- masks, biases and penalties before the draw ---------------------------------------------
def test_logits_adjust_kernel_against_the_plain_function():
    """Allowed and banned ids, biases and the three penalties in the fixed order, on rows
    chosen out of a larger buffer; rows that are not named stay bit for bit."""
    import numpy as np

    from ayaka_b200.kernels import ops

    vocab, rows = 1000, 6
    g = torch.Generator().manual_seed(7)
    logits = (torch.randn(rows, vocab, generator=g) * 3).cuda()
    before = logits.clone()
    cases = {
        4: dict(prompt=[3, 3, 999, 17], output=[17, 5, 5, 5], repetition=1.3, frequency=0.4,
                presence=0.7),
        1: dict(prompt=[1], output=[], allowed={0, 2, 500, 999}, bias={2: 4.5, 500: -100.0},
                banned={999}),
        2: dict(prompt=list(range(0, 700)), output=list(range(600, 900)) + [650] * 5,
                repetition=0.8, frequency=-0.25, presence=-1.0, bias={650: 1.0}, banned={3}),
    }
    header = np.zeros((len(cases), ops.ADJUST_WORDS), dtype=np.int32)
    lists, cursor = [], len(cases) * ops.ADJUST_WORDS

    def place(values):
        nonlocal cursor
        offset = cursor
        lists.append(np.asarray(values, dtype=np.int32))
        cursor += len(values)
        return offset

    for slot, (row, case) in enumerate(cases.items()):
        history = case["prompt"] + case["output"]
        bias = sorted(case.get("bias", {}).items())
        header[slot, 0] = row
        header[slot, 1], header[slot, 2], header[slot, 3] = place(history), len(history), \
            len(case["prompt"])
        header[slot, 4], header[slot, 5] = place([t for t, _ in bias]), len(bias)
        place(np.asarray([v for _, v in bias], dtype=np.float32).view(np.int32))
        allowed = case.get("allowed")
        header[slot, 6], header[slot, 7] = (0, -1) if allowed is None else \
            (place(sorted(allowed)), len(allowed))
        header[slot, 8], header[slot, 9] = place(sorted(case.get("banned", ()))), \
            len(case.get("banned", ()))
        header.view(np.float32)[slot, 10:13] = (case.get("repetition", 1.0),
                                                case.get("frequency", 0.0),
                                                case.get("presence", 0.0))
    desc = torch.from_numpy(np.concatenate([header.reshape(-1)] + lists)).cuda()
    mask = torch.zeros(len(cases) * ((vocab + 31) // 32), dtype=torch.int32, device="cuda")
    ops.logits_adjust(logits, desc, len(cases), mask)
    for row in range(rows):
        if row not in cases:
            assert torch.equal(logits[row], before[row])
            continue
        case = cases[row]
        want = plain.adjust_logits(
            before[row].cpu(), case["prompt"], case["output"],
            repetition=case.get("repetition", 1.0), frequency=case.get("frequency", 0.0),
            presence=case.get("presence", 0.0), bias=case.get("bias"),
            allowed=case.get("allowed"), banned=case.get("banned"))
        torch.testing.assert_close(logits[row].cpu(), want, rtol=1e-6, atol=1e-6)


def test_generation_with_penalties_bias_allowed_ids_and_min_tokens(tmp_path):
    """Greedy generation whose every token is the plain implementation's argmax after the
    same adjustments: the penalties change with every token, the end-of-sequence token cannot
    appear before min_tokens, and a request without adjustments in the same batch is not
    touched (it still runs from the captured graph when alone)."""
    from ayaka_b200 import SamplingParams

    config = dict(TINY_A, eos_token_id=7)
    folder, state = es.make_model(tmp_path / "loud", config, 0, INIT_LOUD, "float32")
    wide = plain.cast_state(state, torch.float64)
    prompts = [random_tokens(256, n, 900 + n) for n in (6, 19, 11)]
    allowed = frozenset(range(0, 256, 3)) | {7}
    params = [
        SamplingParams(temperature=0.0, max_tokens=14, repetition_penalty=1.7,
                       frequency_penalty=0.9, presence_penalty=0.6, ignore_eos=True),
        SamplingParams(temperature=0.0, max_tokens=12, allowed_token_ids=allowed,
                       logit_bias={7: 100.0, 9: 6.0}, min_tokens=5),
        SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True),
    ]
    with _llm(folder, "float32", cuda_graph=True) as llm:
        outputs = llm.generate([tuple(p) for p in prompts], params)
        llm.core.manager.check_integrity()
    for prompt, output, one in zip(prompts, outputs, params):
        got = list(output.outputs[0].token_ids)
        produced: list[int] = []
        for token in got:
            row = plain.logits(wide, config, torch.tensor(prompt + produced))[-1]
            banned = set(one.banned_at(len(produced), 7))
            row = plain.adjust_logits(
                row, prompt, produced, repetition=one.repetition_penalty,
                frequency=one.frequency_penalty, presence=one.presence_penalty,
                bias=dict(one.logit_bias or ()), banned=banned,
                allowed=None if one.allowed_token_ids is None else set(one.allowed_token_ids))
            assert float(row[token]) >= float(row.max()) - 1e-4 * float(row[row > -1e30].abs().max())
            produced.append(token)
    # the biased end-of-sequence token wins as soon as min_tokens allows it, and ends the request
    second = list(outputs[1].outputs[0].token_ids)
    assert second[5] == 7 and len(second) == 6 and 7 not in second[:5]
    assert all(token in allowed for token in second)
    assert outputs[1].outputs[0].finish_reason.value == "stop"
    assert len(outputs[0].outputs[0].token_ids) == 14


def _tokens(outputs):
    return [list(output.outputs[0].token_ids) for output in outputs]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decode_steps_from_graphs_and_launched_ahead(tmp_path, dtype):
    """Decode steps replayed from captured graphs, with and without the next step launched
    before the current tokens reach the host, give the tokens of the step-by-step engine:
    greedy and seeded rows, requests of different lengths, one that ends on a stop token that
    nothing foresaw (the launch ahead then has a row too many), and pages so few that a
    launch ahead sometimes finds no room."""
    from ayaka_b200 import SamplingParams

    folder, state = es.make_model(tmp_path / "loud", TINY_B, 3, INIT_LOUD, dtype)
    prompts = [tuple(random_tokens(503, n, 700 + n)) for n in (4, 33, 18, 7)]
    base = [SamplingParams(temperature=0.0, max_tokens=40),
            SamplingParams(temperature=0.9, top_k=50, max_tokens=29, seed=5),
            SamplingParams(temperature=0.0, max_tokens=35),
            SamplingParams(temperature=1.1, max_tokens=12, seed=6)]
    with _llm(folder, dtype) as llm:
        plainly = _tokens(llm.generate(prompts, base))
    # a stop token for the third request that its plain run produces as its 10th token and
    # not earlier
    third = plainly[2]
    stop = next(token for index, token in enumerate(third) if index >= 9
                and token not in third[:index])
    cut = third.index(stop) + 1
    params = list(base)
    params[2] = SamplingParams(temperature=0.0, max_tokens=35, stop_token_ids=(stop,))
    expected = [plainly[0], plainly[1], third[:cut], plainly[3]]
    slack = 1e-4 if dtype == "float32" else 5e-2
    for pool in (dict(), dict(block_size=4, num_blocks=22)):
        with _llm(folder, dtype, **pool) as llm:
            stepwise = _tokens(llm.generate(prompts, params))
            short = llm.scheduler.stats.shed + llm.scheduler.stats.stalled_rows
        if pool:
            assert short > 0  # the pool is too small for the four of them
        elif dtype == "float32":
            assert stepwise == expected
        for ahead in (False, True):
            with _llm(folder, dtype, cuda_graph=True, decode_ahead=ahead, **pool) as llm:
                outputs = llm.generate(prompts, params)
                llm.core.manager.check_integrity()
                assert llm.core.manager.live_requests() == []
                graphs = llm.graphs
                assert graphs.replays > 0
                if ahead:
                    assert graphs.adopted > 10
                else:
                    assert graphs.adopted == graphs.dropped == 0
            if dtype == "float32":
                assert _tokens(outputs) == stepwise, (pool, ahead)
            if not pool:
                assert outputs[2].outputs[0].finish_reason.value == "stop"
                assert [len(tokens) for tokens in _tokens(outputs)] == [40, 29, cut, 12]
            for prompt, output, one in zip(prompts, outputs, params):
                if one.top_k <= 0 and one.top_p >= 1.0:  # (the check knows no truncation)
                    check_generation(state, TINY_B, prompt, list(output.outputs[0].token_ids),
                                     one, output.seed, slack)


def test_a_launch_ahead_that_the_next_plan_does_not_fit_is_dropped(tmp_path):
    """A request that arrives between two decode steps changes the next plan: the step
    launched ahead is dropped, the plan runs as scheduled, and every token is the one the
    step-by-step engine gives."""
    from ayaka_b200 import SamplingParams

    folder, _ = es.make_model(tmp_path / "loud", TINY_A, 4, INIT_LOUD, "float32")
    first, second = tuple(random_tokens(256, 9, 1)), tuple(random_tokens(256, 21, 2))
    params = SamplingParams(temperature=0.0, max_tokens=24)

    def drive(**options):
        with _llm(folder, "float32", **options) as llm:
            a = llm._add(first, params)
            for _ in range(6):
                llm._advance()
            b = llm._add(second, params)
            while llm.scheduler.has_unfinished:
                llm._advance()
            got = {request_id: [token for event in llm._pending[request_id]
                                for token in event.tokens] for request_id in (a, b)}
            llm.core.manager.check_integrity()
            return got[a], got[b], llm.graphs

    plain_a, plain_b, _ = drive()
    ahead_a, ahead_b, graphs = drive(cuda_graph=True)
    assert (ahead_a, ahead_b) == (plain_a, plain_b)
    assert len(ahead_a) == len(ahead_b) == 24
    assert graphs.dropped >= 1 and graphs.adopted > 10


def test_cancelling_a_stream_while_a_step_is_launched_ahead(tmp_path):
    """A stream closed after a few tokens leaves a decode step in flight that was launched
    ahead for it: its pages go back at once (the stream orders what reuses them after that
    step), the launch is dropped, and the next request gets the step-by-step engine's tokens."""
    from ayaka_b200 import SamplingParams

    folder, state = es.make_model(tmp_path / "a", TINY_A, 0, INIT_LOUD, "float32")
    first, second = random_tokens(256, 13, 21), random_tokens(256, 30, 22)
    params = SamplingParams(temperature=0.0, max_tokens=20)
    with _llm(folder, "float32", cuda_graph=True, num_blocks=8) as llm:
        generator = llm.stream(tuple(first), params)
        seen = [token for _, piece in zip(range(5), generator)
                for token in piece.outputs[0].token_ids]
        assert llm.graphs.adopted >= 2
        generator.close()
        assert llm.core.manager.live_requests() == []
        llm.core.manager.check_integrity()
        output = llm.generate(tuple(second), params)
        assert llm.graphs.dropped >= 1
        llm.core.manager.check_integrity()
    assert seen == plain.greedy_generate(state, TINY_A, first, 20)[:5]
    assert list(output.outputs[0].token_ids) == plain.greedy_generate(state, TINY_A, second, 20)
