"""The scheduler's decisions on the CPU, against a fake step function whose token is a pure
function of (request, position) — the reference tests its scheduler the same way
(``tests/_support/fake_runner.py``, ``tests/scheduler/test_properties.py``): whatever the
batching, the portions and the pressure on the pool, a request's tokens are a prefix of the
expected ones, and the cache bookkeeping stays sound after every call."""

from __future__ import annotations

import random

import pytest

from ayaka_b200.cache.manager import CacheManager
from ayaka_b200.engine.outputs import FinishReason
from ayaka_b200.engine.scheduler import Scheduler, next_chunk
from ayaka_b200.errors import CapacityError, EngineError, InvalidRequestError
from ayaka_b200.parts.base import CacheNeed
from ayaka_b200.sampling.params import SamplingParams

NEED = CacheNeed(2, 16, 0)
VOCAB = 50


def fake_token(prompt: tuple[int, ...], position: int) -> int:
    """The token 'the model' produces at ``position`` of a request: depends on nothing else."""
    return (sum(prompt) * 31 + position * 7) % VOCAB


def make(pages=20, page=4, running=4, budget=16, waiting=8, positions=64, eos=None):
    manager = CacheManager([NEED], [pages], page, running, -(-positions // page))
    return Scheduler(manager, max_running=running, max_tokens_per_step=budget,
                     max_waiting=waiting, max_positions=positions, eos_token_id=eos), manager


def drive(scheduler, manager, prompts, on_plan=None, limit=10_000):
    """Run to completion; returns per request (tokens, final event)."""
    tokens = {rid: [] for rid in prompts}
    final = {}
    for _ in range(limit):
        plan = scheduler.schedule()
        manager.check_integrity()
        events = scheduler.take_events()
        if plan is not None:
            if on_plan:
                on_plan(plan)
            assert sum(len(e.tokens) for e in plan.entries) <= scheduler.max_tokens_per_step
            assert len(plan.entries) <= scheduler.max_running
            picked = {}
            for entry in plan.entries:
                request = scheduler.running[entry.request_id]
                start = request.computed
                full = request.prompt + tuple(request.output)
                assert tuple(entry.tokens) == full[start:start + len(entry.tokens)]
                if entry.want:
                    assert entry.want == (len(entry.tokens) - 1,)
                    picked[entry.request_id] = fake_token(request.prompt,
                                                          start + len(entry.tokens))
            assert tuple(picked) == plan.sampled
            events += scheduler.update(plan, picked)
            manager.check_integrity()
        for event in events:
            tokens.setdefault(event.request_id, []).extend(event.tokens)
            if event.finish_reason is not None:
                final[event.request_id] = event
        if plan is None:
            break
    assert not scheduler.has_unfinished
    return tokens, final


def expected(prompt, count):
    return [fake_token(tuple(prompt), len(prompt) + i) for i in range(count)]


def test_next_chunk_ends_on_a_page_boundary_unless_it_is_the_last():
    assert next_chunk(10, 0, 16, 4) == 10
    assert next_chunk(40, 0, 16, 4) == 16
    assert next_chunk(40, 3, 16, 4) == 13  # 3 + 13 = 16
    assert next_chunk(40, 3, 2, 4) == 1  # 3 + 1 = 4
    assert next_chunk(40, 1, 2, 4) == 2  # cannot reach a boundary: take the budget
    assert next_chunk(40, 38, 16, 4) == 2


def test_admission_checks():
    scheduler, _ = make(positions=32, pages=5)  # 16 tokens of cache
    with pytest.raises(InvalidRequestError):
        scheduler.add_request("a", ())
    with pytest.raises(InvalidRequestError):
        scheduler.add_request("a", tuple(range(32)))  # no room to generate
    with pytest.raises(InvalidRequestError):
        scheduler.add_request("a", (1, 2, 3), SamplingParams(max_tokens=30))
    with pytest.raises(InvalidRequestError):
        scheduler.add_request("a", tuple(range(20)), SamplingParams(max_tokens=1))  # > cache
    scheduler.add_request("a", (1, 2, 3), SamplingParams(max_tokens=4))
    with pytest.raises(InvalidRequestError):
        scheduler.add_request("a", (1,), SamplingParams(max_tokens=4))  # id in use
    small, _ = make(waiting=1)
    small.add_request("x", (1,), SamplingParams(max_tokens=1))
    with pytest.raises(CapacityError):
        small.add_request("y", (1,), SamplingParams(max_tokens=1))


def test_one_request_prompt_in_portions_then_decode():
    scheduler, manager = make(budget=8, page=4)
    prompt = tuple(range(1, 20))
    scheduler.add_request("a", prompt, SamplingParams(max_tokens=5))
    shapes = []
    tokens, final = drive(scheduler, manager, {"a": prompt},
                          on_plan=lambda p: shapes.append([len(e.tokens) for e in p.entries]))
    assert shapes[:3] == [[8], [8], [3]] and shapes[3:] == [[1]] * 4
    assert tokens["a"] == expected(prompt, 5)
    assert final["a"].finish_reason is FinishReason.LENGTH
    assert manager.num_free_pages() == manager.pools[0].num_usable


def test_decodes_run_beside_prompt_portions():
    scheduler, manager = make(budget=8, page=4, running=3)
    scheduler.add_request("a", (1, 2, 3), SamplingParams(max_tokens=6))
    shapes = []

    def on_plan(plan):
        shapes.append([(e.request_id, len(e.tokens)) for e in plan.entries])
        if len(shapes) == 2:
            scheduler.add_request("b", tuple(range(20)), SamplingParams(max_tokens=2))

    prompts = {"a": (1, 2, 3), "b": tuple(range(20))}
    tokens, _ = drive(scheduler, manager, prompts, on_plan=on_plan)
    # after b arrives, a's single decode row comes first and b's portion fills the budget
    assert shapes[2] == [("a", 1), ("b", 4)]  # cut to end on a page boundary
    assert tokens["a"] == expected(prompts["a"], 6) and tokens["b"] == expected(prompts["b"], 2)


def test_queue_order_is_strict():
    scheduler, manager = make(pages=6, page=4, running=4, budget=32)  # 20 tokens of cache
    scheduler.add_request("big", tuple(range(18)), SamplingParams(max_tokens=2))
    scheduler.add_request("big2", tuple(range(18)), SamplingParams(max_tokens=1))
    scheduler.add_request("small", (1,), SamplingParams(max_tokens=1))
    plan = scheduler.schedule()
    # big2 does not fit beside big; small must not overtake it
    assert [e.request_id for e in plan.entries] == ["big"]
    scheduler.update(plan, {"big": 0})


def test_stop_tokens_min_tokens_and_eos():
    prompt = (3, 4)
    stream = expected(prompt, 10)
    stop = stream[2]
    scheduler, manager = make(eos=stream[4])
    scheduler.add_request("s", prompt, SamplingParams(max_tokens=10,
                                                      stop_token_ids=frozenset({stop})))
    scheduler.add_request("m", prompt, SamplingParams(max_tokens=10, min_tokens=3,
                                                      stop_token_ids=frozenset({stop})))
    scheduler.add_request("e", prompt, SamplingParams(max_tokens=10))
    scheduler.add_request("i", prompt, SamplingParams(max_tokens=6, ignore_eos=True))
    tokens, final = drive(scheduler, manager, dict.fromkeys("smei", prompt))
    first_stop = stream.index(stop)
    assert tokens["s"] == stream[:first_stop + 1]  # the stop token is kept
    assert final["s"].finish_reason is FinishReason.STOP and final["s"].stop_reason == stop
    later = next(i for i, t in enumerate(stream) if t in (stop, stream[4]) and i >= 3)
    assert tokens["m"] == stream[:later + 1]
    eos_at = next(i for i, t in enumerate(stream) if t == stream[4])
    assert tokens["e"] == stream[:eos_at + 1] and final["e"].finish_reason is FinishReason.STOP
    assert tokens["i"] == stream[:6] and final["i"].finish_reason is FinishReason.LENGTH


def test_context_limit_ends_a_request():
    scheduler, manager = make(positions=12, pages=10)
    prompt = tuple(range(8))
    scheduler.add_request("a", prompt, SamplingParams(max_tokens=None))
    tokens, final = drive(scheduler, manager, {"a": prompt})
    assert len(tokens["a"]) == 4 and final["a"].finish_reason is FinishReason.LENGTH


def test_a_cache_smaller_than_the_crowd_sheds_the_newest_and_never_leaks():
    scheduler, manager = make(pages=7, page=4, running=4, budget=64)  # 24 tokens of cache
    prompts = {f"r{i}": tuple(range(i + 1, i + 7)) for i in range(4)}  # 6 tokens each
    for rid, prompt in prompts.items():
        scheduler.add_request(rid, prompt, SamplingParams(max_tokens=20))
    tokens, final = drive(scheduler, manager, prompts)
    for rid, prompt in prompts.items():
        got = tokens[rid]
        assert got == expected(prompt, len(got))  # never a wrong token, only fewer
    reasons = {rid: final[rid].finish_reason for rid in prompts}
    assert reasons["r0"] is FinishReason.LENGTH and len(tokens["r0"]) >= len(tokens["r3"])
    assert any(final[rid].error and "cache is full" in final[rid].error for rid in prompts)
    assert scheduler.stats.shed >= 1
    assert manager.num_free_pages() == manager.pools[0].num_usable
    assert manager.live_requests() == []


def test_protocol_errors_and_abort():
    scheduler, manager = make()
    scheduler.add_request("a", (1, 2), SamplingParams(max_tokens=8))
    scheduler.add_request("b", (1, 2, 3), SamplingParams(max_tokens=8))
    plan = scheduler.schedule()
    with pytest.raises(EngineError):
        scheduler.schedule()
    scheduler.abort("a")  # in flight: deferred, pages stay until update
    assert "a" in manager
    with pytest.raises(EngineError):
        scheduler.update(plan, {"a": 1})  # b's token is missing
    scheduler._in_flight = plan  # the failed update consumed nothing else
    events = scheduler.update(plan, {"a": 1, "b": 2})
    assert "a" not in manager
    assert [e.finish_reason for e in events if e.request_id == "a"][-1] is FinishReason.CANCELLED
    scheduler.abort("b")
    assert not scheduler.has_unfinished and manager.live_requests() == []
    manager.check_integrity()


def test_a_failed_step_ends_only_its_requests():
    scheduler, manager = make(running=1)
    scheduler.add_request("a", (1, 2), SamplingParams(max_tokens=3))
    scheduler.add_request("b", (4, 5), SamplingParams(max_tokens=3))
    plan = scheduler.schedule()
    events = scheduler.update(plan, None, error="kernel refused")
    assert events[-1].finish_reason is FinishReason.ERROR and events[-1].request_id == "a"
    manager.check_integrity()
    tokens, final = drive(scheduler, manager, {"a": (1, 2), "b": (4, 5)})
    assert tokens["b"] == expected((4, 5), 3)


@pytest.mark.parametrize("seed", range(25))
def test_random_workloads_keep_every_promise(seed):
    rng = random.Random(seed)
    page = rng.choice([2, 4, 8])
    positions = 64
    scheduler, manager = make(pages=rng.randint(4, 30), page=page, running=rng.randint(1, 5),
                              budget=rng.choice([page, 8, 16, 40]), waiting=50,
                              positions=positions)
    prompts = {}
    arrivals = []
    for index in range(rng.randint(3, 14)):
        prompt = tuple(rng.randrange(VOCAB) for _ in range(rng.randint(1, 30)))
        max_tokens = rng.randint(1, positions - len(prompt))
        arrivals.append((rng.randint(0, 12), f"q{index}", prompt, max_tokens))
    clock = [0]

    def feed(_plan=None):
        for due, rid, prompt, max_tokens in list(arrivals):
            if due <= clock[0]:
                arrivals.remove((due, rid, prompt, max_tokens))
                try:
                    scheduler.add_request(rid, prompt, SamplingParams(max_tokens=max_tokens))
                    prompts[rid] = prompt
                except InvalidRequestError:
                    pass  # a prompt larger than this cache: refused at the door
        clock[0] += 1

    feed()
    while arrivals and not scheduler.has_unfinished:
        feed()
    tokens, final = {}, {}
    while True:
        got, ended = drive(scheduler, manager, prompts, on_plan=feed)
        for rid, values in got.items():
            tokens.setdefault(rid, []).extend(values)
        final.update(ended)
        if not arrivals:
            break
        feed()
    for rid, prompt in prompts.items():
        assert rid in final
        got = tokens[rid]
        assert got == expected(prompt, len(got))
        if final[rid].finish_reason is FinishReason.LENGTH and not final[rid].error:
            assert len(got) >= 1
    assert manager.live_requests() == []
    assert manager.num_free_pages() == manager.pools[0].num_usable


def test_sampling_params_for_logit_adjustments():
    """Penalties, logit bias and allowed ids are validated once, and the parameters say when
    the logits of the next token need adjusting (python/ayaka/core/params.py:56-90, 205-215;
    python/ayaka/sampling/logits.py:105-128)."""
    from ayaka_b200.errors import InvalidRequestError

    plain = SamplingParams()
    assert not plain.penalises and not plain.adjusts_logits(0, 7)
    full = SamplingParams(repetition_penalty=1.2, frequency_penalty=-2.0, presence_penalty=2.0,
                          logit_bias={9: 1.5, 3: -100.0}, allowed_token_ids={4, 9})
    assert full.logit_bias == ((3, -100.0), (9, 1.5)) and full.allowed_token_ids == {4, 9}
    assert full.penalises and full.adjusts_logits(99, None)
    assert SamplingParams(logit_bias=[(5, 0.5)]).logit_bias == ((5, 0.5),)
    assert SamplingParams(logit_bias={}).logit_bias is None
    # the stop ids (and the end-of-sequence id unless ignored) are held back until min_tokens
    held = SamplingParams(min_tokens=3, stop_token_ids={11})
    assert held.banned_at(2, 7) == {7, 11} and held.banned_at(3, 7) == frozenset()
    assert held.adjusts_logits(0, None) and not held.adjusts_logits(3, 7)
    assert SamplingParams(min_tokens=3, ignore_eos=True).banned_at(0, 7) == frozenset()
    for bad in (dict(repetition_penalty=0.0), dict(frequency_penalty=2.5),
                dict(presence_penalty=-2.5), dict(logit_bias={3: 101.0}),
                dict(logit_bias=[(3, 1.0), (3, 2.0)]), dict(logit_bias={-1: 1.0}),
                dict(logit_bias="x"), dict(allowed_token_ids=set()),
                dict(allowed_token_ids={-2}), dict(repetition_penalty=float("nan"))):
        with pytest.raises(InvalidRequestError):
            SamplingParams(**bad)
