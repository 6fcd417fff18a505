"""Random schedules against the plain implementation.

The other engine tests cut the work in chosen ways; here a seed draws everything: which tiny
configuration and dtype, how many requests of which lengths, the page size, how many may be
live, how many pages there are (few enough that they are used again), and step by step which
live requests take part and with how many tokens (single tokens, a few, dozens, hundreds),
decoding requests ahead of the portions or in any order. Every logit of every position is
compared with the plain implementation, and in bfloat16 also with the one that rounds where
the engine does."""

from __future__ import annotations

import random

import pytest

import engine_support as es
from cases import INIT_LOUD, INIT_LOUD_WIDE, TINY_B, TINY_D, random_tokens

pytestmark = pytest.mark.gpu

CONFIGS = {"B": (TINY_B, INIT_LOUD), "D": (TINY_D, INIT_LOUD_WIDE)}
SEEDS_PER_CASE = 12


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    made = {}
    for name, (config, init) in CONFIGS.items():
        for dtype in ("float32", "bfloat16"):
            folder = tmp_path_factory.mktemp(f"random_{name}_{dtype}")
            made[name, dtype] = (*es.make_model(folder, config, seed=ord(name), init=init,
                                                dtype=dtype), config)
    return made


def random_schedule(rng: random.Random, sequences: dict[str, list[int]], pool_tokens: int,
                    live_limit: int) -> list[dict]:
    """Steps in which each live request sits out, brings one token, or a portion of 2 to 400;
    a request is admitted while the pool (each request rounded up to 64 tokens) has room."""
    def rounded(n: int) -> int:
        return -(-n // 64) * 64

    waiting = list(sequences.items())
    rng.shuffle(waiting)
    live: dict[str, int] = {}
    held = 0
    steps = []

    def admit() -> None:
        nonlocal held
        rid, tokens = waiting.pop(0)
        live[rid] = 0
        held += rounded(len(tokens))

    while waiting or live:
        while waiting and len(live) < live_limit and rng.random() < 0.8 and \
                held + rounded(len(waiting[0][1])) <= pool_tokens:
            admit()
        if not live:
            admit()
        entries, end = [], []
        for rid in list(live):
            tokens, done = sequences[rid], live[rid]
            if rng.random() < 0.15 and len(live) > 1:
                continue
            kind = rng.random()
            size = 1 if kind < 0.45 else rng.randint(2, 8) if kind < 0.7 else \
                rng.randint(9, 80) if kind < 0.9 else rng.randint(81, 400)
            size = min(size, len(tokens) - done)
            entries.append({"id": rid, "tokens": tokens[done:done + size],
                            "want": list(range(size))})
            live[rid] = done + size
            if live[rid] == len(tokens):
                end.append(rid)
        if rng.random() < 0.5:
            entries.sort(key=lambda entry: len(entry["tokens"]) != 1)  # single rows first
        for rid in end:
            held -= rounded(len(sequences[rid]))
            del live[rid]
        if entries:
            steps.append({"entries": entries, "end": end})
    return steps


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_random_schedules(models, name, dtype):
    folder, state, config = models[name, dtype]
    limit = config["n_positions"]
    for seed in range(SEEDS_PER_CASE):
        rng = random.Random(f"{name}-{dtype}-{seed}")
        lengths = [rng.choice([rng.randint(1, 20), rng.randint(20, 200), rng.randint(200, limit)])
                   for _ in range(rng.randint(3, 14))]
        sequences = {f"r{index}": random_tokens(config["vocab_size"], length, 1000 * seed + index)
                     for index, length in enumerate(lengths)}
        live_limit = rng.choice([2, 4, 8, 12])
        longest = -(-max(lengths) // 64) * 64
        pool_tokens = max(longest, rng.randint(2, live_limit) * 128) + 64
        steps = random_schedule(rng, sequences, pool_tokens, live_limit)
        page = rng.choice([8, 16, 16, 32])
        peak = es.peak_tokens(steps, sequences)
        every = sum(-(-length // page) for length in lengths)
        pages = max(min(every, -(-peak // page) + live_limit * (64 // page + 1)), live_limit)
        core = es.build_core(folder, dtype, num_blocks=pages + 2, max_running=live_limit,
                             max_tokens_per_step=2048, block_size=page)
        got = es.replay(core, steps)
        label = f"random/{name}/page{page}"
        es.assert_logits_close(got, es.plain_logits(state, config, sequences), dtype, label,
                               page=page)
        if dtype == "bfloat16":
            es.assert_logits_close(got, es.rounded_logits(state, config, sequences), dtype,
                                   label, limits=es.ROUNDED_TOLERANCE, page=page,
                                   row_rms=es.ROUNDED_ROW_RMS)
        assert core.manager.live_requests() == []
        core.manager.check_integrity()
