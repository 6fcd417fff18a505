"""``LLM.generate`` and ``LLM.stream`` under random engine limits against the plain greedy
continuation (float32, where the plain implementation's argmax is the engine's).

A seed draws the requests (prompts of 1 token to nearly the whole context, 1 to 40 tokens to
generate) and the engine: page size, a pool between one request's need and everybody's,
how many may run, a step's token budget (down to 16, so that a prompt is many steps that
return nothing), decode steps from CUDA graphs or not, launched ahead or not. Requests the
cache cuts short must still have a right prefix and say why; every page comes back."""

from __future__ import annotations

import random

import pytest

import engine_support as es
import plain_gpt2 as plain
from cases import INIT_LOUD, TINY_A, TINY_B, random_tokens

pytestmark = pytest.mark.gpu

CONFIGS = {"A": TINY_A, "B": TINY_B}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    return {name: (*es.make_model(tmp_path_factory.mktemp(f"generate_{name}"), config,
                                  seed=ord(name), init=INIT_LOUD, dtype="float32"), config)
            for name, config in CONFIGS.items()}


def draw(rng: random.Random, folder, config: dict, most_tokens: int):
    from ayaka_b200 import EngineConfig, SamplingParams

    limit = config["n_positions"]
    prompts, params = [], []
    for index in range(rng.randint(2, 12)):
        length = rng.choice([rng.randint(1, 8), rng.randint(8, 60), rng.randint(60, limit - 2)])
        prompts.append(tuple(random_tokens(config["vocab_size"], length,
                                           rng.randrange(1 << 30))))
        params.append(SamplingParams(temperature=0.0, ignore_eos=True,
                                     max_tokens=rng.randint(1, min(most_tokens, limit - length))))
    page, running = rng.choice([4, 8, 16]), rng.choice([2, 4, 8])
    need = -(-max(len(p) + q.max_tokens for p, q in zip(prompts, params)) // page)
    blocks = max(need + 1, running + 1, rng.randint(need, need * running + 2)) + 1
    engine = EngineConfig(model=str(folder), dtype="float32", block_size=page, num_blocks=blocks,
                          max_running=running, max_tokens_per_step=rng.choice([16, 64, 2048]),
                          cuda_graph=rng.random() < 0.6, decode_ahead=rng.random() < 0.7)
    return prompts, params, engine


def nothing_left(llm) -> None:
    manager = llm.core.manager
    manager.check_integrity()
    assert manager.live_requests() == []
    assert manager.num_free_pages() == manager.pools[0].num_usable
    assert not llm.scheduler.has_unfinished


@pytest.mark.parametrize("seed", range(10))
def test_generate_under_random_limits(models, seed):
    from ayaka_b200 import LLM

    rng = random.Random(f"generate-{seed}")
    folder, state, config = models[rng.choice(list(models))]
    prompts, params, engine = draw(rng, folder, config, 40)
    with LLM.from_config(engine) as llm:
        outputs = llm.generate(prompts, params)
        nothing_left(llm)
    for prompt, asked, output in zip(prompts, params, outputs):
        got = list(output.outputs[0].token_ids)
        assert got == plain.greedy_generate(state, config, list(prompt), len(got))
        assert len(got) == asked.max_tokens or output.notes  # cut short: it says why


@pytest.mark.parametrize("seed", range(6))
def test_streams_advanced_in_random_order_and_closed_early(models, seed):
    from ayaka_b200 import LLM

    rng = random.Random(f"stream-{seed}")
    folder, state, config = models[rng.choice(list(models))]
    prompts, params, engine = draw(rng, folder, config, 30)
    got: dict[int, list[int]] = {index: [] for index in range(len(prompts))}
    with LLM.from_config(engine) as llm:
        waiting, streams = list(range(len(prompts))), {}
        while waiting or streams:
            if waiting and (not streams or rng.random() < 0.4):
                index = waiting.pop(0)
                streams[index] = llm.stream(prompts[index], params[index])
            index = rng.choice(list(streams))
            if rng.random() < 0.06:
                streams.pop(index).close()  # cancels the request where it stands
                continue
            try:
                output = next(streams[index])
            except StopIteration:
                streams.pop(index)
                continue
            got[index].extend(output.outputs[0].token_ids)
            if output.finished:
                streams.pop(index).close()
        nothing_left(llm)
        assert not llm._pending and not llm._requests
    for index, prompt in enumerate(prompts):
        assert got[index] == plain.greedy_generate(state, config, list(prompt), len(got[index]))
