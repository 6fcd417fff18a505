"""A step that failed ends its requests and leaves the engine usable (CPU, with stand-ins).

The kernels report a bounded wait that ran out, or an id outside its table, through two
sticky words on the device (``ayaka_b200/kernels/flags.py``). These tests put values into a
host stand-in of those words and raise from a stand-in runner; nothing runs on a GPU. The
reference turns a backend refusal into a step error that ends the step's requests
(``python/ayaka/execution/runner.py:227-231``).
"""

from __future__ import annotations

from types import SimpleNamespace

import pytest
import torch

from ayaka_b200.cache.manager import CacheManager
from ayaka_b200.config.engine import EngineConfig
from ayaka_b200.engine import llm as llm_module
from ayaka_b200.engine.outputs import FinishReason
from ayaka_b200.errors import BackendError
from ayaka_b200.kernels.flags import FlagReader, failure
from ayaka_b200.parts.base import CacheNeed
from ayaka_b200.sampling.params import SamplingParams


def test_failure_reads_the_two_words():
    assert failure([0, 0]) is None
    assert "bounded wait" in failure([-5, 0])
    assert "embedding table" in failure([0, 1])
    assert "bounded wait" in failure([-5, 1])  # the wait is the graver one


def test_flag_reader_raises_once_and_clears():
    words = torch.zeros(2, dtype=torch.int32)
    reader = FlagReader(torch.device("cpu"), words)
    reader.read_now()  # nothing set
    words[0] = -5
    with pytest.raises(BackendError) as caught:
        reader.read_now()
    assert caught.value.context["status"] == -5
    assert words.tolist() == [0, 0]
    reader.read_now()  # cleared: the next step starts clean


class _Runner:
    """Stands where the model runner stands: ``run`` fails the way it is told to."""

    def __init__(self, words: torch.Tensor) -> None:
        self.flags = FlagReader(torch.device("cpu"), words)
        self.fail_with: Exception | None = None
        self.steps = 0

    def run(self, entries):  # noqa: ANN001, ANN201
        self.steps += 1
        if self.fail_with is not None:
            raise self.fail_with
        wanted = sum(len(entry.want) for entry in entries)
        return torch.zeros(wanted, 8)


class _Sampler:
    """Stands where the sampler stands: token 1 for every row, after the flag check the real
    sampler makes when it has waited for the ids."""

    def __init__(self, max_rows, device, flags=None) -> None:  # noqa: ANN001
        self.flags = flags

    def sample(self, logits, rows):  # noqa: ANN001, ANN201
        self.flags.snapshot(0)
        self.flags.check(0)
        return [1] * len(rows)


def _llm(monkeypatch: pytest.MonkeyPatch):  # noqa: ANN202
    monkeypatch.setattr(llm_module, "Sampler", _Sampler)
    words = torch.zeros(2, dtype=torch.int32)
    manager = CacheManager([CacheNeed(1, 16)], [9], 4, 4, 8)
    core = SimpleNamespace(
        manager=manager, device=torch.device("cpu"), runner=_Runner(words),
        model=SimpleNamespace(spec=SimpleNamespace(max_positions=32, eos_token_id=None,
                                                   vocab_size=8)))
    config = EngineConfig(model=".", dtype="float32", block_size=4, num_blocks=9,
                          max_running=4, max_tokens_per_step=16, cuda_graph=False)
    return llm_module.LLM(core, config), words


def test_a_kernel_that_gave_up_fails_the_step_not_the_engine(monkeypatch):
    llm, words = _llm(monkeypatch)
    params = SamplingParams(temperature=0.0, max_tokens=3, ignore_eos=True)
    good = llm.generate((1, 2, 3), params)
    assert good.outputs[0].finish_reason is FinishReason.LENGTH
    words[0] = -5  # what a kernel writes when its wait ran out
    bad = llm.generate([(1, 2, 3), (4, 5)], params)
    assert [o.outputs[0].finish_reason for o in bad] == [FinishReason.ERROR] * 2
    assert all("bounded wait" in o.error for o in bad)
    llm.core.manager.check_integrity()
    assert llm.core.manager.num_free_pages() == 8  # everything was given back
    again = llm.generate((1, 2, 3), params)  # the word was cleared: the engine goes on
    assert again.outputs[0].finish_reason is FinishReason.LENGTH


def test_any_exception_inside_a_step_closes_the_step(monkeypatch):
    llm, _ = _llm(monkeypatch)
    params = SamplingParams(temperature=0.0, max_tokens=3, ignore_eos=True)
    llm.core.runner.fail_with = RuntimeError("launch failed")
    with pytest.raises(RuntimeError, match="launch failed"):
        llm.generate((1, 2, 3), params)
    # the scheduler is not left "in flight" and the request holds nothing
    llm.core.manager.check_integrity()
    assert llm.core.manager.num_free_pages() == 8
    assert not llm.scheduler.has_unfinished
    llm.core.runner.fail_with = BackendError("refused")
    refused = llm.generate((1, 2, 3), params)  # a typed error is an output, not a raise
    assert refused.outputs[0].finish_reason is FinishReason.ERROR
    llm.core.runner.fail_with = None
    assert llm.generate((1, 2), params).outputs[0].finish_reason is FinishReason.LENGTH


def test_a_raise_out_of_generate_leaves_nothing_behind(monkeypatch):
    llm, _ = _llm(monkeypatch)
    params = SamplingParams(temperature=0.0, max_tokens=3, ignore_eos=True)
    llm.core.runner.fail_with = RuntimeError("launch failed")
    with pytest.raises(RuntimeError):
        llm.generate([(1, 2, 3), (4, 5, 6, 7, 1, 2, 3, 4, 5, 6, 7, 1, 2, 3, 4, 5, 6)], params)
    assert not llm._pending and not llm._requests
    assert not llm.scheduler.has_unfinished
    llm.core.manager.check_integrity()
    assert llm.core.manager.num_free_pages() == 8
