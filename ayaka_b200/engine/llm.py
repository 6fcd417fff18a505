"""The Python entry point: ``LLM`` generates token ids for token-id prompts.

In the manner of the reference's ``LLM`` (``python/ayaka/engine/llm.py:73-245``):
``LLM.from_config(EngineConfig)``, ``generate(prompts, sampling)`` returning one
``RequestOutput`` per prompt in prompt order (a request that failed is returned with
``finish_reason`` ``ERROR``, not raised), ``stream(prompt, sampling)`` yielding the new
tokens of each step, ``close()`` and the context-manager protocol. A prompt is a tuple or
list of token ids; this engine has no tokenizer, so text is refused with a clear message.
``step(entries)`` exposes the raw step function.
"""

from __future__ import annotations

from collections import deque
from collections.abc import Generator, Mapping, Sequence
from types import TracebackType

import torch

from ayaka_b200.config.engine import EngineConfig
from ayaka_b200.engine.core import EngineCore
from ayaka_b200.engine.outputs import CompletionOutput, FinishReason, RequestOutput, Usage
from ayaka_b200.engine.request import RequestEvent
from ayaka_b200.engine.runner import StepEntry
from ayaka_b200.engine.scheduler import Scheduler
from ayaka_b200.errors import AyakaError, EngineError, InvalidRequestError
from ayaka_b200.sampling.params import SamplingParams
from ayaka_b200.sampling.sampler import SampleRow, Sampler

__all__ = ["LLM"]

Prompt = Sequence[int]


class LLM:
    """Generates for prompts, one batch of steps at a time, on the calling thread."""

    def __init__(self, core: EngineCore, config: EngineConfig) -> None:
        self.core = core
        self.config = config
        spec = core.model.spec
        self.scheduler = Scheduler(
            core.manager, max_running=config.max_running,
            max_tokens_per_step=config.max_tokens_per_step, max_waiting=config.max_waiting,
            max_positions=spec.max_positions, eos_token_id=spec.eos_token_id)
        self.sampler = Sampler(max(config.max_running, 1), core.device, core.runner.flags)
        self._counter = 0
        self._pending: dict[str, deque[RequestEvent]] = {}
        self._requests: dict[str, object] = {}
        self._closed = False
        self.graphs = None
        if config.cuda_graph:
            from ayaka_b200.engine.graph import DecodeGraphs

            self.graphs = DecodeGraphs(core)

    @classmethod
    def from_config(cls, config: EngineConfig,
                    tensors: Mapping[str, torch.Tensor] | None = None) -> LLM:
        """Load the model ``config.model`` names (or fill it from ``tensors``, checkpoint
        named) and build the engine around it."""
        return cls(EngineCore.from_config(config, tensors), config)

    # ---- the raw step function ------------------------------------------------------------
    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor | None:
        """Run one batch of (request, its next tokens) and return fp32 logits at the wanted
        places; see :class:`~ayaka_b200.engine.runner.StepEntry`. Requests fed this way are
        the caller's to ``release``."""
        self._check_open()
        return self.core.step(entries)

    def release(self, request_id: str) -> None:
        self.core.release(request_id)

    # ---- generation -----------------------------------------------------------------------
    def generate(self, prompts: Prompt | Sequence[Prompt],
                 sampling: SamplingParams | Sequence[SamplingParams | None] | None = None
                 ) -> RequestOutput | list[RequestOutput]:
        """Generate a completion for each prompt and wait for all of them."""
        self._check_open()
        single = _is_one_prompt(prompts)
        items: Sequence[Prompt] = [prompts] if single else prompts  # type: ignore[list-item]
        params = _per_prompt(sampling, len(items))
        ids: list[str] = []
        try:
            for prompt, one in zip(items, params):
                ids.append(self._add(prompt, one))
        except AyakaError:
            for request_id in ids:
                self.scheduler.abort(request_id)
                self._forget(request_id)
            raise
        tokens: dict[str, list[int]] = {request_id: [] for request_id in ids}
        final: dict[str, RequestEvent] = {}
        try:
            while len(final) < len(ids):
                for request_id in ids:
                    queue = self._pending.get(request_id)
                    while queue:
                        event = queue.popleft()
                        tokens[request_id].extend(event.tokens)
                        if event.finish_reason is not None:
                            final[request_id] = event
                if len(final) == len(ids):
                    break
                if not self.scheduler.has_unfinished:
                    raise EngineError("requests ended without a final event")
                self._advance()
        except BaseException:
            # nothing of this call is left running or remembered
            for request_id in ids:
                if request_id not in final:
                    self.scheduler.abort(request_id)
                self._forget(request_id)
            self._dispatch(self.scheduler.take_events())
            raise
        outputs = [self._output(request_id, tuple(tokens[request_id]), final[request_id], True)
                   for request_id in ids]
        for request_id in ids:
            self._forget(request_id)
        return outputs[0] if single else outputs

    def stream(self, prompt: Prompt,
               sampling: SamplingParams | None = None) -> Generator[RequestOutput]:
        """Generate for one prompt and yield an output for every step that produced tokens;
        each carries only the new tokens, the last has ``finished`` true. Closing the
        generator early cancels the request."""
        self._check_open()
        request_id = self._add(prompt, sampling)
        finished = False
        try:
            while not finished:
                queue = self._pending.get(request_id)
                if queue:
                    event = queue.popleft()
                    finished = event.finish_reason is not None
                    yield self._output(request_id, event.tokens, event, finished)
                    continue
                if not self.scheduler.has_unfinished:
                    raise EngineError(f"request {request_id!r} ended without a final event")
                self._advance()
        finally:
            if not finished:
                self.scheduler.abort(request_id)
                self._dispatch(self.scheduler.take_events())
            self._forget(request_id)

    # ---- internals ------------------------------------------------------------------------
    def _add(self, prompt: Prompt, sampling: SamplingParams | None) -> str:
        if isinstance(prompt, str):
            raise InvalidRequestError(
                "this engine has no tokenizer: pass the prompt as a sequence of token ids")
        ids = tuple(prompt)
        vocab = self.core.model.spec.vocab_size
        for token in ids:
            if type(token) is not int or not 0 <= token < vocab:
                raise InvalidRequestError(
                    f"prompt token {token!r} is not an integer in [0, {vocab})")
        if sampling is not None:
            named = [token for token, _ in sampling.logit_bias or ()]
            named += list(sampling.allowed_token_ids or ())
            for token in named:
                if token >= vocab:
                    raise InvalidRequestError(
                        f"token id {token} in logit_bias or allowed_token_ids is outside the "
                        f"vocabulary of {vocab}")
        self._counter += 1
        request_id = f"req-{self._counter}"
        request = self.scheduler.add_request(request_id, ids, sampling)
        self._pending[request_id] = deque()
        self._requests[request_id] = request
        return request_id

    def _forget(self, request_id: str) -> None:
        self._pending.pop(request_id, None)
        self._requests.pop(request_id, None)

    def _advance(self) -> None:
        """One scheduler step: plan, run, sample, update, deliver."""
        scheduler = self.scheduler
        plan = scheduler.schedule()
        self._dispatch(scheduler.take_events())  # what shedding ended while planning
        if plan is None:
            return
        try:
            rows = self._sample_rows(plan)
            # (a captured step chooses its tokens inside the graph: rows that want their
            # logits adjusted first take the ordinary step)
            graphs = self.graphs
            if graphs is not None and graphs.can_run(plan) and \
                    not any(row.adjusts for row in rows):
                launch = graphs.launch(plan, rows)
                following = self._rows_ahead(plan) if launch.exact else None
                if following is not None:
                    graphs.launch_ahead(launch, following)
                picked = graphs.finish(launch)
            else:
                if graphs is not None:
                    graphs.drop_ahead()
                logits = self.core.runner.run(plan.entries)
                picked = self.sampler.sample(logits, rows) if plan.sampled else []
        except Exception as error:
            # A step that a kernel refused, or whose kernels gave up a wait, ends its requests
            # and the engine goes on (reference: python/ayaka/execution/runner.py:227-231).
            # Whatever else went wrong between schedule() and update() must still close the
            # step, or the scheduler stays "in flight" and the requests keep their pages.
            if self.graphs is not None:
                try:
                    self.graphs.drop_ahead()
                except Exception:  # noqa: BLE001 - the first error is the one to report
                    pass
            text = str(error) if isinstance(error, AyakaError) else repr(error)
            self._dispatch(scheduler.update(plan, None, error=text))
            self.core.manager.check_integrity()
            if not isinstance(error, AyakaError):
                raise
            return
        self._dispatch(scheduler.update(plan, dict(zip(plan.sampled, picked))))

    def _rows_ahead(self, plan: object) -> list[SampleRow] | None:
        """The sampling rows of the step after ``plan`` if that step can be foreseen: the
        same requests, all decoding, none at the end of its length, nothing waiting and
        room in the cache for one more position each. A stop token cannot be foreseen:
        the launch made ahead then has a row too many, which is left out."""
        scheduler, manager = self.scheduler, self.core.manager
        if not self.config.decode_ahead or scheduler.waiting or \
                len(plan.entries) != len(scheduler.running):  # type: ignore[attr-defined]
            return None
        eos, limit = scheduler.eos_token_id, scheduler.max_positions
        capacity = manager.max_context_tokens
        rows = []
        for request_id in plan.sampled:  # type: ignore[attr-defined]
            request = scheduler.running[request_id]
            params = request.params
            produced = len(request.output) + 1  # once this step's token has arrived
            if limit - len(request.prompt) - produced <= 0 or request.computed + 2 > capacity:
                return None
            if params.max_tokens is not None and params.max_tokens - produced <= 0:
                return None
            row = SampleRow(params, request.seed, len(request.prompt) + produced, (),
                            len(request.prompt), params.banned_at(produced, eos))
            if row.adjusts:
                return None
            rows.append(row)
        for request_id in plan.sampled:  # type: ignore[attr-defined]
            if not manager.allocate(request_id, 2):
                return None
        return rows

    def _sample_rows(self, plan: object) -> list[SampleRow]:
        rows = []
        eos = self.scheduler.eos_token_id
        for request_id in plan.sampled:  # type: ignore[attr-defined]
            request = self.scheduler.running[request_id]
            params = request.params
            history = request.prompt + tuple(request.output) if params.penalises else ()
            rows.append(SampleRow(params, request.seed,
                                  len(request.prompt) + len(request.output), history,
                                  len(request.prompt),
                                  params.banned_at(len(request.output), eos)))
        return rows

    def _dispatch(self, events: list[RequestEvent]) -> None:
        for event in events:
            queue = self._pending.get(event.request_id)
            if queue is not None:
                queue.append(event)

    def _output(self, request_id: str, tokens: tuple[int, ...], event: RequestEvent,
                finished: bool) -> RequestOutput:
        request = self._requests[request_id]
        completion = CompletionOutput(0, tuple(tokens), event.finish_reason, event.stop_reason)
        usage = Usage(len(request.prompt), len(request.output)) if finished else None  # type: ignore
        note = (event.error,) if event.error and event.finish_reason is FinishReason.LENGTH \
            else ()
        error = event.error if event.finish_reason is FinishReason.ERROR else None
        return RequestOutput(request_id, request.prompt, (completion,), finished,  # type: ignore
                             usage, error, request.seed, note)  # type: ignore[attr-defined]

    def _check_open(self) -> None:
        if self._closed:
            raise EngineError("the engine is closed")

    def close(self) -> None:
        """Shut the engine down; later calls raise ``EngineError``."""
        if self.graphs is not None and not self._closed:
            self.graphs.drop_ahead()
        self._closed = True

    def __enter__(self) -> LLM:
        return self

    def __exit__(self, exc_type: type[BaseException] | None, exc: BaseException | None,
                 traceback: TracebackType | None) -> None:
        self.close()


def _is_one_prompt(prompts: object) -> bool:
    if isinstance(prompts, str):
        return True
    if isinstance(prompts, Sequence) and prompts and all(
            type(item) is int for item in prompts):
        return True
    return False


def _per_prompt(sampling: object, count: int) -> list[SamplingParams | None]:
    if sampling is None or isinstance(sampling, SamplingParams):
        return [sampling] * count  # type: ignore[list-item]
    items = list(sampling)  # type: ignore[call-overload]
    if len(items) != count:
        raise InvalidRequestError(f"{len(items)} sampling parameters for {count} prompts")
    return items
