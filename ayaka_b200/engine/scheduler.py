"""The scheduler: which requests run in the next step, with which tokens.

Host logic only; it never touches a tensor. Policy, after the reference's scheduler
(``python/ayaka/scheduler/scheduler.py:176-388, 536-600``, ``scheduler/roster.py:148-180``)
with one change: a step may mix decoding requests and prompt portions.

* Admission (``add_request``): the id is new; the prompt is not empty, shorter than the
  context, and ``prompt + max_tokens`` fits the context; the prompt fits the cache one
  request can get; the queue is not full. Requests wait in arrival order and are admitted
  strictly in that order: one that does not fit is never overtaken by a smaller one.
* A step (``schedule``): first every running request that has a sampled token to feed gets
  one row if the cache gives it a slot; then, under what is left of the token budget,
  running requests that are still reading their prompt get their next portion, in running
  order; then new requests are admitted while the budget and ``max_running`` allow. A
  portion that does not end the prompt is cut to end on a page boundary, and shrinks to the
  pages that are free.
* When pages run out nothing is evicted or preempted: ``allocate`` says no and the step is
  smaller. If *no* running request can move, the one that arrived last is ended with
  ``LENGTH`` and a note that the cache, not the model, was the limit, and its pages go
  back; if nothing runs and the head of the queue still cannot start, it ends with
  ``ERROR``. Either way the engine always makes progress.
* One step is in flight at a time: ``schedule`` twice without ``update`` is an error.
  Pages are only freed in ``update`` (or by ``abort`` between steps), never while a step
  that may read them is running.
"""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field

import numpy as np

from ayaka_b200.cache.manager import CacheManager
from ayaka_b200.engine.outputs import FinishReason
from ayaka_b200.engine.request import Request, RequestEvent, RequestStatus
from ayaka_b200.engine.runner import StepEntry
from ayaka_b200.errors import CapacityError, EngineError, InvalidRequestError
from ayaka_b200.sampling.params import SamplingParams
from ayaka_b200.sampling.rng import resolve_seed

__all__ = ["Scheduler", "SchedulerStats", "StepPlan"]


@dataclass(frozen=True, slots=True)
class StepPlan:
    """One step as the scheduler planned it.

    ``entries`` go to the step function as they are. ``sampled`` lists, in the order of the
    wanted logits rows, the requests that get a token from this step."""

    step_id: int
    entries: tuple[StepEntry, ...]
    sampled: tuple[str, ...]
    num_decode: int
    num_prefill_tokens: int


@dataclass(slots=True)
class SchedulerStats:
    steps: int = 0
    decode_rows: int = 0
    prefill_tokens: int = 0
    shed: int = 0
    finished: int = 0
    stalled_rows: int = 0
    last_step_rows: int = 0
    queue_peak: int = 0
    extra: dict[str, int] = field(default_factory=dict)


def next_chunk(prompt_length: int, computed: int, budget: int, page_size: int) -> int:
    """The next portion of a prompt from ``computed``: the rest if it fits the budget, else
    cut so that it ends on a page boundary (``scheduler.py:566-572`` in the reference)."""
    remaining = prompt_length - computed
    if remaining <= budget:
        return remaining
    size = budget - ((computed + budget) % page_size)
    return size if size > 0 else budget


class Scheduler:
    def __init__(self, manager: CacheManager, *, max_running: int, max_tokens_per_step: int,
                 max_waiting: int, max_positions: int, eos_token_id: int | None = None) -> None:
        self.manager = manager
        self.max_running = min(max_running, manager.max_requests)
        self.max_tokens_per_step = max_tokens_per_step
        self.max_waiting = max_waiting
        self.max_positions = max_positions
        self.eos_token_id = eos_token_id
        self.waiting: deque[Request] = deque()
        self.running: dict[str, Request] = {}
        self.stats = SchedulerStats()
        self._events: list[RequestEvent] = []
        self._known: set[str] = set()
        self._arrivals = 0
        self._in_flight: StepPlan | None = None
        self._step_ids = 0
        self._abort_later: set[str] = set()

    # ---- admission ----------------------------------------------------------------------
    def add_request(self, request_id: str, prompt: tuple[int, ...] | list[int],
                    params: SamplingParams | None = None) -> Request:
        params = params or SamplingParams()
        if request_id in self._known:
            raise InvalidRequestError(f"request id {request_id!r} is already in use")
        prompt = tuple(prompt)
        if not prompt:
            raise InvalidRequestError("the prompt is empty")
        if len(prompt) >= self.max_positions:
            raise InvalidRequestError(
                f"prompt ({len(prompt)}) must be shorter than the model context of "
                f"{self.max_positions} tokens")
        if params.max_tokens is not None and len(prompt) + params.max_tokens > self.max_positions:
            raise InvalidRequestError(
                f"prompt ({len(prompt)}) plus max_tokens ({params.max_tokens}) must be <= the "
                f"model context of {self.max_positions} tokens")
        capacity = self.manager.max_context_tokens
        if len(prompt) > capacity:
            raise InvalidRequestError(
                f"prompt ({len(prompt)} tokens) exceeds the {capacity} tokens of cache this "
                "engine can give one request")
        if len(self.waiting) >= self.max_waiting:
            raise CapacityError(f"the waiting queue is full ({self.max_waiting} requests)")
        request = Request(request_id, prompt, np.asarray(prompt, dtype=np.int64), params,
                          resolve_seed(request_id, params.seed), self._arrivals)
        self._arrivals += 1
        self._known.add(request_id)
        self.waiting.append(request)
        self.stats.queue_peak = max(self.stats.queue_peak, len(self.waiting))
        return request

    @property
    def has_unfinished(self) -> bool:
        return bool(self.waiting or self.running)

    def take_events(self) -> list[RequestEvent]:
        events, self._events = self._events, []
        return events

    # ---- planning -----------------------------------------------------------------------
    def schedule(self) -> StepPlan | None:
        """Plan the next step, or return ``None`` when nothing is left to run."""
        if self._in_flight is not None:
            raise EngineError("schedule() was called twice without update()")
        while True:
            plan = self._plan()
            if plan is not None:
                self._in_flight = plan
                return plan
            if self.running:
                self._shed_stalled()
            elif self.waiting:
                self._shed_unservable_head()
            else:
                return None

    def _grant(self, request: Request, size: int) -> int:
        """Room for ``size`` more tokens, or for as many as the free pages allow."""
        manager = self.manager
        if manager.allocate(request.request_id, size):
            return size
        page = manager.page_size
        held = 0
        if request.request_id in manager:
            held = -(-request.computed // page) * page - request.computed
        free = min(manager.num_free_pages(group) for group in range(len(manager.needs)))
        shrunk = min(size, held + free * page)
        if 1 <= shrunk < size and manager.allocate(request.request_id, shrunk):
            return shrunk
        return 0

    def _plan(self) -> StepPlan | None:
        budget = self.max_tokens_per_step
        entries: list[StepEntry] = []
        sampled: list[str] = []
        decodes = prefill_tokens = stalled = 0
        # 1. decoding requests: one row each
        for request in self.running.values():
            if request.prefilling or budget <= 0:
                continue
            token = request.pending
            if token is None:
                continue
            if self.manager.allocate(request.request_id, 1):
                entries.append(StepEntry(request.request_id, (token,), (0,)))
                sampled.append(request.request_id)
                budget -= 1
                decodes += 1
            else:
                stalled += 1
        # 2. prompts in progress, in running order
        for request in self.running.values():
            if not request.prefilling or budget <= 0:
                continue
            used = self._portion(request, budget, entries, sampled)
            budget -= used
            prefill_tokens += used
            if used == 0:
                stalled += 1
        # 3. new requests, strictly in queue order
        while self.waiting and budget > 0 and len(self.running) < self.max_running:
            request = self.waiting[0]
            used = self._portion(request, budget, entries, sampled)
            if used == 0:
                break
            self.waiting.popleft()
            request.move(RequestStatus.RUNNING)
            self.running[request.request_id] = request
            budget -= used
            prefill_tokens += used
        self.stats.stalled_rows += stalled
        if not entries:
            return None
        self._step_ids += 1
        return StepPlan(self._step_ids, tuple(entries), tuple(sampled), decodes, prefill_tokens)

    def _portion(self, request: Request, budget: int, entries: list[StepEntry],
                 sampled: list[str]) -> int:
        size = next_chunk(len(request.prompt), request.computed, budget, self.manager.page_size)
        size = self._grant(request, size)
        if size == 0:
            return 0
        start = request.computed
        tokens = request.prompt_ids[start:start + size]
        ends_prompt = start + size == len(request.prompt)
        entries.append(StepEntry(request.request_id, tokens, (size - 1,) if ends_prompt else ()))
        if ends_prompt:
            sampled.append(request.request_id)
        return size

    # ---- after the step -----------------------------------------------------------------
    def update(self, plan: StepPlan, tokens: dict[str, int] | None,
               error: str | None = None) -> list[RequestEvent]:
        """Commit what the step computed and take the sampled tokens (``tokens`` maps each id
        of ``plan.sampled`` to its token). With ``error`` the step failed: its requests end
        with ``ERROR`` and nothing is committed."""
        if self._in_flight is None or plan.step_id != self._in_flight.step_id:
            raise EngineError("update() does not answer the step in flight")
        self._in_flight = None
        self.stats.steps += 1
        self.stats.decode_rows += plan.num_decode
        self.stats.prefill_tokens += plan.num_prefill_tokens
        self.stats.last_step_rows = plan.num_decode + plan.num_prefill_tokens
        if error is not None:
            for entry in plan.entries:
                request = self.running.get(entry.request_id)
                if request is not None:
                    self._finish(request, FinishReason.ERROR, error=error)
        else:
            if tokens is None or set(tokens) != set(plan.sampled):
                raise EngineError("update() needs one token for every sampled request")
            context_limit = self.manager.max_context_tokens  # the same for every request
            for entry in plan.entries:
                request = self.running[entry.request_id]
                self.manager.commit(entry.request_id, len(entry.tokens))
                request.computed += len(entry.tokens)
                if entry.request_id in tokens:
                    token = tokens[entry.request_id]
                    reason, stop = request.accept(token, self.eos_token_id, self.max_positions)
                    if reason is None and request.computed + 1 > context_limit:
                        reason = FinishReason.LENGTH
                    if reason is not None:
                        self._finish(request, reason, new_tokens=(token,), stop=stop)
                    else:
                        self._events.append(RequestEvent(request.request_id, (token,)))
        for request_id in list(self._abort_later):
            self._abort_now(request_id)
        self._abort_later.clear()
        return self.take_events()

    def abort(self, request_id: str) -> None:
        """End a request as cancelled. Inside a step in flight the end is deferred to
        ``update`` so that no page is freed while a kernel may read it."""
        if self._in_flight is not None and any(
                entry.request_id == request_id for entry in self._in_flight.entries):
            self._abort_later.add(request_id)
            return
        self._abort_now(request_id)

    def _abort_now(self, request_id: str) -> None:
        request = self.running.get(request_id)
        if request is not None:
            self._finish(request, FinishReason.CANCELLED)
            return
        for request in self.waiting:
            if request.request_id == request_id:
                self.waiting.remove(request)
                self._finish(request, FinishReason.CANCELLED)
                return

    def _finish(self, request: Request, reason: FinishReason, *, new_tokens: tuple[int, ...] = (),
                stop: int | None = None, error: str | None = None) -> None:
        request.finish_reason = reason
        request.move(RequestStatus.FINISHED)
        self.running.pop(request.request_id, None)
        self.manager.free(request.request_id)
        self.stats.finished += 1
        self._events.append(RequestEvent(request.request_id, new_tokens, reason, stop, error))

    def _shed_stalled(self) -> None:
        victim = max(self.running.values(), key=lambda request: request.arrival)
        self.stats.shed += 1
        self._finish(
            victim, FinishReason.LENGTH,
            error=(f"the cache is full: request {victim.request_id!r} stopped at "
                   f"{victim.computed} tokens and no running request can free memory; the "
                   "limit is memory, not the model context"))

    def _shed_unservable_head(self) -> None:
        head = self.waiting.popleft()
        self.stats.shed += 1
        self._finish(head, FinishReason.ERROR,
                     error=(f"request {head.request_id!r} cannot get cache room even with "
                            "nothing else running"))
