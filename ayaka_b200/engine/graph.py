"""Decode steps replayed from CUDA graphs.

A decode-only step (one token per request) launches a few hundred small kernels; launched
one by one from the host they cost more than they compute. For every bucket of batch sizes
(1, 2, 4, 8, ...) the whole step — model forward, final norm, head and token choice — is
captured once into a graph over fixed device buffers. A step then is: fill one pinned
buffer with the step's metadata and sampling parameters, one host-to-device copy, one graph
launch, one device-to-host read of the chosen ids. A step smaller than its bucket is padded
with rows that belong to no request: they store nothing, attend to nothing and their ids
are dropped. The reference does the same for its torch ops (``python/ayaka/execution/
graph.py:89-287``); here one graph per bucket serves greedy and sampling rows alike because
the sampling kernel handles both.
"""

from __future__ import annotations

import numpy as np
import torch

from ayaka_b200.engine.core import EngineCore
from ayaka_b200.kernels import ops
from ayaka_b200.parts.context import GroupStep, StepContext
from ayaka_b200.sampling.sampler import SampleRow

__all__ = ["DecodeGraphs"]


def _align4(n: int) -> int:
    return (n + 3) & ~3


class _Bucket:
    """Fixed buffers, the step context over them and the captured graph of one batch size."""

    def __init__(self, core: EngineCore, size: int) -> None:
        manager = core.manager
        self.size = size
        self.width = manager.max_pages_per_request
        groups = len(manager.needs)
        cursor = 0

        def take(length: int) -> int:
            nonlocal cursor
            offset = cursor
            cursor += _align4(length)
            return offset

        self.o_tokens, self.o_positions, self.o_request = take(size), take(size), take(size)
        self.o_row_start, self.o_kv_len, self.o_state = take(size + 1), take(size), take(size)
        self.o_want = take(size)
        self.o_groups = [(take(size), take(size * self.width)) for _ in range(groups)]
        self.o_temperature, self.o_top_p, self.o_min_p = take(size), take(size), take(size)
        self.o_top_k = take(size)
        self.o_seeds, self.o_sample_positions = take(2 * size), take(2 * size)
        self.words = cursor
        # two launches may be in flight (the step and the one launched ahead of its result):
        # each has its own pinned metadata, pinned result and event
        self.staging = [torch.zeros(cursor, dtype=torch.int32).pin_memory() for _ in range(2)]
        self.out_host = [torch.zeros(size, dtype=torch.int32).pin_memory() for _ in range(2)]
        self.events = [torch.cuda.Event() for _ in range(2)]
        self.turn = 0
        self.meta = torch.zeros(cursor, dtype=torch.int32, device=core.device)
        self.out = torch.zeros(size, dtype=torch.int32, device=core.device)
        meta = self.meta

        def view(offset: int, length: int) -> torch.Tensor:
            return meta[offset:offset + length]

        self.step = StepContext(
            num_rows=size, num_requests=size,
            tokens=view(self.o_tokens, size), positions=view(self.o_positions, size),
            request_of_row=view(self.o_request, size),
            row_start=view(self.o_row_start, size + 1), kv_len=view(self.o_kv_len, size),
            state_slot=view(self.o_state, size),
            host_rows=[1] * size, host_start=[0] * size, host_state_slot=[0] * size,
            groups=[GroupStep(view(o_table, size * self.width).view(size, self.width),
                              view(o_slots, size), manager.page_size)
                    for o_slots, o_table in self.o_groups],
            workspace=core.runner.workspace, bad_index=core.runner._bad_index,
            max_kv_len=core.model.spec.max_positions, decode_only=True)
        self.want_rows = view(self.o_want, size)
        self.argmax_scratch = torch.zeros(2 * size * ops.ARGMAX_PARTS, device=core.device)
        # one graph for steps whose rows are all greedy (argmax), one for any other step
        self.graphs: dict[bool, torch.cuda.CUDAGraph] = {}
        self.kernels = 0

    def launch_body(self, core: EngineCore, greedy: bool) -> None:
        size, meta = self.size, self.meta
        logits = core.model.forward(self.step, core.runner.caches, self.want_rows, size)
        if greedy:
            ops.argmax(logits, self.out, rows=size, scratch=self.argmax_scratch)
            return
        ops.sample(logits, meta[self.o_temperature:self.o_temperature + size].view(torch.float32),
                   meta[self.o_top_k:self.o_top_k + size],
                   meta[self.o_top_p:self.o_top_p + size].view(torch.float32),
                   meta[self.o_min_p:self.o_min_p + size].view(torch.float32),
                   meta[self.o_seeds:self.o_seeds + 2 * size].view(torch.int64),
                   meta[self.o_sample_positions:self.o_sample_positions + 2 * size].view(
                       torch.int64),
                   self.out, rows=size)


class _Launch:
    """A step that was launched: where its result arrives and what it ran."""

    __slots__ = ("bucket", "ids", "positions", "rows", "out_host", "event", "count", "pick",
                 "exact", "slot")

    def __init__(self, bucket: _Bucket, ids: tuple[str, ...], positions: list[int],
                 rows: list[SampleRow], out_host: torch.Tensor, event: torch.cuda.Event,
                 slot: int) -> None:
        self.bucket, self.ids, self.positions, self.rows = bucket, ids, positions, rows
        self.out_host, self.event, self.slot = out_host, event, slot
        self.count = len(ids)
        self.pick = list(range(self.count))  # the launch's row of each entry of its plan
        self.exact = True  # every row of the launch belongs to an entry, in plan order

    def covers(self, ids: tuple[str, ...], positions: list[int],
               rows: list[SampleRow]) -> list[int] | None:
        """The launch's row for each of ``ids`` if it ran every one of them at the given
        position and with the given sampling; else ``None``. Rows of requests that ended
        meanwhile are left out: no row's result depends on another row."""
        if len(rows) != len(ids):
            return None
        where = {request_id: index for index, request_id in enumerate(self.ids)}
        pick = []
        for request_id, position, row in zip(ids, positions, rows):
            index = where.get(request_id)
            if index is None or self.positions[index] != position:
                return None
            mine = self.rows[index]
            if mine.params is not row.params or mine.seed != row.seed or \
                    mine.position != row.position or row.adjusts:
                return None
            pick.append(index)
        return pick


class DecodeGraphs:
    """Captures and replays decode steps; falls back to nothing — a step it cannot run is
    run by the ordinary step function."""

    def __init__(self, core: EngineCore, buckets: tuple[int, ...] | None = None) -> None:
        self.core = core
        limit = core.manager.max_requests
        if buckets is None:
            sizes, size = [], 1
            while size < limit:
                sizes.append(size)
                size *= 2
            sizes.append(limit)
            buckets = tuple(sizes)
        self.sizes = tuple(sorted(set(min(size, limit) for size in buckets)))
        self._buckets: dict[int, _Bucket] = {}
        self._ahead: _Launch | None = None
        self.flags = core.runner.flags
        self.replays = 0
        self.adopted = 0  # launches made ahead that the next plan took over
        self.dropped = 0  # launches made ahead that the next plan did not fit

    def can_run(self, plan: object) -> bool:
        entries = plan.entries  # type: ignore[attr-defined]
        if any(state is not None for state in self.core.cache_plan.run_state):
            return False  # capture runs the step's kernels more than once: pages take that,
            # a running per-request state does not
        return (plan.num_prefill_tokens == 0 and 0 < len(entries) <= self.sizes[-1]  # type: ignore
                and len(plan.sampled) == len(entries))  # type: ignore[attr-defined]

    def bucket_for(self, count: int) -> _Bucket:
        size = next(size for size in self.sizes if size >= count)
        bucket = self._buckets.get(size)
        if bucket is None:
            bucket = _Bucket(self.core, size)
            self._buckets[size] = bucket
        return bucket

    def run(self, plan: object, rows: list[SampleRow]) -> list[int]:
        """Run a decode-only plan through its bucket's graph; returns one id per entry."""
        return self.finish(self.launch(plan, rows))

    def launch(self, plan: object, rows: list[SampleRow]) -> _Launch:
        """Start a decode-only plan, or take over the launch made ahead for it."""
        manager = self.core.manager
        entries = plan.entries  # type: ignore[attr-defined]
        ids = tuple(entry.request_id for entry in entries)
        held = [manager.held(request_id) for request_id in ids]
        positions = [h.committed for h in held]
        ahead, self._ahead = self._ahead, None
        if ahead is not None:
            pick = ahead.covers(ids, positions, rows)
            if pick is not None:
                self.adopted += 1
                ahead.pick = pick
                ahead.exact = pick == list(range(ahead.count))
                return ahead
            # The plan is not the one foreseen. What the launch stored in the cache is what
            # this step stores again (or lies in pages that were given back); only its
            # buffers have to be free before they are filled anew.
            ahead.event.synchronize()
            self.dropped += 1
        tokens = [entry.tokens[0] for entry in entries]
        return self._launch(ids, [h.row for h in held], positions, rows, tokens, None)

    def launch_ahead(self, after: _Launch, rows: list[SampleRow]) -> None:
        """Start the step that follows ``after`` before ``after``'s tokens have reached the
        host: same requests in the same rows, one position on, each row fed the id the
        earlier launch chose, copied on the device. The caller has made room for the next
        position of every request. :meth:`launch` hands the result to the next plan if that
        plan turns out as foreseen, and drops it otherwise."""
        if not after.exact or self._ahead is not None:
            raise RuntimeError("a launch ahead follows a launch whose rows are all live")
        manager = self.core.manager
        table_rows = [manager.held(request_id).row for request_id in after.ids]
        self._ahead = self._launch(after.ids, table_rows,
                                   [position + 1 for position in after.positions], rows,
                                   None, after)

    def drop_ahead(self) -> None:
        """Forget a launch made ahead (waits for it: its buffers are filled anew later)."""
        ahead, self._ahead = self._ahead, None
        if ahead is not None:
            ahead.event.synchronize()
            self.dropped += 1

    def finish(self, launch: _Launch) -> list[int]:
        """Wait for a launch and return the chosen id of each of its plan's entries; raises
        :class:`BackendError` if a kernel up to and including this launch gave up."""
        launch.event.synchronize()
        self.flags.check(launch.slot)
        chosen = launch.out_host.tolist()
        return [chosen[index] for index in launch.pick]

    def _launch(self, ids: tuple[str, ...], table_rows: list[int], positions: list[int],
                rows: list[SampleRow], tokens: list[int] | None,
                after: _Launch | None) -> _Launch:
        count = len(ids)
        bucket = self.bucket_for(count)
        if after is not None and after.bucket is not bucket:
            raise RuntimeError("a launch ahead stays in the bucket of the launch before it")
        slot = bucket.turn
        bucket.turn ^= 1
        staging = bucket.staging[slot]
        self._fill(bucket, staging, table_rows, positions, rows, tokens)
        bucket.meta.copy_(staging, non_blocking=True)
        if after is not None:
            bucket.meta[bucket.o_tokens:bucket.o_tokens + count].copy_(
                bucket.out[:count], non_blocking=True)
        greedy = all(row.params.greedy for row in rows)
        if greedy not in bucket.graphs:
            self._capture(bucket, greedy)  # (runs the step it captures: the same stores)
        bucket.graphs[greedy].replay()
        bucket.out_host[slot].copy_(bucket.out, non_blocking=True)
        self.flags.snapshot(slot)
        event = bucket.events[slot]
        event.record(torch.cuda.current_stream(self.core.device))
        self.replays += 1
        return _Launch(bucket, ids, positions, rows, bucket.out_host[slot], event, slot)

    def _capture(self, bucket: _Bucket, greedy: bool) -> None:
        core = self.core
        with torch.cuda.device(core.device):
            # twice without capture: allocates the workspace, builds and configures kernels
            side = torch.cuda.Stream(core.device)
            side.wait_stream(torch.cuda.current_stream(core.device))
            with torch.cuda.stream(side):
                bucket.launch_body(core, greedy)
                bucket.launch_body(core, greedy)
            torch.cuda.current_stream(core.device).wait_stream(side)
            torch.cuda.synchronize(core.device)
            graph = torch.cuda.CUDAGraph()
            before = ops.launch_count()
            with torch.cuda.graph(graph):
                bucket.launch_body(core, greedy)
            bucket.kernels = ops.launch_count() - before
            bucket.graphs[greedy] = graph

    def _fill(self, bucket: _Bucket, staging: torch.Tensor, table_rows: list[int],
              positions_of: list[int], rows: list[SampleRow], tokens: list[int] | None) -> None:
        manager = self.core.manager
        size, width, page = bucket.size, bucket.width, manager.page_size
        host = staging.numpy()
        floats = host.view(np.float32)
        count = len(table_rows)
        host[bucket.o_request:bucket.o_request + size] = -1
        host[bucket.o_tokens:bucket.o_tokens + size] = 0
        host[bucket.o_positions:bucket.o_positions + size] = 0
        host[bucket.o_kv_len:bucket.o_kv_len + size] = 0
        host[bucket.o_want:bucket.o_want + size] = np.arange(size)
        host[bucket.o_row_start:bucket.o_row_start + size + 1] = np.arange(size + 1)
        floats[bucket.o_temperature:bucket.o_temperature + size] = 0.0
        slots = np.asarray(table_rows, dtype=np.int32)
        positions = np.asarray(positions_of, dtype=np.int32)
        if tokens is not None:
            host[bucket.o_tokens:bucket.o_tokens + count] = tokens
        host[bucket.o_positions:bucket.o_positions + count] = positions
        host[bucket.o_request:bucket.o_request + count] = np.arange(count)
        host[bucket.o_kv_len:bucket.o_kv_len + count] = positions + 1
        host[bucket.o_state:bucket.o_state + count] = slots
        live = np.arange(count)
        for group, (o_slots, o_table) in enumerate(bucket.o_groups):
            host[o_slots:o_slots + size] = -1
            block = host[o_table:o_table + size * width].reshape(size, width)
            block[:count] = manager.tables[group][slots]
            host[o_slots:o_slots + count] = (block[live, positions // page] * page
                                             + positions % page)
        longs_seed = host[bucket.o_seeds:bucket.o_seeds + 2 * size].view(np.int64)
        longs_pos = host[bucket.o_sample_positions:
                         bucket.o_sample_positions + 2 * size].view(np.int64)
        longs_seed[:] = 0
        longs_pos[:] = 0
        for b, row in enumerate(rows):
            params = row.params
            floats[bucket.o_temperature + b] = 0.0 if params.greedy else params.temperature
            floats[bucket.o_top_p + b] = params.top_p
            floats[bucket.o_min_p + b] = params.min_p
            host[bucket.o_top_k + b] = max(params.top_k, 0)
            longs_seed[b] = row.seed
            longs_pos[b] = row.position
