"""The step function: run one batch of (request, its next tokens) through the model.

A step carries, for every request in it, the next tokens of that request: a portion of its
prompt of any length or a single decoded token, any mix of the two across requests. Only
these tokens are computed; everything earlier comes from the cache. The step returns fp32
logits at the places the caller asks for. Rows are concatenated in the order of the entries
(the reference's conventions: ``python/ayaka/ops/attention.py:10-30``,
``python/ayaka/execution/inputs.py:244-301``); unlike the reference's scheduler-level steps
(``python/ayaka/scheduler/step.py:43-44``) a step here may mix prompt portions and decodes.

Metadata travels in one packed int32 buffer: filled on the host in pinned memory, sent with
one asynchronous copy, viewed on the device at fixed 16-byte aligned offsets.
"""

from __future__ import annotations

from collections.abc import Sequence
from dataclasses import dataclass

import numpy as np
import torch

from ayaka_b200.cache.manager import CacheManager
from ayaka_b200.cache.storage import CacheStorage
from ayaka_b200.errors import CapacityError, EngineError, InvalidRequestError
from ayaka_b200.kernels.flags import FlagReader
from ayaka_b200.models.decoder import DecoderModel
from ayaka_b200.parts.context import GroupStep, StepContext, Workspace

__all__ = ["ModelRunner", "StepEntry"]


@dataclass(frozen=True, slots=True)
class StepEntry:
    """One request's share of a step.

    Attributes:
        request_id: a request the cache manager has allocated ``len(tokens)`` tokens for.
        tokens: its next tokens, in order (at least one).
        want: indices into ``tokens`` whose logits the step returns (may be empty).
    """

    request_id: str
    tokens: Sequence[int]
    want: Sequence[int] = ()


def _align4(n: int) -> int:
    return (n + 3) & ~3


class ModelRunner:
    """Owns the workspace and the metadata buffers; turns entries into logits."""

    def __init__(self, model: DecoderModel, manager: CacheManager, storage: CacheStorage,
                 max_rows: int, device: torch.device) -> None:
        self.model = model
        self.manager = manager
        self.storage = storage
        self.max_rows = max_rows
        self.device = device
        self.workspace = Workspace(max_rows, device)
        self.caches = storage.layer_caches()
        groups = len(manager.needs)
        capacity = (_align4(max_rows) * (4 + groups) + 3 * _align4(manager.max_requests + 1)
                    + groups * _align4(manager.max_requests * manager.max_pages_per_request)
                    + 64)
        self._capacity = capacity
        # Two pinned buffers in turn. A step that returns no logits ends without waiting for
        # the device (a prompt cut into many portions: dozens of such steps in a row), so the
        # host may be several steps ahead of the copies it queued: before a buffer is filled
        # again, the copy that last read it must have run (an event per buffer).
        self._staging = [torch.empty(capacity, dtype=torch.int32).pin_memory() for _ in range(2)]
        self._staging_read: list[torch.cuda.Event | None] = [None, None]
        self._turn = 0
        self._device_meta = torch.zeros(capacity, dtype=torch.int32, device=device)
        #: the device's status word and bad-index word, read wherever a step synchronises
        self.flags = FlagReader(device)
        self._bad_index = self.flags.flags[1:2]
        self.steps_run = 0

    # ------------------------------------------------------------------------------------
    def run(self, entries: Sequence[StepEntry]) -> torch.Tensor | None:
        """Compute the step and return fp32 logits ``[wanted, vocab]`` in the order of the
        entries and of each ``want`` (a view of a persistent buffer, valid until the next
        step), or ``None`` when nothing is wanted. The caller commits afterwards."""
        step, want_rows, num_want = self.prepare(entries)
        if step.num_rows == 0:
            return None
        with torch.cuda.device(self.device):
            logits = self.model.forward(step, self.caches, want_rows, num_want)
        self.steps_run += 1
        return logits

    def check_device_flags(self) -> None:
        """Raise :class:`BackendError` if, since the last check, a kernel gave up a bounded
        wait or flagged an id outside its table (a synchronising read of two ints; the
        replay program and tests call it, generation reads the words with its token ids)."""
        self.flags.read_now()

    # ------------------------------------------------------------------------------------
    def prepare(self, entries: Sequence[StepEntry]) -> tuple[StepContext, torch.Tensor, int]:
        """Validate the entries and put the step's metadata on the device."""
        manager, spec = self.manager, self.model.spec
        num_requests = len(entries)
        if num_requests > manager.max_requests:
            raise CapacityError(f"a step of {num_requests} requests exceeds max_requests "
                                f"{manager.max_requests}")
        seen: set[str] = set()
        rows, starts, table_rows = [], [], []
        for entry in entries:
            if entry.request_id in seen:
                raise EngineError(f"request {entry.request_id!r} appears twice in one step")
            seen.add(entry.request_id)
            if entry.request_id not in manager:
                raise EngineError(f"request {entry.request_id!r} has no cache allocation")
            count = len(entry.tokens)
            if count < 1:
                raise InvalidRequestError(f"request {entry.request_id!r} brings no token")
            start = manager.committed(entry.request_id)
            if start + count > spec.max_positions:
                raise InvalidRequestError(
                    f"request {entry.request_id!r} would reach position {start + count - 1}, "
                    f"past the model's {spec.max_positions} positions")
            rows.append(count)
            starts.append(start)
            table_rows.append(manager.row(entry.request_id))
        total = sum(rows)
        if total > self.max_rows:
            raise CapacityError(f"a step of {total} tokens exceeds max_tokens_per_step "
                                f"{self.max_rows}")
        self.storage.zero_state_rows(manager.take_fresh_rows())

        page_size = manager.page_size
        turn = self._turn
        staging = self._staging[turn]
        self._turn ^= 1
        if self._staging_read[turn] is not None:
            self._staging_read[turn].synchronize()  # type: ignore[union-attr]
        host = staging.numpy()
        cursor = 0

        def segment(length: int) -> tuple[np.ndarray, int]:
            nonlocal cursor
            offset = cursor
            cursor += _align4(max(length, 1))
            return host[offset:offset + length], offset

        tokens, o_tokens = segment(total)
        positions, o_positions = segment(total)
        request_of_row, o_request = segment(total)
        row_start, o_row_start = segment(num_requests + 1)
        kv_len, o_kv_len = segment(num_requests)
        state_slot, o_state = segment(num_requests)
        want_total = sum(len(entry.want) for entry in entries)
        want_rows, o_want = segment(want_total)

        at = 0
        want_at = 0
        row_start[0] = 0
        for b, entry in enumerate(entries):
            count, start = rows[b], starts[b]
            ids = np.asarray(entry.tokens, dtype=np.int64)
            if ids.min() < 0 or ids.max() >= spec.vocab_size:
                raise InvalidRequestError(
                    f"request {entry.request_id!r} has a token id outside [0, "
                    f"{spec.vocab_size})")
            tokens[at:at + count] = ids
            positions[at:at + count] = np.arange(start, start + count, dtype=np.int32)
            request_of_row[at:at + count] = b
            for place in entry.want:
                if not 0 <= place < count:
                    raise InvalidRequestError(
                        f"request {entry.request_id!r} wants place {place} of {count} tokens")
                want_rows[want_at] = at + place
                want_at += 1
            at += count
            row_start[b + 1] = at
            kv_len[b] = start + count
            state_slot[b] = table_rows[b]
        max_kv_len = max((starts[b] + rows[b] for b in range(num_requests)), default=0)
        width = max(1, -(-max_kv_len // page_size))
        group_offsets = []
        for group in range(len(manager.needs)):
            table = manager.tables[group]
            slots, o_slots = segment(total)
            block, o_block = segment(num_requests * width)
            block2d = block.reshape(num_requests, width) if num_requests else block
            at = 0
            for b in range(num_requests):
                block2d[b] = table[table_rows[b], :width]
                pos = positions[at:at + rows[b]]
                pages = block2d[b][pos // page_size]
                if np.any(pages == 0):
                    raise EngineError(
                        f"request {entries[b].request_id!r} has no page for a position of "
                        "this step; allocate before running")
                slots[at:at + rows[b]] = pages * page_size + pos % page_size
                at += rows[b]
            group_offsets.append((o_slots, o_block))
        if cursor > self._capacity:
            raise CapacityError("the step's metadata exceeds its buffer")

        meta = self._device_meta
        meta[:cursor].copy_(staging[:cursor], non_blocking=True)
        if self._staging_read[turn] is None:
            self._staging_read[turn] = torch.cuda.Event()
        self._staging_read[turn].record(  # type: ignore[union-attr]
            torch.cuda.current_stream(self.device))

        def view(offset: int, length: int) -> torch.Tensor:
            return meta[offset:offset + max(length, 1)][:length] if length else \
                meta[offset:offset]

        groups = [GroupStep(block_table=view(o_block, num_requests * width).view(
                                num_requests, width),
                            slot_mapping=view(o_slots, total), page_size=page_size)
                  for o_slots, o_block in group_offsets]
        step = StepContext(
            num_rows=total, num_requests=num_requests,
            tokens=view(o_tokens, total), positions=view(o_positions, total),
            request_of_row=view(o_request, total),
            row_start=view(o_row_start, num_requests + 1), kv_len=view(o_kv_len, num_requests),
            state_slot=view(o_state, num_requests),
            host_rows=rows, host_start=starts, host_state_slot=table_rows,
            groups=groups, workspace=self.workspace, bad_index=self._bad_index,
            max_kv_len=max_kv_len, decode_only=all(count == 1 for count in rows),
        )
        return step, view(o_want, want_total), want_total
