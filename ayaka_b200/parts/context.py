"""What a part sees of one step: the batch's metadata, its cache, and scratch buffers.

Rows of all requests in a step are concatenated in request order. ``request_of_row[i]`` is
the batch index of row ``i``'s request (also its row of every ``block_table``);
``positions[i]`` its index in its sequence. ``kv_len[b]`` counts request ``b``'s tokens
*after* this step, as in the reference's metadata (``python/ayaka/ops/attention.py:61-95``).
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch

__all__ = ["GroupStep", "LayerCache", "StepContext", "Workspace"]


class Workspace:
    """Scratch activations that live as long as the runner: fixed addresses, no allocation
    after the first step that needs a buffer. Buffers are named; layers run one after the
    other, so every layer uses the same ones."""

    def __init__(self, max_rows: int, device: torch.device) -> None:
        self.max_rows = max_rows
        self.device = device
        self._buffers: dict[tuple[str, int, torch.dtype], torch.Tensor] = {}
        # a buffer that had to grow is kept: a captured graph may still hold its address
        self._retired: list[torch.Tensor] = []

    def buffer(self, name: str, width: int, dtype: torch.dtype,
               rows: int | None = None) -> torch.Tensor:
        """A ``[max_rows (or rows), width]`` tensor; the same tensor at every call."""
        key = (name, width, dtype)
        found = self._buffers.get(key)
        want = self.max_rows if rows is None else rows
        if found is None or found.shape[0] < want:
            if found is not None:
                self._retired.append(found)
            found = torch.zeros((want, width), dtype=dtype, device=self.device)
            self._buffers[key] = found
        return found

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self._buffers.values())


@dataclass(slots=True)
class GroupStep:
    """One cache group's view of the step."""

    block_table: torch.Tensor  # int32 [B, pages_per_request]; 0 = no page
    slot_mapping: torch.Tensor  # int32 [N]; page * page_size + slot, negative = store nothing
    page_size: int


@dataclass(slots=True)
class LayerCache:
    """What one run of a layer may touch of the cache."""

    group: int | None  # index into StepContext.groups, None when the mixer has no pages
    k_pages: torch.Tensor | None  # [pages, kv_heads, page_size, head_dim]
    v_pages: torch.Tensor | None
    writes: bool  # False when this run reads the cache another run wrote
    state: torch.Tensor | None = None  # [max_requests, *StateNeed.shape]


@dataclass(slots=True)
class StepContext:
    """One step's batch, on the device and (the small lists) on the host."""

    num_rows: int
    num_requests: int
    tokens: torch.Tensor  # int32 [>= N]
    positions: torch.Tensor  # int32 [>= N]
    request_of_row: torch.Tensor  # int32 [>= N]
    row_start: torch.Tensor  # int32 [>= B + 1]; rows of request b are row_start[b]..row_start[b+1]
    kv_len: torch.Tensor  # int32 [>= B]
    state_slot: torch.Tensor  # int32 [>= B]; the request's row of every per-request state tensor
    host_rows: list[int]
    host_start: list[int]  # position of each request's first row in this step
    host_state_slot: list[int]
    groups: list[GroupStep]
    workspace: Workspace
    bad_index: torch.Tensor  # one int32 the embedding sets on an id outside its table
    max_kv_len: int = 0
    decode_only: bool = False
    extra: dict[str, object] = field(default_factory=dict)
