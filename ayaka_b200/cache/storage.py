"""The cache's device tensors, and the plan that groups a model's runs by what they need.

Layout of a group's keys (and, separately, values):
``[cache slot, page, kv_head, token in page, head_dim]``. One cache slot per run of the
execution order that writes a cache; a run that reads another run's cache shares its slot.
All of one head's tokens in a page are contiguous (``page_size * head_dim`` elements), so an
attention kernel fetches a head's page in one bulk copy.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ayaka_b200.errors import ConfigError
from ayaka_b200.parts.base import CacheNeed, StateNeed
from ayaka_b200.parts.context import LayerCache
from ayaka_b200.parts.spec import Run

__all__ = ["CachePlan", "CacheStorage", "plan_cache"]


@dataclass(frozen=True, slots=True)
class CachePlan:
    """Which group and cache slot every run of the order uses.

    Attributes:
        groups: the distinct needs, in order of first use.
        run_group: per run, its group index or ``None`` (a mixer without pages).
        run_slot: per run, its slot inside the group's tensors or ``None``.
        run_writes: per run, whether it writes that slot (``False`` for a reader).
        slots_per_group: cache slots each group's tensors hold.
        run_state: per run, the fixed-size state its mixer asks for, or ``None``.
    """

    groups: tuple[CacheNeed, ...]
    run_group: tuple[int | None, ...]
    run_slot: tuple[int | None, ...]
    run_writes: tuple[bool, ...]
    slots_per_group: tuple[int, ...]
    run_state: tuple[StateNeed | None, ...]

    def bytes_per_page(self, group: int, itemsize: int, page_size: int) -> int:
        need = self.groups[group]
        return (2 * self.slots_per_group[group] * need.num_kv_heads * page_size
                * need.head_dim * itemsize)

    def bytes_per_token(self, itemsize: int) -> int:
        """Key and value bytes one cached token takes over all groups (windows ignored)."""
        return sum(self.bytes_per_page(g, itemsize, 1) for g in range(len(self.groups)))


def plan_cache(order: tuple[Run, ...],
               needs: list[tuple[CacheNeed | None, StateNeed | None]]) -> CachePlan:
    groups: list[CacheNeed] = []
    slots: list[int] = []
    run_group: list[int | None] = []
    run_slot: list[int | None] = []
    run_writes: list[bool] = []
    for index, (run, (need, _)) in enumerate(zip(order, needs)):
        if need is None:
            run_group.append(None)
            run_slot.append(None)
            run_writes.append(False)
            continue
        if run.reads_cache_of is not None:
            owner = run.reads_cache_of
            if run_group[owner] is None or needs[owner][0] != need:
                raise ConfigError(
                    "model.order", "CACHE_MISMATCH",
                    f"run {index} reads the cache of run {owner}, whose geometry differs")
            run_group.append(run_group[owner])
            run_slot.append(run_slot[owner])
            run_writes.append(False)
            continue
        if need not in groups:
            groups.append(need)
            slots.append(0)
        group = groups.index(need)
        run_group.append(group)
        run_slot.append(slots[group])
        run_writes.append(True)
        slots[group] += 1
    return CachePlan(tuple(groups), tuple(run_group), tuple(run_slot), tuple(run_writes),
                     tuple(slots), tuple(state for _, state in needs))


class CacheStorage:
    """Keys, values and per-request state on the device, as the plan lays them out."""

    def __init__(self, plan: CachePlan, num_pages: list[int], page_size: int, max_requests: int,
                 dtype: torch.dtype, device: torch.device, poison: bool = False) -> None:
        self.plan = plan
        self.page_size = page_size
        self.keys: list[torch.Tensor] = []
        self.values: list[torch.Tensor] = []
        for need, slots, pages in zip(plan.groups, plan.slots_per_group, num_pages):
            shape = (slots, pages, need.num_kv_heads, page_size, need.head_dim)
            self.keys.append(torch.zeros(shape, dtype=dtype, device=device))
            self.values.append(torch.zeros(shape, dtype=dtype, device=device))
        if poison:
            self.poison()
        self.states: list[torch.Tensor | None] = [
            None if need is None else
            torch.zeros((max_requests, *need.shape), dtype=need.dtype, device=device)
            for need in plan.run_state]

    def poison(self) -> None:
        """Fill every page with NaN (tests: a slot read before it is written then shows)."""
        for tensor in (*self.keys, *self.values):
            tensor.fill_(float("nan"))

    def layer_caches(self) -> list[LayerCache]:
        """One :class:`LayerCache` per run of the order."""
        out = []
        for index, group in enumerate(self.plan.run_group):
            if group is None:
                out.append(LayerCache(None, None, None, False, self.states[index]))
            else:
                slot = self.plan.run_slot[index]
                out.append(LayerCache(group, self.keys[group][slot], self.values[group][slot],
                                      self.plan.run_writes[index], self.states[index]))
        return out

    def zero_state_rows(self, rows: list[int]) -> None:
        if not rows:
            return
        for state in self.states:
            if state is not None:
                state[rows] = 0

    def nbytes(self) -> int:
        total = sum(t.numel() * t.element_size() for t in (*self.keys, *self.values))
        return total + sum(t.numel() * t.element_size() for t in self.states if t is not None)
