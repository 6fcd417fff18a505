"""Building an engine from a configuration, and the loop-free core the replay program and
the scheduler share: model, cache manager, cache storage, step function."""

from __future__ import annotations

from collections.abc import Mapping, Sequence
from pathlib import Path

import torch

from ayaka_b200.cache.manager import CacheManager
from ayaka_b200.cache.storage import CacheStorage, plan_cache
from ayaka_b200.config.engine import EngineConfig
from ayaka_b200.errors import BackendError, CapacityError
from ayaka_b200.engine.runner import ModelRunner, StepEntry
from ayaka_b200.models import load_model
from ayaka_b200.models.decoder import DecoderModel

__all__ = ["EngineCore"]

_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


class EngineCore:
    """A loaded model with its cache and step function on one CUDA device.

    ``step`` is the whole of what happens between a request's tokens and its logits:
    allocate pages, run the batch, commit. The scheduler calls ``allocate`` / ``runner.run``
    / ``commit`` itself because it decides what to do when pages run out.
    """

    def __init__(self, model: DecoderModel, model_config: object, *, dtype: str,
                 device: torch.device, block_size: int, num_blocks: int, max_running: int,
                 max_tokens_per_step: int, poison_cache: bool = False) -> None:
        self.model = model
        self.model_config = model_config
        self.dtype = dtype
        self.device = device
        spec = model.spec
        self.cache_plan = plan_cache(spec.order, model.needs())
        groups = len(self.cache_plan.groups)
        pages_per_request = -(-spec.max_positions // block_size)
        self.manager = CacheManager(list(self.cache_plan.groups), [num_blocks] * groups,
                                    block_size, max_running, pages_per_request)
        self.storage = CacheStorage(self.cache_plan, [num_blocks] * groups, block_size,
                                    max_running, _DTYPES[dtype], device, poison=poison_cache)
        self.runner = ModelRunner(model, self.manager, self.storage, max_tokens_per_step, device)

    @classmethod
    def from_config(cls, config: EngineConfig,
                    tensors: Mapping[str, torch.Tensor] | None = None,
                    poison_cache: bool = False) -> EngineCore:
        """Load ``config.model`` and size the cache.

        The page count is ``num_blocks`` if given; else enough pages for
        ``kv_reserve_tokens`` tokens (each request may waste part of a page) or, when that
        is absent too, for ``max_running`` full contexts, bounded by ``memory_ratio`` of the
        device memory that is free after the weights are loaded.
        """
        if not torch.cuda.is_available():
            raise BackendError("no CUDA device is available; this engine has no CPU path")
        device = torch.device(config.device if ":" in config.device else "cuda:0")
        torch.cuda.set_device(device)
        model, model_config = load_model(Path(config.model), config.dtype, device, tensors)
        spec = model.spec
        plan = plan_cache(spec.order, model.needs())
        itemsize = 4 if config.dtype == "float32" else 2
        num_blocks = config.num_blocks
        if num_blocks is None:
            wanted_tokens = config.kv_reserve_tokens or config.max_running * spec.max_positions
            num_blocks = -(-wanted_tokens // config.block_size) + config.max_running + 1
            per_page = sum(plan.bytes_per_page(g, itemsize, config.block_size)
                           for g in range(len(plan.groups)))
            free, _ = torch.cuda.mem_get_info(device)
            affordable = int(free * config.memory_ratio) // max(per_page, 1)
            if affordable < 2:
                raise CapacityError("the device has no memory left for a single cache page")
            if config.kv_reserve_tokens and affordable < num_blocks:
                raise CapacityError(
                    f"{config.kv_reserve_tokens} cache tokens need {num_blocks} pages, the "
                    f"device has room for {affordable}")
            num_blocks = min(num_blocks, affordable)
        return cls(model, model_config, dtype=config.dtype, device=device,
                   block_size=config.block_size, num_blocks=num_blocks,
                   max_running=config.max_running,
                   max_tokens_per_step=config.max_tokens_per_step, poison_cache=poison_cache)

    # ------------------------------------------------------------------------------------
    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor | None:
        """Allocate, run and commit one batch; returns fp32 logits at the wanted places.

        Raises :class:`CapacityError` (and changes nothing) if the cache cannot hold the
        step's tokens."""
        started: list[str] = []
        for entry in entries:
            known = entry.request_id in self.manager
            if self.manager.allocate(entry.request_id, len(entry.tokens)):
                if not known:
                    started.append(entry.request_id)
            else:
                for request_id in started:
                    self.manager.free(request_id)
                raise CapacityError(
                    f"the cache has no room for {len(entry.tokens)} more tokens of request "
                    f"{entry.request_id!r} ({self.manager.num_free_pages()} pages free)")
        logits = self.runner.run(entries)
        for entry in entries:
            self.manager.commit(entry.request_id, len(entry.tokens))
        return logits

    def release(self, request_id: str) -> None:
        """Give back what a finished request holds."""
        self.manager.free(request_id)
