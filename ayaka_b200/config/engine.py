"""What to load and how to run it: the engine's own configuration.

Field names and defaults follow the reference's ``CacheConfig`` / ``SchedulerConfig`` /
``DeviceConfig`` (``python/ayaka/configs/cache.py:53-57``, ``configs/scheduler.py:54-58``,
``configs/device.py:61-65``) where it has them: page (``block_size``) 16, 2048 tokens a
step, 1024 waiting requests, a memory ratio of 0.9. Cross-field checks are those of
``python/ayaka/configs/engine.py:92-107``.
"""

from __future__ import annotations

from dataclasses import dataclass

from ayaka_b200.errors import ConfigError

__all__ = ["DTYPE_NAMES", "EngineConfig"]

#: spellings of ``--dtype`` -> canonical name
DTYPE_NAMES = {
    "bf16": "bfloat16", "bfloat16": "bfloat16",
    "fp32": "float32", "float32": "float32",
}


@dataclass(frozen=True, slots=True)
class EngineConfig:
    """One engine: a model folder, a dtype, the cache's size and the scheduler's limits.

    Attributes:
        model: folder with ``config.json`` and ``model.safetensors``.
        dtype: ``bfloat16`` (serving kernels) or ``float32`` (everything in true 32-bit).
        device: the CUDA device, ``cuda`` or ``cuda:N``.
        block_size: tokens per cache page.
        num_blocks: pages per pool (page 0 is padding), or ``None`` to size the pool from
            ``kv_reserve_tokens`` or ``memory_ratio``.
        memory_ratio: share of the free device memory the cache may take when nothing
            else sizes it.
        kv_reserve_tokens: tokens the cache must hold in total; ``None`` means
            ``max_running`` full contexts (bounded by ``memory_ratio``).
        max_running: most requests live at once (rows of the block table).
        max_tokens_per_step: token budget of one step.
        max_waiting: longest queue of requests not yet admitted.
        cuda_graph: replay decode-only steps from CUDA graphs.
        decode_ahead: with ``cuda_graph``, launch the next decode step while the tokens of
            the current one are still on their way to the host (the device feeds them
            on); the launch is dropped if the next plan turns out otherwise.
    """

    model: str
    dtype: str = "float32"
    device: str = "cuda"
    block_size: int = 16
    num_blocks: int | None = None
    memory_ratio: float = 0.90
    kv_reserve_tokens: int | None = None
    max_running: int = 8
    max_tokens_per_step: int = 2048
    max_waiting: int = 1024
    cuda_graph: bool = False
    decode_ahead: bool = True

    def __post_init__(self) -> None:
        if self.dtype not in DTYPE_NAMES:
            raise ConfigError("engine.dtype", "INVALID_CHOICE",
                              f"must be one of {sorted(DTYPE_NAMES)}, got {self.dtype!r}")
        object.__setattr__(self, "dtype", DTYPE_NAMES[self.dtype])
        if not (self.device == "cuda" or self.device.startswith("cuda:")):
            raise ConfigError("engine.device", "INVALID_CHOICE",
                              f"this engine runs on CUDA devices only, got {self.device!r}")
        for name, minimum in (("block_size", 1), ("max_running", 1), ("max_tokens_per_step", 1),
                              ("max_waiting", 1)):
            value = getattr(self, name)
            if type(value) is not int or value < minimum:
                raise ConfigError(f"engine.{name}", "INVALID_RANGE",
                                  f"must be an integer >= {minimum}, got {value!r}")
        if not 0.0 < float(self.memory_ratio) <= 1.0:
            raise ConfigError("engine.memory_ratio", "INVALID_RANGE",
                              f"must be in (0, 1], got {self.memory_ratio}")
        if self.kv_reserve_tokens is not None and (
                type(self.kv_reserve_tokens) is not int or self.kv_reserve_tokens < 1):
            raise ConfigError("engine.kv_reserve_tokens", "INVALID_RANGE", "must be >= 1")
        if self.num_blocks is not None:
            if type(self.num_blocks) is not int or self.num_blocks < 2:
                raise ConfigError("engine.num_blocks", "NUM_BLOCKS_TOO_SMALL",
                                  f"must be >= 2 (page 0 is padding), got {self.num_blocks!r}")
            if self.max_running > self.num_blocks - 1:
                raise ConfigError(
                    "engine.max_running", "RUNNING_EXCEEDS_BLOCKS",
                    f"{self.max_running} running requests need a page each, but "
                    f"num_blocks={self.num_blocks} leaves {self.num_blocks - 1}")
        if self.max_tokens_per_step < self.block_size:
            raise ConfigError(
                "engine.max_tokens_per_step", "STEP_SMALLER_THAN_BLOCK",
                f"a step of {self.max_tokens_per_step} tokens cannot fill one page of "
                f"{self.block_size}")
