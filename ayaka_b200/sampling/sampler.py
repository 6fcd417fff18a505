"""From logits rows to token ids: the per-step batch of sampling parameters and the launch.

A step whose rows are all greedy takes the argmax kernel; any other step takes the sampling
kernel, which handles greedy rows too (``python/ayaka/sampling/sampler.py:46-117`` has the
same short path). Parameters travel in one pinned buffer and one copy; the sampled ids come
back in the step's only device-to-host read."""

from __future__ import annotations

from collections.abc import Sequence
from dataclasses import dataclass

import numpy as np
import torch

from ayaka_b200.kernels import ops
from ayaka_b200.sampling.params import SamplingParams

__all__ = ["SampleRow", "Sampler"]


@dataclass(frozen=True, slots=True)
class SampleRow:
    """One logits row's parameters: the request's, its seed, and the index in the sequence
    (prompt plus output) of the token this row produces."""

    params: SamplingParams
    seed: int
    position: int


class Sampler:
    def __init__(self, max_rows: int, device: torch.device) -> None:
        self.max_rows = max_rows
        self.device = device
        # layout of the staging buffer, in 4-byte words per row: temperature, top_p, min_p
        # (float32), top_k (int32), then seeds and positions (int64, two words each)
        self._host = torch.empty(8 * max_rows, dtype=torch.int32).pin_memory()
        self._dev = torch.zeros(8 * max_rows, dtype=torch.int32, device=device)
        self._out = torch.zeros(max_rows, dtype=torch.int32, device=device)
        self._out_host = torch.empty(max_rows, dtype=torch.int32).pin_memory()
        self._argmax_scratch = torch.zeros(2 * max_rows * ops.ARGMAX_PARTS, device=device)

    def sample(self, logits: torch.Tensor, rows: Sequence[SampleRow]) -> list[int]:
        """Pick one token per row of ``logits`` (``[len(rows), vocab]`` fp32)."""
        count = len(rows)
        if count == 0:
            return []
        if count > self.max_rows or logits.shape[0] < count:
            raise ValueError("more rows than the sampler was built for")
        if all(row.params.greedy for row in rows):
            ops.argmax(logits, self._out, rows=count, scratch=self._argmax_scratch)
        else:
            n = self.max_rows
            host = self._host.numpy()
            floats = host.view(np.float32)
            longs = host[4 * n:].view(np.int64)
            for index, row in enumerate(rows):
                params = row.params
                floats[index] = 0.0 if params.greedy else params.temperature
                floats[n + index] = params.top_p
                floats[2 * n + index] = params.min_p
                host[3 * n + index] = max(params.top_k, 0)
                longs[index] = row.seed
                longs[n + index] = row.position
            self._dev.copy_(self._host, non_blocking=True)
            dev = self._dev
            ops.sample(logits, dev[:n].view(torch.float32), dev[3 * n:4 * n],
                       dev[n:2 * n].view(torch.float32), dev[2 * n:3 * n].view(torch.float32),
                       dev[4 * n:6 * n].view(torch.int64), dev[6 * n:8 * n].view(torch.int64),
                       self._out, rows=count)
        self._out_host[:count].copy_(self._out[:count], non_blocking=True)
        torch.cuda.current_stream(self.device).synchronize()
        return self._out_host[:count].tolist()
