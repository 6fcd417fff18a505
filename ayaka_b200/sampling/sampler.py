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
from ayaka_b200.kernels.flags import FlagReader
from ayaka_b200.sampling.params import SamplingParams

__all__ = ["SampleRow", "Sampler"]


@dataclass(frozen=True, slots=True)
class SampleRow:
    """One logits row's parameters: the request's, its seed, and the index in the sequence
    (prompt plus output) of the token this row produces. ``history`` (the prompt followed by
    the output, ``prompt_len`` tokens of it prompt) is needed only by penalties; ``banned``
    are the ids that cannot be chosen now (stop ids before ``min_tokens``)."""

    params: SamplingParams
    seed: int
    position: int
    history: Sequence[int] = ()
    prompt_len: int = 0
    banned: frozenset[int] = frozenset()

    @property
    def adjusts(self) -> bool:
        params = self.params
        return params.penalises or params.logit_bias is not None or \
            params.allowed_token_ids is not None or bool(self.banned)


class Sampler:
    def __init__(self, max_rows: int, device: torch.device,
                 flags: FlagReader | None = None) -> None:
        self.max_rows = max_rows
        self.device = device
        #: the kernels' failure words, copied beside the ids and checked after the wait
        self.flags = flags
        # layout of the staging buffer, in 4-byte words per row: temperature, top_p, min_p
        # (float32), top_k (int32), then seeds and positions (int64, two words each)
        self._host = torch.empty(8 * max_rows, dtype=torch.int32).pin_memory()
        self._dev = torch.zeros(8 * max_rows, dtype=torch.int32, device=device)
        self._out = torch.zeros(max_rows, dtype=torch.int32, device=device)
        self._out_host = torch.empty(max_rows, dtype=torch.int32).pin_memory()
        self._argmax_scratch = torch.zeros(2 * max_rows * ops.ARGMAX_PARTS, device=device)
        # descriptor and mask scratch of the logit adjustments, grown on demand
        self._adjust_host: torch.Tensor | None = None
        self._adjust_dev: torch.Tensor | None = None
        self._mask: torch.Tensor | None = None

    def _adjust(self, logits: torch.Tensor, rows: Sequence[SampleRow]) -> None:
        """Masks, biases and penalties of the rows that ask for them, in place, before the
        token is chosen (one descriptor, one copy, one kernel)."""
        picked = [(index, row) for index, row in enumerate(rows) if row.adjusts]
        if not picked:
            return
        words = ops.ADJUST_WORDS
        header = np.zeros((len(picked), words), dtype=np.int32)
        floats = header.view(np.float32)
        lists: list[np.ndarray] = []
        cursor = len(picked) * words
        masked = False

        def place(values: np.ndarray) -> int:
            nonlocal cursor
            offset = cursor
            lists.append(values)
            cursor += values.shape[0]
            return offset

        for slot, (index, row) in enumerate(picked):
            params = row.params
            history = np.asarray(row.history if params.penalises else (), dtype=np.int32)
            header[slot, 0] = index
            header[slot, 1] = place(history)
            header[slot, 2] = history.shape[0]
            header[slot, 3] = min(row.prompt_len, history.shape[0])
            bias = params.logit_bias or ()
            header[slot, 4] = place(np.asarray([token for token, _ in bias], dtype=np.int32))
            header[slot, 5] = len(bias)
            place(np.asarray([value for _, value in bias], dtype=np.float32).view(np.int32))
            if params.allowed_token_ids is None:
                header[slot, 6], header[slot, 7] = 0, -1
            else:
                allowed = np.asarray(sorted(params.allowed_token_ids), dtype=np.int32)
                header[slot, 6], header[slot, 7] = place(allowed), allowed.shape[0]
                masked = True
            banned = np.asarray(sorted(row.banned), dtype=np.int32)
            header[slot, 8], header[slot, 9] = place(banned), banned.shape[0]
            floats[slot, 10] = params.repetition_penalty
            floats[slot, 11] = params.frequency_penalty
            floats[slot, 12] = params.presence_penalty
        packed = np.concatenate([header.reshape(-1)] + lists)
        if self._adjust_host is None or self._adjust_host.shape[0] < packed.shape[0]:
            size = max(4096, 2 * packed.shape[0])
            self._adjust_host = torch.empty(size, dtype=torch.int32).pin_memory()
            self._adjust_dev = torch.zeros(size, dtype=torch.int32, device=self.device)
        assert self._adjust_dev is not None
        self._adjust_host.numpy()[:packed.shape[0]] = packed
        self._adjust_dev[:packed.shape[0]].copy_(self._adjust_host[:packed.shape[0]],
                                                 non_blocking=True)
        mask = None
        if masked:
            need = len(picked) * ((logits.shape[1] + 31) // 32)
            if self._mask is None or self._mask.shape[0] < need:
                self._mask = torch.zeros(need, dtype=torch.int32, device=self.device)
            mask = self._mask
        ops.logits_adjust(logits, self._adjust_dev, len(picked), mask)

    def sample(self, logits: torch.Tensor, rows: Sequence[SampleRow]) -> list[int]:
        """Pick one token per row of ``logits`` (``[len(rows), vocab]`` fp32)."""
        count = len(rows)
        if count == 0:
            return []
        if count > self.max_rows or logits.shape[0] < count:
            raise ValueError("more rows than the sampler was built for")
        self._adjust(logits, rows)
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
        if self.flags is not None:
            self.flags.snapshot(0)
        torch.cuda.current_stream(self.device).synchronize()
        if self.flags is not None:
            self.flags.check(0)  # raises BackendError: the ids of a failed step are not used
        return self._out_host[:count].tolist()
