"""What kernels report back without failing: two int32 words per device.

Word 0 is the *status word*: a kernel whose bounded wait ran out (an mbarrier that never
completed within its limit) writes its refusal code there, skips its stores and returns
normally, so the context stays usable. Word 1 is set to 1 by the embedding kernel when an id
lies outside its table. Both are sticky until the host clears them. The step function reads
them where it synchronises anyway (with the chosen ids), so a step whose kernels gave up
fails as a step instead of delivering tokens made from stale activations; the reference turns
a backend's refusal into a step error the same way (``python/ayaka/execution/runner.py:227-231``).
"""

from __future__ import annotations

from collections.abc import Sequence

import torch

from ayaka_b200.errors import BackendError

__all__ = ["FlagReader", "bad_index", "device_flags", "failure", "status_word"]

STATUS, BAD_INDEX, WORDS = 0, 1, 2
_flags: dict[int, torch.Tensor] = {}


def device_flags(device: torch.device) -> torch.Tensor:
    """The device's two words (int32 ``[2]``), created zeroed on first use."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    words = _flags.get(index)
    if words is None:
        words = torch.zeros(WORDS, dtype=torch.int32, device=torch.device("cuda", index))
        _flags[index] = words
    return words


_status_views: dict[int | None, torch.Tensor] = {}


def status_word(device: torch.device) -> torch.Tensor:
    """One int32 that a kernel sets when a bounded wait ran out (the same view every call:
    hundreds of launches a step ask for it)."""
    view = _status_views.get(device.index)
    if view is None:
        view = device_flags(device)[STATUS:STATUS + 1]
        _status_views[device.index] = view
    return view


def bad_index(device: torch.device) -> torch.Tensor:
    """One int32 that the embedding kernel sets when an id is outside its table."""
    return device_flags(device)[BAD_INDEX:BAD_INDEX + 1]


def failure(values: Sequence[int]) -> str | None:
    """What a host copy of the two words says went wrong, or ``None``."""
    status, bad = int(values[STATUS]), int(values[BAD_INDEX])
    if status:
        return (f"a kernel gave up a bounded wait (status {status}); it skipped its stores, "
                "so the step's activations are not to be trusted")
    if bad:
        return "a token or position id was outside its embedding table"
    return None


class FlagReader:
    """Copies the words to pinned host memory beside a step's result and checks the copy.

    ``snapshot`` queues an 8-byte device-to-host copy on the current stream and costs no
    synchronisation; ``check`` is called once the stream (or an event recorded after the
    snapshot) has been waited for. Two slots, because two decode steps may be in flight.
    """

    def __init__(self, device: torch.device, flags: torch.Tensor | None = None) -> None:
        self.device = device
        self.flags = device_flags(device) if flags is None else flags
        pin = self.flags.is_cuda
        self.host = [torch.zeros(WORDS, dtype=torch.int32) for _ in range(2)]
        if pin:
            self.host = [buffer.pin_memory() for buffer in self.host]

    def snapshot(self, slot: int = 0) -> None:
        self.host[slot].copy_(self.flags, non_blocking=True)

    def check(self, slot: int = 0) -> None:
        """Raise :class:`BackendError` if the snapshot shows a failure; the words are cleared
        so that the next step starts clean."""
        values = self.host[slot].tolist()
        what = failure(values)
        if what is not None:
            self.flags.zero_()
            for buffer in self.host:
                buffer.zero_()
            raise BackendError(what, context={"status": values[STATUS],
                                              "bad_index": values[BAD_INDEX]})

    def read_now(self) -> None:
        """Synchronising read and check (the replay program and tests)."""
        self.snapshot(0)
        if self.flags.is_cuda:
            torch.cuda.current_stream(self.device).synchronize()
        self.check(0)
