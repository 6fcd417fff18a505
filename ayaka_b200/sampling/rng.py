"""The random numbers of sampling, on the host: seeds and the Philox reference.

A draw is a pure function of ``(seed, position)``: ``u = (philox4x32_10((pos_lo, pos_hi,
stream, sequence), (seed_lo, seed_hi))[0] >> 8) / 2**24`` with ``position`` the index, in
prompt plus output, of the token being produced (the reference's scheme,
``python/ayaka/ops/sampling.py:25-39``, ``python/ayaka/sampling/rng.py:29-117``). Nothing
advances, so how requests are batched or cut cannot change a draw. The kernel computes the
same function on the device; this module serves seeds and tests.
"""

from __future__ import annotations

import hashlib

from ayaka_b200.sampling.params import MAX_SEED

__all__ = ["draw_uniform", "philox4x32_10", "resolve_seed"]

_WORD = 0xFFFFFFFF


def philox4x32_10(counter: tuple[int, int, int, int],
                  key: tuple[int, int]) -> tuple[int, int, int, int]:
    """Philox-4x32 with 10 rounds (Salmon et al., SC11) on Python integers."""
    c0, c1, c2, c3 = counter
    k0, k1 = key
    for index in range(10):
        if index:
            k0 = (k0 + 0x9E3779B9) & _WORD
            k1 = (k1 + 0xBB67AE85) & _WORD
        low, high = 0xD2511F53 * c0, 0xCD9E8D57 * c2
        c0, c1, c2, c3 = (high >> 32) ^ c1 ^ k0, high & _WORD, (low >> 32) ^ c3 ^ k1, low & _WORD
    return c0, c1, c2, c3


def draw_uniform(seed: int, position: int) -> float:
    """The number in [0, 1) that picks the token at ``position`` for ``seed``."""
    words = philox4x32_10((position & _WORD, position >> 32, 0, 0), (seed & _WORD, seed >> 32))
    return (words[0] >> 8) / float(1 << 24)


def resolve_seed(request_id: str, seed: int | None) -> int:
    """The seed a request samples with: the caller's, or one derived from the request id by
    blake2b so that it is the same in every process."""
    if seed is not None:
        return seed
    digest = hashlib.blake2b(request_id.encode("utf-8"), digest_size=8).digest()
    return int.from_bytes(digest, "big") & MAX_SEED
