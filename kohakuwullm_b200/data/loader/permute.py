"""Deterministic epoch shuffling without materialising a permutation.

``FeistelPermutation(n, key)`` is a bijection on ``[0, n)``: a 4-round Feistel network on the smallest
even-bit-width domain that covers ``n``, with cycle-walking to stay inside ``[0, n)``. Position ``i`` of
epoch ``e`` is ``perm(i)`` with ``key = splitmix64(seed, e)``, so any position of any epoch costs O(1)
and a resumed run needs only ``(epoch, cursor)``. ``ShardIndices`` gives rank/worker ``k`` of ``n`` the
strided positions ``k, k+n, ...``. ``is_validation`` is a hash split that does not depend on the epoch.
Reference: src/kohakuwullm/data/loader/permute.py:19-142.
"""

from __future__ import annotations

MASK64 = (1 << 64) - 1


def splitmix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & MASK64
    z = x
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & MASK64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & MASK64
    return z ^ (z >> 31)


def epoch_key(seed: int, epoch: int) -> int:
    return splitmix64(splitmix64(seed & MASK64) ^ (epoch & MASK64))


class FeistelPermutation:
    ROUNDS = 4

    def __init__(self, n: int, key: int):
        if n <= 0:
            raise ValueError("n must be positive")
        self.n = n
        bits = max(2, (n - 1).bit_length())
        bits += bits & 1
        self.half = bits // 2
        self.mask = (1 << self.half) - 1
        self.keys = [splitmix64(key + r) for r in range(self.ROUNDS)]

    def _encrypt(self, x: int) -> int:
        left, right = x >> self.half, x & self.mask
        for k in self.keys:
            left, right = right, left ^ (splitmix64(right ^ k) & self.mask)
        return (left << self.half) | right

    def __call__(self, i: int) -> int:
        if not 0 <= i < self.n:
            raise IndexError(i)
        x = self._encrypt(i)
        while x >= self.n:  # cycle-walk back into the domain
            x = self._encrypt(x)
        return x

    def __len__(self) -> int:
        return self.n


class ShardIndices:
    """Positions ``shard, shard + shards, ...`` of an ``n``-long (permuted) epoch."""

    def __init__(self, n: int, shard: int, shards: int, seed: int = 0, shuffle: bool = True):
        if not 0 <= shard < shards:
            raise ValueError(f"shard {shard} not in [0, {shards})")
        self.n, self.shard, self.shards, self.seed, self.shuffle = n, shard, shards, seed, shuffle

    def length(self) -> int:
        return (self.n - self.shard + self.shards - 1) // self.shards if self.n > self.shard else 0

    def index(self, epoch: int, cursor: int) -> int:
        pos = self.shard + cursor * self.shards
        if pos >= self.n:
            raise IndexError(cursor)
        if not self.shuffle:
            return pos
        return FeistelPermutation(self.n, epoch_key(self.seed, epoch))(pos)

    def iterate(self, epoch: int, start: int = 0):
        perm = FeistelPermutation(self.n, epoch_key(self.seed, epoch)) if self.shuffle else None
        for cursor in range(start, self.length()):
            pos = self.shard + cursor * self.shards
            yield cursor, (perm(pos) if perm else pos)


def is_validation(key: int | str, fraction: float, seed: int = 0) -> bool:
    """Epoch-independent hash split: the same record is always on the same side."""
    if isinstance(key, str):
        h = 0
        for ch in key.encode():
            h = splitmix64(h ^ ch)
        key = h
    return (splitmix64(key ^ splitmix64(seed)) >> 11) / float(1 << 53) < fraction
