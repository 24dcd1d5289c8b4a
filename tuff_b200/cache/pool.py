"""A pool of numbered units (pages or slots) with a free list.

Units freed last are handed out first, so a small pool reuses its units at
once.  The pool refuses to free a unit that is not held (freed twice, or never
given out) and to give out more than it has.
"""
from __future__ import annotations

from typing import List


class OutOfPages(RuntimeError):
    """The pool cannot cover what was asked; nothing was taken."""


class PoolError(RuntimeError):
    """Misuse of the pool: a unit freed twice or one the pool never gave out."""


class UnitPool:
    def __init__(self, n_units: int, what: str = "page"):
        if n_units < 0:
            raise ValueError("a pool cannot have a negative size")
        self.n_units, self.what = int(n_units), what
        self._free: List[int] = list(range(self.n_units - 1, -1, -1))   # pop() hands out 0 first
        self._held = [False] * self.n_units

    @property
    def n_free(self) -> int:
        return len(self._free)

    @property
    def n_held(self) -> int:
        return self.n_units - len(self._free)

    def take(self, n: int = 1) -> List[int]:
        if n > len(self._free):
            raise OutOfPages(f"{n} {self.what}(s) wanted, {len(self._free)} of {self.n_units} free")
        out = [self._free.pop() for _ in range(n)]
        for u in out:
            self._held[u] = True
        return out

    def give_back(self, unit: int) -> None:
        if not 0 <= unit < self.n_units:
            raise PoolError(f"{self.what} {unit} is not of this pool (0..{self.n_units - 1})")
        if not self._held[unit]:
            raise PoolError(f"{self.what} {unit} freed twice or never taken")
        self._held[unit] = False
        self._free.append(unit)

    def held_units(self) -> List[int]:
        return [u for u in range(self.n_units) if self._held[u]]

    def check(self) -> None:
        """Raises if the free list and the held flags disagree (no unit lost or held twice)."""
        free = sorted(self._free)
        if len(set(free)) != len(free):
            raise PoolError(f"a {self.what} is on the free list twice")
        if any(self._held[u] for u in free):
            raise PoolError(f"a free {self.what} is marked held")
        if len(free) + sum(self._held) != self.n_units:
            raise PoolError(f"{self.what}s lost: {len(free)} free + {sum(self._held)} held != {self.n_units}")
