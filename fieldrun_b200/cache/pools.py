"""Bookkeeping of what a cache hands out: sequence slots and pages of tokens.

Pure host code.  Both pools refuse to give out what is held and to take back
what is free, so a leak or a double free shows as an error at the place it
happens, not as a wrong logit later.
"""
from __future__ import annotations


class CacheFull(RuntimeError):
    """No free slot or page is left."""


class IndexPool:
    """Indices 0..n-1, each either free or held.  The lowest free index is given
    out first, so a freed index is used again by the next request."""

    def __init__(self, n: int, what: str):
        if n < 0:
            raise ValueError(f"a pool of {what}s cannot have {n} entries")
        self.n = n
        self.what = what
        self._held = [False] * n
        self._free = list(range(n - 1, -1, -1))       # a stack; the lowest index on top
        self._free_sorted = True

    def alloc(self) -> int:
        if not self._free:
            raise CacheFull(f"no free {self.what}: all {self.n} are held")
        if not self._free_sorted:
            self._free.sort(reverse=True)
            self._free_sorted = True
        index = self._free.pop()
        self._held[index] = True
        return index

    def free(self, index: int) -> None:
        if not 0 <= index < self.n:
            raise ValueError(f"{self.what} {index} does not exist (there are {self.n})")
        if not self._held[index]:
            raise ValueError(f"{self.what} {index} is freed twice (or was never given out)")
        self._held[index] = False
        self._free.append(index)
        self._free_sorted = False

    def is_held(self, index: int) -> bool:
        return 0 <= index < self.n and self._held[index]

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_held(self) -> int:
        return self.n - len(self._free)

    def held(self) -> list[int]:
        return [i for i, h in enumerate(self._held) if h]

    def check(self) -> None:
        """Every index is exactly free or held."""
        free = sorted(self._free)
        if len(set(free)) != len(free):
            raise AssertionError(f"a {self.what} is on the free list twice")
        for i in free:
            if self._held[i]:
                raise AssertionError(f"{self.what} {i} is both free and held")
        if len(free) + sum(self._held) != self.n:
            raise AssertionError(f"a {self.what} is lost: {len(free)} free + {sum(self._held)} held != {self.n}")
