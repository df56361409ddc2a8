"""Bookkeeping of what sequences hold: slots and pages, handed out and taken back.

Pure host code.  Both allocators refuse what would corrupt the cache later: freeing what is
not held, or holding more than there is.  `check()` verifies that nothing is lost or held
twice; the tests call it after every operation.
"""


class CacheError(RuntimeError):
    """The cache cannot do what was asked: no slot or page left, a slot used that is not held,
    a sequence longer than the position table."""


class FreeList:
    """`n` numbered things; `take()` hands out the lowest free number (so that reuse is easy to
    see in tests), `give(i)` takes it back."""

    def __init__(self, n, what):
        self.n, self.what = int(n), what
        self._free = list(range(self.n - 1, -1, -1))  # a stack whose top is the lowest number
        self._held = set()

    def available(self):
        return len(self._free)

    def held(self):
        return set(self._held)

    def take(self):
        if not self._free:
            raise CacheError(f"no free {self.what} (all {self.n} are held)")
        i = self._free.pop()
        self._held.add(i)
        return i

    def give(self, i):
        if i not in self._held:
            raise CacheError(f"{self.what} {i} is given back but is not held")
        self._held.remove(i)
        self._free.append(i)
        if len(self._free) > 1 and self._free[-2] < i:
            self._free.sort(reverse=True)

    def check(self):
        free = set(self._free)
        assert len(free) == len(self._free), f"a {self.what} is on the free list twice"
        assert not (free & self._held), f"a {self.what} is both free and held"
        assert free | self._held == set(range(self.n)), f"a {self.what} is lost"
