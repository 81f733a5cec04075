"""Host-side bookkeeping of slots and pages.  No tensor lives here, so it runs anywhere."""
from __future__ import annotations

from ..errors import CacheError


class FreeList:
    """A pool of integer handles.  A handle is held by at most one owner and freed at most once."""

    def __init__(self, count: int, what: str):
        self.what = what
        self.count = count
        self._free = list(range(count - 1, -1, -1))   # pop() hands out 0 first
        self._held = [False] * count

    @property
    def free(self) -> int:
        return len(self._free)

    @property
    def held(self) -> int:
        return self.count - len(self._free)

    def take(self) -> int:
        if not self._free:
            raise CacheError(f"no free {self.what}: all {self.count} are in use")
        handle = self._free.pop()
        self._held[handle] = True
        return handle

    def take_many(self, n: int) -> list[int]:
        if n > len(self._free):
            raise CacheError(f"{n} {self.what}s needed, {len(self._free)} of {self.count} free")
        return [self.take() for _ in range(n)]

    def give_back(self, handle: int) -> None:
        if not (0 <= handle < self.count):
            raise CacheError(f"{self.what} {handle} does not exist")
        if not self._held[handle]:
            raise CacheError(f"{self.what} {handle} is not in use (freed twice?)")
        self._held[handle] = False
        self._free.append(handle)

    def is_held(self, handle: int) -> bool:
        return 0 <= handle < self.count and self._held[handle]

    def check(self) -> None:
        """Every handle is either free or held, none twice."""
        if sorted(self._free + [h for h in range(self.count) if self._held[h]]) != list(range(self.count)):
            raise CacheError(f"{self.what} bookkeeping is corrupt")
