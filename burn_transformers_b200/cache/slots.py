"""Pools of integer handles (slots, pages).  The books are kept by the host library (csrc/host/page_book.cpp);
no tensor lives here, so it runs anywhere."""
from __future__ import annotations

from ..errors import CacheError
from . import native


class FreeList:
    """A pool of integer handles.  A handle is held by at most one owner and freed at most once."""

    def __init__(self, count: int, what: str):
        self.what = what
        self.count = count
        self._lib = native.library()
        self._pool = self._lib.bth_pool_create(count, what.encode())
        if not self._pool:
            raise native.error()

    def __del__(self):
        pool, self._pool = getattr(self, "_pool", None), None
        if pool:
            self._lib.bth_pool_destroy(pool)

    @property
    def free(self) -> int:
        return self._lib.bth_pool_free(self._pool)

    @property
    def held(self) -> int:
        return self.count - self.free

    def take(self) -> int:
        handle = self._lib.bth_pool_take(self._pool)
        if handle < 0:
            raise native.error()
        return handle

    def take_many(self, n: int) -> list[int]:
        if n > self.free:
            raise CacheError(f"{n} {self.what}s needed, {self.free} of {self.count} free")
        return [self.take() for _ in range(n)]

    def give_back(self, handle: int) -> None:
        if self._lib.bth_pool_give_back(self._pool, int(handle)) < 0:
            raise native.error()

    def is_held(self, handle: int) -> bool:
        return bool(self._lib.bth_pool_is_held(self._pool, int(handle)))

    def check(self) -> None:
        """Every handle is either free or held, none twice."""
        if self._lib.bth_pool_check(self._pool) < 0:
            raise native.error()
