"""Free lists for sequence slots and for cache pages.

Both hand out small integers, take them back, and refuse what would corrupt the
cache: a slot or page held twice, freed twice, or never handed out. `check()`
verifies that held and free ids partition the range; the cache tests call it after
every operation.
"""
from __future__ import annotations

from typing import Iterable, List, Set

from ..errors import invalid_argument, runtime_error


class IdAllocator:
    def __init__(self, count: int, what: str):
        if count < 0:
            raise invalid_argument(f"cannot make {count} {what}s")
        self.count = count
        self.what = what
        # Lowest ids first on a fresh allocator; a freed id is the next one handed
        # out, so reuse happens at once and tests of reuse meet it.
        self._free: List[int] = list(range(count - 1, -1, -1))
        self._held: Set[int] = set()

    @property
    def free_count(self) -> int:
        return len(self._free)

    @property
    def held(self) -> Set[int]:
        return set(self._held)

    def acquire(self) -> int:
        if not self._free:
            raise runtime_error(f"no free {self.what} (all {self.count} are held)")
        item = self._free.pop()
        self._held.add(item)
        return item

    def acquire_many(self, count: int) -> List[int]:
        if count > len(self._free):
            raise runtime_error(f"need {count} free {self.what}s, {len(self._free)} of {self.count} are free")
        return [self.acquire() for _ in range(count)]

    def release(self, item: int) -> None:
        if not isinstance(item, int) or item < 0 or item >= self.count:
            raise invalid_argument(f"{self.what} {item!r} does not exist")
        if item not in self._held:
            raise invalid_argument(f"{self.what} {item} is not held (freed twice?)")
        self._held.remove(item)
        self._free.append(item)

    def release_many(self, items: Iterable[int]) -> None:
        for item in list(items):
            self.release(item)

    def is_held(self, item: int) -> bool:
        return item in self._held

    def check(self) -> None:
        free = set(self._free)
        if len(free) != len(self._free):
            raise runtime_error(f"a {self.what} is on the free list twice")
        if free & self._held:
            raise runtime_error(f"a {self.what} is both free and held")
        if free | self._held != set(range(self.count)):
            raise runtime_error(f"a {self.what} is lost")
