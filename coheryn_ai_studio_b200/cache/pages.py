"""Host-side bookkeeping of cache pages and of per-request state slots.

A :class:`PagePool` owns ``num_pages`` page ids.  Every page is either free or held
with a reference count >= 1 (more than one holder when requests share a prefix).  A
page that was filled completely and carries a content hash stays findable after its
last holder lets go of it: it waits in a least-recently-used list and is only wiped
when the pool has no plain free page left.  Freed pages are handed out again last-in
first-out, so reuse happens at once (and stale contents would show in tests).
"""
from __future__ import annotations

from collections import OrderedDict
from typing import Dict, List, Optional


class CacheError(RuntimeError):
    """A bookkeeping invariant was broken (double free, unknown page or slot)."""


class PagePool:
    def __init__(self, num_pages: int):
        if num_pages < 0:
            raise ValueError("a pool cannot have a negative number of pages")
        self.num_pages = num_pages
        self._free: List[int] = list(range(num_pages - 1, -1, -1))   # stack; page 0 first out
        self._refs: List[int] = [0] * num_pages
        self._hash_of: Dict[int, bytes] = {}            # page -> content hash
        self._page_of: Dict[bytes, int] = {}            # content hash -> page
        self._idle: "OrderedDict[int, None]" = OrderedDict()   # hashed pages with no holder, LRU first

    # ---- queries
    @property
    def available(self) -> int:
        """Pages that an allocation can get right now (free + idle hashed pages)."""
        return len(self._free) + len(self._idle)

    def refcount(self, page: int) -> int:
        return self._refs[page]

    # ---- allocation
    def allocate(self, n: int) -> Optional[List[int]]:
        """n pages with reference count 1, or None (and no change) if fewer are available."""
        if n < 0:
            raise ValueError("cannot allocate a negative number of pages")
        if n > self.available:
            return None
        out = []
        for _ in range(n):
            if self._free:
                p = self._free.pop()
            else:
                p, _ = self._idle.popitem(last=False)    # evict the least recently used
                self._forget(p)
            self._refs[p] = 1
            out.append(p)
        return out

    def retain(self, page: int) -> None:
        """One more holder of a page (a shared prefix); revives an idle hashed page."""
        self._known(page)
        if self._refs[page] == 0:
            if page not in self._idle:
                raise CacheError(f"page {page} is free and cannot be retained")
            del self._idle[page]
        self._refs[page] += 1

    def release(self, page: int) -> None:
        self._known(page)
        if self._refs[page] <= 0:
            raise CacheError(f"page {page} is released but nobody holds it")
        self._refs[page] -= 1
        if self._refs[page] == 0:
            if page in self._hash_of:
                self._idle[page] = None
            else:
                self._free.append(page)

    # ---- content hashes (prefix reuse)
    def set_hash(self, page: int, digest: bytes) -> None:
        """Record that ``page`` holds the full block identified by ``digest``.  If
        another page already carries that digest the record stays with the older one."""
        self._known(page)
        if self._refs[page] <= 0:
            raise CacheError(f"page {page} is not held")
        if digest in self._page_of or page in self._hash_of:
            return
        self._hash_of[page] = digest
        self._page_of[digest] = page

    def lookup(self, digest: bytes) -> Optional[int]:
        return self._page_of.get(digest)

    def _forget(self, page: int) -> None:
        d = self._hash_of.pop(page, None)
        if d is not None:
            self._page_of.pop(d, None)

    def drop_hashes(self) -> None:
        """Forget every content hash (idle pages become plain free pages)."""
        for p in list(self._idle):
            self._free.append(p)
        self._idle.clear()
        self._hash_of.clear()
        self._page_of.clear()

    def _known(self, page: int) -> None:
        if not 0 <= page < self.num_pages:
            raise CacheError(f"page {page} is not in the pool (0..{self.num_pages - 1})")

    # ---- invariants
    def check(self, held: Optional[Dict[int, int]] = None) -> None:
        """Every page is in exactly one place; with ``held`` (page -> number of holders as
        the caller counts them) the reference counts must agree."""
        seen = [0] * self.num_pages
        for p in self._free:
            seen[p] += 1
        for p in self._idle:
            seen[p] += 1
        for p in range(self.num_pages):
            if self._refs[p] < 0:
                raise CacheError(f"page {p} has a negative reference count")
            if self._refs[p] > 0:
                seen[p] += 1
            if seen[p] != 1:
                raise CacheError(f"page {p} is in {seen[p]} places (free / idle / held)")
            if p in self._idle and p not in self._hash_of:
                raise CacheError(f"idle page {p} has no hash")
        if held is not None:
            for p in range(self.num_pages):
                if self._refs[p] != held.get(p, 0):
                    raise CacheError(f"page {p}: pool counts {self._refs[p]} holders, "
                                     f"requests hold it {held.get(p, 0)} times")


class SlotPool:
    """Slots for per-request state of fixed size."""

    def __init__(self, num_slots: int):
        self.num_slots = num_slots
        self._free = list(range(num_slots - 1, -1, -1))
        self._used = set()

    @property
    def available(self) -> int:
        return len(self._free)

    def allocate(self) -> Optional[int]:
        if not self._free:
            return None
        s = self._free.pop()
        self._used.add(s)
        return s

    def release(self, slot: int) -> None:
        if slot not in self._used:
            raise CacheError(f"slot {slot} is released but not in use")
        self._used.remove(slot)
        self._free.append(slot)

    def check(self) -> None:
        if len(self._free) + len(self._used) != self.num_slots or self._used & set(self._free):
            raise CacheError("slot pool lost or duplicated a slot")
