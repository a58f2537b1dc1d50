"""Host-side bookkeeping of cache pages and of per-request state slots.

A :class:`PagePool` owns ``num_pages`` page ids.  Every page is either free or held
with a reference count >= 1 (more than one holder when requests share a prefix).  A
page that was filled completely and carries a content hash stays findable after its
last holder lets go of it: it waits in a least-recently-used list and is only wiped
when the pool has no plain free page left.  Freed pages are handed out again last-in
first-out, so reuse happens at once (and stale contents would show in tests).

The books themselves are kept by the native host runtime (``csrc/host_pages.cpp``, plain
C++ behind a C interface); the classes here own a handle and turn its status codes into
exceptions.
"""
from __future__ import annotations

import ctypes
from typing import Dict, List, Optional

from ..csrc import build


class CacheError(RuntimeError):
    """A bookkeeping invariant was broken (double free, unknown page or slot)."""


_lib = None


def _host():
    global _lib
    if _lib is None:
        lib = build.host_library()
        lib.coheryn_pool_new.restype = ctypes.c_void_p
        lib.coheryn_pool_new.argtypes = [ctypes.c_int]
        lib.coheryn_slots_new.restype = ctypes.c_void_p
        lib.coheryn_slots_new.argtypes = [ctypes.c_int]
        for name in ("coheryn_pool_delete", "coheryn_slots_delete", "coheryn_pool_drop_hashes"):
            getattr(lib, name).restype = None
            getattr(lib, name).argtypes = [ctypes.c_void_p]
        for name in ("coheryn_pool_available", "coheryn_slots_available", "coheryn_slots_acquire"):
            getattr(lib, name).argtypes = [ctypes.c_void_p]
        for name in ("coheryn_pool_refcount", "coheryn_pool_retain", "coheryn_pool_release",
                     "coheryn_slots_release", "coheryn_slots_held"):
            getattr(lib, name).argtypes = [ctypes.c_void_p, ctypes.c_int]
        lib.coheryn_pool_allocate.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.POINTER(ctypes.c_int)]
        lib.coheryn_pool_set_hash.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_char_p, ctypes.c_int]
        lib.coheryn_pool_lookup.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_int]
        lib.coheryn_pool_check.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int),
                                           ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int)]
        P, I, L = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
        IP, S = ctypes.POINTER(ctypes.c_int), ctypes.c_char_p
        sig = {
            "coheryn_book_new": (P, [I, I, I, I, I, IP]), "coheryn_book_delete": (None, [P]),
            "coheryn_book_prefix_reuse": (I, [P]), "coheryn_book_set_prefix_reuse": (None, [P, I]),
            "coheryn_book_pool": (P, [P, I]), "coheryn_book_slots": (P, [P]), "coheryn_book_count": (I, [P]),
            "coheryn_book_has": (I, [P, S]), "coheryn_book_admit": (I, [P, S, IP, I, IP, IP, ctypes.POINTER(L)]),
            "coheryn_book_number": (L, [P, S, I]), "coheryn_book_pages_needed": (I, [P, S, I, IP]),
            "coheryn_book_reserve": (I, [P, S, IP, I]), "coheryn_book_commit": (I, [P, S]),
            "coheryn_book_rollback": (I, [P, S]), "coheryn_book_free": (I, [P, S]),
            "coheryn_book_mark_unknown": (I, [P, S, I]), "coheryn_book_patch_token": (I, [P, S, I, I]),
            "coheryn_book_table": (I, [P, S, I, IP, I]), "coheryn_book_slot_ids": (I, [P, S, I, IP, I]),
            "coheryn_book_available": (None, [P, IP]), "coheryn_book_check": (I, [P, IP, IP, IP]),
            "coheryn_book_tables": (I, [P, I, ctypes.POINTER(S), I, IP, I, IP]),
            "coheryn_book_layout": (I, [P, I, ctypes.POINTER(S), IP, IP, IP, I, IP, IP, IP, ctypes.POINTER(L)]),
            "coheryn_planner_new": (P, [P, I, I, I]), "coheryn_planner_delete": (None, [P]),
            "coheryn_planner_max_seqs": (I, [P]),
            "coheryn_planner_add": (I, [P, S, IP, I, I, IP, I, I, IP]),
            "coheryn_planner_adopt": (I, [P, S, IP, I, I, I, IP]), "coheryn_planner_has_work": (I, [P]),
            "coheryn_planner_schedule": (I, [P]), "coheryn_planner_lookahead": (I, [P, I, IP, IP, IP]),
            "coheryn_planner_plan": (I, [P, IP, IP, IP, IP, I]), "coheryn_planner_list": (I, [P, I, IP, I]),
            "coheryn_planner_tokens": (I, [P, I, I, I, IP]), "coheryn_planner_job": (L, [P, I, I]),
            "coheryn_planner_set_computed": (None, [P, I, I]), "coheryn_planner_advance": (None, [P, I, IP, IP]),
            "coheryn_planner_append_token": (I, [P, I, I]), "coheryn_planner_finish": (I, [P, I, I]),
            "coheryn_planner_stats": (None, [P, ctypes.POINTER(L)]),
        }
        for name, (res, args) in sig.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


def host():
    """The native host runtime with every entry point declared."""
    return _host()


UNKNOWN_PAGE, NOT_HELD, FREE_PAGE, NOT_ENOUGH, BAD_ARGUMENT = 1, 2, 3, 4, 5


class PagePool:
    def __init__(self, num_pages: int):
        if num_pages < 0:
            raise ValueError("a pool cannot have a negative number of pages")
        self.num_pages = num_pages
        self._lib = _host()
        self._owned = True
        self._h = self._lib.coheryn_pool_new(num_pages)
        if not self._h:
            raise CacheError("the native page pool could not be made")

    @classmethod
    def borrowed(cls, handle, num_pages: int, keep_alive=None) -> "PagePool":
        """A face on a pool that someone else owns (a group's pool inside the cache book)."""
        self = cls.__new__(cls)
        self.num_pages, self._lib, self._h, self._owned, self._keep = num_pages, _host(), handle, False, keep_alive
        return self

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h and getattr(self, "_owned", False):
            self._lib.coheryn_pool_delete(h)

    def _fail(self, code: int, page: int, doing: str):
        if code == UNKNOWN_PAGE:
            raise CacheError(f"page {page} is not in the pool (0..{self.num_pages - 1})")
        if code == NOT_HELD:
            raise CacheError(f"page {page} is {doing} but nobody holds it")
        if code == FREE_PAGE:
            raise CacheError(f"page {page} is free and cannot be retained")
        raise CacheError(f"page pool: status {code} while page {page} is {doing}")

    # ---- queries
    @property
    def available(self) -> int:
        """Pages that an allocation can get right now (free + idle hashed pages)."""
        return self._lib.coheryn_pool_available(self._h)

    def refcount(self, page: int) -> int:
        r = self._lib.coheryn_pool_refcount(self._h, page)
        if r < 0:
            self._fail(UNKNOWN_PAGE, page, "asked for")
        return r

    # ---- allocation
    def allocate(self, n: int) -> Optional[List[int]]:
        """n pages with reference count 1, or None (and no change) if fewer are available."""
        if n < 0:
            raise ValueError("cannot allocate a negative number of pages")
        out = (ctypes.c_int * max(n, 1))()
        code = self._lib.coheryn_pool_allocate(self._h, n, out)
        if code == NOT_ENOUGH:
            return None
        if code:
            raise CacheError(f"page pool: status {code} while {n} pages are allocated")
        return list(out[:n])

    def retain(self, page: int) -> None:
        """One more holder of a page (a shared prefix); revives an idle hashed page."""
        code = self._lib.coheryn_pool_retain(self._h, page)
        if code:
            self._fail(code, page, "retained")

    def release(self, page: int) -> None:
        code = self._lib.coheryn_pool_release(self._h, page)
        if code:
            self._fail(code, page, "released")

    # ---- content hashes (prefix reuse)
    def set_hash(self, page: int, digest: bytes) -> None:
        """Record that ``page`` holds the full block identified by ``digest``.  If
        another page already carries that digest the record stays with the older one."""
        code = self._lib.coheryn_pool_set_hash(self._h, page, digest, len(digest))
        if code == NOT_HELD:
            raise CacheError(f"page {page} is not held")
        if code:
            self._fail(code, page, "given a hash")

    def lookup(self, digest: bytes) -> Optional[int]:
        page = self._lib.coheryn_pool_lookup(self._h, digest, len(digest))
        return None if page < 0 else page

    def drop_hashes(self) -> None:
        """Forget every content hash (idle pages become plain free pages)."""
        self._lib.coheryn_pool_drop_hashes(self._h)

    # ---- invariants
    def check(self, held: Optional[Dict[int, int]] = None) -> None:
        """Every page is in exactly one place; with ``held`` (page -> number of holders as
        the caller counts them) the reference counts must agree."""
        counts = None
        if held is not None:
            counts = (ctypes.c_int * max(self.num_pages, 1))()
            for page, n in held.items():
                if not 0 <= page < self.num_pages:
                    raise CacheError(f"page {page} is not in the pool (0..{self.num_pages - 1})")
                counts[page] = n
        bad, info = ctypes.c_int(-1), ctypes.c_int(0)
        code = self._lib.coheryn_pool_check(self._h, counts, ctypes.byref(bad), ctypes.byref(info))
        p = bad.value
        if code == 1:
            raise CacheError(f"page {p} has a negative reference count")
        if code == 2:
            raise CacheError(f"page {p} is in {info.value} places (free / idle / held)")
        if code == 3:
            raise CacheError(f"idle page {p} has no hash")
        if code == 4:
            raise CacheError(f"page {p}: pool counts {info.value} holders, "
                             f"requests hold it {held.get(p, 0)} times")
        if code:
            raise CacheError(f"page pool: check returned {code}")


class SlotPool:
    """Slots for per-request state of fixed size."""

    def __init__(self, num_slots: int):
        if num_slots < 0:
            raise ValueError("a pool cannot have a negative number of slots")
        self.num_slots = num_slots
        self._lib = _host()
        self._owned = True
        self._h = self._lib.coheryn_slots_new(num_slots)
        if not self._h:
            raise CacheError("the native slot pool could not be made")

    @classmethod
    def borrowed(cls, handle, num_slots: int, keep_alive=None) -> "SlotPool":
        self = cls.__new__(cls)
        self.num_slots, self._lib, self._h, self._owned, self._keep = num_slots, _host(), handle, False, keep_alive
        return self

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h and getattr(self, "_owned", False):
            self._lib.coheryn_slots_delete(h)

    @property
    def available(self) -> int:
        return self._lib.coheryn_slots_available(self._h)

    def allocate(self) -> Optional[int]:
        s = self._lib.coheryn_slots_acquire(self._h)
        return None if s < 0 else s

    def release(self, slot: int) -> None:
        if self._lib.coheryn_slots_release(self._h, slot):
            raise CacheError(f"slot {slot} is released but not in use")

    def check(self) -> None:
        held = sum(1 for s in range(self.num_slots) if self._lib.coheryn_slots_held(self._h, s) == 1)
        if held + self.available != self.num_slots:
            raise CacheError("slot pool lost or duplicated a slot")
