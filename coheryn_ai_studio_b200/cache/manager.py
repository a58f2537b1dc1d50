"""The cache manager: keys and values in pages with a block table per request, one pool
per group of layers with the same needs, and slots for per-request state of fixed size.

Schedule entries whose mixers ask for the same :class:`PagedKV` (kv heads, head size,
window) form a group: they share page ids and block tables, and each has its own slice
of the group's pool ``[entry, K/V, page, kv head, slot in page, head_dim]``.  A group
with a window gives a page back as soon as every later query lies past it; a finished
request gives everything back.  Full, hashed pages of groups without a window can be
found again by a later request with the same token prefix (the reference hands a whole
session's keys and values to the next request with a common prefix, capped at
prompt_len - 1 so the last prompt token is always recomputed:
crates/coheryn-engine/src/inference/generation.rs:189-202; here the unit is a page).
Prefix reuse is switched off when any group has a window or any mixer keeps fixed
state, because those cannot be rebuilt from pages alone.

The books (which request holds which page in which group, what is reserved and what
committed, the hash chain of full pages, the pages a window has passed, the state slots) are
kept by the native host runtime (``csrc/host_engine.cpp``: ``CacheBook``, over the pools of
``csrc/host_pools.h``).  This class owns the device tensors and is the book's Python face; the
scheduler's native planner works on the same book.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..parts.base import FixedState, LayerCache, PagedKV
from .pages import CacheError, PagePool, SlotPool, host

_ALREADY, _NO_SLOT, _UNKNOWN, _UNCOMMITTED, _NOT_ENOUGH = 6, 7, 8, 9, 4


@dataclass
class _Group:
    need: PagedKV
    entries: List[int]                   # schedule entries that own a slice
    pool: Optional[PagePool] = None      # a face on the book's pool of this group
    tensor: Optional[torch.Tensor] = None


class _Requests:
    """The live requests as the book knows them: ``id in requests``, ``len(requests)``, truth."""

    def __init__(self, manager: "CacheManager"):
        self._m = manager

    def __contains__(self, req_id) -> bool:
        return bool(self._m._lib.coheryn_book_has(self._m._book, str(req_id).encode()))

    def __len__(self) -> int:
        return int(self._m._lib.coheryn_book_count(self._m._book))

    def __bool__(self) -> bool:
        return len(self) > 0


def _ints(values: Sequence[int]):
    n = len(values)
    return (ctypes.c_int * max(n, 1))(*[int(v) for v in values]), n


class CacheManager:
    def __init__(self, requirements: Sequence, cache_from: Sequence[Optional[int]], dtype: torch.dtype,
                 device, page_size: int = 16, num_pages: int = 0, max_requests: int = 64,
                 prefix_reuse: bool = True):
        if page_size < 1:
            raise ValueError("page_size must be positive")
        self.page_size, self.num_pages, self.max_requests = page_size, num_pages, max_requests
        self.dtype, self.device = dtype, device
        self.groups: List[_Group] = []
        self._entry_group: List[Optional[Tuple[int, int]]] = [None] * len(requirements)
        self._state: Dict[int, torch.Tensor] = {}
        self._cache_from = list(cache_from)
        for e, need in enumerate(requirements):
            if need is None:
                continue
            if isinstance(need, PagedKV):
                for gi, g in enumerate(self.groups):
                    if g.need == need:
                        self._entry_group[e] = (gi, len(g.entries))
                        g.entries.append(e)
                        break
                else:
                    self.groups.append(_Group(need, [e]))
                    self._entry_group[e] = (len(self.groups) - 1, 0)
            elif isinstance(need, FixedState):
                self._state[e] = torch.zeros((max_requests,) + tuple(need.shape), dtype=need.dtype,
                                             device=device)
            else:
                raise TypeError(f"schedule entry {e}: unknown cache requirement {need!r}")
        # One page more than the pool hands out: page ``num_pages`` belongs to no request and takes
        # the writes of padding rows (a decode batch padded up to a captured width).
        for g in self.groups:
            n = g.need
            g.tensor = torch.zeros((len(g.entries), 2, num_pages + 1, n.num_kv_heads, page_size, n.head_dim),
                                   dtype=dtype, device=device)
        reuse = bool(prefix_reuse) and not self._state and all(g.need.window is None for g in self.groups)
        self._lib = host()
        windows, n_groups = _ints([g.need.window or 0 for g in self.groups])
        self._book = self._lib.coheryn_book_new(page_size, num_pages, max_requests, 1 if reuse else 0, n_groups, windows)
        if not self._book:
            raise CacheError("the native cache book could not be made")
        for gi, g in enumerate(self.groups):
            g.pool = PagePool.borrowed(self._lib.coheryn_book_pool(self._book, gi), num_pages, keep_alive=self)
        self.slots = SlotPool.borrowed(self._lib.coheryn_book_slots(self._book), max_requests, keep_alive=self)
        self.requests = _Requests(self)

    def __del__(self):
        book, self._book = getattr(self, "_book", None), None
        if book:
            self._lib.coheryn_book_delete(book)

    @property
    def book_handle(self):
        """The native book, for the planner that schedules over it."""
        return self._book

    @property
    def prefix_reuse(self) -> bool:
        return bool(self._lib.coheryn_book_prefix_reuse(self._book))

    # ------------------------------------------------------------------ views for the model
    def layer_caches(self) -> List[Optional[LayerCache]]:
        out: List[Optional[LayerCache]] = []
        for e in range(len(self._entry_group)):
            src = self._cache_from[e]
            owner = e if src is None else src
            if owner in self._state:
                out.append(LayerCache(kind="state", state=self._state[owner], writes=src is None))
            elif self._entry_group[owner] is not None:
                gi, idx = self._entry_group[owner]
                g = self.groups[gi]
                out.append(LayerCache(kind="paged", group=gi, page_size=self.page_size,
                                      k=g.tensor[idx, 0], v=g.tensor[idx, 1], writes=src is None))
            else:
                out.append(None)
        return out

    @property
    def spare_page(self) -> int:
        """Index of the page that no request owns (see the constructor)."""
        return self.num_pages

    @property
    def has_fixed_state(self) -> bool:
        return bool(self._state)

    def state_tensors(self) -> List[torch.Tensor]:
        """The fixed-state pools ([slots, *shape] each), for a caller that must put them back as
        they were (the warm-up runs before a CUDA-graph capture)."""
        return list(self._state.values())

    def bytes_per_token(self) -> int:
        item = torch.empty((), dtype=self.dtype).element_size()
        return sum(2 * len(g.entries) * g.need.num_kv_heads * g.need.head_dim * item for g in self.groups)

    # ------------------------------------------------------------------ requests
    def _key(self, req_id) -> bytes:
        return str(req_id).encode()

    def _number(self, req_id, what: int) -> int:
        v = int(self._lib.coheryn_book_number(self._book, self._key(req_id), what))
        if v < 0:
            raise KeyError(req_id)
        return v

    def zero_state(self, req_id) -> None:
        """A request starts from zero state: called for every admission (also those the native
        planner makes)."""
        if self._state:
            slot = self.state_slot(req_id)
            for st in self._state.values():
                st[slot].zero_()

    def admit(self, req_id: str, prompt: Optional[Sequence[int]] = None) -> Optional[int]:
        """Give the request a state slot (zeroed) and, when a prompt is given and prefix
        reuse is on, map the leading full pages that are already cached.  Returns the
        number of prompt tokens reused, or None when no slot is free."""
        reused, slot, serial = ctypes.c_int(0), ctypes.c_int(-1), ctypes.c_longlong(0)
        if prompt is None:
            arr, n = None, -1
        else:
            arr, n = _ints(prompt)
        rc = self._lib.coheryn_book_admit(self._book, self._key(req_id), arr, n, ctypes.byref(reused),
                                          ctypes.byref(slot), ctypes.byref(serial))
        if rc == _ALREADY:
            raise CacheError(f"request {req_id!r} is already admitted")
        if rc == _NO_SLOT:
            return None
        if rc:
            raise CacheError(f"cache book: status {rc} while request {req_id!r} is admitted")
        self.zero_state(req_id)
        return reused.value

    def length(self, req_id: str) -> int:
        return self._number(req_id, 0)

    def pages_needed(self, req_id: str, n: int) -> List[int]:
        out = (ctypes.c_int * max(len(self.groups), 1))()
        if self._lib.coheryn_book_pages_needed(self._book, self._key(req_id), int(n), out):
            raise KeyError(req_id)
        return list(out[:len(self.groups)])

    def can_reserve(self, req_id: str, n: int) -> bool:
        return all(need <= avail for need, avail in zip(self.pages_needed(req_id, n), self.available_pages()))

    def reserve(self, req_id: str, tokens: Sequence[int]) -> bool:
        """Pages for ``tokens`` after what the request already holds.  All groups or none:
        returns False and changes nothing when any pool is short."""
        arr, n = _ints(tokens)
        rc = self._lib.coheryn_book_reserve(self._book, self._key(req_id), arr, n)
        if rc == _NOT_ENOUGH:
            return False
        if rc == _UNCOMMITTED:
            raise CacheError(f"request {req_id!r} has a reservation that was not committed")
        if rc == _UNKNOWN:
            raise KeyError(req_id)
        if rc:
            raise CacheError(f"cache book: status {rc} while pages are reserved for {req_id!r}")
        return True

    def slot_ids(self, req_id: str, group: int) -> List[int]:
        """Cache slot (page * page_size + offset) of every reserved, uncommitted token."""
        n = self._number(req_id, 1) - self._number(req_id, 0)
        out = (ctypes.c_int * max(n, 1))()
        if self._lib.coheryn_book_slot_ids(self._book, self._key(req_id), group, out, n) < 0:
            raise KeyError(req_id)
        return list(out[:n])

    def block_table(self, req_id: str, group: int) -> List[int]:
        cap = -(-max(self._number(req_id, 1), 1) // self.page_size) + 1
        out = (ctypes.c_int * cap)()
        n = self._lib.coheryn_book_table(self._book, self._key(req_id), group, out, cap)
        if n < 0:
            raise KeyError(req_id)
        if n > cap:
            out = (ctypes.c_int * n)()
            self._lib.coheryn_book_table(self._book, self._key(req_id), group, out, n)
        return list(out[:n])

    def state_slot(self, req_id: str) -> int:
        return self._number(req_id, 2)

    def serial(self, req_id: str) -> int:
        """A number unique to this admission of the request."""
        return self._number(req_id, 5)

    def commit(self, req_id: str) -> None:
        """The reserved tokens' keys and values are written: advance the length, hash the
        pages that became full, give back the pages a window has passed."""
        if self._lib.coheryn_book_commit(self._book, self._key(req_id)):
            raise KeyError(req_id)

    def mark_unknown(self, req_id: str, index: int) -> None:
        """Token ``index`` of the request was reserved with a placeholder id: the step that runs
        it was launched before the id was read back.  Pages holding it are not hashed until
        ``patch_token`` supplies the id."""
        if self._lib.coheryn_book_mark_unknown(self._book, self._key(req_id), int(index)):
            raise KeyError(req_id)

    def patch_token(self, req_id: str, index: int, token: int) -> None:
        rc = self._lib.coheryn_book_patch_token(self._book, self._key(req_id), int(index), int(token))
        if rc == _UNKNOWN:
            raise KeyError(req_id)
        if rc:
            raise IndexError(f"request {req_id!r} holds no token {index}")

    def rollback(self, req_id: str) -> None:
        """Drop a reservation that was not committed (pages beyond the committed length
        go back)."""
        if self._lib.coheryn_book_rollback(self._book, self._key(req_id)):
            raise KeyError(req_id)

    def free(self, req_id: str) -> None:
        if self._lib.coheryn_book_free(self._book, self._key(req_id)):
            raise CacheError(f"request {req_id!r} is not admitted")

    def available_pages(self) -> List[int]:
        out = (ctypes.c_int * max(len(self.groups), 1))()
        self._lib.coheryn_book_available(self._book, out)
        return list(out[:len(self.groups)])

    def check(self) -> None:
        """No page lost, held twice or freed twice; no slot lost."""
        group, page, info = ctypes.c_int(-1), ctypes.c_int(-1), ctypes.c_int(0)
        rc = self._lib.coheryn_book_check(self._book, ctypes.byref(group), ctypes.byref(page), ctypes.byref(info))
        if rc == 0:
            return
        g, p = group.value, page.value
        raise CacheError({
            1: f"group {g}: page {p} has a negative reference count",
            2: f"group {g}: page {p} is in {info.value} places (free / idle / held)",
            3: f"group {g}: idle page {p} has no hash",
            4: f"group {g}: page {p}: the pool counts {info.value} holders, the requests hold it otherwise",
            5: "slot pool lost or duplicated a slot",
            6: "two requests share a state slot"}.get(rc, f"cache book: check returned {rc}"))
