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
"""
from __future__ import annotations

import hashlib
import struct
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..parts.base import FixedState, LayerCache, PagedKV
from .pages import CacheError, PagePool, SlotPool


@dataclass
class _Group:
    need: PagedKV
    entries: List[int]                   # schedule entries that own a slice
    pool: PagePool
    tensor: Optional[torch.Tensor] = None


@dataclass
class _Request:
    slot: int
    serial: int = 0                      # unique per admission: tells a re-admitted id from the old one
    length: int = 0                      # tokens whose keys/values are committed
    tokens: List[int] = field(default_factory=list)    # committed + reserved token ids
    tables: List[List[int]] = field(default_factory=list)   # per group: page per block, -1 once given back
    unknown_at: Optional[int] = None     # index of a token whose id is not known yet (a step launched ahead)
    hashed_blocks: int = 0
    last_hash: bytes = b""
    reused: int = 0


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
                    self.groups.append(_Group(need, [e], PagePool(num_pages)))
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
        self.slots = SlotPool(max_requests)
        self.requests: Dict[str, _Request] = {}
        self._admissions = 0
        self.prefix_reuse = bool(prefix_reuse) and not self._state and all(
            g.need.window is None for g in self.groups)

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
    def _block_hash(self, prev: bytes, block_tokens: Sequence[int]) -> bytes:
        return hashlib.sha256(prev + struct.pack(f"<{len(block_tokens)}i", *block_tokens)).digest()

    def admit(self, req_id: str, prompt: Optional[Sequence[int]] = None) -> Optional[int]:
        """Give the request a state slot (zeroed) and, when a prompt is given and prefix
        reuse is on, map the leading full pages that are already cached.  Returns the
        number of prompt tokens reused, or None when no slot is free."""
        if req_id in self.requests:
            raise CacheError(f"request {req_id!r} is already admitted")
        slot = self.slots.allocate()
        if slot is None:
            return None
        for st in self._state.values():
            st[slot].zero_()
        self._admissions += 1
        r = _Request(slot=slot, serial=self._admissions, tables=[[] for _ in self.groups])
        self.requests[req_id] = r
        if prompt is not None and self.prefix_reuse and self.groups and len(prompt) > 1:
            limit = (len(prompt) - 1) // self.page_size
            h = b""
            found: List[List[int]] = []
            for b in range(limit):
                h = self._block_hash(h, prompt[b * self.page_size:(b + 1) * self.page_size])
                pages = [g.pool.lookup(h) for g in self.groups]
                if any(p is None for p in pages):
                    break
                found.append(pages)
                r.last_hash = h
            for pages in found:
                for gi, p in enumerate(pages):
                    self.groups[gi].pool.retain(p)
                    r.tables[gi].append(p)
            n = len(found) * self.page_size
            r.length = r.reused = n
            r.tokens = list(prompt[:n])
            r.hashed_blocks = len(found)
        return r.reused

    def length(self, req_id: str) -> int:
        return self.requests[req_id].length

    def _first_needed_block(self, g: _Group, next_position: int) -> int:
        if g.need.window is None:
            return 0
        return max(0, next_position - g.need.window + 1) // self.page_size

    def pages_needed(self, req_id: str, n: int) -> List[int]:
        r = self.requests[req_id]
        blocks = -(-(r.length + n) // self.page_size)
        return [max(0, blocks - len(t)) for t in r.tables]

    def can_reserve(self, req_id: str, n: int) -> bool:
        return all(need <= g.pool.available for need, g in zip(self.pages_needed(req_id, n), self.groups))

    def reserve(self, req_id: str, tokens: Sequence[int]) -> bool:
        """Pages for ``tokens`` after what the request already holds.  All groups or none:
        returns False and changes nothing when any pool is short."""
        r = self.requests[req_id]
        if len(r.tokens) != r.length:
            raise CacheError(f"request {req_id!r} has a reservation that was not committed")
        need = self.pages_needed(req_id, len(tokens))
        if any(n > g.pool.available for n, g in zip(need, self.groups)):
            return False
        for n, g, t in zip(need, self.groups, r.tables):
            t.extend(g.pool.allocate(n))
        r.tokens.extend(int(x) for x in tokens)
        return True

    def slot_ids(self, req_id: str, group: int) -> List[int]:
        """Cache slot (page * page_size + offset) of every reserved, uncommitted token."""
        r = self.requests[req_id]
        ps, table = self.page_size, r.tables[group]
        return [table[p // ps] * ps + p % ps for p in range(r.length, len(r.tokens))]

    def block_table(self, req_id: str, group: int) -> List[int]:
        return self.requests[req_id].tables[group]

    def state_slot(self, req_id: str) -> int:
        return self.requests[req_id].slot

    def serial(self, req_id: str) -> int:
        """A number unique to this admission of the request."""
        return self.requests[req_id].serial

    def commit(self, req_id: str) -> None:
        """The reserved tokens' keys and values are written: advance the length, hash the
        pages that became full, give back the pages a window has passed."""
        r = self.requests[req_id]
        r.length = len(r.tokens)
        ps = self.page_size
        if self.prefix_reuse:
            known = r.length if r.unknown_at is None else min(r.length, r.unknown_at)   # hashing waits for the id
            while (r.hashed_blocks + 1) * ps <= known:
                b = r.hashed_blocks
                r.last_hash = self._block_hash(r.last_hash, r.tokens[b * ps:(b + 1) * ps])
                for g, t in zip(self.groups, r.tables):
                    g.pool.set_hash(t[b], r.last_hash)
                r.hashed_blocks += 1
        for g, t in zip(self.groups, r.tables):
            if g.need.window is None:
                continue
            for b in range(min(self._first_needed_block(g, r.length), len(t))):
                if t[b] >= 0:
                    g.pool.release(t[b])
                    t[b] = -1

    def mark_unknown(self, req_id: str, index: int) -> None:
        """Token ``index`` of the request was reserved with a placeholder id: the step that runs
        it was launched before the id was read back.  Pages holding it are not hashed until
        ``patch_token`` supplies the id."""
        self.requests[req_id].unknown_at = index

    def patch_token(self, req_id: str, index: int, token: int) -> None:
        r = self.requests[req_id]
        r.tokens[index] = int(token)
        if r.unknown_at == index:
            r.unknown_at = None

    def rollback(self, req_id: str) -> None:
        """Drop a reservation that was not committed (pages beyond the committed length
        go back)."""
        r = self.requests[req_id]
        del r.tokens[r.length:]
        keep = -(-r.length // self.page_size)
        for g, t in zip(self.groups, r.tables):
            for p in t[keep:]:
                if p >= 0:
                    g.pool.release(p)
            del t[keep:]

    def free(self, req_id: str) -> None:
        r = self.requests.pop(req_id, None)
        if r is None:
            raise CacheError(f"request {req_id!r} is not admitted")
        for g, t in zip(self.groups, r.tables):
            for p in t:
                if p >= 0:
                    g.pool.release(p)
        self.slots.release(r.slot)

    def available_pages(self) -> List[int]:
        return [g.pool.available for g in self.groups]

    def check(self) -> None:
        """No page lost, held twice or freed twice; no slot lost."""
        for gi, g in enumerate(self.groups):
            held: Dict[int, int] = {}
            for r in self.requests.values():
                for p in r.tables[gi]:
                    if p >= 0:
                        held[p] = held.get(p, 0) + 1
            g.pool.check(held)
        self.slots.check()
        if len({r.slot for r in self.requests.values()}) != len(self.requests):
            raise CacheError("two requests share a state slot")
