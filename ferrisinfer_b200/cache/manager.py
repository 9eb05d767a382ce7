"""The cache manager: pages and block tables per request and page group, and fixed-size state slots.

What the reference has: one cache per session, per-layer pages ``[page, kv heads, head dim]``
with a per-layer table from logical block (position / page size) to page
(crates/ferrisinfer-runtime/src/paged_kv.rs:131-172, 469-527, 605-613); everything is returned
when the session is reset or dropped (crates/ferrisinfer-runtime/src/paged_kv.rs:529-549;
crates/ferrisinfer-runtime/src/scheduler.rs:590-599); the per-request state of fixed size (position,
last sample, RNG state) lives in the session (crates/ferrisinfer-runtime/src/session.rs:92-102).

Here ONE manager serves all requests:

* Mixers that keep keys and values declare a ``PagedKV`` need.  Run-order entries with the same
  need (kv heads, head size, window) form a **page group**: the group has one pool of page ids and
  one block table per request, and each entry of the group has key and value tensors of its own
  ``[pages, kv heads, page size, head dim]`` addressed by the group's page ids.  Groups with
  different needs (all keys / a window of them) have pools and tables of their own.
* A request's pages are allocated before a step for every token the step brings (``extend``),
  counted as held after it (``commit``), and given back when the request ends (``release``) or, in a
  window group, as soon as the window has passed them (in ``commit``); a page that is given back is
  the next one handed out.
* Mixers with a ``FixedState`` need, and the engine itself (sampler state), get a tensor
  ``[slots, *shape]``; a request holds one slot id from admission to release, and the slot's rows
  are zeroed at admission.
* Every pool has one page more than it hands out, and every state tensor one slot more
  (``padding_page``, ``padding_slot``): rows that only fill a step up to a recorded batch size write
  their key, value and state there, where no request ever reads.
* A need of another kind than these two brings its own builder (``register_cache_need``).
* With prefix sharing, full pages of prompts are found by later requests through a chain hash and
  shared, not copied.  With ``keep_finished`` the index holds a reference of its own, so the pages of
  a prompt outlive the request that computed them; they count as free, and the least recently used
  of them are given up (ends of chains first) when a request needs pages that the free list lacks.
"""

from __future__ import annotations

from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Any, Optional

import torch

from ..errors import CacheError, OutOfPages
from ..parts.base import FixedState, LayerCache, PagedKV
from .pages import PagePool

NO_PAGE = -1


@dataclass
class PageGroup:
    gid: int
    need: PagedKV
    members: list  # run-order entries whose k/v tensors this group's page ids address
    page_size: int
    pool: PagePool

    @property
    def window(self) -> Optional[int]:
        return self.need.window


@dataclass
class RequestCache:
    request_id: Any
    slot: int
    num_tokens: int = 0  # tokens whose keys/values (or state) are in the cache
    tables: dict = field(default_factory=dict)  # gid -> list of page ids (NO_PAGE = hole)
    arrays: dict = field(default_factory=dict)  # gid -> int32 array copy of the table, dropped when it changes
    prompt: Optional[list] = None  # the request's known tokens, when its full pages may be shared
    registered_blocks: int = 0  # leading blocks of the prompt that are in the prefix index
    block_keys: list = field(default_factory=list)  # chain hash of each registered or borrowed block
    shared_tokens: int = 0  # tokens that came from other requests' pages at admission
    revived_pages: int = 0  # of those pages, how many had outlived their last holder


class PrefixIndex:
    """Full pages of prompts that live requests hold, by the hash of all tokens up to the page's end.

    The reference finds a donor by scanning live sequences for the longest common prompt prefix and
    COPIES its pages (crates/ferrisinfer-runtime/src/prefix_index.rs:42-108;
    crates/ferrisinfer-runtime/src/paged_kv.rs:329-389), counting references only as metadata
    (crates/ferrisinfer-runtime/src/block_manager.rs:84-122).  Here the pages themselves are shared:
    a chain hash key_i = H(key_{i-1}, tokens of page i) names a block; a borrower's block tables point at
    the same page ids and the pool counts the holders.  An entry lives as long as its pages do."""

    def __init__(self):
        self.blocks: dict = {}  # key -> (page ids, one per page group; previous key; the page's tokens)
        self.by_page: dict = {}  # (gid, page) -> key

    @staticmethod
    def chain(prev, tokens) -> int:
        return hash((prev, tuple(tokens)))

    def lookup(self, key, prev, tokens):
        """The pages of the block, or None; a hash that collides is told apart by the tokens themselves."""
        entry = self.blocks.get(key)
        if entry is None or entry[1] != prev or entry[2] != tuple(tokens):
            return None
        return entry[0]

    def insert(self, key, prev, tokens, pages: tuple) -> bool:
        """True if the block is new to the index."""
        if key in self.blocks:
            return False
        self.blocks[key] = (pages, prev, tuple(tokens))
        for gid, page in enumerate(pages):
            self.by_page[(gid, page)] = key
        return True

    def remove(self, key):
        """Forget the block; returns its pages (or None)."""
        entry = self.blocks.pop(key, None)
        if entry is None:
            return None
        for gid, page in enumerate(entry[0]):
            self.by_page.pop((gid, page), None)
        return entry[0]

    def forget_page(self, gid: int, page: int) -> None:
        key = self.by_page.pop((gid, page), None)
        if key is not None:
            entry = self.blocks.pop(key, None)
            if entry is not None:
                for g2, p2 in enumerate(entry[0]):
                    self.by_page.pop((g2, p2), None)


# need class -> builder(manager, run-order index, need) -> LayerCache.  A builder may use ``manager.page_group(need)``
# (pages by block table) and ``manager.new_state(shape, dtype)`` (one row per request slot, zeroed at admission).
_NEED_BUILDERS: dict = {}


def register_cache_need(need_cls, builder) -> None:
    """How the cache manager serves a kind of need that it does not know: ``builder(manager, index, need)``
    returns the ``LayerCache`` that the mixer of run-order entry ``index`` gets."""
    _NEED_BUILDERS[need_cls] = builder


def _build_paged(manager, index, need):
    g = manager.page_group(need)
    g.members.append(index)
    cache = LayerCache(need=need, group=g.gid)
    if manager.device is not None:
        # one page beyond the pool's: the padding page.  Keys and values are the two planes of one tensor, so that
        # a kernel can fetch a tile of keys and the tile of values of the same tokens with one copy.
        shape = (2, g.pool.num_pages + 1, need.num_kv_heads, manager.page_size, need.head_dim)
        planes = torch.zeros(shape, dtype=manager.dtype, device=manager.device)
        cache.k, cache.v = planes[0], planes[1]
    return cache


def _build_state(manager, index, need):
    return LayerCache(need=need, state=manager.new_state(need.shape, need.dtype))


register_cache_need(PagedKV, _build_paged)
register_cache_need(FixedState, _build_state)


class CacheManager:
    def __init__(self, needs: list, page_size: int, num_pages, max_requests: int,
                 dtype: torch.dtype = torch.float32, device=None, extra_states: Optional[dict] = None,
                 prefix_sharing: bool = False, min_prefix_share_tokens: int = 0, keep_finished: bool = False):
        """``needs[i]``: the cache need of run-order entry i (PagedKV, FixedState, a kind registered with
        ``register_cache_need``, or None).
        ``num_pages``: pages per group (an int for all groups, or a dict gid -> int).
        ``device`` None: bookkeeping only (no tensors), as the CPU tests use it.
        ``keep_finished`` (with prefix sharing): shareable pages stay in the cache after their last
        holder has gone, until their room is needed."""
        if page_size <= 0:
            raise CacheError(f"page size must be positive, not {page_size}")
        if max_requests <= 0:
            raise CacheError(f"at least one request slot is needed, not {max_requests}")
        self.page_size = int(page_size)
        self.max_requests = int(max_requests)
        self.dtype, self.device = dtype, device
        self.groups: list = []
        self.layer_caches: list = [None] * len(needs)
        self.state_tensors: dict = {}
        self._by_need: dict = {}
        self._num_pages = num_pages
        for i, need in enumerate(needs):
            if need is None:
                continue
            builder = next((b for cls, b in _NEED_BUILDERS.items() if isinstance(need, cls)), None)
            if builder is None:
                raise CacheError(f"run-order entry {i} has an unknown cache need {need!r}")
            self.layer_caches[i] = builder(self, i, need)
        for name, need in (extra_states or {}).items():
            if device is not None:
                self.state_tensors[name] = self.new_state(need.shape, need.dtype)
        self._free_slots = list(range(self.max_requests - 1, -1, -1))
        self.requests: dict = {}
        # Pages of prompts are shared only where a page means the same for every layer: all page groups keep
        # every key (no window) and no mixer keeps a state of its own.
        shareable = bool(self.groups) and all(g.window is None for g in self.groups) and not any(
            isinstance(n, FixedState) for n in needs)
        self.prefix = PrefixIndex() if (prefix_sharing and shareable) else None
        self.min_prefix_share_tokens = int(min_prefix_share_tokens)
        self.keep_finished = bool(keep_finished) and self.prefix is not None
        # blocks of the index that no request holds (the index's own reference keeps their pages), least
        # recently used first; a block's descendants in a chain always come before it
        self._idle: OrderedDict = OrderedDict()
        self.stats = {"shared_tokens": 0, "shared_pages": 0, "revived_pages": 0, "evicted_pages": 0}

    # ------------------------------------------------------------------- set-up
    def page_group(self, need: PagedKV) -> PageGroup:
        """The page group of ``need`` (made at its first call): entries with the same need share page ids."""
        gid = self._by_need.get(need)
        if gid is None:
            gid = len(self.groups)
            n = self._num_pages[gid] if isinstance(self._num_pages, dict) else self._num_pages
            self.groups.append(PageGroup(gid, need, [], self.page_size, PagePool(n)))
            self._by_need[need] = gid
        return self.groups[gid]

    def new_state(self, shape, dtype) -> Optional[torch.Tensor]:
        """A zeroed tensor with one row of ``shape`` per request slot and one more, the padding slot's
        (None without a device)."""
        if self.device is None:
            return None
        return torch.zeros((self.max_requests + 1, *shape), dtype=dtype, device=self.device)

    @property
    def padding_slot(self) -> int:
        """A state slot that no request ever holds."""
        return self.max_requests

    def padding_page(self, gid: int) -> int:
        """A page of group ``gid`` that no request ever holds."""
        return self.groups[gid].pool.num_pages

    def state_bytes(self) -> int:
        """Bytes of the per-request state tensors (mixers' and the engine's)."""
        total = 0
        for cache in self.layer_caches:
            if cache is not None and cache.state is not None:
                total += cache.state.numel() * cache.state.element_size()
        for t in self.state_tensors.values():
            total += t.numel() * t.element_size()
        return total

    # ------------------------------------------------------------------ requests
    def has(self, request_id) -> bool:
        return request_id in self.requests

    @property
    def num_free_slots(self) -> int:
        return len(self._free_slots)

    def admit(self, request_id, prompt: Optional[list] = None) -> RequestCache:
        """Give ``request_id`` a state slot (zeroed) and empty block tables.  With ``prompt`` (its known
        tokens) and prefix sharing on, leading full pages that another live request already holds are
        borrowed: the request then starts with ``num_tokens`` > 0.  At least one token is always left to
        compute, and fewer than ``min_prefix_share_tokens`` are not worth sharing."""
        if request_id in self.requests:
            raise CacheError(f"request {request_id!r} is already admitted")
        if not self._free_slots:
            raise CacheError(f"all {self.max_requests} request slots are taken")
        slot = self._free_slots.pop()
        rc = RequestCache(request_id, slot, 0, {g.gid: [] for g in self.groups})
        self.requests[request_id] = rc
        if self.prefix is not None and prompt is not None:
            rc.prompt = prompt
            ps = self.page_size
            most = (len(prompt) - 1) // ps  # never the whole prompt
            key, found = None, []
            for b in range(most):
                tokens = prompt[b * ps:(b + 1) * ps]
                prev, key = key, PrefixIndex.chain(key, tokens)
                pages = self.prefix.lookup(key, prev, tokens)
                if pages is None:
                    break
                found.append((key, pages))
            if found and len(found) * ps >= self.min_prefix_share_tokens:
                for key, pages in found:
                    for g, page in zip(self.groups, pages):
                        g.pool.retain(page)
                        rc.tables[g.gid].append(page)
                    rc.block_keys.append(key)
                    if key in self._idle:  # pages that had outlived their last holder
                        del self._idle[key]
                        rc.revived_pages += len(self.groups)
                        self.stats["revived_pages"] += len(self.groups)
                rc.registered_blocks = len(found)
                rc.num_tokens = rc.shared_tokens = len(found) * ps
                self.stats["shared_tokens"] += rc.shared_tokens
                self.stats["shared_pages"] += len(found) * len(self.groups)
        for cache in self.layer_caches:
            if cache is not None and cache.state is not None:
                cache.state[slot].zero_()
        for t in self.state_tensors.values():
            t[slot].zero_()
        return rc

    def get(self, request_id) -> RequestCache:
        try:
            return self.requests[request_id]
        except KeyError:
            raise CacheError(f"request {request_id!r} is not admitted") from None

    # --------------------------------------------------------------------- pages
    def _first_needed_block(self, g: PageGroup, num_tokens: int) -> int:
        """Lowest block that a query at position >= num_tokens can still read."""
        if g.window is None:
            return 0
        return max(0, num_tokens - g.window + 1) // self.page_size

    def pages_needed(self, request_id, new_total: int) -> dict:
        """gid -> pages that ``extend(request_id, new_total)`` would take from the pool."""
        rc = self.get(request_id)
        out = {}
        blocks = -(-new_total // self.page_size)
        for g in self.groups:
            table = rc.tables[g.gid]
            first = self._first_needed_block(g, rc.num_tokens)
            # every block from `first` up to the table's end has a page (extend fills them, commit frees
            # only below `first`), so what is missing lies beyond the table's end
            out[g.gid] = max(0, blocks - max(len(table), first))
        return out

    def free_pages(self) -> dict:
        """gid -> pages that a request can get: the free list and the pages that only the prefix index holds."""
        return {g.gid: g.pool.num_free + len(self._idle) for g in self.groups}

    @property
    def num_idle_blocks(self) -> int:
        """Blocks of finished prompts that are kept for later requests (one page per group each)."""
        return len(self._idle)

    def can_extend(self, request_id, new_total: int, reserve: Optional[dict] = None) -> bool:
        """Whether the pools can cover ``new_total`` tokens of the request, leaving ``reserve``
        (gid -> pages) for others."""
        need = self.pages_needed(request_id, new_total)
        free = self.free_pages()
        return all(need[g.gid] + (reserve or {}).get(g.gid, 0) <= free[g.gid] for g in self.groups)

    def _evict_idle(self, count: int) -> int:
        """Give up to ``count`` idle blocks' pages back to the free lists, least recently used first."""
        done = 0
        while done < count and self._idle:
            key, _ = self._idle.popitem(last=False)
            pages = self.prefix.remove(key)
            if pages is None:
                continue
            for g, page in zip(self.groups, pages):
                if not g.pool.release(page):
                    raise CacheError(f"idle page {page} of group {g.gid} still had a holder")
            self.stats["evicted_pages"] += len(self.groups)
            done += 1
        return done

    def drop_idle(self) -> int:
        """Forget every kept prompt page that no request holds; returns the blocks dropped."""
        return self._evict_idle(len(self._idle))

    def extend(self, request_id, new_total: int) -> None:
        """Make every position below ``new_total`` that the next step can read or write addressable.
        All groups or none: raises OutOfPages without taking a page if any pool is short."""
        rc = self.get(request_id)
        if new_total < rc.num_tokens:
            raise CacheError(f"request {request_id!r} holds {rc.num_tokens} tokens; cannot extend to {new_total}")
        need = self.pages_needed(request_id, new_total)
        free = self.free_pages()
        for g in self.groups:
            if need[g.gid] > free[g.gid]:
                raise OutOfPages(
                    f"request {request_id!r} needs {need[g.gid]} more pages in group {g.gid} "
                    f"({free[g.gid]} of {g.pool.num_pages} free)"
                )
        short = max(need[g.gid] - g.pool.num_free for g in self.groups) if self.groups else 0
        if short > 0:
            self._evict_idle(short)
        blocks = -(-new_total // self.page_size)
        for g in self.groups:
            table = rc.tables[g.gid]
            if blocks <= len(table):
                continue
            first = self._first_needed_block(g, rc.num_tokens)
            start = len(table)
            if first > start:  # blocks that the window has passed before they were ever needed
                table.extend([NO_PAGE] * (first - start))
                start = first
            table.extend(g.pool.alloc(blocks - start))
            rc.arrays.pop(g.gid, None)

    def commit(self, request_id, new_total: int) -> int:
        """The step that brought the request to ``new_total`` tokens is done: count them, and give
        back the pages of window groups that no later query can read.  Returns pages freed."""
        rc = self.get(request_id)
        if new_total < rc.num_tokens:
            raise CacheError(f"request {request_id!r} cannot shrink from {rc.num_tokens} to {new_total} tokens")
        rc.num_tokens = new_total
        if self.prefix is not None and rc.prompt is not None:
            # full pages of the prompt that are now in the cache can be borrowed by later requests
            ps = self.page_size
            upto = min(new_total, len(rc.prompt)) // ps
            while rc.registered_blocks < upto:
                b = rc.registered_blocks
                prev = rc.block_keys[-1] if rc.block_keys else None
                tokens = rc.prompt[b * ps:(b + 1) * ps]
                key = PrefixIndex.chain(prev, tokens)
                rc.block_keys.append(key)
                pages = tuple(rc.tables[g.gid][b] for g in self.groups)
                if self.prefix.insert(key, prev, tokens, pages) and self.keep_finished:
                    for g, page in zip(self.groups, pages):
                        g.pool.retain(page)  # the index's own reference
                rc.registered_blocks += 1
        freed = 0
        for g in self.groups:
            if g.window is None:
                continue
            table = rc.tables[g.gid]
            upto = min(self._first_needed_block(g, new_total), len(table))
            b = upto - 1
            while b >= 0 and table[b] != NO_PAGE:  # everything below an earlier hole went back before
                g.pool.release(table[b])
                table[b] = NO_PAGE
                freed += 1
                b -= 1
            if freed:
                rc.arrays.pop(g.gid, None)
        return freed

    def release(self, request_id) -> int:
        """The request is over (finished, cancelled or preempted): pages and slot go back."""
        rc = self.requests.pop(request_id, None)
        if rc is None:
            raise CacheError(f"request {request_id!r} is released twice (or was never admitted)")
        if rc.num_tokens == rc.shared_tokens and rc.shared_tokens:
            # admitted and sent away again before it computed a token (its first portion did not fit): what it
            # borrowed does not count as shared
            self.stats["shared_tokens"] -= rc.shared_tokens
            self.stats["shared_pages"] -= (rc.shared_tokens // self.page_size) * len(self.groups)
            self.stats["revived_pages"] -= rc.revived_pages
        freed = 0
        for g in self.groups:
            for page in rc.tables[g.gid]:
                if page != NO_PAGE and g.pool.release(page):
                    freed += 1
                    if self.prefix is not None:
                        self.prefix.forget_page(g.gid, page)
        if self.keep_finished:
            # blocks that only the index holds now wait for a later request or for their room to be needed;
            # the end of the chain first, so that it is given up before what leads to it
            for key in reversed(rc.block_keys):
                entry = self.prefix.blocks.get(key)
                if entry is not None and all(g.pool.refcount(p) == 1 for g, p in zip(self.groups, entry[0])):
                    self._idle.pop(key, None)
                    self._idle[key] = None
        self._free_slots.append(rc.slot)
        return freed

    # ----------------------------------------------------------------- addressing
    def block_table(self, request_id, gid: int) -> list:
        return self.get(request_id).tables[gid]

    def block_table_array(self, request_id, gid: int):
        """The block table as an int32 array (cached until the table changes)."""
        import numpy as np

        rc = self.get(request_id)
        arr = rc.arrays.get(gid)
        if arr is None:
            arr = np.asarray(rc.tables[gid], dtype=np.int32)
            rc.arrays[gid] = arr
        return arr

    def slots_for(self, request_id, gid: int, start: int, count: int) -> list:
        """Cache slot (page * page_size + offset) of positions start .. start + count - 1."""
        table = self.get(request_id).tables[gid]
        ps = self.page_size
        out = []
        for pos in range(start, start + count):
            page = table[pos // ps]
            if page == NO_PAGE:
                raise CacheError(f"request {request_id!r}: position {pos} has no page in group {gid}")
            out.append(page * ps + pos % ps)
        return out

    # ----------------------------------------------------------------- invariants
    def check_invariants(self) -> None:
        """No page lost, held twice without a count, or freed twice; no slot lost or held twice."""
        for g in self.groups:
            holders: dict = {}
            for rc in self.requests.values():
                for page in rc.tables[g.gid]:
                    if page != NO_PAGE:
                        holders[page] = holders.get(page, 0) + 1
            if self.keep_finished:
                for entry in self.prefix.blocks.values():
                    holders[entry[0][g.gid]] = holders.get(entry[0][g.gid], 0) + 1
            g.pool.check(holders)
        for key in self._idle:
            entry = self.prefix.blocks.get(key)
            if entry is None or any(g.pool.refcount(p) != 1 for g, p in zip(self.groups, entry[0])):
                raise CacheError("a block is listed as idle but is held by a request or gone from the index")
        if self.prefix is not None:
            for key, entry in self.prefix.blocks.items():
                for g, page in zip(self.groups, entry[0]):
                    if g.pool.refcount(page) <= 0:
                        raise CacheError(f"the prefix index names page {page} of group {g.gid}, which nobody holds")
        held = [rc.slot for rc in self.requests.values()]
        if len(set(held)) != len(held):
            raise CacheError("a state slot is held by two requests")
        if set(held) & set(self._free_slots) or len(held) + len(self._free_slots) != self.max_requests:
            raise CacheError("a state slot is lost or both free and held")
