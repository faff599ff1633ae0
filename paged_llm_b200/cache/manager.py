"""Bookkeeping of the paged cache: which page holds which tokens of which request.

The design follows the reference's `BlockManager` (pagedllm/block_manager.py:48-243):
fixed-size pages with reference counts; a free queue in least-recently-freed
order whose pages keep their content hash until they are handed out again
("cached but evictable"); a chained hash over full pages for prefix lookup that
never covers a request's last token; copy-on-write when a shared, partly filled
page is appended to; all-or-nothing allocation.

What is added here:

* **Groups.**  Layers with different needs (all keys, or a window of them; other
  head counts or head sizes) form groups with pages, tables and free queues of
  their own.  A request has one block table per group.  A group with a window
  gives pages back as soon as the window has passed them
  (`release_behind_window`); their table entries become `NO_PAGE`.
* **State slots.**  A pool of slot numbers for per-request state of fixed size,
  taken at admission and given back with the pages.
* The hash is a 64-bit BLAKE2 digest (stable across processes) and a hit is
  confirmed by comparing the tokens.
* A page whose content is already cached elsewhere stays un-hashed, but the
  chain goes on behind it (the reference stops hashing that request there,
  block_manager.py:147-155).

Prefix lookup needs every group to keep all keys and no state slots; otherwise
it is switched off (a shared prefix would need a snapshot of the state, or keys
that a window has dropped).
"""

from __future__ import annotations

import hashlib
import struct
from collections import OrderedDict
from dataclasses import dataclass

from ..engine.sequence import NO_PAGE, Sequence


@dataclass
class Page:
    page_id: int
    ref_count: int = 0
    content_hash: int | None = None
    tokens: tuple[int, ...] | None = None      # what the hash stands for (hit confirmation)


@dataclass(frozen=True)
class PageCopy:
    """A physical copy of one page that has to happen before the next step."""

    group: int
    src: int
    dst: int


@dataclass(frozen=True)
class GroupSpec:
    num_pages: int
    window: int | None = None


def chain_hash(prev: int | None, tokens) -> int:
    h = hashlib.blake2b(digest_size=8)
    h.update(struct.pack("<q", -1 if prev is None else prev & 0x7FFFFFFFFFFFFFFF))
    h.update(struct.pack(f"<{len(tokens)}q", *tokens))
    return int.from_bytes(h.digest(), "little") & 0x7FFFFFFFFFFFFFFF


class PagePool:
    """Pages of one group: reference counts, the free queue, the hash table."""

    def __init__(self, num_pages: int, keep_hash_when_free: bool):
        if num_pages <= 0:
            raise ValueError("num_blocks must be positive")
        self.num_pages = num_pages
        self.keep_hash_when_free = keep_hash_when_free
        self.pages = [Page(i) for i in range(num_pages)]
        self.free: OrderedDict[int, None] = OrderedDict((i, None) for i in range(num_pages))
        self.cached: dict[int, int] = {}       # content hash -> page id

    def take(self) -> Page:
        page_id, _ = self.free.popitem(last=False)       # least recently freed
        page = self.pages[page_id]
        assert page.ref_count == 0
        self._forget(page)
        page.ref_count = 1
        return page

    def _forget(self, page: Page) -> None:
        if page.content_hash is not None:
            if self.cached.get(page.content_hash) == page.page_id:
                del self.cached[page.content_hash]
            page.content_hash, page.tokens = None, None

    def touch(self, page_id: int) -> None:
        page = self.pages[page_id]
        if page.ref_count == 0:
            del self.free[page_id]
        page.ref_count += 1

    def release(self, page_id: int) -> None:
        page = self.pages[page_id]
        if page.ref_count <= 0:
            raise AssertionError(f"double free of block {page_id}")
        page.ref_count -= 1
        if page.ref_count == 0:
            if not self.keep_hash_when_free:
                self._forget(page)
            self.free[page_id] = None                    # most recently freed: last to go


class CacheManager:
    """`BlockManager` of the reference, over one or more groups."""

    def __init__(self, num_blocks: int | list[GroupSpec], block_size: int, enable_prefix_caching: bool = True,
                 num_state_slots: int = 0):
        groups = [GroupSpec(num_blocks)] if isinstance(num_blocks, int) else list(num_blocks)
        if not groups:
            groups = [GroupSpec(1)]
        if block_size <= 0:
            raise ValueError("block_size must be positive")
        self.block_size = block_size
        self.group_specs = groups
        all_keys = all(g.window is None for g in groups)
        self.enable_prefix_caching = bool(enable_prefix_caching and all_keys and num_state_slots == 0)
        self.pools = [PagePool(g.num_pages, self.enable_prefix_caching) for g in groups]
        self._pending_copies: list[PageCopy] = []
        self._pending_state_copies: list[tuple[int, int]] = []
        self._free_state_slots = list(range(num_state_slots - 1, -1, -1))
        self.num_state_slots = num_state_slots
        self.num_cache_queries = 0
        self.num_cache_hits = 0

    # ---- introspection (first group = the reference's single pool) -----------
    @property
    def num_blocks(self) -> int:
        return self.pools[0].num_pages

    @property
    def blocks(self) -> list[Page]:
        return self.pools[0].pages

    @property
    def num_free_blocks(self) -> int:
        return len(self.pools[0].free)

    @property
    def num_cached_blocks(self) -> int:
        return len(self.pools[0].cached)

    def num_free_in_group(self, g: int) -> int:
        return len(self.pools[g].free)

    def usage(self) -> float:
        return 1.0 - sum(len(p.free) for p in self.pools) / sum(p.num_pages for p in self.pools)

    def pages_for(self, num_tokens: int) -> int:
        return -(-num_tokens // self.block_size)

    def max_tokens_per_request(self) -> int:
        """The longest request the pools can ever hold."""
        return min(p.num_pages for p in self.pools) * self.block_size

    def _tables(self, seq: Sequence) -> list[list[int]]:
        while len(seq.block_tables) < len(self.pools):
            seq.block_tables.append([])
        return seq.block_tables

    # ---- prefix cache ----------------------------------------------------------
    def get_computed_blocks(self, seq: Sequence) -> tuple[list[list[int]] | list[int], int]:
        """Longest cached prefix in whole pages, never covering the last token, so
        that the step still has a row to produce logits from
        (block_manager.py:111-133).  Returns (page ids, tokens); page ids is a
        plain list for a single group, a list per group otherwise."""
        single = len(self.pools) == 1
        if not self.enable_prefix_caching or seq.num_computed_tokens > 0:
            return ([] if single else [[] for _ in self.pools]), 0
        self.num_cache_queries += 1
        bs = self.block_size
        limit = (seq.num_tokens - 1) // bs
        hits: list[list[int]] = [[] for _ in self.pools]
        prev = None
        n = 0
        for i in range(limit):
            tokens = tuple(seq.token_ids[i * bs:(i + 1) * bs])
            h = chain_hash(prev, tokens)
            found = []
            for pool in self.pools:
                pid = pool.cached.get(h)
                if pid is None or pool.pages[pid].tokens != tokens:
                    found = None
                    break
                found.append(pid)
            if found is None:
                break
            for g, pid in enumerate(found):
                hits[g].append(pid)
            prev = h
            n += 1
        if n:
            self.num_cache_hits += 1
        return (hits[0] if single else hits), n * bs

    def cache_full_blocks(self, seq: Sequence, num_computed_before: int, num_computed_after: int) -> None:
        """Give a hash to the pages that became full between the two watermarks
        (block_manager.py:135-158)."""
        if not self.enable_prefix_caching:
            return
        bs = self.block_size
        last_full = num_computed_after // bs
        tables = self._tables(seq)
        while len(seq.page_hashes) < last_full:
            i = len(seq.page_hashes)
            tokens = tuple(seq.token_ids[i * bs:(i + 1) * bs])
            h = chain_hash(seq.page_hashes[-1] if seq.page_hashes else None, tokens)
            seq.page_hashes.append(h)
            for g, pool in enumerate(self.pools):
                page = pool.pages[tables[g][i]]
                if page.content_hash is None and h not in pool.cached:
                    page.content_hash, page.tokens = h, tokens
                    pool.cached[h] = page.page_id

    # ---- allocation ------------------------------------------------------------
    def _normalise_hits(self, computed_blocks) -> list[list[int]]:
        if not computed_blocks:
            return [[] for _ in self.pools]
        if isinstance(computed_blocks[0], int):
            return [list(computed_blocks)] + [[] for _ in self.pools[1:]]
        return [list(c) for c in computed_blocks]

    def _pages_needed(self, g: int, seq: Sequence, num_new: int, num_cached: int) -> int:
        total = seq.num_computed_tokens + num_cached + num_new
        have = len(self._tables(seq)[g]) + num_cached // self.block_size
        return max(0, self.pages_for(total) - have)

    def can_allocate(self, seq: Sequence, num_new_tokens: int, computed_blocks=None) -> bool:
        hits = self._normalise_hits(computed_blocks)
        num_cached = len(hits[0]) * self.block_size
        for g, pool in enumerate(self.pools):
            free = len(pool.free) - sum(1 for b in hits[g] if pool.pages[b].ref_count == 0)
            need = self._pages_needed(g, seq, num_new_tokens, num_cached)
            if num_new_tokens > 0 and self._cow_target(g, seq, num_cached, hits[g]) is not None:
                need += 1
            if need > free:
                return False
        return True

    def _cow_target(self, g: int, seq: Sequence, num_cached: int, hits_g: list[int]) -> int | None:
        """Table index of a shared, partly filled page that the next write would
        land in (block_manager.py:195-202), or None."""
        first_write = seq.num_computed_tokens + num_cached
        if first_write % self.block_size == 0:
            return None
        idx = first_write // self.block_size
        table = self._tables(seq)[g] + hits_g
        if idx >= len(table) or table[idx] == NO_PAGE:
            return None
        return idx if self.pools[g].pages[table[idx]].ref_count > 1 else None

    def _covered(self, seq: Sequence, num_new_tokens: int) -> bool:
        """True if every group's table already covers the new tokens and the page that takes
        the first of them is this request's alone (no page to take, no copy to make)."""
        bs = self.block_size
        first = seq.num_computed_tokens
        need = -(-(first + num_new_tokens) // bs)
        tables = seq.block_tables
        if len(tables) < len(self.pools):
            return False
        for g, pool in enumerate(self.pools):
            table = tables[g]
            if len(table) < need:
                return False
            if first % bs:
                page = table[first // bs]
                if page == NO_PAGE or pool.pages[page].ref_count != 1:
                    return False
        return True

    def allocate_slots(self, seq: Sequence, num_new_tokens: int, computed_blocks=None) -> list[int] | None:
        """Make every group's table cover computed + cached + new tokens.  Returns
        the new page ids of the first group, or None, having changed nothing, if
        any group cannot cover it (block_manager.py:171-217)."""
        if not computed_blocks and self._covered(seq, num_new_tokens):
            return []                                  # the usual decode step: the last page has room
        if not self.can_allocate(seq, num_new_tokens, computed_blocks):
            return None
        hits = self._normalise_hits(computed_blocks)
        num_cached = len(hits[0]) * self.block_size
        tables = self._tables(seq)
        seq.table_version += 1
        first_group_new: list[int] = []
        for g, pool in enumerate(self.pools):
            cow_idx = self._cow_target(g, seq, num_cached, hits[g]) if num_new_tokens > 0 else None
            need = self._pages_needed(g, seq, num_new_tokens, num_cached)
            for b in hits[g]:
                pool.touch(b)
            tables[g].extend(hits[g])
            new = [pool.take().page_id for _ in range(need)]
            tables[g].extend(new)
            if cow_idx is not None:
                shared = tables[g][cow_idx]
                fresh = pool.take().page_id
                self._pending_copies.append(PageCopy(g, shared, fresh))
                pool.release(shared)
                tables[g][cow_idx] = fresh
                new.append(fresh)
            if g == 0:
                first_group_new = new
        if hits[0] and not seq.page_hashes:
            # the chain of a request that starts on cached pages continues from them
            seq.page_hashes = [self.pools[0].pages[b].content_hash for b in hits[0]]
        return first_group_new

    def release_behind_window(self, seq: Sequence) -> int:
        """Give back the pages that no later query of `seq` can read: with `c`
        tokens computed, a window w needs keys from position c - w + 1 on.
        Returns the number of pages released."""
        released = 0
        bs = self.block_size
        for g, spec in enumerate(self.group_specs):
            if spec.window is None:
                continue
            first_needed = seq.num_computed_tokens - spec.window + 1
            table = self._tables(seq)[g]
            j = 0
            while j < len(table) and (j + 1) * bs <= first_needed:
                if table[j] != NO_PAGE:
                    self.pools[g].release(table[j])
                    table[j] = NO_PAGE
                    released += 1
                    seq.table_version += 1
                j += 1
        return released

    def free(self, seq: Sequence) -> None:
        """Give back every page of `seq`, deepest first, so that the pages least
        likely to be shared are the first to be reused (block_manager.py:219-223),
        and its state slot."""
        for g, table in enumerate(self._tables(seq)):
            for b in reversed(table):
                if b != NO_PAGE:
                    self.pools[g].release(b)
        seq.block_tables = [[] for _ in self.pools]
        seq.page_hashes = []
        seq.table_version += 1
        self.release_state_slot(seq)

    def fork(self, parent: Sequence, child: Sequence) -> None:
        """`child` shares every page of `parent` (block_manager.py:225-231).  State of fixed
        size cannot be shared (a step overwrites it): the child gets a slot of its own and a copy
        of the parent's state is queued for the next step (`take_pending_state_copies`)."""
        assert not any(self._tables(child)), "child already owns pages"
        if self.num_state_slots and parent.state_slot is not None:
            if not self.acquire_state_slot(child):
                raise RuntimeError("fork: no state slot is free for the child")
            self._pending_state_copies.append((parent.state_slot, child.state_slot))
        for g, table in enumerate(self._tables(parent)):
            for b in table:
                if b != NO_PAGE:
                    self.pools[g].touch(b)
        child.block_tables = [list(t) for t in parent.block_tables]
        child.table_version += 1
        child.page_hashes = list(parent.page_hashes)
        child.num_computed_tokens = parent.num_computed_tokens

    def take_pending_copies(self) -> list[PageCopy]:
        ops, self._pending_copies = self._pending_copies, []
        return ops

    def take_pending_state_copies(self) -> list[tuple[int, int]]:
        """(source slot, destination slot) pairs that forks have queued, in order."""
        ops, self._pending_state_copies = self._pending_state_copies, []
        return ops

    def slot_mapping(self, seq: Sequence, start_token: int, num_tokens: int, group: int = 0) -> list[int]:
        """Flat slot (page * block_size + offset) of each token of a range
        (block_manager.py:237-243).  The kernels compute this themselves from the
        block table; the list is for tests."""
        bs = self.block_size
        table = self._tables(seq)[group]
        return [table[t // bs] * bs + t % bs for t in range(start_token, start_token + num_tokens)]

    # ---- state slots -----------------------------------------------------------
    def acquire_state_slot(self, seq: Sequence) -> bool:
        """Give `seq` a state slot if the model has any.  False if none is free."""
        if self.num_state_slots == 0 or seq.state_slot is not None:
            return True
        if not self._free_state_slots:
            return False
        seq.state_slot = self._free_state_slots.pop()
        return True

    def release_state_slot(self, seq: Sequence) -> None:
        if seq.state_slot is not None:
            assert seq.state_slot not in self._free_state_slots, f"state slot {seq.state_slot} freed twice"
            self._free_state_slots.append(seq.state_slot)
            seq.state_slot = None

    @property
    def num_free_state_slots(self) -> int:
        return len(self._free_state_slots)

    def check_invariants(self, live: list[Sequence]) -> None:
        """Every page is either free with no holder or held exactly as often as
        its reference count says.  For tests."""
        for g, pool in enumerate(self.pools):
            held = [0] * pool.num_pages
            for seq in live:
                for b in self._tables(seq)[g]:
                    if b != NO_PAGE:
                        held[b] += 1
            for page in pool.pages:
                assert page.ref_count == held[page.page_id], \
                    f"group {g} page {page.page_id}: ref_count {page.ref_count}, held {held[page.page_id]} times"
                assert (page.page_id in pool.free) == (page.ref_count == 0), \
                    f"group {g} page {page.page_id}: free-queue membership does not match ref_count"
            assert len(pool.free) + sum(1 for p in pool.pages if p.ref_count > 0) == pool.num_pages
