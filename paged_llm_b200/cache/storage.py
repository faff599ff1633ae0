"""Device memory of the cache: page pools and state slots.

The reference keeps, per layer, one K and one V tensor
[num_blocks, block_size, kv_heads, head_dim], zero-initialised
(pagedllm/kv_cache.py:16-54).  Here a group of layers shares one tensor

    [layers, pages, 2 (K, V), kv_heads, page_size, head_dim]

so that the page_size x head_dim tile of one (layer, page, K or V, kv head) is
contiguous: an attention kernel reads a page of one head as one block.  A page id
indexes the same row of every layer of its group, as in the reference.

State slots: [slots, *shape] per scheduled run of a layer that asks for fixed
state.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ..parts.base import FixedState, PagedKV
from .manager import GroupSpec, PageCopy


@dataclass
class LayerCache:
    """What a mixer gets for one run of its layer."""

    kind: str                         # "paged_kv" | "fixed_state"
    group: int                        # index of the block table to use (paged_kv)
    owner: bool                       # False: reads another run's cache, writes nothing
    kv: torch.Tensor | None = None    # [pages, 2, kv_heads, page_size, head_dim]
    state: torch.Tensor | None = None  # [slots, *shape]
    window: int | None = None


class CacheStorage:
    """Allocates the device tensors that a model's cache slots ask for and
    hands out per-run views."""

    def __init__(self, cache_slots, num_pages: int, page_size: int, dtype: torch.dtype, device,
                 num_state_slots: int = 0):
        self.page_size, self.dtype, self.device = page_size, dtype, torch.device(device)
        self.num_pages = num_pages
        # group paged requirements: same (heads, head_dim, window) -> same group
        self.group_keys: list[PagedKV] = []
        members: list[list[int]] = []
        for slot in cache_slots:
            if slot.shares is None and isinstance(slot.requirement, PagedKV):
                if slot.requirement not in self.group_keys:
                    self.group_keys.append(slot.requirement)
                    members.append([])
                members[self.group_keys.index(slot.requirement)].append(slot.entry)
        self.pools: list[torch.Tensor] = []
        for key, entries in zip(self.group_keys, members):
            shape = (len(entries), num_pages, 2, key.num_kv_heads, page_size, key.head_dim)
            self.pools.append(torch.zeros(shape, dtype=dtype, device=self.device))
        self.layer_caches: list[LayerCache | None] = [None] * len(cache_slots)
        self.num_state_slots = 0
        for slot in cache_slots:
            req = slot.requirement
            if slot.shares is not None:
                continue
            if isinstance(req, PagedKV):
                g = self.group_keys.index(req)
                self.layer_caches[slot.entry] = LayerCache(
                    "paged_kv", g, True, kv=self.pools[g][members[g].index(slot.entry)], window=req.window)
            elif isinstance(req, FixedState):
                self.num_state_slots = max(1, num_state_slots)
                state = torch.zeros((self.num_state_slots, *req.shape), dtype=req.dtype, device=self.device)
                self.layer_caches[slot.entry] = LayerCache("fixed_state", -1, True, state=state)
        for slot in cache_slots:
            if slot.shares is not None:
                src = self.layer_caches[slot.shares]
                self.layer_caches[slot.entry] = LayerCache(src.kind, src.group, False, kv=src.kv, state=src.state,
                                                           window=src.window)

    @property
    def num_groups(self) -> int:
        return len(self.group_keys)

    def group_specs(self) -> list[GroupSpec]:
        return [GroupSpec(self.num_pages, key.window) for key in self.group_keys]

    def page_bytes(self) -> int:
        """Bytes of one page id across all groups and layers."""
        return sum(p[:, 0].numel() * p.element_size() for p in self.pools)

    @staticmethod
    def page_bytes_for(cache_slots, page_size: int, dtype: torch.dtype) -> int:
        elem = torch.tensor([], dtype=dtype).element_size()
        return sum(2 * s.requirement.num_kv_heads * s.requirement.head_dim * page_size * elem
                   for s in cache_slots if s.shares is None and isinstance(s.requirement, PagedKV))

    def fill(self, value: float) -> None:
        """Overwrite every page (tests poison the pool to show stale reads)."""
        for p in self.pools:
            p.fill_(value)

    def apply_copies(self, copies: list[PageCopy], ops) -> None:
        """Copy-on-write: page `src` -> page `dst` in every layer of the group
        (reference: kv_cache.py:47-54)."""
        for g in range(len(self.pools)):
            pairs = [(c.src, c.dst) for c in copies if c.group == g]
            if pairs:
                ops.copy_pages(self.pools[g], pairs)

    def _state_tensors(self):
        return [lc.state for lc in self.layer_caches if lc is not None and lc.kind == "fixed_state" and lc.owner]

    def zero_state(self, slots) -> None:
        """Zero the state of the given slots (an int or a list of them) in every stateful run:
        one indexed fill per state tensor, whatever the number of slots."""
        slots = [slots] if isinstance(slots, int) else list(slots)
        if not slots:
            return
        states = self._state_tensors()
        if not states:
            return
        idx = torch.tensor(slots, dtype=torch.long).to(self.device, non_blocking=True)
        for state in states:
            state.index_fill_(0, idx, 0)

    def save_state(self) -> list[torch.Tensor]:
        """Copies of all state tensors (the runner takes them around the trial runs of a graph
        capture, which must leave no trace: a stateful mixer's step is not idempotent)."""
        return [state.clone() for state in self._state_tensors()]

    def restore_state(self, saved: list[torch.Tensor]) -> None:
        for state, old in zip(self._state_tensors(), saved):
            state.copy_(old)

    def copy_state(self, pairs) -> None:
        """state[dst] = state[src] for each (src, dst), in order (a forked request starts from
        its parent's state)."""
        for src, dst in pairs:
            for state in self._state_tensors():
                state[dst].copy_(state[src])
