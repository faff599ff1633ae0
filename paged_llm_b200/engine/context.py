"""What one step carries to the parts: the batch's metadata on the device and
on the host, the cache views, and the kernel library.

The reference builds `AttentionMetadata` (slot_mapping, block_tables,
cu_seqlens_q, seq_lens_k, max_q_len) plus input ids, positions and
logits_indices from Python lists every step (pagedllm/engine.py:62-91;
pagedllm/model/llama.py:63-71).  Here the same facts travel as int32 views into
one packed device buffer that is filled by a single host-to-device copy; the
slot mapping is not materialised (the kernel that writes keys and values
derives it from the block table and the position).
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch


@dataclass
class HostBatch:
    """The step's shape on the host, for planning and for parts written in
    plain tensor code."""

    q_lens: list[int]            # new tokens of each request
    starts: list[int]            # position of each request's first new token
    state_slots: list[int]       # state slot of each request (-1: none)
    seq_ids: list[int] = field(default_factory=list)

    @property
    def k_lens(self) -> list[int]:
        return [s + n for s, n in zip(self.starts, self.q_lens)]

    @property
    def cu(self) -> list[int]:
        out = [0]
        for n in self.q_lens:
            out.append(out[-1] + n)
        return out


@dataclass
class AttentionPlan:
    """Work lists of one attention shape (query heads per kv head, window) for
    the step: items are int32 quadruples (request, row tile, split, splits)."""

    small: torch.Tensor | None       # [n_small, 4]: requests with few query rows (decode)
    large: torch.Tensor | None       # [n_large, 4]: the others (prefill portions)
    splits: torch.Tensor             # [S]: splits of each request (1: written directly)
    n_small: int
    n_large: int
    max_splits: int
    small_tokens: int = 0            # tokens of the requests in `small` (scratch rows)
    long_context: bool = False       # a decode step whose contexts are split through the work list, not as clusters


@dataclass
class StepContext:
    ops: object
    num_tokens: int
    num_seqs: int
    num_logits: int
    input_ids: torch.Tensor          # [T] int32
    positions: torch.Tensor          # [T] int32
    token_seq: torch.Tensor          # [T] int32: row of the request each token belongs to (-1: padding)
    cu_seqlens_q: torch.Tensor       # [S+1] int32
    seq_lens_k: torch.Tensor         # [S] int32: context length including the new tokens
    state_slots: torch.Tensor        # [S] int32
    logits_indices: torch.Tensor     # [num_logits] int32
    block_tables: list[torch.Tensor]  # per cache group: [S, stride] int32
    layer_caches: list
    page_size: int
    max_q_len: int
    host: HostBatch
    attention_plans: dict = field(default_factory=dict)    # (group size, window) -> AttentionPlan
    logits_all: bool = False        # logits are wanted at every token, in order (decode steps): no row gather
    padded: bool = False            # built for a captured graph of mixed items: token rows and lists have spare capacity
