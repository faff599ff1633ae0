"""One request and its bookkeeping (reference: pagedllm/sequence.py:23-112).

`token_ids` is prompt plus generated tokens; `num_computed_tokens` is the
watermark: how many leading tokens have their keys and values in the cache.
Block tables are kept per cache group (`block_tables[g]`); `block_table` is the
first group's, which is all a Llama has.
"""

from __future__ import annotations

import itertools
import time
from dataclasses import dataclass, field
from enum import Enum, auto

from ..config.sampling import SamplingParams


class SequenceStatus(Enum):
    WAITING = auto()
    RUNNING = auto()
    FINISHED_STOPPED = auto()      # EOS or a stop token
    FINISHED_LENGTH = auto()       # max_tokens or max_model_len
    FINISHED_ABORTED = auto()

    @property
    def finished(self) -> bool:
        return self.name.startswith("FINISHED")


_ids = itertools.count()

NO_PAGE = -1      # block-table entry of a page that a window has passed


@dataclass(eq=False)
class Sequence:
    prompt_token_ids: list[int]
    sampling_params: SamplingParams = field(default_factory=SamplingParams)
    seq_id: int = field(default_factory=lambda: next(_ids))
    status: SequenceStatus = SequenceStatus.WAITING
    num_computed_tokens: int = 0
    arrival_time: float = field(default_factory=time.perf_counter)
    num_cached_tokens: int = 0         # prefix-cache hit at the (last) admission
    num_preemptions: int = 0

    def __post_init__(self) -> None:
        if len(self.prompt_token_ids) == 0:
            raise ValueError("empty prompt")
        self.prompt_token_ids = [int(t) for t in self.prompt_token_ids]
        self.token_ids: list[int] = list(self.prompt_token_ids)
        self.block_tables: list[list[int]] = [[]]
        self.page_hashes: list[int] = []      # chained content hash of each full page so far
        self.table_version: int = 0           # bumped by the cache manager whenever a block table changes
        self.state_slot: int | None = None    # slot of fixed-size per-request state
        self.max_tokens: int = self.sampling_params.max_tokens   # may be clamped at admission
        self.num_unresolved: int = 0          # trailing tokens that are sampled on the device but not yet known here

    # the first cache group's table, which is what a single-group model has
    @property
    def block_table(self) -> list[int]:
        return self.block_tables[0]

    @block_table.setter
    def block_table(self, value: list[int]) -> None:
        self.block_tables[0] = value

    @property
    def num_prompt_tokens(self) -> int:
        return len(self.prompt_token_ids)

    @property
    def num_tokens(self) -> int:
        return len(self.token_ids)

    @property
    def num_generated_tokens(self) -> int:
        return len(self.token_ids) - len(self.prompt_token_ids)

    @property
    def num_uncomputed_tokens(self) -> int:
        return len(self.token_ids) - self.num_computed_tokens

    @property
    def output_token_ids(self) -> list[int]:
        return self.token_ids[len(self.prompt_token_ids):]

    @property
    def is_finished(self) -> bool:
        return self.status.finished

    @property
    def is_prefill_done(self) -> bool:
        return self.num_computed_tokens >= len(self.prompt_token_ids)

    def append_token(self, token_id: int) -> None:
        self.token_ids.append(int(token_id))

    def reset_for_recompute(self) -> None:
        """Preemption by recompute: what the cache held is dropped, generated
        tokens are kept, so the request comes back as a longer prompt
        (sequence.py:101-106)."""
        self.num_computed_tokens = 0
        self.block_tables = [[] for _ in self.block_tables]
        self.page_hashes = []
        self.table_version += 1
        self.status = SequenceStatus.WAITING
        self.num_preemptions += 1
