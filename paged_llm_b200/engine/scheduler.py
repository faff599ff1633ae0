"""Continuous batching with a token budget, chunked prefill and preemption by
recompute.  The rules are the reference's (pagedllm/scheduler.py:53-187):

* every step has `max_num_batched_tokens` tokens to give out; a decoding request
  takes one, a request still in its prompt takes what is left of the prompt or
  of the budget (prompts are cut purely by the budget, not at page edges);
* running requests are served first, in admission order; if pages run out, the
  most recently admitted running request is preempted (its pages are freed, its
  generated tokens are kept, it goes to the FRONT of the waiting queue and is
  later recomputed as a longer prompt) until the allocation succeeds or the
  request itself was the victim;
* then waiting requests are admitted strictly first-in first-out while budget,
  `max_num_seqs` and pages allow; admission stops at the first that does not fit;
* a request samples in the step that computes its last known token.

Decided here, where the reference leaves a trap: a request that could never
fit the pool (more pages than exist), or never fit a step with chunking off, is
refused by `add` with an error instead of spinning forever; `max_tokens` is
clamped on the request, never on the caller's `SamplingParams` object.
"""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field

from ..cache.manager import CacheManager
from ..config.engine import EngineConfig
from .sequence import Sequence, SequenceStatus


@dataclass
class ScheduledSequence:
    seq: Sequence
    num_new_tokens: int
    needs_sampling: bool = field(init=False)    # fixed when scheduled

    def __post_init__(self) -> None:
        self.needs_sampling = self.seq.num_computed_tokens + self.num_new_tokens == self.seq.num_tokens


@dataclass
class SchedulerOutput:
    scheduled: list[ScheduledSequence] = field(default_factory=list)
    preempted: list[Sequence] = field(default_factory=list)
    num_prefill_tokens: int = 0
    num_decode_tokens: int = 0

    def grant(self, seq: Sequence, num_tokens: int) -> None:
        """`seq` brings `num_tokens` tokens in this step; they count as decoding once its prompt is through."""
        if seq.is_prefill_done:
            self.num_decode_tokens += num_tokens
        else:
            self.num_prefill_tokens += num_tokens
        self.scheduled.append(ScheduledSequence(seq, num_tokens))

    @property
    def is_empty(self) -> bool:
        return not self.scheduled

    @property
    def total_tokens(self) -> int:
        return self.num_prefill_tokens + self.num_decode_tokens


class Scheduler:
    def __init__(self, config: EngineConfig, block_manager: CacheManager, eos_token_id: int | None):
        self.config = config
        self.bm = block_manager
        self.eos_token_id = eos_token_id
        self.waiting: deque[Sequence] = deque()     # admission order; a preempted request goes to the front
        self.running: list[Sequence] = []           # admission order: the last one is the first to be preempted
        self.finished: list[Sequence] = []
        self.num_preemptions = 0

    # ---- queues ------------------------------------------------------------------
    def add(self, seq: Sequence) -> None:
        cfg = self.config
        n = seq.num_prompt_tokens
        if n >= cfg.max_model_len:
            raise ValueError(f"prompt has {n} tokens, max_model_len={cfg.max_model_len}")
        if not cfg.enable_chunked_prefill and n > cfg.max_num_batched_tokens:
            raise ValueError(f"prompt of {n} tokens exceeds max_num_batched_tokens={cfg.max_num_batched_tokens} and "
                             "chunked prefill is off")
        seq.max_tokens = seq.sampling_params.max_tokens
        if n + seq.max_tokens > cfg.max_model_len:
            seq.max_tokens = max(1, cfg.max_model_len - n)
        # The longest this request can get must fit the pool on its own, else it
        # would preempt itself for ever.
        longest = n + seq.max_tokens
        if not cfg.enable_chunked_prefill:
            # a preempted request comes back as prompt + generated tokens in one portion
            longest_portion = longest - 1
            if longest_portion > cfg.max_num_batched_tokens:
                seq.max_tokens = max(1, cfg.max_num_batched_tokens - n + 1)
                longest = n + seq.max_tokens
        capacity = self.bm.max_tokens_per_request()
        if longest - 1 > capacity:
            if n > capacity:
                raise ValueError(f"prompt of {n} tokens can never fit the cache pool of {capacity} tokens")
            seq.max_tokens = max(1, capacity - n + 1)
        seq.status = SequenceStatus.WAITING
        self.waiting.append(seq)

    def _retire(self, seq: Sequence, status: SequenceStatus) -> None:
        """The request leaves for good: what it holds in the cache goes back."""
        self.bm.free(seq)
        seq.status = status
        self.finished.append(seq)

    def abort(self, seq_id: int) -> None:
        seq = next((s for s in (*self.waiting, *self.running) if s.seq_id == seq_id), None)
        if seq is None:
            return
        (self.waiting if seq.status is SequenceStatus.WAITING else self.running).remove(seq)
        self._retire(seq, SequenceStatus.FINISHED_ABORTED)

    @property
    def has_unfinished(self) -> bool:
        return len(self.waiting) + len(self.running) > 0

    @property
    def num_unfinished(self) -> int:
        return len(self.waiting) + len(self.running)

    # ---- one step's decisions ----------------------------------------------------
    def _portion(self, need: int, left: int) -> int:
        """Tokens a request that still has `need` to compute may bring when `left` remain of the
        step's budget: all of them, a cut prompt if chunking is on, else none this step."""
        if need <= left:
            return need
        return left if self.config.enable_chunked_prefill else 0

    def _evict_last(self, out: SchedulerOutput) -> Sequence:
        """Preemption by recompute of the most recently admitted running request."""
        victim = self.running.pop()
        self.bm.free(victim)
        victim.reset_for_recompute()
        self.waiting.appendleft(victim)
        out.preempted.append(victim)
        self.num_preemptions += 1
        return victim

    def _make_room(self, seq: Sequence, num_tokens: int, out: SchedulerOutput) -> bool:
        """Pages for `num_tokens` more tokens of a running request, evicting from the end of
        `running` while the pool is short.  False if `seq` itself had to go."""
        while self.bm.allocate_slots(seq, num_tokens) is None:
            if self._evict_last(out) is seq:
                return False
        return True

    def _serve_running(self, out: SchedulerOutput, left: int) -> int:
        """Running requests in admission order.  Evictions only ever shorten `running` from its
        end, so walking it by index never meets a request that was preempted in this pass."""
        i = 0
        while i < len(self.running) and left > 0:
            seq = self.running[i]
            n = self._portion(seq.num_uncomputed_tokens, left)
            if n > 0 and self._make_room(seq, n, out):
                out.grant(seq, n)
                left -= n
            i += 1
        return left

    def _admit_waiting(self, out: SchedulerOutput, left: int) -> int:
        """Waiting requests strictly in order, until one does not fit (budget, request limit,
        state slot or pages): it keeps its place and is tried again next step."""
        while self.waiting and left > 0 and len(self.running) < self.config.max_num_seqs:
            seq = self.waiting[0]
            hits, num_cached = self.bm.get_computed_blocks(seq)
            n = self._portion(seq.num_tokens - num_cached, left)
            if n == 0 or not self.bm.acquire_state_slot(seq):
                break
            if self.bm.allocate_slots(seq, n, hits) is None:
                self.bm.release_state_slot(seq)
                break
            self.waiting.popleft()
            seq.num_computed_tokens = seq.num_cached_tokens = num_cached
            seq.status = SequenceStatus.RUNNING
            self.running.append(seq)
            out.grant(seq, n)
            left -= n
        return left

    def schedule(self) -> SchedulerOutput:
        out = SchedulerOutput()
        left = self._serve_running(out, self.config.max_num_batched_tokens)
        self._admit_waiting(out, left)
        return out

    # ---- after the step ----------------------------------------------------------
    PLACEHOLDER = 0      # stands in `token_ids` for a token that is sampled but not yet read back

    def update(self, out: SchedulerOutput, sampled: dict[int, int]) -> list[Sequence]:
        """Advance watermarks, register full pages, append sampled tokens, retire
        what finished (scheduler.py:161-187).  Returns the requests that finished.
        It is `advance` followed by `resolve`; an engine that launches the next step
        before it has read this step's tokens calls the two apart."""
        self.advance(out)
        return self.resolve(out, sampled)

    def advance(self, out: SchedulerOutput) -> None:
        """The step is launched: its tokens count as computed, and a request that
        samples in it gets a place for the token to come."""
        for item in out.scheduled:
            seq = item.seq
            seq.num_computed_tokens += item.num_new_tokens
            self.bm.release_behind_window(seq)
            if item.needs_sampling:
                seq.append_token(self.PLACEHOLDER)
                seq.num_unresolved += 1

    def _status_after(self, seq: Sequence, token: int, known: int) -> SequenceStatus | None:
        """The finished status a request takes once `token` is its newest of `known` known tokens,
        or None if it goes on: a stop token or (unless ignored) the end-of-sequence token stops it,
        its own token limit or the model's length limit ends it."""
        sp = seq.sampling_params
        if token in sp.stop_token_ids or (token == self.eos_token_id and not sp.ignore_eos):
            return SequenceStatus.FINISHED_STOPPED
        if known - seq.num_prompt_tokens >= seq.max_tokens or known >= self.config.max_model_len:
            return SequenceStatus.FINISHED_LENGTH
        return None

    def resolve(self, out: SchedulerOutput, sampled: dict[int, int]) -> list[Sequence]:
        """The step's tokens are known: they take their places, pages that are full of
        known tokens get their hashes, finished requests are retired.  A request that
        finished in an earlier step (while this one was already running) is skipped."""
        done: list[Sequence] = []
        for item in out.scheduled:
            seq = item.seq
            if seq.is_finished:
                continue
            if item.needs_sampling:
                token = int(sampled[seq.seq_id])
                seq.token_ids[seq.num_tokens - seq.num_unresolved] = token
                seq.num_unresolved -= 1
            known = seq.num_tokens - seq.num_unresolved
            self.bm.cache_full_blocks(seq, 0, min(seq.num_computed_tokens, known))
            if item.needs_sampling:
                seq.status = self._status_after(seq, token, known) or seq.status
            if seq.is_finished:
                if seq.num_unresolved:                     # places of a step that ran ahead in vain
                    del seq.token_ids[known:]
                    seq.num_unresolved = 0
                self.running.remove(seq)
                self._retire(seq, seq.status)
                done.append(seq)
        return done
