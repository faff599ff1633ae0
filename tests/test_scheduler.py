"""Scheduler decisions with a fake sampler: admission, token budget, portions,
mixed steps, preemption when pages run out, finishing and freeing.  The cases
follow the reference's (tests/test_scheduler.py) plus what this engine decides
differently (requests that can never fit)."""

import pytest

from paged_llm_b200.cache import CacheManager
from paged_llm_b200.config import EngineConfig, SamplingParams
from paged_llm_b200.engine.scheduler import Scheduler
from paged_llm_b200.engine.sequence import Sequence, SequenceStatus


def make(num_blocks=64, block_size=4, **kw):
    cfg = EngineConfig(block_size=block_size, num_gpu_blocks=num_blocks, device="cpu",
                       **{"max_num_batched_tokens": 16, "max_model_len": 64, **kw})
    cm = CacheManager(num_blocks, block_size, cfg.enable_prefix_caching)
    return Scheduler(cfg, cm, eos_token_id=2), cm


def run_step(sched, next_token=7):
    out = sched.schedule()
    sampled = {s.seq.seq_id: next_token for s in out.scheduled if s.needs_sampling}
    return out, sched.update(out, sampled)


def req(n, max_tokens=4, **kw):
    return Sequence(list(range(10, 10 + n)), SamplingParams(temperature=0.0, max_tokens=max_tokens, **kw))


def test_prefill_then_decode_then_finish():
    sched, cm = make()
    s = req(5, max_tokens=3)
    sched.add(s)
    out, done = run_step(sched)
    assert [(x.num_new_tokens, x.needs_sampling) for x in out.scheduled] == [(5, True)]
    assert out.num_prefill_tokens == 5 and s.num_generated_tokens == 1 and not done
    out, done = run_step(sched)
    assert out.num_decode_tokens == 1 and out.scheduled[0].num_new_tokens == 1
    out, done = run_step(sched)
    assert done == [s] and s.status is SequenceStatus.FINISHED_LENGTH and s.output_token_ids == [7, 7, 7]
    assert cm.num_free_blocks == cm.num_blocks and not sched.has_unfinished


def test_eos_and_stop_tokens():
    sched, _ = make()
    a, b, c = req(3), req(3, ignore_eos=True, max_tokens=2), req(3, stop_token_ids=(7,), ignore_eos=True)
    for s in (a, b, c):
        sched.add(s)
    run_step(sched, next_token=2)
    assert a.status is SequenceStatus.FINISHED_STOPPED and a.output_token_ids == [2]
    assert b.status is SequenceStatus.RUNNING
    assert c.status is SequenceStatus.RUNNING
    run_step(sched, next_token=7)
    assert b.status is SequenceStatus.FINISHED_LENGTH and c.status is SequenceStatus.FINISHED_STOPPED


def test_portions_honour_the_budget_and_do_not_sample_mid_prompt():
    sched, _ = make()
    s = req(40)
    sched.add(s)
    sizes = []
    for _ in range(3):
        out, _ = run_step(sched)
        sizes.append((out.scheduled[0].num_new_tokens, out.scheduled[0].needs_sampling))
    assert sizes == [(16, False), (16, False), (8, True)] and s.num_generated_tokens == 1


def test_mixed_step_decode_beside_portion():
    sched, _ = make()
    a = req(4)
    sched.add(a)
    run_step(sched)
    b = req(30)
    sched.add(b)
    out, _ = run_step(sched)
    assert [(x.seq, x.num_new_tokens) for x in out.scheduled] == [(a, 1), (b, 15)]
    assert out.num_decode_tokens == 1 and out.num_prefill_tokens == 15


def test_fifo_and_max_num_seqs():
    sched, _ = make(max_num_seqs=2)
    seqs = [req(3) for _ in range(3)]
    for s in seqs:
        sched.add(s)
    out, _ = run_step(sched)
    assert [x.seq for x in out.scheduled] == seqs[:2] and seqs[2].status is SequenceStatus.WAITING


def test_preemption_when_pages_run_out_and_lossless_recovery():
    sched, cm = make(num_blocks=6, block_size=4, enable_prefix_caching=False)
    a, b = req(10, max_tokens=8), req(9, max_tokens=8)
    sched.add(a)
    sched.add(b)
    preempted = 0
    for _ in range(100):
        if not sched.has_unfinished:
            break
        out, _ = run_step(sched)
        preempted += len(out.preempted)
        cm.check_invariants(sched.running)
    assert not sched.has_unfinished and preempted > 0
    assert b.num_preemptions > 0 and a.num_preemptions == 0     # the most recently admitted is the victim
    assert len(a.output_token_ids) == 8 and len(b.output_token_ids) == 8
    assert cm.num_free_blocks == 6


def test_preempted_request_goes_to_the_front_and_keeps_its_tokens():
    sched, cm = make(num_blocks=4, block_size=4, enable_prefix_caching=False)
    a, b, c = req(8, max_tokens=6), req(6, max_tokens=6), req(2)
    sched.add(a); sched.add(b)
    run_step(sched)                                     # both prefilled: 2 + 2 pages
    sched.add(c)
    out, _ = run_step(sched)                            # a needs a 3rd page: b is preempted
    assert out.preempted == [b] and sched.waiting[0] is b and b.num_computed_tokens == 0
    assert b.num_generated_tokens == 1 and b.block_table == []


def test_prefix_cache_across_requests():
    sched, cm = make(max_num_batched_tokens=64)
    a = req(13, max_tokens=1)
    sched.add(a)
    run_step(sched)
    b = Sequence(list(a.prompt_token_ids[:12]) + [99, 98], SamplingParams(max_tokens=1))
    sched.add(b)
    out, _ = run_step(sched)
    assert b.num_cached_tokens == 12 and out.scheduled[0].num_new_tokens == 2 and cm.num_cache_hits == 1


def test_no_chunking():
    sched, _ = make(enable_chunked_prefill=False)
    with pytest.raises(ValueError, match="chunked"):
        sched.add(req(17))
    a, b = req(10), req(10)
    sched.add(a); sched.add(b)
    out, _ = run_step(sched)
    assert [x.seq for x in out.scheduled] == [a]        # b does not fit what is left of the budget: it waits whole


def test_limits_at_add():
    sched, _ = make()
    with pytest.raises(ValueError, match="max_model_len"):
        sched.add(req(64))
    shared = SamplingParams(max_tokens=100)
    s = Sequence(list(range(60)), shared)
    sched.add(s)
    assert s.max_tokens == 4 and shared.max_tokens == 100   # clamped on the request, not on the caller's object


def test_request_that_can_never_fit_is_refused():
    sched, _ = make(num_blocks=4, block_size=4)             # 16 tokens in all
    with pytest.raises(ValueError, match="never fit"):
        sched.add(req(17))
    s = req(10, max_tokens=50)
    sched.add(s)
    assert s.max_tokens == 7                                # 10 + 7 - 1 = 16 tokens held at most
    for _ in range(20):
        if not sched.has_unfinished:
            break
        run_step(sched)
    assert s.status is SequenceStatus.FINISHED_LENGTH and len(s.output_token_ids) == 7


def test_abort():
    sched, cm = make()
    a, b = req(5), req(5)
    sched.add(a); sched.add(b)
    run_step(sched)
    sched.abort(a.seq_id)
    assert a.status is SequenceStatus.FINISHED_ABORTED and sched.running == [b]
    sched.abort(b.seq_id)
    assert cm.num_free_blocks == cm.num_blocks


@pytest.mark.parametrize("seed", range(8))
def test_random_arrivals_and_aborts_keep_the_rules(seed):
    """Requests arrive, are aborted and finish in random order on a pool so small that
    preemption happens: every step honours the token budget and the request limit, a
    step's entries are distinct running requests, prompts are never sampled midway, the
    cache's books balance, and in the end every request finished with its own length and
    every page is free."""
    import random

    rng = random.Random(seed)
    bs = rng.choice([2, 4, 8])
    budget = rng.choice([8, 16, 24])
    chunked = seed % 4 != 3
    max_seqs = rng.choice([2, 3, 5])
    num_blocks = rng.randrange(12, 28)
    max_len = 48
    sched, cm = make(num_blocks=num_blocks, block_size=bs, max_num_batched_tokens=budget, max_model_len=max_len,
                     max_num_seqs=max_seqs, enable_chunked_prefill=chunked, enable_prefix_caching=seed % 2 == 0)
    pending = []
    for i in range(25):
        n = rng.randrange(1, budget + 1 if not chunked else 30)
        pending.append(Sequence([rng.randrange(3, 40) for _ in range(n)],
                                SamplingParams(temperature=0.0, max_tokens=rng.randrange(1, 9), ignore_eos=True)))
    added, aborted, refused = [], set(), set()
    steps = 0
    while pending or sched.has_unfinished:
        steps += 1
        assert steps < 5000, "the scheduler makes no progress"
        while pending and rng.random() < 0.4:
            s = pending.pop()
            try:
                sched.add(s)
                added.append(s)
            except ValueError:
                refused.add(s.seq_id)               # a request the pool or the budget can never hold
        if added and rng.random() < 0.05:
            victim = rng.choice(added)
            if not victim.is_finished:
                sched.abort(victim.seq_id)
                aborted.add(victim.seq_id)
        out = sched.schedule()
        ids = [x.seq.seq_id for x in out.scheduled]
        assert len(set(ids)) == len(ids) and out.total_tokens <= budget and len(sched.running) <= max_seqs
        assert sum(x.num_new_tokens for x in out.scheduled) == out.total_tokens
        for x in out.scheduled:
            assert x.seq in sched.running and x.num_new_tokens >= 1
            reaches_end = x.seq.num_computed_tokens + x.num_new_tokens == x.seq.num_tokens
            assert x.needs_sampling == reaches_end
            if not chunked:
                assert x.num_new_tokens in (1, x.seq.num_tokens - x.seq.num_computed_tokens)
        for v in out.preempted:                     # back in the queue, or admitted again in this very step
            assert v.seq_id in ids or (v.status is SequenceStatus.WAITING and v.num_computed_tokens == 0
                                       and not v.block_table)
        cm.check_invariants(list(sched.running))
        sched.update(out, {x.seq.seq_id: rng.randrange(3, 40) for x in out.scheduled if x.needs_sampling})
        cm.check_invariants(list(sched.running))
    assert cm.num_free_blocks == cm.num_blocks
    for s in added:
        if s.seq_id in aborted:
            assert s.status is SequenceStatus.FINISHED_ABORTED
        else:
            # its own length, cut to what the model length, the pool and (without chunking: a preempted
            # request comes back as one portion) the token budget can ever hold
            n = s.num_prompt_tokens
            want = min(s.sampling_params.max_tokens, max_len - n, cm.max_tokens_per_request() - n + 1)
            if not chunked:
                want = min(want, budget - n + 1)
            assert s.status is SequenceStatus.FINISHED_LENGTH and s.num_generated_tokens == max(1, want), s
