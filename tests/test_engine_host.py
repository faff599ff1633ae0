"""The engine's host logic (runner metadata, cache, scheduler, replay, entry
point) on the CPU, with the kernel library replaced by tests/torch_ops.py:
tokens must equal the plain implementation's under chunking, mixing, preemption,
prefix hits and fork, and every page must come back."""

import numpy as np
import pytest
import torch

from paged_llm_b200 import EngineConfig, LLMEngine, SamplingParams
from paged_llm_b200.engine.replay import TraceReplayer
from paged_llm_b200.engine.runner import StepItem
from paged_llm_b200.engine.sequence import Sequence
from tests import plain_llama, schedules
from tests.helpers import assert_logits_close
from tests.tiny import TINIES, make_folder, random_tokens, read_folder
from tests.torch_ops import TorchOps


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for name, (hf, init) in TINIES.items():
        d = tmp_path_factory.mktemp(f"tiny{name}")
        make_folder(d, hf, init)
        out[name] = str(d)
    return out


def engine(folder, **kw):
    cfg = dict(dtype="float32", device="cpu", block_size=8, num_gpu_blocks=64, max_model_len=128,
               max_num_batched_tokens=24)
    cfg.update(kw)
    return LLMEngine(folder, ops=TorchOps(), **cfg)


def plain_greedy(folder, prompt, n):
    cfg, w = read_folder(folder)
    return plain_llama.greedy_generate(cfg, w, prompt, n)


def test_chunked_and_mixed_generation_equals_plain(folders):
    eng = engine(folders["A"])
    prompts = [random_tokens(256, n, n) for n in (5, 30, 13, 41)]
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=10))
    for p, o in zip(prompts, outs):
        assert o.token_ids == plain_greedy(folders["A"], p, 10) and o.finish_reason == "length"
    assert eng.block_manager.num_free_blocks == 64
    assert eng.stats.num_prefill_tokens == sum(map(len, prompts)) and eng.stats.num_decode_tokens == 4 * 9


def plain_greedy_with_stop(folder, prompt, n, stop):
    toks = plain_greedy(folder, prompt, n)
    for i, t in enumerate(toks):
        if t in stop:
            return toks[:i + 1]
    return toks


@pytest.mark.parametrize("tiny", ["A", "B"])
def test_steps_that_run_ahead_change_no_token(folders, tiny):
    """Decoding overlapped (the next step launched before the last one's tokens are read)
    and not: the same tokens, the same reasons to stop, every page back.  Requests end at
    different lengths and on stop tokens that only show once the step after is on its way."""
    vocab = TINIES[tiny][0]["vocab_size"]
    prompts = [random_tokens(vocab, n, 10 + n) for n in (7, 19, 3, 26)]
    lengths = (14, 5, 22, 9)
    free_run = [plain_greedy(folders[tiny], p, n) for p, n in zip(prompts, lengths)]
    stops = [[], [free_run[1][2]], [free_run[2][9]], []]            # requests 1 and 2 stop early on a token
    sps = [SamplingParams(temperature=0.0, max_tokens=n, stop_token_ids=st) for n, st in zip(lengths, stops)]
    results = {}
    for overlap in (True, False):
        eng = engine(folders[tiny], overlap_decode=overlap, max_num_batched_tokens=64)
        outs = eng.generate(prompts, sps)
        results[overlap] = [(o.token_ids, o.finish_reason) for o in outs]
        assert eng.block_manager.num_free_blocks == 64 and not eng.has_unfinished_requests
        assert (eng.stats.num_steps_ahead > 0) == overlap
    assert results[True] == results[False]
    for (toks, reason), p, n, st in zip(results[True], prompts, lengths, stops):
        want = plain_greedy_with_stop(folders[tiny], p, n, st)
        assert toks == want and reason == ("stop" if st and want[-1] in st else "length")


def test_running_ahead_with_sampling_arrivals_and_abort(folders):
    """Seeded sampling gives the same tokens overlapped or not; a request that arrives or is
    aborted while a step is on its way is handled between steps."""
    prompts = [random_tokens(256, n, 70 + n) for n in (9, 15, 4)]
    sps = [SamplingParams(temperature=0.8, top_k=20, max_tokens=12, seed=5 + i) for i in range(3)]
    tokens = {}
    for overlap in (True, False):
        eng = engine(folders["A"], overlap_decode=overlap)
        ids = [eng.add_request(p, sp) for p, sp in zip(prompts[:2], sps[:2])]
        got: dict[int, list[int]] = {}
        steps = 0
        while eng.has_unfinished_requests:
            for o in eng.step():
                if o.new_token is not None:
                    got.setdefault(o.seq_id, []).append(o.new_token)
            steps += 1
            if steps == 4:
                ids.append(eng.add_request(prompts[2], sps[2]))      # arrives while the others decode
            if steps == 7:
                eng.abort_request(ids[1])
        tokens[overlap] = [got[i] for i in ids]
        assert eng.block_manager.num_free_blocks == 64
        assert len(got[ids[0]]) == 12 and len(got[ids[2]]) == 12 and len(got[ids[1]]) < 12
    assert tokens[True][0] == tokens[False][0] and tokens[True][2] == tokens[False][2]
    n = min(len(tokens[True][1]), len(tokens[False][1]))
    assert tokens[True][1][:n] == tokens[False][1][:n]


def test_prefix_hit(folders):
    eng = engine(folders["B"], max_num_batched_tokens=128)
    shared = random_tokens(509, 24, 7)
    prompts = [shared + [3, 4], shared + [5, 6, 7, 8]]
    first = eng.generate([prompts[0]], SamplingParams(temperature=0.0, max_tokens=6))[0]
    second = eng.generate([prompts[1]], SamplingParams(temperature=0.0, max_tokens=6))[0]
    assert first.num_cached_tokens == 0 and second.num_cached_tokens == 24
    assert first.token_ids == plain_greedy(folders["B"], prompts[0], 6)
    assert second.token_ids == plain_greedy(folders["B"], prompts[1], 6)


def test_preemption_is_lossless(folders):
    eng = engine(folders["A"], num_gpu_blocks=14, enable_prefix_caching=False)
    prompts = [random_tokens(256, n, 40 + n) for n in (20, 22, 18, 25)]
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=16))
    assert eng.stats.num_preemptions > 0 and sum(o.num_preemptions for o in outs) == eng.stats.num_preemptions
    for p, o in zip(prompts, outs):
        assert o.token_ids == plain_greedy(folders["A"], p, 16)
    assert eng.block_manager.num_free_blocks == 14


def test_fork_copies_the_shared_page(folders):
    eng = engine(folders["A"], enable_prefix_caching=False, num_gpu_blocks=32)
    sched, cm, runner = eng.scheduler, eng.block_manager, eng.runner
    base = random_tokens(256, 11, 3)                        # one full page and 3 slots of the next
    root = Sequence(base, SamplingParams(temperature=0.0, max_tokens=100))
    sched.add(root)
    out = sched.schedule(); sched.update(out, runner.run(out))
    children = []
    for tok in (50, 60):
        child = Sequence(base, SamplingParams(temperature=0.0, max_tokens=3))
        cm.fork(root, child)
        child.token_ids = base + [tok]
        child.status = root.status
        sched.running.append(child)
        children.append(child)
    sched.abort(root.seq_id)
    assert cm.blocks[children[0].block_table[1]].ref_count == 2
    while sched.has_unfinished:
        out = sched.schedule(); sched.update(out, runner.run(out))
    assert eng.ops.calls.get("copy_pages", 0) >= 1
    for child, tok in zip(children, (50, 60)):
        assert child.output_token_ids == [tok] + plain_greedy(folders["A"], base + [tok], 2)
    assert cm.num_free_blocks == 32


def test_text_prompt_without_tokenizer_and_bad_ids(folders):
    eng = engine(folders["A"])
    with pytest.raises(ValueError, match="tokenizer"):
        eng.add_request("hello")
    with pytest.raises(ValueError, match="vocabulary"):
        eng.add_request([1, 2, 999])
    with pytest.raises(ValueError, match="empty prompt"):
        eng.add_request([])


def test_pool_too_small_is_an_error_not_a_hang(folders):
    eng = engine(folders["A"], num_gpu_blocks=2)
    with pytest.raises(ValueError, match="never fit"):
        eng.generate([random_tokens(256, 40, 1)], SamplingParams(max_tokens=4))


def test_temperature_sampling_is_reproducible_and_batch_independent(folders):
    prompts = [random_tokens(509, n, n) for n in (1, 9, 40, 64, 100)]
    sp = [SamplingParams(temperature=0.7, max_tokens=12, seed=3 + i) for i in range(5)]
    together = engine(folders["B"], num_gpu_blocks=24, max_model_len=256).generate(prompts, sp)
    assert sum(o.num_preemptions for o in together) > 0           # 24 pages of 8 force preemption
    alone = [engine(folders["B"], num_gpu_blocks=24, max_model_len=256).generate([p], [s])[0]
             for p, s in zip(prompts, sp)]
    assert [o.token_ids for o in together] == [o.token_ids for o in alone]
    other = engine(folders["B"], max_model_len=256).generate(
        prompts[:1], [SamplingParams(temperature=0.7, max_tokens=12, seed=99)])
    assert other[0].token_ids != together[0].token_ids


@pytest.mark.parametrize("schedule", ["whole", "tail", "portions", "mixed"])
def test_replay_schedules_on_the_host(folders, schedule):
    hf, _ = TINIES["C"]
    reqs = {f"r{i}": random_tokens(hf["vocab_size"], n, i) for i, n in enumerate((3, 70, 90, 48, 33))}
    steps, max_tokens = getattr(schedules, schedule)(reqs)
    rp = TraceReplayer(folders["C"], "float32", max_tokens, device="cpu", ops=TorchOps(), block_size=16,
                       poison=float("nan"))
    outputs = {rec["step"]: out for rec in steps if (out := rp.step(rec)) is not None}
    got = schedules.collect(steps, outputs)
    cfg, w = read_folder(folders["C"])
    for rid, toks in reqs.items():
        want = plain_llama.forward_logits(cfg, w, toks).numpy()
        assert np.abs(got[rid] - want).max() < 2e-5, (schedule, rid)
    assert rp.cm.num_free_blocks == rp.cm.num_blocks


def test_replay_reports_a_pool_that_is_too_small(folders):
    rp = TraceReplayer(folders["A"], "float32", 32, device="cpu", ops=TorchOps())
    with pytest.raises(RuntimeError, match="max-tokens"):
        rp.step({"step": 0, "entries": [{"id": "a", "tokens": list(range(40)), "want": []}], "end": []})


def test_toy_architecture_with_state_steps_on_the_host(tmp_path):
    """A mixer with state of its own, a layer run twice and a run that reads
    another run's cache: registered by the test, no change to the package."""
    from paged_llm_b200.weights import write_model_folder
    from tests.toy_parts import TOY, ToyConfig, plain_toy_logits

    write_model_folder(str(tmp_path), ToyConfig.from_hf_dict(TOY), seed=4, std=0.1, norm_std=0.05)
    cfg, w = read_folder(tmp_path)
    reqs = {"a": random_tokens(61, 50, 1), "b": random_tokens(61, 37, 2), "c": random_tokens(61, 64, 3)}
    steps, max_tokens = schedules.mixed(reqs, live=2, seed=4)
    rp = TraceReplayer(str(tmp_path), "float32", max_tokens, device="cpu", ops=TorchOps())
    assert rp.storage.num_state_slots > 0 and rp.storage.num_groups == 1
    assert len(rp.storage.pools[0]) == 1                     # two runs of the attention layer share one cache
    outputs = {rec["step"]: out for rec in steps if (out := rp.step(rec)) is not None}
    got = schedules.collect(steps, outputs)
    for rid, toks in reqs.items():
        assert np.abs(got[rid] - plain_toy_logits(cfg, w, toks).numpy()).max() < 2e-5, rid
    assert rp.cm.num_free_state_slots == rp.cm.num_state_slots


@pytest.mark.parametrize("which", ["A", "B"])
def test_routed_toy_steps_on_the_host(tmp_path, which):
    """A position encoding, an embedding and a routed feed-forward of the test's own:
    registered, built from a written folder and stepped, no change to the package."""
    from paged_llm_b200.weights import write_model_folder
    from tests.toy_parts import ROUTED_TOY_A, ROUTED_TOY_B, RoutedToyConfig, plain_routed_toy_logits

    hf = {"A": ROUTED_TOY_A, "B": ROUTED_TOY_B}[which]
    write_model_folder(str(tmp_path), RoutedToyConfig.from_hf_dict(hf), seed=6, std=0.1, norm_std=0.05)
    cfg, w = read_folder(tmp_path)
    assert cfg == hf
    V = hf["vocab_size"]
    reqs = {"a": random_tokens(V, 45, 1), "b": random_tokens(V, 70, 2), "c": random_tokens(V, 33, 3)}
    steps, max_tokens = schedules.mixed(reqs, live=2, seed=5)
    rp = TraceReplayer(str(tmp_path), "float32", max_tokens, device="cpu", ops=TorchOps())
    assert rp.storage.num_state_slots == 0 and rp.storage.num_groups == 1
    outputs = {rec["step"]: out for rec in steps if (out := rp.step(rec)) is not None}
    got = schedules.collect(steps, outputs)
    for rid, toks in reqs.items():
        assert_logits_close(got[rid], plain_routed_toy_logits(cfg, w, toks).numpy(), "float32", rid)


def test_learned_positions_refuse_a_position_beyond_the_table(tmp_path):
    from paged_llm_b200.weights import write_model_folder
    from tests.toy_parts import ROUTED_TOY_A, RoutedToyConfig

    hf = {**ROUTED_TOY_A, "max_position_embeddings": 8}
    write_model_folder(str(tmp_path), RoutedToyConfig.from_hf_dict(hf), seed=6, std=0.2)
    rp = TraceReplayer(str(tmp_path), "float32", 64, device="cpu", ops=TorchOps())
    with pytest.raises(ValueError, match="the table has 8 rows"):
        rp.step({"step": 0, "entries": [{"id": "a", "tokens": list(range(9)), "want": []}], "end": []})


# ---- what a replayed graph has baked in -----------------------------------------------------

class PlanningOps(TorchOps):
    """The test double with the B200's planning figures, so that the runner's graph keys and
    in-place metadata patches can be exercised on the host."""

    num_sms, MAX_SPLITS, MAX_CLUSTER, CLUSTER_KEYS, MIN_SPLIT_KEYS = 148, 32, 8, 600, 128

    def long_context_class(self, num_requests, num_kv_heads, max_context):
        from paged_llm_b200.kernels.plan import is_long_context
        return is_long_context(num_requests, num_kv_heads, self.num_sms, self.MAX_SPLITS, self.MAX_CLUSTER,
                               self.CLUSTER_KEYS, max_context)

    def plan_attention(self, q_lens, k_lens, group_size, num_kv_heads, window, head_dim, pad_requests=None,
                       fixed_capacity=False, pad_tokens=None):
        from paged_llm_b200.kernels.plan import plan_attention
        return plan_attention(q_lens, k_lens, group_size, num_kv_heads, window, small_rows=16, large_rows=64,
                              min_split_keys=self.MIN_SPLIT_KEYS, num_sms=self.num_sms, max_splits=self.MAX_SPLITS,
                              pad_requests=pad_requests, fixed_capacity=fixed_capacity,
                              cluster_max=self.MAX_CLUSTER, long_keys=self.CLUSTER_KEYS, pad_tokens=pad_tokens)


def runner_with_two_plan_keys(folder, max_tokens=8192):
    rp = TraceReplayer(folder, "float32", max_tokens, device="cpu", ops=PlanningOps(), block_size=16)
    runner = rp.runner
    runner.use_graphs = True
    # two attention shapes in one model: 4 kv heads and 37 kv heads (the second splits less, so the
    # two change class at different context lengths)
    runner.plan_keys = [(8, 4, None, 64), (1, 37, None, 64)]
    return rp, runner


def test_graph_key_keeps_the_context_class_of_every_attention_shape(folders):
    rp, runner = runner_with_two_plan_keys(folders["A"])
    ops = rp.ops

    def key_at(context):
        seq = Sequence([1] * (context + 1), SamplingParams())
        seq.num_computed_tokens = context
        return runner._graph_key([StepItem(seq, 1, (0,))])

    assert key_at(100) == ("decode", 1)
    edges = [min(c for c in range(1, 20000, 7) if ops.long_context_class(1, nkv, c + 1)) for nkv in (4, 37)]
    assert edges[0] != edges[1], "the two shapes must change class at different contexts for this test"
    lo, hi = sorted(edges)
    first = (edges[0] == lo, edges[1] == lo)
    assert key_at(lo + 7) == ("decode", 1, first)
    assert key_at(hi + 7) == ("decode", 1, (True, True))
    # every class tuple is a graph of its own, so no graph is replayed with a plan of another class
    assert len({key_at(c) for c in (100, lo + 7, hi + 7)}) == 3


def test_patched_metadata_never_outgrows_the_captured_sections(folders):
    """A plan whose lists, split count or class differ from what the graph was captured with is
    not patched into the packed buffer (it would overrun the next section)."""
    from paged_llm_b200.engine.runner import _Graph
    rp, runner = runner_with_two_plan_keys(folders["A"], max_tokens=8 * 4096)
    seqs = []
    for _ in range(8):
        seq = Sequence([1] * 4000, SamplingParams())
        seq.num_computed_tokens = 100
        seq.block_tables = [list(range(250))]
        seqs.append(seq)
    items = [StepItem(seq, 1, (0,)) for seq in seqs]
    pk, host, info = runner._gather(items, pad_to=8, table_stride=runner._table_stride())
    entry = _Graph(None, None, None, pk.size, 0, 8)
    entry.packed = np.zeros(pk.size, np.int32)
    for _, off, data in pk.sections:
        entry.packed[off:off + data.size] = data
    entry.offsets = {name: off for name, off, _ in pk.sections}
    entry.seq_ids, entry.versions, entry.strides = tuple(s.seq_id for s in seqs), [s.table_version for s in seqs], info["strides"]
    entry.plan_shapes = runner._plan_shapes(info["plans"])
    for seq in seqs:
        seq.num_computed_tokens = 101
    assert runner._patch_decode(items, entry) and entry.packed[entry.offsets["pos"]] == 101
    for seq in seqs:
        seq.num_computed_tokens = 3900                # long-context class for the first shape: other capacity
    assert not runner._patch_decode(items, entry) and entry.packed is None
    sizes = {name: data.size for name, _, data in pk.sections}
    key = runner.plan_keys[0]
    other = rp.ops.plan_attention([1] * 8, [3901] * 8, *key, pad_requests=8, fixed_capacity=True)
    assert other["small"].size > sizes[f"small{key}"], "the other class has longer lists: patching would overrun"
    assert other["max_splits"] != info["plans"][key]["max_splits"]


def test_step_refuses_positions_past_the_table(folders):
    rp = TraceReplayer(folders["A"], "float32", 64, device="cpu", ops=TorchOps(), block_size=16)
    seq = Sequence([1] * 80, SamplingParams())
    with pytest.raises(ValueError, match="max_model_len"):
        rp.runner.step([StepItem(seq, 65, ())])


class FaultyOps(TorchOps):
    """A kernel library one of whose bounded waits has given up."""

    def check_kernels(self):
        from paged_llm_b200.kernels.errors import KernelError
        raise KernelError("1 bounded wait(s) inside kernels gave up")


def test_a_kernel_fault_is_an_error_not_a_token(folders):
    from paged_llm_b200.kernels.errors import KernelError
    eng = LLMEngine(folders["A"], ops=FaultyOps(), dtype="float32", device="cpu", block_size=8, num_gpu_blocks=64,
                    max_model_len=128)
    with pytest.raises(KernelError, match="gave up"):
        eng.generate([random_tokens(256, 5, 1)], SamplingParams(temperature=0.0, max_tokens=3))
    rp = TraceReplayer(folders["A"], "float32", 64, device="cpu", ops=FaultyOps(), block_size=16)
    with pytest.raises(KernelError, match="gave up"):
        rp.step({"step": 0, "entries": [{"id": "a", "tokens": [1, 2, 3], "want": [2]}], "end": []})


def test_tiny_b_workload_preempts_and_hits_the_prefix_cache(folders):
    """The workload of tests/test_generate_gpu.py::tiny_b_workload on the host: its requests are
    preempted, one of them finds the shared prefix in the cache, and every token is the plain draw."""
    from tests.plain_sampling import gumbel_scores
    from tests.test_generate_gpu import tiny_b_workload
    prompts, sps = tiny_b_workload()
    eng = engine(folders["B"], num_gpu_blocks=24, max_model_len=256, max_num_batched_tokens=32)
    outs = eng.generate(prompts, sps)
    assert eng.stats.num_preemptions > 0 and eng.block_manager.num_cache_hits > 0
    assert max(o.num_cached_tokens for o in outs) >= 16 and eng.block_manager.num_free_blocks == 24
    cfg, w = read_folder(folders["B"])
    for p, sp, o in zip(prompts, sps, outs):
        seq = list(p)
        for tok in o.token_ids:
            scores = gumbel_scores(plain_llama.forward_logits(cfg, w, seq)[-1].numpy(), 0.7, -1, 1.0, sp.seed, len(seq))
            assert scores.max() - scores[tok] < 1e-3
            seq.append(tok)


def test_score_modifiers_reach_the_attention_part(tmp_path):
    """The Llama with a bias by distance and a score cap (tests/toy_parts.py) on the host."""
    from tests.toy_parts import biased_llama_case
    hf, w, reqs, plain = biased_llama_case(tmp_path)
    steps, max_tokens = schedules.mixed(reqs, live=3, seed=6)
    rp = TraceReplayer(str(tmp_path), "float32", max_tokens, device="cpu", ops=TorchOps(), poison=float("nan"))
    outputs = {rec["step"]: out for rec in steps if (out := rp.step(rec)) is not None}
    got = schedules.collect(steps, outputs)
    for rid, toks in reqs.items():
        assert np.abs(got[rid] - plain(toks)).max() < 2e-5, rid
    without = plain_llama.forward_logits(hf, w, reqs["a"]).numpy()
    assert np.abs(without - plain(reqs["a"])).max() > 0.05 * np.abs(without).max(), "the modifiers must matter here"


def test_fork_gives_the_child_a_copy_of_the_state(tmp_path):
    """A model with state of fixed size: `fork` hands the child a slot of its own and queues a
    copy of the parent's state, which the next step carries out before it runs."""
    from paged_llm_b200.weights import write_model_folder
    from tests.toy_parts import TOY, ToyConfig, plain_toy_logits
    write_model_folder(str(tmp_path), ToyConfig.from_hf_dict(TOY), seed=4, std=0.1, norm_std=0.05)
    cfg, w = read_folder(tmp_path)
    eng = LLMEngine(str(tmp_path), ops=TorchOps(), dtype="float32", device="cpu", block_size=8, num_gpu_blocks=32,
                    max_model_len=128, max_num_seqs=4)
    sched, cm, runner = eng.scheduler, eng.block_manager, eng.runner
    base = random_tokens(61, 21, 3)
    root = Sequence(base, SamplingParams(temperature=0.0, max_tokens=50, ignore_eos=True))
    sched.add(root)
    out = sched.schedule(); sched.update(out, runner.run(out))
    child = Sequence(base, SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True))
    cm.fork(root, child)
    assert child.state_slot is not None and child.state_slot != root.state_slot
    child.token_ids = base + [7]
    child.status = root.status
    sched.running.append(child)
    while sched.has_unfinished and not child.is_finished:
        out = sched.schedule(); sched.update(out, runner.run(out))
    toks = base + [7]
    for tok in child.output_token_ids[1:]:
        assert tok == int(plain_toy_logits(cfg, w, toks)[-1].argmax())
        toks.append(tok)
    # the parent went on from its own state, untouched by the child
    toks = list(base)
    for tok in root.output_token_ids[:5]:
        assert tok == int(plain_toy_logits(cfg, w, toks)[-1].argmax())
        toks.append(tok)
    sched.abort(root.seq_id)
    assert cm.num_free_state_slots == cm.num_state_slots and cm.num_free_blocks == 32


def test_plan_of_a_mixed_step_with_fixed_capacity():
    """The work lists of a step of mixed items that replays a graph: their sizes depend on the token and request
    capacity only, items beyond the step's own are request -1, and a step that does not fit is refused."""
    from paged_llm_b200.kernels.plan import PlanCapacityError, large_capacity, plan_attention
    kw = dict(small_rows=16, large_rows=128, min_split_keys=128, num_sms=148, pad_requests=64, fixed_capacity=True,
              pad_tokens=256)
    sizes = set()
    for q_lens, k_lens in (([1, 1, 100], [30, 500, 100]), ([2] * 20 + [7, 9], [50] * 20 + [7, 300]), ([200], [1200]),
                           ([1] * 64, [9] * 64)):
        plan = plan_attention(q_lens, k_lens, 8, 4, None, **kw)
        small, large = plan["small"].reshape(-1, 4), plan["large"].reshape(-1, 4)
        sizes.add((small.shape[0], large.shape[0], plan["max_splits"], plan["num_small_tokens"]))
        assert large.shape[0] == large_capacity(256, 8, 16, 128)
        real_large = large[large[:, 0] >= 0]
        want_tiles = sum(-(-q * 8 // 128) for q in q_lens if q * 8 > 16)
        assert len(real_large) == want_tiles and (large[len(real_large):, 0] == -1).all()
        real_small = small[small[:, 0] >= 0]
        assert sorted(set(real_small[:, 0].tolist())) == [s for s, q in enumerate(q_lens) if q * 8 <= 16]
        assert plan["num_small_tokens"] >= sum(q for q in q_lens if q * 8 <= 16)
    assert len(sizes) == 1, "the capacity must not depend on the step's items"
    with pytest.raises(PlanCapacityError):
        plan_attention([300], [300], 8, 4, None, **kw)                     # more tokens than the graph holds


def test_small_mixed_steps_get_a_graph_key_and_metadata_of_one_size(folders):
    """Steps of mixed items: the key is the bucket of 64 tokens (from the second time on), every step of a bucket
    packs metadata of the same size whatever its items, padding is what the kernels skip (request -1, no keys),
    and a step that does not fit is refused so that it runs as launches."""
    from paged_llm_b200.kernels.plan import PlanCapacityError
    rp, runner = runner_with_two_plan_keys(folders["A"], max_tokens=64 * 1024)
    runner.mixed_graphs = True

    def items_of(specs):
        out = []
        for context, new, want in specs:
            seq = Sequence([1] * (context + new), SamplingParams())
            seq.num_computed_tokens = context
            seq.block_tables = [list(range(-(-(context + new) // 16)))]
            out.append(StepItem(seq, new, want))
        return out

    a = items_of([(300, 1, (0,)), (20, 1, (0,)), (0, 90, (89,))])              # 92 tokens: bucket 128
    b = items_of([(0, 100, ()), (0, 7, (6,)), (700, 2, (1,)), (5, 1, (0,))])   # 110 tokens: bucket 128
    c = items_of([(0, 200, (199,)), (50, 1, (0,))])                            # bucket 256
    assert runner._graph_key(a) is None, "a bucket is captured when it comes the second time"
    assert runner._graph_key(b) == ("mixed", 128) and runner._graph_key(c) is None
    assert runner._graph_key(items_of([(0, 1100, (1099,)), (50, 1, (0,))])) is None        # more than 1,024 tokens
    sizes = set()
    for items in (a, b):
        pk, host, info = runner._gather(items, table_stride=runner._table_stride(), pad_mixed=(128, runner.MIXED_GRAPH_SEQS))
        sizes.add((pk.size, str(runner._plan_shapes(info["plans"]))))
        sec = {name: data for name, _, data in pk.sections}
        T, S = sum(i.num_new_tokens for i in items), len(items)
        assert info["T"] == 128 and info["S"] == runner.MIXED_GRAPH_SEQS and info["padded"] and not info["logits_all"]
        assert (sec["tseq"][T:] == -1).all() and (sec["tseq"][:T] >= 0).all()
        assert (sec["cu"][S:] == T).all() and (sec["klen"][S:] == 0).all()
        assert sec["lidx"].size == runner.MIXED_GRAPH_SEQS and info["L"] == sum(len(i.want) for i in items)
    assert len(sizes) == 1, "every step of a bucket must pack metadata of the same layout"
    with pytest.raises(PlanCapacityError):
        runner._gather(c, table_stride=runner._table_stride(), pad_mixed=(128, runner.MIXED_GRAPH_SEQS))


def test_a_graph_that_does_not_fit_the_memory_is_given_up_for_launches(folders, monkeypatch):
    """Capturing a graph that runs out of device memory: the step runs as launches, the key is not tried
    again, other keys still are."""
    rp = TraceReplayer(folders["A"], "float32", 256, device="cpu", ops=TorchOps(), block_size=16)
    runner = rp.runner
    runner.use_graphs = True
    calls = []

    def no_room(key, *a, **k):
        calls.append(key)
        raise torch.OutOfMemoryError("CUDA out of memory (made up by the test)")
    monkeypatch.setattr(runner, "_capture", no_room)
    for step in range(3):
        out = rp.step({"step": step, "entries": [{"id": "a", "tokens": [5 + step], "want": [0]}], "end": []})
        assert out is not None and np.isfinite(out).all()
    assert calls == [("decode", 1)] and ("decode", 1) in runner._no_graph and runner.num_graph_steps == 0
    assert runner.num_eager_steps == 3
