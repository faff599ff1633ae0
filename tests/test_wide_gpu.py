"""Logits at the layer widths of the benchmarks and on the step shapes that only the benchmark
runs: a 2,048-token portion (the tcgen05 product with the fused SiLU epilogue, the tcgen05
attention kernel, the replayed portion graph), decode steps of 17 to 257 live requests (library
products between this package's kernels, the graph buckets 24 to 64, no graph above 256), at
TinyLlama-1.1B and Llama-3-8B widths with two layers each.

Three-way comparison: the float32 engine against the plain implementation (tight), the bfloat16
engine against the float32 engine (rounding of activations only: both load the same bfloat16
weight values), and the bfloat16 engine against the plain implementation.  The reference
checks its GPU model against a dense oracle on a real model in tests/test_model_gpu.py:47-54."""

import numpy as np
import pytest

from tests import plain_llama, schedules
from tests.helpers import assert_bf16_close_to_f32, assert_logits_close
from tests.tiny import random_tokens, read_folder
from tests.wide import WIDES, wide_folder

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    made = {}

    def get(name):
        if name not in made:
            made[name] = wide_folder(tmp_path_factory, name)
        return made[name]
    return get


_plain_cache: dict = {}


def plain_rows(folder, key, tokens, rows):
    """Plain logits of one request at `rows`, computed once per (test data, request)."""
    k = (folder, key)
    if k not in _plain_cache:
        cfg, w = read_folder(folder)
        _plain_cache[k] = plain_llama.forward_logits(cfg, w, tokens, rows=rows).numpy()
    return _plain_cache[k]


def replay(folder, dtype, steps, max_tokens, **kw):
    from paged_llm_b200.engine.replay import TraceReplayer

    rp = TraceReplayer(folder, dtype, max_tokens, poison=float("nan"), **kw)
    outputs = {rec["step"]: out for rec in steps if (out := rp.step(rec)) is not None}
    assert not rp.live
    rp.cm.check_invariants([])
    assert rp.cm.num_free_blocks == rp.cm.num_blocks, "pages were lost"
    timeouts = getattr(rp.ops, "kernel_timeouts", lambda: 0)()
    assert timeouts == 0, f"{timeouts} bounded waits inside kernels gave up"
    return outputs, rp


def compare_three_ways(folder, tag, reqs, steps, got32, got16):
    wanted = schedules.wanted_positions(steps)
    a, b = schedules.collect(steps, got32), schedules.collect(steps, got16)
    for rid, rows in wanted.items():
        if not rows:
            continue
        want = plain_rows(folder, (tag, rid, tuple(rows)), reqs[rid], rows)
        assert_logits_close(a[rid], want, "float32", f"{tag}/float32/{rid}")
        assert_bf16_close_to_f32(b[rid], a[rid], f"{tag}/bfloat16 against float32/{rid}")
        assert_logits_close(b[rid], want, "bfloat16", f"{tag}/bfloat16/{rid}")


# ----------------------------------------------------------------------------- prompt portions

def portion_and_tail_trace(toks, portion=2048):
    """The same 2,048 tokens as the whole first step of three requests (the second captures the
    portion graph, the third replays it), the third then decodes the remaining tokens one by
    one; a fourth brings all tokens in one step and asks for logits at many places."""
    head = toks[:portion]
    steps = [{"step": i, "entries": [{"id": rid, "tokens": head, "want": [portion - 1]}],
              "end": [rid] if rid != "c" else []} for i, rid in enumerate("abc")]
    for i in range(portion, len(toks)):
        steps.append({"step": len(steps), "entries": [{"id": "c", "tokens": [toks[i]], "want": [0]}],
                      "end": ["c"] if i == len(toks) - 1 else []})
    places = sorted(set(range(0, len(toks), 97)) | set(range(len(toks) - 40, len(toks))) | {0, 1, 15, 16, 17, 127, 128})
    steps.append({"step": len(steps), "entries": [{"id": "d", "tokens": toks, "want": places}], "end": ["d"]})
    return steps


@pytest.mark.parametrize("name", ["T", "8B"])
def test_portion_of_2048_tokens_and_decoded_tail(folders, name):
    hf, _ = WIDES[name]
    toks = random_tokens(hf["vocab_size"], 2048 + 32, 11)
    steps = portion_and_tail_trace(toks)
    reqs = {"a": toks[:2048], "b": toks[:2048], "c": toks, "d": toks}
    got = {}
    for dtype in ("float32", "bfloat16"):
        got[dtype], rp = replay(folders(name), dtype, steps, 2 * 2112)
        if dtype == "bfloat16":
            assert ("portion", 2048, 1) in rp.runner._graphs, sorted(rp.runner._graphs)
            assert rp.runner.num_graph_steps >= 2 + 32
    # a and b brought c's first tokens: one plain run of c serves all three
    rows_c = list(range(2047, 2080))
    want_c = plain_rows(folders(name), ("tail", "c"), toks, rows_c)
    wanted = schedules.wanted_positions(steps)
    a, b = schedules.collect(steps, got["float32"]), schedules.collect(steps, got["bfloat16"])
    assert wanted["c"] == rows_c and wanted["a"] == [2047]
    for rid, want in (("a", want_c[:1]), ("b", want_c[:1]), ("c", want_c)):
        assert_logits_close(a[rid], want, "float32", f"{name}/float32/{rid}")
        assert_bf16_close_to_f32(b[rid], a[rid], f"{name}/bfloat16 against float32/{rid}")
        assert_logits_close(b[rid], want, "bfloat16", f"{name}/bfloat16/{rid}")
    want_d = plain_rows(folders(name), ("whole", "d"), toks, wanted["d"])
    assert_logits_close(a["d"], want_d, "float32", f"{name}/float32/d")
    assert_bf16_close_to_f32(b["d"], a["d"], f"{name}/bfloat16 against float32/d")
    assert_logits_close(b["d"], want_d, "bfloat16", f"{name}/bfloat16/d")


WIDE_PORTIONS = (300, 2, 64, 513, 17, 129, 7, 33, 256, 3, 100, 48, 600)


def test_portions_of_changing_size(folders):
    hf, _ = WIDES["T"]
    reqs = {"p": random_tokens(hf["vocab_size"], 2080, 12), "q": random_tokens(hf["vocab_size"], 150, 13)}
    steps, max_tokens = schedules.portions(reqs, sizes=WIDE_PORTIONS)
    edges = {rid: set() for rid in reqs}
    at = {rid: 0 for rid in reqs}
    for rec in steps:
        for e in rec["entries"]:
            n = len(e["tokens"])
            edges[e["id"]] |= {at[e["id"]], at[e["id"]] + n - 1, at[e["id"]] + n // 2}
            at[e["id"]] += n
    steps = schedules.keep_wanted(steps, lambda rid, p: p in edges[rid])
    got32, _ = replay(folders("T"), "float32", steps, max_tokens)
    got16, _ = replay(folders("T"), "bfloat16", steps, max_tokens)
    compare_three_ways(folders("T"), "portions", reqs, steps, got32, got16)


def test_mixed_requests_with_reused_pages(folders):
    hf, _ = WIDES["T"]
    lengths = (700, 300, 520, 90, 410, 260, 33)
    reqs = {f"m{i}": random_tokens(hf["vocab_size"], n, 40 + i) for i, n in enumerate(lengths)}
    steps, max_tokens = schedules.mixed(reqs, live=4, seed=2, choices=(2, 5, 16, 40, 64, 130, 257))
    steps = schedules.keep_wanted(steps, lambda rid, p: p % 5 == 0 or p >= len(reqs[rid]) - 8)
    got32, rp = replay(folders("T"), "float32", steps, max_tokens)
    assert sum(-(-n // 16) for n in lengths) > rp.cm.num_blocks, "the trace must reuse pages"
    got16, _ = replay(folders("T"), "bfloat16", steps, max_tokens)
    compare_three_ways(folders("T"), "mixed", reqs, steps, got32, got16)


# ----------------------------------------------------------------------------- many requests decoding

def decode_trace(vocab, n_requests, seed, tail=3, longest=100, group=8):
    """Prompts in steps of `group` requests, then `tail` steps in which every request brings one token."""
    rng = np.random.default_rng(seed)
    lengths = rng.integers(tail + 1, longest, n_requests)
    lengths[::7] *= 5                                     # a few long ones, so that contexts are split
    reqs = {f"r{i}": random_tokens(vocab, int(n), seed * 1000 + i) for i, n in enumerate(lengths)}
    ids = list(reqs)
    steps = []
    for i in range(0, len(ids), group):
        steps.append({"step": len(steps), "end": [], "entries": [
            {"id": rid, "tokens": reqs[rid][:-tail], "want": []} for rid in ids[i:i + group]]})
    for j in range(tail):
        steps.append({"step": len(steps), "end": ids if j == tail - 1 else [], "entries": [
            {"id": rid, "tokens": [reqs[rid][len(reqs[rid]) - tail + j]], "want": [0]} for rid in ids]})
    return reqs, steps, int(sum(schedules._round64(len(t)) for t in reqs.values()))


@pytest.mark.parametrize("n_requests", [17, 24, 33, 64, 257])
def test_decode_steps_of_many_requests(folders, n_requests):
    hf, _ = WIDES["T"]
    reqs, steps, max_tokens = decode_trace(hf["vocab_size"], n_requests, seed=n_requests,
                                           longest=100 if n_requests <= 64 else 30)
    got32, _ = replay(folders("T"), "float32", steps, max_tokens, max_num_seqs=n_requests)
    got16, rp = replay(folders("T"), "bfloat16", steps, max_tokens, max_num_seqs=n_requests)
    if n_requests <= rp.runner.GRAPH_BUCKETS[-1]:
        bucket = next(b for b in rp.runner.GRAPH_BUCKETS if b >= n_requests)
        # (the three decode steps; a step of prompts in front of them may replay a graph of small mixed steps too)
        assert any(k[:2] == ("decode", bucket) for k in rp.runner._graphs) and rp.runner.num_graph_steps >= 3
        eager, rp_e = replay(folders("T"), "bfloat16", steps, max_tokens, max_num_seqs=n_requests, enforce_eager=True)
        assert rp_e.runner.num_graph_steps == 0
        for k in got16:
            assert_bf16_close_to_f32(got16[k], eager[k], f"graph against eager, step {k}")
    else:
        # more requests than the largest bucket: the decode steps run as launches (the short prompts in front of
        # them may replay graphs of small mixed steps)
        assert not any(k[0] == "decode" for k in rp.runner._graphs)
    compare_three_ways(folders("T"), f"decode{n_requests}", reqs, steps, got32, got16)


def test_random_serving_workload_for_a_few_seconds(folders):
    """Five seconds of requests arriving at random at the benchmark's widths: prompts of 1 to 1,500 tokens (half of
    them behind one of three shared prefixes), 1 to 200 output tokens, greedy / temperature / top-k / top-p, 48
    request slots, a budget of 1,024 tokens and so few pages that requests are preempted.  Nothing raises, no page
    is lost, no bounded wait in a kernel gives up, and nearly every step replays a graph."""
    import random
    import time
    from paged_llm_b200 import EngineConfig, LLMEngine, SamplingParams
    hf, _ = WIDES["T"]
    vocab = hf["vocab_size"]
    eng = LLMEngine(folders("T"), EngineConfig(dtype="bfloat16", block_size=16, max_model_len=2048, max_num_seqs=48,
                                               max_num_batched_tokens=1024, enable_prefix_caching=True,
                                               num_gpu_blocks=1200))
    eng.warm_up()
    rng = random.Random(1)
    prefixes = [[rng.randrange(vocab) for _ in range(rng.randint(16, 750))] for _ in range(3)]
    t_end, n_req, tokens = time.time() + 5.0, 0, 0
    while time.time() < t_end or eng.has_unfinished_requests:
        if time.time() < t_end and rng.random() < 0.2:
            for _ in range(rng.randint(1, 4)):
                body = [rng.randrange(vocab) for _ in range(rng.randint(1, 750))]
                prompt = rng.choice(prefixes) + body if rng.random() < 0.5 else body
                kind = rng.random()
                how = dict(temperature=0.0) if kind < 0.5 else dict(temperature=0.8, seed=n_req) if kind < 0.7 else \
                    dict(temperature=0.9, top_k=rng.choice([0, 5, 50]), top_p=rng.choice([1.0, 0.9, 0.5]), seed=n_req)
                eng.add_request(prompt[:1500], SamplingParams(max_tokens=rng.randint(1, 200), ignore_eos=True, **how))
                n_req += 1
        for out in eng.step():
            if out.new_token is not None:
                assert 0 <= out.new_token < vocab
                tokens += 1
    eng.block_manager.check_invariants([])
    assert eng.block_manager.num_free_blocks == eng.block_manager.num_blocks, "pages were lost"
    assert eng.ops.kernel_timeouts() == 0
    assert n_req > 100 and tokens > 10 * n_req and eng.stats.num_preemptions > 0
    assert eng.runner.num_graph_steps > 20 * max(1, eng.runner.num_eager_steps), (
        eng.runner.num_graph_steps, eng.runner.num_eager_steps)
