"""Generation through the Python entry point and the command line on the GPU:
greedy tokens against the plain implementation, long decoding, the first tokens
of a sequence, temperature sampling, preemption, prefix hits."""

import os
import subprocess
import sys

import numpy as np
import pytest

from tests import plain_llama
from tests.helpers import assert_logits_close, model_folder, plain_logits
from tests.tiny import TINIES, random_tokens, read_folder

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {name: model_folder(tmp_path_factory, name) for name in TINIES}


def plain_greedy(folder, prompt, n):
    cfg, w = read_folder(folder)
    return plain_llama.greedy_generate(cfg, w, prompt, n)


@pytest.mark.parametrize("name,block,blocks", [("A", 16, 32), ("B", 8, 24)])
def test_greedy_generation_float32(folders, name, block, blocks):
    from paged_llm_b200 import LLMEngine, SamplingParams
    hf, _ = TINIES[name]
    lengths = (5, 17, 33) if name == "A" else (1, 9, 40, 64, 100)
    prompts = [random_tokens(hf["vocab_size"], n, 10 + n) for n in lengths]
    eng = LLMEngine(folders[name], dtype="float32", block_size=block, num_gpu_blocks=blocks, max_model_len=128,
                    max_num_batched_tokens=32)
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=8))
    for p, o in zip(prompts, outs):
        assert o.token_ids == plain_greedy(folders[name], p, 8)
    if name == "B":
        assert eng.stats.num_preemptions > 0, "24 pages of 8 tokens cannot hold all five requests"
    assert eng.block_manager.num_free_blocks == blocks
    assert eng.runner.num_graph_steps > 0 and eng.ops.launches > 0


def test_steps_that_run_ahead_change_no_token_on_the_device(folders):
    """The next decode step launched before the last one's tokens are read (its input ids taken
    from the device) against the step-by-step engine: the same tokens, greedy and sampled, with
    requests that end at different lengths and on a stop token."""
    from paged_llm_b200 import LLMEngine, SamplingParams
    hf, _ = TINIES["A"]
    prompts = [random_tokens(hf["vocab_size"], n, 30 + n) for n in (6, 21, 2, 12)]
    free_run = plain_greedy(folders["A"], prompts[1], 12)
    sps = [SamplingParams(temperature=0.0, max_tokens=15),
           SamplingParams(temperature=0.0, max_tokens=12, stop_token_ids=[free_run[6]]),
           SamplingParams(temperature=0.9, top_p=0.9, max_tokens=20, seed=11),
           SamplingParams(temperature=0.0, max_tokens=4)]
    got = {}
    for overlap in (True, False):
        eng = LLMEngine(folders["A"], dtype="float32", block_size=16, num_gpu_blocks=32, max_model_len=128,
                        overlap_decode=overlap)
        got[overlap] = [(o.token_ids, o.finish_reason) for o in eng.generate(prompts, sps)]
        assert (eng.stats.num_steps_ahead > 0) == overlap
        assert eng.block_manager.num_free_blocks == 32 and not eng.has_unfinished_requests
    assert got[True] == got[False]
    assert got[True][0][0] == plain_greedy(folders["A"], prompts[0], 15)
    assert got[True][1] == (free_run[:free_run.index(free_run[6]) + 1], "stop")


def test_greedy_generation_bfloat16_follows_the_plain_model(folders):
    """bfloat16 may flip a near-tie; every generated token must be the argmax or
    within rounding of it in the plain model's logits for the same prefix."""
    from paged_llm_b200 import LLMEngine, SamplingParams
    hf, _ = TINIES["C"]
    prompts = [random_tokens(hf["vocab_size"], n, 20 + n) for n in (3, 30, 77)]
    eng = LLMEngine(folders["C"], dtype="bfloat16", num_gpu_blocks=64, max_model_len=256)
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=10))
    for p, o in zip(prompts, outs):
        seq = list(p)
        for tok in o.token_ids:
            ref = plain_logits(folders["C"], seq)[-1]
            assert ref.max() - ref[tok] <= 3e-2 * np.abs(ref).max()
            seq.append(tok)


def test_warm_up_captures_the_decode_graphs(folders):
    from paged_llm_b200 import LLMEngine, SamplingParams
    eng = LLMEngine(folders["A"], dtype="float32", block_size=16, num_gpu_blocks=32, max_model_len=128, max_num_seqs=8)
    # the decode buckets up to max_num_seqs, and the one bucket of small mixed steps that fits max_model_len=128
    want = {("decode", b) for b in (1, 2, 4, 8)} | ({("mixed", 64)} if eng.runner.mixed_graphs else set())
    assert eng.warm_up() == len(want) and set(eng.runner._graphs) == want
    assert eng.block_manager.num_free_blocks == 32 and eng.stats.num_steps == 0
    hf, _ = TINIES["A"]
    prompt = random_tokens(hf["vocab_size"], 9, 3)
    out = eng.generate([prompt], SamplingParams(temperature=0.0, max_tokens=6))[0]
    assert out.token_ids == plain_greedy(folders["A"], prompt, 6)
    assert set(eng.runner._graphs) == want


def test_decoding_across_the_context_classes(folders):
    """A decode step is planned as clusters while contexts are short and through the work list
    once they are long, with a CUDA graph per class.  The limit is lowered here so that a short
    generation crosses it: tokens must follow the plain model on both sides of the change."""
    from paged_llm_b200 import LLMEngine, SamplingParams
    hf, _ = TINIES["C"]
    prompts = [random_tokens(hf["vocab_size"], n, 50 + n) for n in (5, 21)]
    eng = LLMEngine(folders["C"], dtype="bfloat16", num_gpu_blocks=64, max_model_len=256)
    if not eng.ops.cluster_attention:
        pytest.skip("without clusters there is one decode class only")
    eng.ops.CLUSTER_KEYS = 5                      # 5 keys x 8 blocks: contexts above 40 tokens are "long"
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=40))
    keys = set(eng.runner._graphs)
    assert ("decode", 2) in keys and ("decode", 2, (True,)) in keys, keys
    for p, o in zip(prompts, outs):
        seq = list(p)
        for tok in o.token_ids:
            ref = plain_logits(folders["C"], seq)[-1]
            assert ref.max() - ref[tok] <= 3e-2 * np.abs(ref).max()
            seq.append(tok)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(folders, dtype):
    """300 decoded tokens from a short prompt, teacher-forced, against the plain logits."""
    from paged_llm_b200.engine.replay import TraceReplayer
    hf, _ = TINIES["C"]
    toks = random_tokens(hf["vocab_size"], 305, 77)
    rp = TraceReplayer(folders["C"], dtype, 320)
    rows = [rp.step({"step": 0, "entries": [{"id": "a", "tokens": toks[:5], "want": [4]}], "end": []})[0]]
    for i in range(5, 305):
        rows.append(rp.step({"step": i, "entries": [{"id": "a", "tokens": [toks[i]], "want": [0]}], "end": []})[0])
    assert_logits_close(np.stack(rows), plain_logits(folders["C"], toks)[4:], dtype, "long decoding")
    assert rp.runner.num_graph_steps == 300


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_of_a_sequence(folders, dtype):
    """A prompt of one token, then single tokens: positions 0, 1, 2, ... each on their own."""
    from paged_llm_b200.engine.replay import TraceReplayer
    hf, _ = TINIES["B"]
    toks = random_tokens(hf["vocab_size"], 12, 5)
    rp = TraceReplayer(folders["B"], dtype, 64, block_size=8)
    rows = [rp.step({"step": i, "entries": [{"id": "a", "tokens": [t], "want": [0]}], "end": []})[0]
            for i, t in enumerate(toks)]
    assert_logits_close(np.stack(rows), plain_logits(folders["B"], toks), dtype, "first tokens")


def test_temperature_sampling_follows_the_plain_draw(folders):
    """Tiny B, temperature 0.7: each sampled token is what the plain sampler draws
    from the plain logits with the same stream."""
    from paged_llm_b200 import LLMEngine, SamplingParams
    from tests.plain_sampling import gumbel_scores
    hf, _ = TINIES["B"]
    prompts = [random_tokens(hf["vocab_size"], n, n) for n in (1, 9, 40)]
    sps = [SamplingParams(temperature=0.7, max_tokens=12, seed=3 + i) for i in range(3)]
    eng = LLMEngine(folders["B"], dtype="float32", block_size=8, num_gpu_blocks=24, max_model_len=256)
    outs = eng.generate(prompts, sps)
    for p, sp, o in zip(prompts, sps, outs):
        seq = list(p)
        for tok in o.token_ids:
            scores = gumbel_scores(plain_logits(folders["B"], seq)[-1], 0.7, -1, 1.0, sp.seed, len(seq))
            assert scores.max() - scores[tok] < 1e-3
            seq.append(tok)
    again = LLMEngine(folders["B"], dtype="float32", block_size=8, num_gpu_blocks=24, max_model_len=256).generate(prompts, sps)
    assert [o.token_ids for o in again] == [o.token_ids for o in outs]


def tiny_b_workload():
    """The second tiny configuration's workload: prompts of 1, 9, 40, 64 and 100 tokens, the
    100-token one opening with the first 16 tokens (two pages of 8) of the 40-token one,
    temperature 0.7 with seed 3, 12 tokens each, on 24 pages of 8 tokens."""
    from paged_llm_b200 import SamplingParams
    hf, _ = TINIES["B"]
    prompts = [random_tokens(hf["vocab_size"], n, 60 + n) for n in (1, 9, 40, 64, 100)]
    prompts[4][:16] = prompts[2][:16]
    sps = [SamplingParams(temperature=0.7, max_tokens=12, seed=3, ignore_eos=True) for _ in prompts]
    return prompts, sps


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_tiny_b_workload_with_preemption_and_a_shared_prefix(tmp_path_factory, dtype):
    """Sampled generation under preemption by recompute with a prefix hit, in both precisions:
    every token is what the plain sampler draws from the plain logits of the same prefix.  The
    folder holds bfloat16 values, so both precisions and the plain model use the same weights."""
    from paged_llm_b200 import LLMEngine
    from tests.helpers import BF16_VS_F32_TOL
    from tests.plain_sampling import gumbel_scores
    folder = model_folder(tmp_path_factory, "B", dtype="bfloat16")
    prompts, sps = tiny_b_workload()
    eng = LLMEngine(folder, dtype=dtype, block_size=8, num_gpu_blocks=24, max_model_len=256, max_num_batched_tokens=32)
    outs = eng.generate(prompts, sps)
    assert eng.stats.num_preemptions > 0, "24 pages of 8 tokens cannot hold all five requests"
    assert eng.block_manager.num_cache_hits > 0 and max(o.num_cached_tokens for o in outs) >= 16
    assert eng.block_manager.num_free_blocks == 24
    for p, sp, o in zip(prompts, sps, outs):
        assert len(o.token_ids) == 12
        seq = list(p)
        for tok in o.token_ids:
            row = plain_logits(folder, seq)[-1]
            scores = gumbel_scores(row, 0.7, -1, 1.0, sp.seed, len(seq))
            slack = 1e-3 if dtype == "float32" else 2 * BF16_VS_F32_TOL * float(np.abs(row).max()) / 0.7
            assert scores.max() - scores[tok] <= slack, (dtype, len(p), len(seq))
            seq.append(tok)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_fork_copies_the_shared_page_on_the_device(folders, dtype):
    """fork -> both children write into the shared, partly filled page -> copy-on-write -> both
    decode: the copied page is read through the attention kernels (reference:
    pagedllm/block_manager.py:195-231)."""
    from paged_llm_b200 import LLMEngine, SamplingParams
    from paged_llm_b200.engine.sequence import Sequence
    eng = LLMEngine(folders["A"], dtype=dtype, block_size=8, num_gpu_blocks=32, max_model_len=128,
                    enable_prefix_caching=False)
    eng.kv_cache.fill(float("nan"))
    sched, cm, runner = eng.scheduler, eng.block_manager, eng.runner
    base = random_tokens(256, 11, 3)                        # one full page and 3 slots of the next
    root = Sequence(base, SamplingParams(temperature=0.0, max_tokens=100))
    sched.add(root)
    out = sched.schedule()
    sched.update(out, runner.run(out))
    children = []
    for tok in (50, 60):
        child = Sequence(base, SamplingParams(temperature=0.0, max_tokens=4))
        cm.fork(root, child)
        child.token_ids = base + [tok]
        child.status = root.status
        sched.running.append(child)
        children.append(child)
    sched.abort(root.seq_id)
    assert cm.blocks[children[0].block_table[1]].ref_count == 2
    copies, take = [], cm.take_pending_copies

    def counted():
        got = take()
        copies.extend(got)
        return got
    cm.take_pending_copies = counted
    while sched.has_unfinished:
        out = sched.schedule()
        sched.update(out, runner.run(out))
    assert len(copies) == 1, "the first child to write gets a copy of the shared page, the second keeps the page"
    for child, tok in zip(children, (50, 60)):
        seq = base + [tok]
        for got in child.output_token_ids[1:]:
            ref = plain_logits(folders["A"], seq)[-1]
            assert ref.max() - ref[got] <= (1e-4 if dtype == "float32" else 3e-2 * np.abs(ref).max())
            seq.append(got)
        assert len(child.output_token_ids) == 4
    assert cm.num_free_blocks == 32


def test_pool_sized_from_measured_memory(folders):
    """`num_gpu_blocks=None`: the pool is sized from the device's free memory and the measured
    peak of one largest step (reference: pagedllm/engine.py:161-179)."""
    import torch
    from paged_llm_b200 import LLMEngine, SamplingParams
    hf, _ = TINIES["A"]
    free0, total = torch.cuda.mem_get_info()
    eng = LLMEngine(folders["A"], dtype="bfloat16", block_size=16, max_model_len=128, max_num_seqs=8,
                    max_num_batched_tokens=256, gpu_memory_utilization=0.5)
    blocks = eng.block_manager.num_blocks
    # capped by what eight requests of full length can use; far below half of the device
    assert blocks == 8 * (128 // 16) + 16
    assert eng.activation_peak_bytes is not None and eng.activation_peak_bytes > 256 * hf["hidden_size"] * 4
    free1, _ = torch.cuda.mem_get_info()
    assert total - free1 <= 0.5 * total + (total - free0)
    prompt = random_tokens(hf["vocab_size"], 9, 3)
    out = eng.generate([prompt], SamplingParams(temperature=0.0, max_tokens=6))[0]
    seq = list(prompt)
    for tok in out.token_ids:
        ref = plain_logits(folders["A"], seq)[-1]
        assert ref.max() - ref[tok] <= 3e-2 * np.abs(ref).max()
        seq.append(tok)
    # without the cap of the request limit the pool takes what the budget allows
    big = LLMEngine(folders["A"], dtype="bfloat16", block_size=16, max_model_len=4096, max_num_seqs=256,
                    max_num_batched_tokens=256, gpu_memory_utilization=0.02 + (total - free1) / total)
    page_bytes = big.kv_cache.page_bytes()
    assert 16 <= big.block_manager.num_blocks * page_bytes <= 0.025 * total


def test_prefix_hit_and_stats(folders):
    from paged_llm_b200 import LLMEngine, SamplingParams
    hf, _ = TINIES["A"]
    shared = random_tokens(hf["vocab_size"], 48, 1)
    eng = LLMEngine(folders["A"], dtype="float32", num_gpu_blocks=32, max_model_len=128)
    a = eng.generate([shared + [1, 2]], SamplingParams(temperature=0.0, max_tokens=4))[0]
    b = eng.generate([shared + [3, 4, 5]], SamplingParams(temperature=0.0, max_tokens=4))[0]
    assert a.num_cached_tokens == 0 and b.num_cached_tokens == 48
    assert b.token_ids == plain_greedy(folders["A"], shared + [3, 4, 5], 4)
    assert eng.block_manager.num_cache_hits == 1


def test_command_line(folders):
    proc = subprocess.run(
        [sys.executable, os.path.join(ROOT, "examples", "generate.py"), "--model", folders["A"], "--dtype", "float32",
         "--max-tokens", "5", "--temperature", "0.0", "--prompt-ids", "5,17,3", "--prompt-ids", "9", "--num-blocks", "32",
         "--max-model-len", "128"],
        capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    want = [plain_greedy(folders["A"], p, 5) for p in ([5, 17, 3], [9])]
    for w in want:
        assert str(w) in proc.stdout, proc.stdout
    assert "steps=" in proc.stdout and "preemptions=0" in proc.stdout


def test_random_arrivals_with_graphs_and_as_launches(folders):
    """Sixty requests of random lengths arriving in random order between steps, with a small token budget and few
    pages, so that most steps are mixed ones and some requests are preempted: greedy tokens in float32 with every
    kind of graph (decode buckets, recurring portions, small mixed steps) against the engine that launches every
    kernel, and against the plain model for a few of them."""
    import random
    from paged_llm_b200 import LLMEngine, SamplingParams
    hf, _ = TINIES["A"]
    rng = random.Random(4)
    work = [(random_tokens(hf["vocab_size"], rng.randint(1, 60), 100 + i), rng.randint(1, 24)) for i in range(60)]
    arrive = sorted(rng.randint(0, 40) for _ in work)          # the step before which each request arrives
    results = {}
    for eager in (False, True):
        eng = LLMEngine(folders["A"], dtype="float32", block_size=16, num_gpu_blocks=24, max_model_len=128,
                        max_num_seqs=8, max_num_batched_tokens=64, enforce_eager=eager)
        ids, step, nxt, done = {}, 0, 0, {}
        while nxt < len(work) or eng.has_unfinished_requests:
            while nxt < len(work) and arrive[nxt] <= step:
                prompt, n = work[nxt]
                ids[eng.add_request(prompt, SamplingParams(temperature=0.0, max_tokens=n, ignore_eos=True))] = nxt
                nxt += 1
            for o in eng.step():
                if o.new_token is not None:
                    done.setdefault(ids[o.seq_id], []).append(o.new_token)
            step += 1
        results[eager] = done
        assert eng.block_manager.num_free_blocks == 24
        if not eager:
            kinds = {k[0] for k in eng.runner._graphs}
            assert "decode" in kinds and (not eng.runner.mixed_graphs or "mixed" in kinds), kinds
            assert eng.runner.num_graph_steps > eng.runner.num_eager_steps
        else:
            assert eng.runner.num_graph_steps == 0
    assert results[False] == results[True]
    for i in (0, 17, 59):
        prompt, n = work[i]
        assert results[True][i] == plain_greedy(folders["A"], prompt, n)
