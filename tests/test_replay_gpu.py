"""Trace replay on the GPU: the same requests whole, with the tail decoded, in
portions and mixed, in float32 and bfloat16, against the plain implementation."""

import json
import os
import subprocess
import sys

import numpy as np
import pytest

from tests import schedules
from tests.helpers import assert_bf16_close_to_f32, assert_logits_close, model_folder, plain_logits, requests_for
from tests.tiny import TINIES

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LENGTHS = {"A": (5, 17, 33, 100, 81, 64, 2), "B": (1, 9, 40, 64, 100, 129, 77), "C": (3, 70, 150, 48, 97)}


def replay(folder, dtype, steps, max_tokens, block_size=16, **kw):
    from paged_llm_b200.engine.replay import TraceReplayer

    rp = TraceReplayer(folder, dtype, max_tokens, block_size=block_size, poison=float("nan"), **kw)
    outputs = {}
    for rec in steps:
        out = rp.step(rec)
        if out is not None:
            outputs[rec["step"]] = out
    assert not rp.live, "requests left alive at the end of the trace"
    rp.cm.check_invariants([])
    assert rp.cm.num_free_blocks == rp.cm.num_blocks, "pages were lost"
    return outputs, rp


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {name: model_folder(tmp_path_factory, name) for name in TINIES}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
@pytest.mark.parametrize("schedule", ["whole", "tail", "portions", "mixed"])
def test_schedule_matches_plain(folders, name, dtype, schedule):
    hf, _ = TINIES[name]
    reqs = requests_for(hf["vocab_size"], LENGTHS[name], seed=ord(name))
    steps, max_tokens = getattr(schedules, schedule)(reqs)
    outputs, rp = replay(folders[name], dtype, steps, max_tokens, block_size=8 if name == "B" else 16)
    got = schedules.collect(steps, outputs)
    for rid, toks in reqs.items():
        assert_logits_close(got[rid], plain_logits(folders[name], toks), dtype, f"{schedule}/{name}/{rid}")
    if schedule == "mixed":
        total = sum(-(-len(t) // rp.cm.block_size) for t in reqs.values())
        assert total > rp.cm.num_blocks, "the mixed trace must need more pages than the pool has, so that they are reused"


@pytest.mark.parametrize("name", ["A", "B", "C"])
@pytest.mark.parametrize("schedule", ["whole", "tail", "portions", "mixed"])
def test_bfloat16_against_the_float32_engine(tmp_path_factory, name, schedule):
    """Both engines on a folder of bfloat16 values: the weights are the same numbers, so the
    logits differ by the rounding of activations only, which is held much tighter than the
    distance to the plain float32 model."""
    folder = model_folder(tmp_path_factory, name, dtype="bfloat16")
    hf, _ = TINIES[name]
    reqs = requests_for(hf["vocab_size"], LENGTHS[name], seed=ord(name))
    steps, max_tokens = getattr(schedules, schedule)(reqs)
    block = 8 if name == "B" else 16
    a, _ = replay(folder, "float32", steps, max_tokens, block_size=block)
    b, _ = replay(folder, "bfloat16", steps, max_tokens, block_size=block)
    for k in a:
        assert_bf16_close_to_f32(b[k], a[k], f"{schedule}/{name}/step {k}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_eager_and_graph_decode_agree(folders, dtype):
    hf, _ = TINIES["A"]
    reqs = requests_for(hf["vocab_size"], (60, 45), seed=3)
    steps, max_tokens = schedules.tail(reqs, last=20)
    a, rp_a = replay(folders["A"], dtype, steps, max_tokens)
    b, rp_b = replay(folders["A"], dtype, steps, max_tokens, enforce_eager=True)
    assert rp_a.runner.num_graph_steps > 0 and rp_b.runner.num_graph_steps == 0
    for k in a:
        assert_logits_close(a[k], b[k], dtype, f"graph vs eager step {k}")


def test_trace_run_program(folders, tmp_path):
    """The program itself, as a user runs it: JSON lines in, `done` lines and .f32 files out."""
    hf, _ = TINIES["A"]
    reqs = requests_for(hf["vocab_size"], (21, 40, 9), seed=5)
    steps, max_tokens = schedules.mixed(reqs, live=3, seed=1)
    out_dir = tmp_path / "out"
    proc = subprocess.run(
        [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folders["A"], "--dtype", "float32",
         "--out", str(out_dir), "--max-tokens", str(max_tokens)],
        input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    done = [line for line in proc.stdout.splitlines() if line.startswith("done ")]
    assert done == [f"done {s['step']}" for s in steps]
    outputs = {}
    for s in steps:
        n = sum(len(e["want"]) for e in s["entries"])
        if n:
            outputs[s["step"]] = np.fromfile(out_dir / f"{s['step']}.f32", dtype="<f4").reshape(n, hf["vocab_size"])
    got = schedules.collect(steps, outputs)
    for rid, toks in reqs.items():
        assert_logits_close(got[rid], plain_logits(folders["A"], toks), "float32", f"trace_run/{rid}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_repeated_portions_replay_a_graph(folders, dtype):
    """A prompt cut into equal portions: from the second portion on the step replays a captured
    graph (other context lengths, same shapes) and still matches the plain logits."""
    hf, _ = TINIES["C"]
    toks = requests_for(hf["vocab_size"], (64 * 5 + 7,), seed=9)["r0"]
    steps = []
    for i in range(5):
        steps.append({"step": i, "entries": [{"id": "a", "tokens": toks[64 * i:64 * (i + 1)], "want": [63]}], "end": []})
    steps.append({"step": 5, "entries": [{"id": "a", "tokens": toks[320:], "want": list(range(7))}], "end": ["a"]})
    outputs, rp = replay(folders["C"], dtype, steps, 384)
    # (the portions from the second on; the tail of 7 tokens may replay a graph of small mixed steps as well)
    assert rp.runner.num_graph_steps >= 4 and ("portion", 64, 1) in rp.runner._graphs
    want = plain_logits(folders["C"], toks)
    got = np.concatenate([outputs[i] for i in range(6)])
    rows = [64 * i + 63 for i in range(5)] + list(range(320, 327))
    assert_logits_close(got, want[rows], dtype, "portion graph")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_small_mixed_steps_replay_graphs(folders, name, dtype):
    """Steps of mixed items of few tokens (portions beside decoded tokens, cut anywhere) replay graphs captured
    with spare capacity for tokens, requests, wanted rows and attention work items: the same logits as the
    plain model and as the run that launches every kernel, in both precisions."""
    hf, _ = TINIES[name]
    reqs = requests_for(hf["vocab_size"], LENGTHS[name], seed=ord(name) + 1)
    steps, max_tokens = schedules.mixed(reqs)
    block = 8 if name == "B" else 16
    outputs, rp = replay(folders[name], dtype, steps, max_tokens, block_size=block)
    if not rp.runner.mixed_graphs:
        pytest.skip("graphs of small mixed steps are switched off")
    mixed = [k for k in rp.runner._graphs if k[0] == "mixed"]
    assert mixed and rp.runner.num_graph_steps > len(steps) // 3, "the mixed steps did not replay graphs"
    got = schedules.collect(steps, outputs)
    for rid, toks in reqs.items():
        assert_logits_close(got[rid], plain_logits(folders[name], toks), dtype, f"mixed graphs/{name}/{rid}")
    eager, rp_e = replay(folders[name], dtype, steps, max_tokens, block_size=block, enforce_eager=True)
    assert rp_e.runner.num_graph_steps == 0
    for k in outputs:
        if dtype == "float32":
            np.testing.assert_allclose(outputs[k], eager[k], rtol=0, atol=2e-5 * max(1.0, float(np.abs(eager[k]).max())))
        else:
            assert_bf16_close_to_f32(outputs[k], eager[k], f"graph against launches, step {k}")
