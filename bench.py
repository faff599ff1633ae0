"""Headline benchmark: decode tokens per second of the TinyLlama-1.1B-sized Llama
(random bfloat16 weights) at batch 8 with 512-token prompts, on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A step is one decode step.  The timed region is exactly K steps after W warm-up
steps, timed with CUDA events on the launching stream.  One JSON line is
printed; beside `value` (device-timed loop: tokens stay on the device) it holds

* `e2e`: the same through `LLMEngine.step()`: host token ids in, host token ids
  out, every step (metadata host-to-device from pinned memory, sampled ids
  device-to-host);
* `prefill`: one step of a 2,048-token prompt, with the fraction of the bf16 peak;
* `roofline`: bytes a decode step must read (weights once, the live cache)
  divided by its time, against the measured HBM bandwidth;
* `points`: decode tokens per second at batch 1 and 64;
* `clocks`: SM clock and throttle reasons sampled during the timed region;
* `gpu_launches`: kernels of this package launched in the timed region.

Weights (2.2 GB) are larger than the 126 MB L2, so every step re-reads them from
HBM; no L2 flush is needed between iterations.

`--impl reference` runs the unmodified reference (xiyiji/paged-llm, installed
under baseline/_ref) through its own `LLMEngine` on the same model folder and
prints the same line with "impl": "reference".
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}

SIZES = {
    # TinyLlama 1.1B layer sizes (22 layers, 32 query / 4 kv heads of 64, hidden 2048, context 2048)
    "tinyllama-1.1b": dict(vocab_size=32000, hidden_size=2048, intermediate_size=5632, num_hidden_layers=22,
                           num_attention_heads=32, num_key_value_heads=4, head_dim=64, rope_theta=10000.0,
                           rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=2048),
    # Llama-3.2-1B layer sizes (16 layers, 32 query / 8 kv heads of 64, llama3 rotary scaling, tied head)
    "llama-3.2-1b": dict(vocab_size=128256, hidden_size=2048, intermediate_size=8192, num_hidden_layers=16,
                         num_attention_heads=32, num_key_value_heads=8, head_dim=64, rope_theta=500000.0,
                         rope_scaling=dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                           original_max_position_embeddings=8192),
                         rms_norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=8192),
    # Llama-3-8B layer sizes (32 layers, 32 query / 8 kv heads of 128, hidden 4096); about 16 GB at full depth
    "llama-3-8b": dict(vocab_size=128256, hidden_size=4096, intermediate_size=14336, num_hidden_layers=32,
                       num_attention_heads=32, num_key_value_heads=8, head_dim=128, rope_theta=500000.0,
                       rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=8192),
    # for trying the script out on small hardware; never the default
    "tiny-a": dict(vocab_size=256, hidden_size=64, intermediate_size=172, num_hidden_layers=2,
                   num_attention_heads=4, num_key_value_heads=2, head_dim=16, max_position_embeddings=4096),
}
PROMPT_LEN, DECODE_LEN, PREFILL_TOKENS, BLOCK_SIZE = 512, 256, 2048, 16
RAGGED_PROMPTS, RAGGED_OUTPUTS = (128, 4096), (64, 512)      # the ragged serving workload: lengths drawn uniformly


def load_peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                raw = json.load(f)
            flat = {}

            def walk(d):
                for k, v in d.items():
                    if isinstance(v, dict):
                        walk(v)
                    elif isinstance(v, (int, float)):
                        flat.setdefault(k, float(v))
            walk(raw)
            out = {"source": "measured"}
            out["hbm_gbs"] = flat.get("hbm_gbs") or FALLBACK_PEAKS["hbm_gbs"]
            out["bf16_tflops"] = flat.get("bf16_tflops") or FALLBACK_PEAKS["bf16_tflops"]
            if "bf16_tflops_sustained" in flat:
                out["bf16_tflops_sustained"] = flat["bf16_tflops_sustained"]
            return out
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """nvidia-smi in a loop during the timed region (reads settings, changes none)."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int = 0):
        self.proc = None
        self.path = None
        self.uuid = None
        try:
            import torch
            self.uuid = "GPU-" + str(torch.cuda.get_device_properties(device_index).uuid)
        except Exception:
            self.uuid = None

    def __enter__(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            cmd = ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100"]
            if self.uuid:
                cmd += ["-i", self.uuid]
            self.proc = subprocess.Popen(cmd, stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self) -> dict:
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            with open(self.path) as f:
                for line in f:
                    parts = [p.strip() for p in line.split(",")]
                    if len(parts) < 7:
                        continue
                    try:
                        sm.append(float(parts[0]))
                        mx.append(float(parts[1]))
                    except ValueError:
                        continue
                    for name, flag in zip(names, parts[3:7]):
                        if flag.lower().startswith("active"):
                            reasons.add(name)
            os.unlink(self.path)
        except (OSError, TypeError):
            pass
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def write_tokenizer(folder: str, vocab: int) -> None:
    """A word-level tokenizer over token names t0..tN, only so that the
    reference's engine, which loads a tokenizer unconditionally, starts."""
    from tokenizers import Tokenizer, models, pre_tokenizers

    tok = Tokenizer(models.WordLevel({f"t{i}": i for i in range(vocab)}, unk_token="t0"))
    tok.pre_tokenizer = pre_tokenizers.Whitespace()
    tok.save(os.path.join(folder, "tokenizer.json"))
    with open(os.path.join(folder, "tokenizer_config.json"), "w") as f:
        json.dump({"tokenizer_class": "PreTrainedTokenizerFast", "unk_token": "t0", "eos_token": "t1"}, f)


STUB_ABOVE_PARAMS = 2_000_000_000      # larger models get their random weights drawn on the device


def make_model(folder: str, size: str, layers: int | None, with_tokenizer: bool = False, on_device: bool | None = None):
    """Writes a model folder of the named layer sizes with random weights N(0, 0.02), seed 0.  Models of
    more than two billion parameters (or `on_device`) get a folder without tensors whose weights the
    engine draws on the device (weights/random_init.py: write_random_stub); the reference arm always
    gets tensors."""
    from paged_llm_b200.config.registry import parse_model_config
    from paged_llm_b200.weights import write_model_folder, write_random_stub

    hf = {"architectures": ["LlamaForCausalLM"], **SIZES[size]}
    full_layers = hf["num_hidden_layers"]
    if layers:
        hf["num_hidden_layers"] = layers
    _, cfg = parse_model_config(hf)          # the architecture named in the configuration decides the config class
    if on_device is None:
        on_device = cfg.num_parameters > STUB_ABOVE_PARAMS and not with_tokenizer
    if on_device:
        write_random_stub(folder, cfg, seed=0, std=0.02, dtype="bfloat16")
    else:
        write_model_folder(folder, cfg, seed=0, std=0.02, dtype="bfloat16")
    if with_tokenizer:
        write_tokenizer(folder, cfg.vocab_size)
    return cfg, full_layers


def prompts_for(vocab: int, batch: int, length: int, seed: int = 0):
    import torch
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (length,), generator=g).tolist() for _ in range(batch)]


def step_flops(cfg, tokens: int, context_start: int = 0) -> float:
    """Multiply-adds x 2 of one step of `tokens` new tokens of one request."""
    h, d = cfg.hidden_size, cfg.head_dim
    per_layer = (cfg.num_attention_heads + 2 * cfg.num_key_value_heads) * d * h + cfg.num_attention_heads * d * h \
        + 3 * cfg.intermediate_size * h
    gemm = 2.0 * tokens * per_layer * cfg.num_hidden_layers + 2.0 * cfg.vocab_size * h
    keys = sum(context_start + i + 1 for i in range(tokens))
    attn = 4.0 * cfg.num_attention_heads * d * keys * cfg.num_hidden_layers
    return gemm + attn


# ------------------------------------------------------------------------------ ours

def device_decode_loop(engine, batch: int, steps: int, warmup: int, prompt_len: int):
    """Prefills `batch` requests, then times `steps` decode steps on the device:
    sampled tokens stay on the device and feed the next step.  Returns
    (ms per step, launches per step, context length at the middle of the run)."""
    import torch
    from paged_llm_b200.config import SamplingParams
    from paged_llm_b200.engine.runner import StepItem
    from paged_llm_b200.engine.sequence import Sequence

    cm, runner, ops = engine.block_manager, engine.runner, engine.ops
    vocab = engine.model_config.vocab_size
    seqs = [Sequence(p, SamplingParams(temperature=0.0, max_tokens=steps + warmup + 2))
            for p in prompts_for(vocab, batch, prompt_len, seed=batch)]
    chunk = max(1, engine.config.max_num_batched_tokens // prompt_len)
    for i in range(0, batch, chunk):
        group = seqs[i:i + chunk]
        for s in group:
            ok = cm.allocate_slots(s, prompt_len)
            assert ok is not None, "pool too small for the benchmark"
        logits = runner.step([StepItem(s, prompt_len, (prompt_len - 1,)) for s in group])
        toks = ops.argmax(logits).tolist()
        for s, t in zip(group, toks):
            s.num_computed_tokens = prompt_len
            s.append_token(t)
    items = [StepItem(s, 1, (0,)) for s in seqs]

    def one_step(first: bool):
        for s in seqs:
            ok = cm.allocate_slots(s, 1)
            assert ok is not None, "pool too small for the benchmark"
        logits = runner.step(items)
        nxt = ops.argmax(logits)
        for s in seqs:
            s.num_computed_tokens += 1
            s.token_ids.append(0)            # the id lives on the device; the host list only keeps the length
        return nxt

    # device-resident feedback: the ids section of the next step's metadata is overwritten on the device
    def run(n):
        nonlocal last
        for _ in range(n):
            if last is not None:
                runner.next_ids_override = last
            last = one_step(False)

    last = None
    run(warmup)
    torch.cuda.synchronize()
    launches0 = ops.launches + runner.graph_launches
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ctx_mid = seqs[0].num_computed_tokens + steps // 2
    start.record()
    run(steps)
    end.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(end) / steps
    launches = (ops.launches + runner.graph_launches - launches0) / steps
    for s in seqs:
        cm.free(s)
    return ms, launches, ctx_mid


def decode_kernel_times(engine, batch: int, steps: int, warmup: int, prompt_len: int) -> dict:
    """Device time of every kernel inside replayed decode steps (torch's profiler, i.e. CUPTI activity
    records of the real step, not serialised launches): name -> [launches per step, mean microseconds].
    Kernels launched with programmatic dependent launch overlap, so the sum can exceed the step."""
    import collections
    import torch
    from torch.profiler import ProfilerActivity, profile

    device_decode_loop(engine, batch, steps, warmup, prompt_len)            # graphs captured, caches warm
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        _, launches, _ = device_decode_loop(engine, batch, steps, warmup, prompt_len)
        torch.cuda.synchronize()
    events = sorted((e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA),
                    key=lambda e: e.time_range.start)
    # the decode steps are the tail of the record: per step the package's kernels, the library's, and two copies
    per_step = collections.Counter()
    tail = events[-int(round(launches + 4)) * steps:]
    total = collections.defaultdict(float)
    for e in tail:
        name = e.name.replace("(anonymous namespace)::", "").replace("<unnamed>::", "").replace("void ", "")
        name = name.split("(")[0][:72]
        per_step[name] += 1
        total[name] += e.time_range.end - e.time_range.start
    return {k: [round(per_step[k] / steps, 1), round(total[k] / per_step[k], 2)]
            for k in sorted(total, key=lambda k: -total[k])[:14]}


def prefill_kernel_times(engine, tokens: int) -> dict:
    """The same for one prompt portion of `tokens` tokens: name -> [launches in the step, mean microseconds]."""
    import collections
    import torch
    from torch.profiler import ProfilerActivity, profile

    prefill_once(engine, tokens, iters=1, warmup=3)                          # graph captured, caches warm
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        prefill_once(engine, tokens, iters=1, warmup=0)
        torch.cuda.synchronize()
    count, total = collections.Counter(), collections.defaultdict(float)
    for e in prof.events():
        if e.device_type != torch.autograd.DeviceType.CUDA:
            continue
        name = e.name.replace("(anonymous namespace)::", "").replace("<unnamed>::", "").replace("void ", "")
        name = name.split("(")[0][:72]
        count[name] += 1
        total[name] += e.time_range.end - e.time_range.start
    return {k: [count[k], round(total[k] / count[k], 2)] for k in sorted(total, key=lambda k: -total[k])[:14]}


def e2e_decode(engine, batch: int, steps: int, warmup: int, prompt_len: int):
    """The same decode steps through the public `LLMEngine.step()`: token ids
    come back to the host every step."""
    import torch
    from paged_llm_b200.config import SamplingParams

    vocab = engine.model_config.vocab_size
    # no request ends inside the timed steps (the requests of the second prefill step are a token
    # behind the others): all of them are steady decoding of the whole batch
    sp = SamplingParams(temperature=0.0, max_tokens=steps + warmup + 8, ignore_eos=True)
    for p in prompts_for(vocab, batch, prompt_len, seed=100 + batch):
        engine.add_request(p, sp)
    while any(not s.is_prefill_done or s.num_generated_tokens == 0 for s in engine.scheduler.running) \
            or engine.scheduler.waiting:
        engine.step()
    for _ in range(warmup):
        engine.step()
    torch.cuda.synchronize()
    h2d0 = engine.runner.h2d_bytes
    t0 = time.perf_counter()
    n_tokens = 0
    for _ in range(steps):
        n_tokens += sum(1 for o in engine.step() if o.new_token is not None)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    h2d = (engine.runner.h2d_bytes - h2d0) / steps
    while engine.has_unfinished_requests:
        engine.step()
    return n_tokens / dt, h2d, batch * 4


def ragged_generate(engine, num_requests: int, prompt_range, output_range, seed: int = 0):
    """Ragged requests through the public `LLMEngine.generate`: prompt and output lengths drawn
    uniformly, uniform token ids, greedy, prompts cut into portions under the token budget while
    others decode.  Wall-clock seconds around the call, tokens counted from what comes back."""
    import random
    from paged_llm_b200.config import SamplingParams

    rng = random.Random(seed)
    vocab = engine.model_config.vocab_size
    prompts, params = [], []
    for _ in range(num_requests):
        n = rng.randint(*prompt_range)
        prompts.append([rng.randrange(vocab) for _ in range(n)])
        params.append(SamplingParams(temperature=0.0, max_tokens=rng.randint(*output_range), ignore_eos=True))
    steps0, pre0 = engine.stats.num_steps, engine.stats.num_preemptions
    graph0 = engine.runner.num_graph_steps
    t0 = time.perf_counter()
    outs = engine.generate(prompts, params)
    dt = time.perf_counter() - t0
    generated = sum(len(o.token_ids) for o in outs)
    assert generated == sum(p.max_tokens for p in params), "every request runs to its own length"
    return {"seconds": round(dt, 3), "requests": num_requests, "prompt_tokens": sum(map(len, prompts)),
            "generated_tokens": generated, "generated_tok_s": round(generated / dt, 1),
            "total_tok_s": round((generated + sum(map(len, prompts))) / dt, 1),
            "steps": engine.stats.num_steps - steps0,
            "graph_steps": engine.runner.num_graph_steps - graph0, "preemptions": engine.stats.num_preemptions - pre0}


def prefill_once(engine, tokens: int, iters: int = 5, warmup: int = 3):
    import torch
    from paged_llm_b200.config import SamplingParams
    from paged_llm_b200.engine.runner import StepItem
    from paged_llm_b200.engine.sequence import Sequence

    cm, runner = engine.block_manager, engine.runner
    vocab = engine.model_config.vocab_size
    times = []
    for i in range(warmup + iters):
        seq = Sequence(prompts_for(vocab, 1, tokens, seed=7 + i)[0], SamplingParams())
        ok = cm.allocate_slots(seq, tokens)
        assert ok is not None, "pool too small for the benchmark"
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        runner.step([StepItem(seq, tokens, (tokens - 1,))])
        end.record()
        torch.cuda.synchronize()
        if i >= warmup:
            times.append(start.elapsed_time(end))
        cm.free(seq)
    return statistics.median(times)


def mixed_step(engine, batch: int, portion: int, context: int, iters: int = 5, warmup: int = 3):
    """One step that carries `batch` decoding requests (context `context`) beside one prompt portion of
    `portion` tokens of a new request: the step a serving engine runs while a long prompt arrives.
    Returns the median milliseconds of the step (CUDA events)."""
    import torch
    from paged_llm_b200.config import SamplingParams
    from paged_llm_b200.engine.runner import StepItem
    from paged_llm_b200.engine.sequence import Sequence

    cm, runner, ops = engine.block_manager, engine.runner, engine.ops
    vocab = engine.model_config.vocab_size
    seqs = [Sequence(p, SamplingParams()) for p in prompts_for(vocab, batch, context, seed=3)]
    chunk = max(1, engine.config.max_num_batched_tokens // context)
    for i in range(0, batch, chunk):
        group = seqs[i:i + chunk]
        for s in group:
            ok = cm.allocate_slots(s, context)
            assert ok is not None, "pool too small for the benchmark"
        runner.step([StepItem(s, context, ()) for s in group])
        for s in group:
            s.num_computed_tokens = context
            s.append_token(1)
    times = []
    for i in range(warmup + iters):
        new = Sequence(prompts_for(vocab, 1, portion, seed=50 + i)[0], SamplingParams())
        ok = cm.allocate_slots(new, portion)
        assert ok is not None
        for s in seqs:
            ok = cm.allocate_slots(s, 1)
            assert ok is not None
        items = [StepItem(s, 1, (0,)) for s in seqs] + [StepItem(new, portion, (portion - 1,))]
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        ops.argmax(runner.step(items))
        end.record()
        torch.cuda.synchronize()
        if i >= warmup:
            times.append(start.elapsed_time(end))
        for s in seqs:
            s.num_computed_tokens += 1
            s.append_token(1)
        cm.free(new)
    for s in seqs:
        cm.free(s)
    return statistics.median(times)


def chunked_prefill(engine, tokens: int, iters: int = 3, warmup: int = 2):
    """One prompt of `tokens` tokens through the public `LLMEngine.generate` with one output token: the
    scheduler cuts it into portions of `max_num_batched_tokens`.  Median wall-clock milliseconds."""
    import torch
    from paged_llm_b200.config import SamplingParams

    vocab = engine.model_config.vocab_size
    times = []
    for i in range(warmup + iters):
        prompt = prompts_for(vocab, 1, tokens, seed=20 + i)[0]
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        engine.generate([prompt], SamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True))
        torch.cuda.synchronize()
        if i >= warmup:
            times.append((time.perf_counter() - t0) * 1e3)
    return statistics.median(times)


def sampling_times(args) -> dict:
    """Microseconds per call of the sampler's kernels on `--batch` rows of a vocabulary of the named size: the
    calls are issued back to back (each with its one copy of parameters from pinned memory) and timed with CUDA
    events, so a call that takes the device less than the host takes to issue it shows the host's time."""
    import numpy as np
    import torch
    from paged_llm_b200.kernels.ops import CudaOps

    ops = CudaOps(torch.device("cuda:0"))
    rows, vocab = args.batch, SIZES[args.size]["vocab_size"]
    logits = torch.randn(rows, vocab, device="cuda") * 2.0

    def timed(fn, n=50):
        for _ in range(5):
            fn()
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(n):
            fn()
        end.record()
        torch.cuda.synchronize()
        return round(start.elapsed_time(end) / n * 1e3, 1)

    out = {"only": "sample", "size": args.size, "rows": rows, "vocab": vocab, "unit": "us per call",
           "argmax": timed(lambda: ops.argmax(logits))}
    for name, k, p in (("temperature", 0, 1.0), ("top_k_50", 50, 1.0), ("top_p_0.9", 0, 0.9), ("top_k_50_top_p_0.9", 50, 0.9)):
        arrays = (np.full(rows, 0.7, np.float32), np.full(rows, k, np.int32), np.full(rows, p, np.float32),
                  np.arange(rows, dtype=np.uint64), np.arange(rows, dtype=np.uint64))
        out[name] = timed(lambda: ops.sample(logits, *arrays))
    return out


def validate(args) -> dict:
    """The float32 validation run at the benchmark's layer sizes: the same trace (a 2,048-token
    portion, 32 decoded tokens, portions of changing size, a mixed batch) through the bfloat16 engine
    and the true-float32 engine on the same weight values, and the float32 engine against the plain
    implementation of tests/plain_llama.py on a shorter request.  Reports the largest differences
    relative to the largest logit."""
    import numpy as np
    from paged_llm_b200.engine.replay import TraceReplayer
    from tests import plain_llama, schedules
    from tests.tiny import random_tokens, read_folder

    with tempfile.TemporaryDirectory() as folder:
        cfg, full_layers = make_model(folder, args.size, args.layers, on_device=False)
        V = cfg.vocab_size
        long_req = random_tokens(V, 2048 + 32, 1)
        reqs = {"w": long_req, "p": random_tokens(V, 700, 2), "q": random_tokens(V, 333, 3), "r": random_tokens(V, 90, 4)}
        # whole + tail for the long request, portions and a mixed batch for the others
        steps = [{"step": 0, "entries": [{"id": "w", "tokens": long_req[:2048], "want": [0, 1, 511, 1024, 2047]}], "end": []}]
        for i in range(2048, len(long_req)):
            steps.append({"step": len(steps), "entries": [{"id": "w", "tokens": [long_req[i]], "want": [0]}],
                          "end": ["w"] if i == len(long_req) - 1 else []})
        more, _ = schedules.mixed({k: reqs[k] for k in "pqr"}, live=3, seed=1, choices=(2, 5, 16, 40, 64, 130, 257))
        more = schedules.keep_wanted(more, lambda rid, p: p % 16 == 0 or p >= len(reqs[rid]) - 4)
        for rec in more:
            steps.append({**rec, "step": len(steps)})
        max_tokens = 2112 + sum(schedules._round64(len(reqs[k])) for k in "pqr")
        out = {}
        for dtype in ("float32", "bfloat16"):
            rp = TraceReplayer(folder, dtype, max_tokens)
            res = {rec["step"]: o for rec in steps if (o := rp.step(rec)) is not None}
            out[dtype] = schedules.collect(steps, res)
            del rp
        worst16 = max(float(np.abs(out["bfloat16"][k] - out["float32"][k]).max() / np.abs(out["float32"][k]).max())
                      for k in out["float32"])
        hf, w = read_folder(folder)
        rows = schedules.wanted_positions(steps)["q"]
        want = plain_llama.forward_logits(hf, w, reqs["q"], rows=rows).numpy()
        worst32 = float(np.abs(out["float32"]["q"] - want).max() / max(1.0, np.abs(want).max()))
    return {"only": "validate", "size": args.size, "layers": cfg.num_hidden_layers, "layers_full": full_layers,
            "positions_compared": int(sum(len(v) for v in out["float32"].values())),
            "bf16_vs_f32_engine_rel": round(worst16, 6), "f32_engine_vs_plain_rel": round(worst32, 8),
            "trace": "2,048-token portion + 32 decoded tokens; three requests of 700/333/90 tokens mixed, portions of 2 to 257 tokens"}


def run_ours(args) -> dict:
    import torch
    from paged_llm_b200 import EngineConfig, LLMEngine

    peaks = load_peaks()
    if args.only == "validate":
        return validate(args)
    if args.only == "sample":
        return sampling_times(args)
    with tempfile.TemporaryDirectory() as folder:
        cfg, full_layers = make_model(folder, args.size, args.layers)
        prompt_len = args.context if args.only in ("decode", "mixed") and args.context else PROMPT_LEN
        pre_tokens = args.prefill_tokens if args.only in ("prefill", "mixed") and args.prefill_tokens else PREFILL_TOKENS
        max_len = max(prompt_len + args.steps + args.warmup + DECODE_LEN, pre_tokens) + 64
        if args.only == "ragged":
            p_hi = int(args.prompt_range.split(",")[1]) if args.prompt_range else RAGGED_PROMPTS[1]
            o_hi = int(args.output_range.split(",")[1]) if args.output_range else RAGGED_OUTPUTS[1]
            max_len = max(p_hi, 512) + max(o_hi, 32) + 64          # (the untimed first requests are up to 512 + 32 long)
        seqs = max(args.batch, 64) if prompt_len == PROMPT_LEN else args.batch
        if args.only == "mixed":
            max_len = max(max_len, prompt_len + 64, pre_tokens + 64)
            seqs = args.batch + 2
        engine = LLMEngine(folder, EngineConfig(
            dtype="bfloat16", block_size=BLOCK_SIZE, max_model_len=max_len, max_num_seqs=max(seqs, 64),
            max_num_batched_tokens=args.chunk if args.only == "prefill" and args.chunk else max(2048, pre_tokens),
            enable_prefix_caching=False,
            num_gpu_blocks=seqs * (-(-max_len // BLOCK_SIZE)) + 64))
    B = args.batch
    if args.only == "ragged":            # 64 ragged requests under a 2,048-token budget, end to end
        engine.warm_up()
        ragged_generate(engine, 8, (128, 512), (16, 32), seed=1)          # untimed: first-use costs
        # untimed too: the same workload with other lengths and tokens, so that the graphs of its batch buckets
        # and context classes exist (a server runs for longer than its first two seconds)
        n_req = args.requests
        p_range = tuple(int(v) for v in args.prompt_range.split(",")) if args.prompt_range else RAGGED_PROMPTS
        o_range = tuple(int(v) for v in args.output_range.split(",")) if args.output_range else RAGGED_OUTPUTS
        ragged_generate(engine, n_req, p_range, o_range, seed=1)
        return {"only": "ragged", "size": args.size, "layers": cfg.num_hidden_layers,
                "prompt_range": list(p_range), "output_range": list(o_range),
                **ragged_generate(engine, n_req, p_range, o_range, seed=0)}
    if args.only == "decode":            # a short run of one part, for profilers and other context lengths
        ms, launches, ctx_mid = device_decode_loop(engine, B, args.steps, args.warmup, prompt_len)
        step_bytes = engine.model.weight_bytes_per_step() + B * ctx_mid * (engine.kv_cache.page_bytes() // BLOCK_SIZE)
        gbs = step_bytes / (ms * 1e-3) / 1e9
        extra = {"kernel_times": decode_kernel_times(engine, B, min(args.steps, 8), args.warmup, prompt_len)} \
            if args.kernel_times else {}
        return {**extra, "only": "decode", "size": args.size, "batch": B, "context": ctx_mid, "ms_per_step": round(ms, 4),
                "tokens_per_s": round(B * 1000.0 / ms, 1), "launches_per_step": launches,
                "layers": cfg.num_hidden_layers, "layers_full": full_layers, "gb_per_s": round(gbs, 1),
                "frac": round(gbs / peaks["hbm_gbs"], 4), "peaks_source": peaks["source"]}
    if args.only == "mixed":             # B decoding requests beside one prompt portion, in one step
        portion = args.prefill_tokens or PREFILL_TOKENS
        ms = mixed_step(engine, B, portion, prompt_len, iters=max(3, min(args.steps, 10)), warmup=args.warmup)
        flops = step_flops(cfg, portion) + B * step_flops(cfg, 1, prompt_len)
        return {"only": "mixed", "size": args.size, "layers": cfg.num_hidden_layers, "layers_full": full_layers,
                "decoding_requests": B, "context": prompt_len, "portion": portion, "ms": round(ms, 3),
                "tokens_per_s": round((portion + B) * 1000.0 / ms, 1),
                "tflops": round(flops / (ms * 1e-3) / 1e12, 1),
                "frac": round(flops / (ms * 1e-3) / 1e12 / peaks["bf16_tflops"], 4), "peaks_source": peaks["source"]}
    if args.only == "prefill" and args.chunk:
        ms = chunked_prefill(engine, pre_tokens, iters=max(1, args.steps), warmup=args.warmup)
        tflops = step_flops(cfg, pre_tokens) / (ms * 1e-3) / 1e12
        return {"only": "prefill", "size": args.size, "tokens": pre_tokens, "portions_of": args.chunk, "ms": round(ms, 3),
                "through": "LLMEngine.generate, one output token, wall clock", "layers": cfg.num_hidden_layers,
                "layers_full": full_layers, "tokens_per_s": round(pre_tokens * 1000.0 / ms, 1), "tflops": round(tflops, 1),
                "frac": round(tflops / peaks["bf16_tflops"], 4), "peaks_source": peaks["source"]}
    if args.only == "prefill":
        pre_ms = prefill_once(engine, pre_tokens, iters=max(1, args.steps), warmup=args.warmup)
        tflops = step_flops(cfg, pre_tokens) / (pre_ms * 1e-3) / 1e12
        extra = {"kernel_times": prefill_kernel_times(engine, pre_tokens)} if args.kernel_times else {}
        return {**extra, "only": "prefill", "size": args.size, "tokens": pre_tokens, "ms": round(pre_ms, 3),
                "layers": cfg.num_hidden_layers, "tflops": round(tflops, 1),
                "frac": round(tflops / peaks["bf16_tflops"], 4), "peaks_source": peaks["source"]}
    weight_bytes = engine.model.weight_bytes_per_step()
    kv_bytes_per_token = engine.kv_cache.page_bytes() // BLOCK_SIZE

    with ClockSampler() as clocks:
        ms, launches, ctx_mid = device_decode_loop(engine, B, args.steps, args.warmup, PROMPT_LEN)
    clock_summary = clocks.summary()
    value = B * 1000.0 / ms
    step_bytes = weight_bytes + B * ctx_mid * kv_bytes_per_token
    achieved = step_bytes / (ms * 1e-3) / 1e9

    e2e_value, h2d, d2h = e2e_decode(engine, B, args.steps, args.warmup, PROMPT_LEN)
    points = {}
    for b in (1, 64):
        pms, _, _ = device_decode_loop(engine, b, min(args.steps, 128), args.warmup, PROMPT_LEN)
        points[f"decode_b{b}"] = round(b * 1000.0 / pms, 1)
    pre_ms = prefill_once(engine, PREFILL_TOKENS)
    flops = step_flops(cfg, PREFILL_TOKENS)
    peak_flops = peaks["bf16_tflops"] * 1e12

    return {
        "metric": "decode tok/s at batch 8 (TinyLlama 1.1B sizes, 512-token prompts, bf16, one B200)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights N(0, 0.02) seed 0, uniform random token ids",
        "impl": "ours",
        "config": {
            "model": "TinyLlama-1.1B layer sizes" if args.size == "tinyllama-1.1b" else args.size,
            "global_batch": B, "seq_len": PROMPT_LEN + DECODE_LEN, "prompt_len": PROMPT_LEN,
            "decode_len": DECODE_LEN, "parallelism": "single GPU", "layers": cfg.num_hidden_layers,
            "layers_full": full_layers, "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads,
            "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size,
            "vocab": cfg.vocab_size, "block_size": BLOCK_SIZE, "params": cfg.num_parameters,
            "l2": "weights (2.2 GB) exceed the 126 MB L2: no flush between iterations",
            "peaks": peaks["source"], "cuda_graphs": not engine.config.enforce_eager,
        },
        "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s", "h2d_bytes_per_step": int(h2d),
                "d2h_bytes_per_step": int(d2h)},
        "gpu_launches": int(round(launches * args.steps)),
        "clocks": clock_summary,
        "prefill": {"value": round(PREFILL_TOKENS * 1000.0 / pre_ms, 1), "tokens": PREFILL_TOKENS,
                    "ms": round(pre_ms, 3), "frac": round(flops / (pre_ms * 1e-3) / peak_flops, 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4)},
        "points": points,
    }


# ------------------------------------------------------------------------------ reference

def run_reference(args) -> dict:
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "pagedllm")):
        return {"impl": "reference", "unavailable": "baseline/_ref holds no installed reference (pip install --target failed or was not run)"}
    try:
        import torch
        if not torch.cuda.is_available():
            return {"impl": "reference", "unavailable": "no CUDA device"}
        sys.path.insert(0, ref_dir)
        from pagedllm import EngineConfig, SamplingParams
        from pagedllm.engine import LLMEngine
    except Exception as e:                                            # noqa: BLE001
        return {"impl": "reference", "unavailable": f"import of the reference failed: {type(e).__name__}: {e}"[:300]}
    B = args.batch
    try:
        with tempfile.TemporaryDirectory() as folder:
            cfg, full_layers = make_model(folder, args.size, args.layers, with_tokenizer=True)
            max_len = PROMPT_LEN + args.steps + args.warmup + DECODE_LEN + 64
            engine = LLMEngine(folder, EngineConfig(
                dtype="bfloat16", block_size=BLOCK_SIZE, max_model_len=max_len, max_num_seqs=64,
                max_num_batched_tokens=4096, enable_prefix_caching=False,
                num_gpu_blocks=64 * (-(-max_len // BLOCK_SIZE)) + 64))
        sp = SamplingParams(temperature=0.0, max_tokens=args.steps + args.warmup + 1, ignore_eos=True)
        for p in prompts_for(cfg.vocab_size, B, PROMPT_LEN, seed=100 + B):
            engine.add_request(p, sp)
        while engine.scheduler.waiting or any(s.num_generated_tokens == 0 for s in engine.scheduler.running):
            engine.step()
        for _ in range(args.warmup):
            engine.step()
        torch.cuda.synchronize()
        with ClockSampler() as clocks:
            t0 = time.perf_counter()
            n = 0
            for _ in range(args.steps):
                n += sum(1 for o in engine.step() if o.new_token is not None)
            torch.cuda.synchronize()
            dt = time.perf_counter() - t0
        value = n / dt
        return {
            "metric": "decode tok/s at batch 8 (TinyLlama 1.1B sizes, 512-token prompts, bf16, one B200)",
            "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(dt * 1000.0 / args.steps, 4), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic: random weights, uniform random token ids",
            "impl": "reference",
            "config": {"model": "TinyLlama-1.1B layer sizes" if args.size == "tinyllama-1.1b" else args.size,
                       "global_batch": B, "seq_len": PROMPT_LEN + DECODE_LEN, "prompt_len": PROMPT_LEN,
                       "layers": cfg.num_hidden_layers, "layers_full": full_layers, "parallelism": "single GPU",
                       "attention": engine.attention_backend, "timing": "wall clock around LLMEngine.step()"},
            "e2e": {"value": round(value, 1), "unit": "tokens/s"},
            "clocks": clocks.summary(),
        }
    except Exception as e:                                            # noqa: BLE001
        return {"impl": "reference", "unavailable": f"the reference failed to run: {type(e).__name__}: {e}"[:300]}


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=None,
                    help="with --only decode or mixed: prompt length of the decoding requests instead of 512")
    ap.add_argument("--prefill-tokens", type=int, default=None,
                    help="with --only prefill: length of the prompt (one step) instead of 2,048")
    ap.add_argument("--size", choices=sorted(SIZES), default="tinyllama-1.1b")
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the named size (reported in config)")
    ap.add_argument("--chunk", type=int, default=None,
                    help="with --only prefill: the prompt goes through LLMEngine.generate in portions of this many tokens")
    ap.add_argument("--requests", type=int, default=64, help="with --only ragged: number of requests")
    ap.add_argument("--prompt-range", default=None, help="with --only ragged: LO,HI prompt lengths (default 128,4096)")
    ap.add_argument("--output-range", default=None, help="with --only ragged: LO,HI output lengths (default 64,512)")
    ap.add_argument("--kernel-times", action="store_true",
                    help="with --only decode or --only prefill: add the device time of every kernel inside the replayed steps")
    ap.add_argument("--only", choices=["decode", "prefill", "ragged", "mixed", "validate", "sample"], default=None,
                    help="run only the decode loop, only the prefill step, the ragged serving workload through "
                         "LLMEngine.generate, one mixed step (--batch decoding requests of --context tokens beside one "
                         "portion of --prefill-tokens), the float32 validation run, or the sampler's kernels on --batch rows, and print "
                         "a short line")
    args = ap.parse_args()
    if args.gpus != 1 or int(os.environ.get("WORLD_SIZE", "1")) > 1:
        if int(os.environ.get("RANK", "0")) == 0:
            print(json.dumps({"unavailable": f"this engine runs on one GPU; --gpus {args.gpus} is not supported",
                              "n_gpus": args.gpus}))
        return 2
    if args.warmup < 3:
        args.warmup = 3
    line = run_reference(args) if args.impl == "reference" else run_ours(args)
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
