"""Trace replay: feed given token ids through a model step by step, write logits.

Nothing is sampled and nothing is scheduled: the trace says which request
brings which tokens in which step.  The model, the step function, the cache
manager and the kernels are the ones generation uses; this file only turns
trace lines into `StepItem`s.  (The reference has no such program; the nearest
is driving `schedule -> build_inputs -> model` by hand in
tests/test_model_gpu.py:47-52.)

Input, one JSON object per line on standard input:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

`entries`: per request its next tokens and the places among them whose logits
are wanted; all entries of a step run as one batch.  `end`: requests that are
finished after the step; their pages are given back.  For a step that wants
something, `<out>/<step>.f32` holds the logits [wanted, vocab] as little-endian
float32 in the order of the entries and of `want`.  After every step a line
`done <step>` is printed and flushed.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np

from ..cache.manager import CacheManager
from ..cache.storage import CacheStorage
from ..config.engine import EngineConfig
from ..config.sampling import SamplingParams
from ..weights.loader import load_model
from .runner import ModelRunner, StepItem
from .sequence import Sequence


class TraceReplayer:
    def __init__(self, model_dir: str, dtype: str, max_tokens: int, device: str = "cuda", ops=None,
                 block_size: int = 16, enforce_eager: bool = False, poison: float | None = None,
                 max_num_seqs: int = 64):
        import torch

        self.device = torch.device(device)
        if ops is None:
            from ..kernels.ops import CudaOps
            ops = CudaOps(self.device)
        self.ops = ops
        self.model, self.model_config, self.dtype = load_model(model_dir, dtype, self.device, ops=ops)
        ops.set_compute_dtype(self.dtype)
        num_pages = max(1, -(-int(max_tokens) // block_size))
        max_len = num_pages * block_size
        self.model.prepare(max_len, self.device, ops)
        self.config = EngineConfig(block_size=block_size, num_gpu_blocks=num_pages, max_model_len=max(max_len, 2),
                                   max_num_batched_tokens=max(max_len, block_size), max_num_seqs=max_num_seqs,
                                   enable_prefix_caching=False, dtype=dtype, device=device,
                                   enforce_eager=enforce_eager)
        slots = self.model.cache_slots()
        self.storage = CacheStorage(slots, num_pages, block_size, self.dtype, self.device,
                                    num_state_slots=max_num_seqs if self.model.has_fixed_state else 0)
        if poison is not None:
            self.storage.fill(poison)
        self.cm = CacheManager(self.storage.group_specs() or num_pages, block_size, enable_prefix_caching=False,
                               num_state_slots=self.storage.num_state_slots)
        self.runner = ModelRunner(self.model, self.storage, self.cm, self.config, ops)
        self.live: dict[str, Sequence] = {}

    def step(self, record: dict) -> np.ndarray | None:
        """Runs one trace step.  Returns the wanted logits [wanted, vocab] as a
        float32 array, or None if nothing was wanted."""
        items = []
        vocab = self.model_config.vocab_size
        for e in record.get("entries", []):
            rid, tokens = str(e["id"]), [int(t) for t in e["tokens"]]
            if not tokens:
                continue
            bad = [t for t in tokens if not 0 <= t < vocab]
            if bad:
                raise ValueError(f"step {record.get('step')}: token ids {bad[:5]} outside the vocabulary of {vocab}")
            seq = self.live.get(rid)
            if seq is None:
                seq = Sequence(tokens, SamplingParams())
                self.live[rid] = seq
                if not self.cm.acquire_state_slot(seq):
                    raise RuntimeError(f"no state slot free: more than {self.config.max_num_seqs} live requests "
                                       "(raise --max-requests)")
            else:
                seq.token_ids.extend(tokens)
            if self.cm.allocate_slots(seq, len(tokens)) is None:
                held = {k: s.num_computed_tokens for k, s in self.live.items()}
                raise RuntimeError(f"step {record.get('step')}: the cache pool of {self.cm.num_blocks} pages x "
                                   f"{self.cm.block_size} tokens cannot take {len(tokens)} more tokens of request "
                                   f"{rid!r} (live requests hold {held}); raise --max-tokens")
            items.append(StepItem(seq, len(tokens), tuple(int(w) for w in e.get("want", []))))
        logits = self.runner.step(items) if items else None
        for it in items:
            it.seq.num_computed_tokens += it.num_new_tokens
            self.cm.release_behind_window(it.seq)
        for rid in record.get("end", []):
            seq = self.live.pop(str(rid), None)
            if seq is not None:
                self.cm.free(seq)
        if logits is None:
            return None
        out = logits.float().cpu().numpy().astype("<f4", copy=False)
        check = getattr(self.ops, "check_kernels", None)
        if check is not None:
            check()                      # a wait inside a kernel that gave up is an error, not a row of logits
        return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to a multiple of 64)")
    ap.add_argument("--block-size", type=int, default=16)
    ap.add_argument("--max-requests", type=int, default=64, help="most requests live at a time (state slots)")
    ap.add_argument("--enforce-eager", action="store_true", help="no CUDA-graph replay of decode steps")
    args = ap.parse_args(argv)
    os.makedirs(args.out, exist_ok=True)
    replayer = TraceReplayer(args.model, args.dtype, args.max_tokens, block_size=args.block_size,
                             enforce_eager=args.enforce_eager, max_num_seqs=args.max_requests)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        logits = replayer.step(record)
        if logits is not None:
            logits.tofile(os.path.join(args.out, f"{record['step']}.f32"))
        print(f"done {record['step']}", flush=True)
    return 0
