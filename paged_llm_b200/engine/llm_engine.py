"""`LLMEngine`: model folder in, generated tokens out.

The surface is the reference's (pagedllm/engine.py:105-234): `LLMEngine(model,
config=None, **overrides)`, `add_request`, `abort_request`, `step`, `generate`,
`has_unfinished_requests`, `stats`; `RequestOutput`, `StepOutput` and
`EngineStats` carry the same fields.  Prompts are lists of token ids, or text if
the model folder has tokenizer files.
"""

from __future__ import annotations

import dataclasses
import logging
import os
import time
from dataclasses import dataclass, field

import torch

from ..cache.manager import CacheManager
from ..cache.storage import CacheStorage
from ..config.engine import EngineConfig
from ..config.sampling import SamplingParams
from ..sampling.sampler import Sampler
from ..weights.loader import load_model, read_hf_config
from .runner import ModelRunner, StepItem
from .scheduler import Scheduler
from .sequence import Sequence

log = logging.getLogger("paged_llm_b200")


@dataclass
class StepOutput:
    seq_id: int
    new_token: int | None
    finished: bool


@dataclass
class RequestOutput:
    seq_id: int
    prompt_token_ids: list[int]
    token_ids: list[int]            # generated tokens only
    text: str
    finish_reason: str              # "stop" | "length" | "abort"
    num_cached_tokens: int
    num_preemptions: int


@dataclass
class EngineStats:
    num_steps: int = 0
    num_prefill_tokens: int = 0
    num_decode_tokens: int = 0
    num_preemptions: int = 0
    step_times: list[float] = field(default_factory=list)
    num_steps_ahead: int = 0           # steps launched before the tokens of the step in front were read


@dataclass
class _InFlight:
    """A step that is launched but whose tokens have not been read yet."""
    out: object                     # its SchedulerOutput
    sampled: list                   # the requests that sample in it, in the order of `ids`
    ids: torch.Tensor | None        # their token ids on the device
    host: torch.Tensor | None       # the same on their way to pinned host memory
    event: object                   # recorded behind that copy
    t0: float


_FINISH = {"FINISHED_STOPPED": "stop", "FINISHED_LENGTH": "length", "FINISHED_ABORTED": "abort"}
_TOKENIZER_FILES = ("tokenizer.json", "tokenizer.model", "tokenizer_config.json")


def _load_tokenizer(path: str):
    if not any(os.path.exists(os.path.join(path, f)) for f in _TOKENIZER_FILES):
        return None
    from transformers import AutoTokenizer       # tokenizer only, as in the reference (engine.py:112-114)
    return AutoTokenizer.from_pretrained(path)


def _eos_from_config(hf_config: dict):
    eos = hf_config.get("eos_token_id")
    if isinstance(eos, list):
        eos = eos[0] if eos else None
    return eos


class LLMEngine:
    def __init__(self, model: str, config: EngineConfig | None = None, ops=None, **overrides):
        self.config = cfg = config or EngineConfig(**overrides)
        self.device = torch.device(cfg.device)
        if not os.path.isdir(model):
            raise FileNotFoundError(f"{model!r} is not a model folder (config.json + *.safetensors); "
                                    "downloading from a hub is not supported")
        if ops is None:
            from ..kernels.ops import CudaOps
            ops = CudaOps(self.device)
        self.ops = ops
        self.tokenizer = _load_tokenizer(model)
        hf_config = read_hf_config(model)
        t0 = time.perf_counter()
        self.model, self.model_config, self.dtype = load_model(model, cfg.dtype, self.device, ops=ops)
        ops.set_compute_dtype(self.dtype)
        self.model.prepare(cfg.max_model_len, self.device, ops)
        log.info("loaded %s in %.1fs (dtype=%s)", model, time.perf_counter() - t0, self.dtype)

        slots = self.model.cache_slots()
        has_state = self.model.has_fixed_state
        self.sampler = Sampler(ops, cfg.seed)
        self.activation_peak_bytes = None      # measured when the pool is sized here (num_gpu_blocks not given)
        num_blocks = cfg.num_gpu_blocks or self._size_pool(slots, has_state)
        self.kv_cache = CacheStorage(slots, num_blocks, cfg.block_size, self.dtype, self.device,
                                     num_state_slots=cfg.max_num_seqs if has_state else 0)
        self.block_manager = CacheManager(self.kv_cache.group_specs() or num_blocks, cfg.block_size,
                                          cfg.enable_prefix_caching, num_state_slots=self.kv_cache.num_state_slots)
        eos = self.tokenizer.eos_token_id if self.tokenizer is not None else _eos_from_config(hf_config)
        self.scheduler = Scheduler(cfg, self.block_manager, eos)
        self.runner = ModelRunner(self.model, self.kv_cache, self.block_manager, cfg, ops, self.sampler)
        self.stats = EngineStats()
        self._seqs: dict[int, Sequence] = {}
        self._in_flight: _InFlight | None = None
        self._unreported: list[StepOutput] = []
        self._pinned: list[torch.Tensor] = []
        self._pinned_pos = 0
        self._steps_since_check = 0
        log.info("KV cache: %d blocks x %d tokens = %d tokens (%.2f GiB)", num_blocks, cfg.block_size,
                 num_blocks * cfg.block_size, num_blocks * self.kv_cache.page_bytes() / 2 ** 30)

    # ---- sizing -------------------------------------------------------------------
    def _activation_peak(self, slots, has_state: bool) -> int:
        """Bytes the largest step needs beyond weights and cache: measured, as the reference does
        (engine.py:161-179), by running one step of `max_num_batched_tokens` tokens of one request
        that samples at `max_num_seqs` places, on a throw-away pool just large enough for it, and
        reading the allocator's peak."""
        cfg = self.config
        n_tok = min(cfg.max_num_batched_tokens, cfg.max_model_len)
        pages = -(-n_tok // cfg.block_size) + 1
        torch.cuda.synchronize(self.device)
        torch.cuda.empty_cache()
        base = torch.cuda.memory_allocated(self.device)
        storage = CacheStorage(slots, pages, cfg.block_size, self.dtype, self.device,
                               num_state_slots=1 if has_state else 0)
        manager = CacheManager(storage.group_specs() or pages, cfg.block_size, False,
                               num_state_slots=storage.num_state_slots)
        eager = dataclasses.replace(cfg, enforce_eager=True, num_gpu_blocks=pages)
        runner = ModelRunner(self.model, storage, manager, eager, self.ops)
        seq = Sequence([0] * n_tok, SamplingParams())
        manager.acquire_state_slot(seq)
        if manager.allocate_slots(seq, n_tok) is None:
            raise RuntimeError("the throw-away pool of the sizing step is too small")
        held = torch.cuda.memory_allocated(self.device) - base
        torch.cuda.reset_peak_memory_stats(self.device)
        rows = min(n_tok, cfg.max_num_seqs)
        logits = runner.step([StepItem(seq, n_tok, tuple(range(n_tok - rows, n_tok)))])
        if logits is not None and self.sampler is not None:
            self.ops.argmax(logits)
        torch.cuda.synchronize(self.device)
        peak = torch.cuda.max_memory_allocated(self.device) - base - held
        del logits, runner, manager, storage
        torch.cuda.empty_cache()
        return int(peak)

    def _size_pool(self, slots, has_state: bool = False) -> int:
        """Pages that fit in `gpu_memory_utilization` of the device beside the weights, what other
        processes hold, and the measured peak of one largest step (`_activation_peak`)."""
        cfg = self.config
        page_bytes = CacheStorage.page_bytes_for(slots, cfg.block_size, self.dtype)
        if self.device.type != "cuda" or page_bytes == 0:
            return max(64, cfg.max_model_len * 4 // cfg.block_size)
        peak = self._activation_peak(slots, has_state)
        free, total = torch.cuda.mem_get_info(self.device)
        ours = torch.cuda.memory_reserved(self.device)
        used_by_others = total - free - ours
        budget = int(total * cfg.gpu_memory_utilization) - used_by_others - torch.cuda.memory_allocated(self.device) - peak
        num_blocks = budget // page_bytes
        # no request can use more than max_model_len tokens: more pages than every
        # running request at full length would never be touched
        num_blocks = min(num_blocks, cfg.max_num_seqs * (-(-cfg.max_model_len // cfg.block_size)) + 16)
        if num_blocks < 16:
            raise RuntimeError(f"not enough GPU memory for the KV cache ({num_blocks} blocks); lower "
                               "max_num_batched_tokens or raise gpu_memory_utilization")
        self.activation_peak_bytes = peak
        return int(num_blocks)

    # ---- requests -----------------------------------------------------------------
    def add_request(self, prompt: str | list[int], sampling_params: SamplingParams | None = None) -> int:
        if isinstance(prompt, str):
            if self.tokenizer is None:
                raise ValueError("this model folder has no tokenizer files; pass prompts as lists of token ids")
            ids = self.tokenizer.encode(prompt)
        else:
            ids = [int(t) for t in prompt]
        vocab = self.model_config.vocab_size
        bad = [t for t in ids if not 0 <= t < vocab]
        if bad:
            raise ValueError(f"token ids {bad[:5]} are outside the vocabulary of {vocab}")
        seq = Sequence(ids, sampling_params or SamplingParams())
        self.scheduler.add(seq)
        self._seqs[seq.seq_id] = seq
        return seq.seq_id

    def abort_request(self, seq_id: int) -> None:
        if self._in_flight is not None:              # its tokens first, then the request may go
            flight, self._in_flight = self._in_flight, None
            self._unreported += self._resolve(flight)
        self.scheduler.abort(seq_id)

    @property
    def has_unfinished_requests(self) -> bool:
        return self.scheduler.has_unfinished or self._in_flight is not None or bool(self._unreported)

    # ---- stepping -----------------------------------------------------------------
    def step(self) -> list[StepOutput]:
        """One step of the engine: returns, for each request of the step whose tokens are read,
        its new token (None for a portion of a prompt that samples nothing) and whether it
        finished (reference: pagedllm/engine.py:186-211).

        While requests only decode, the steps overlap: the step after is launched from what is
        known on the host (positions, pages) with its input tokens taken from the device, and
        only then are the tokens of the step in front read, appended and checked.  The device
        never waits for the host that way.  A request that turns out to have stopped (EOS, a
        stop token) has then run one step in vain; its token of that step is dropped.  A step
        is never launched ahead when a request is about to reach its length limit, when
        requests wait for admission, or when pages could run out."""
        t0 = time.perf_counter()
        outputs, self._unreported = self._unreported, []
        flight = self._in_flight
        if flight is None:
            flight = self._launch(None, t0)
            if flight is None:
                return outputs
        self._in_flight = self._launch(flight, t0) if self._may_run_ahead(flight) else None
        outputs += self._resolve(flight)
        self._check_kernels(force=not self.scheduler.has_unfinished and self._in_flight is None)
        self.stats.step_times.append(time.perf_counter() - t0)
        return outputs

    def _launch(self, ahead_of: _InFlight | None, t0: float) -> _InFlight | None:
        """Schedules and launches a step.  `ahead_of`: the step whose tokens, still on the
        device, are this step's input."""
        out = self.scheduler.schedule()
        if out.is_empty:
            if self.scheduler.has_unfinished and ahead_of is None:
                raise RuntimeError("no request can be scheduled although some are unfinished: the cache pool is "
                                   "too small for the oldest waiting request")
            return None
        if ahead_of is not None:
            assert [i.seq.seq_id for i in out.scheduled] == [s.seq_id for s in ahead_of.sampled]
            self.runner.next_ids_override = ahead_of.ids
            self.stats.num_steps_ahead += 1
        sampled, ids = self.runner.launch(out)
        self.scheduler.advance(out)
        host = event = None
        if ids is not None and ids.is_cuda:
            if len(self._pinned) < 2 or self._pinned[0].numel() < ids.numel():
                self._pinned = [torch.empty(max(ids.numel(), 256), dtype=ids.dtype, pin_memory=True) for _ in range(2)]
            self._pinned_pos ^= 1
            host = self._pinned[self._pinned_pos][:ids.numel()]
            host.copy_(ids, non_blocking=True)
            event = torch.cuda.Event()
            event.record()
        st = self.stats
        st.num_steps += 1
        st.num_prefill_tokens += out.num_prefill_tokens
        st.num_decode_tokens += out.num_decode_tokens
        st.num_preemptions += len(out.preempted)
        return _InFlight(out, sampled, ids, host, event, t0)

    def _may_run_ahead(self, flight: _InFlight) -> bool:
        """Whether the step after `flight` can be launched before its tokens are read: it is
        the same requests decoding one token further, whatever those tokens are."""
        sch, cfg = self.scheduler, self.config
        if not cfg.overlap_decode or flight.ids is None or sch.waiting:
            return False
        out = flight.out
        if out.num_prefill_tokens or out.preempted or len(out.scheduled) != len(sch.running):
            return False
        for item, seq in zip(out.scheduled, sch.running):
            if item.seq is not seq or not item.needs_sampling or seq.num_unresolved != 1:
                return False
            # its length limit would end it with the token on its way: nothing to run ahead for
            if seq.num_generated_tokens >= seq.max_tokens or seq.num_tokens >= cfg.max_model_len:
                return False
        # a page each at most, and none must be taken from a running request
        bm = self.block_manager
        return min(bm.num_free_in_group(g) for g in range(len(bm.pools))) >= len(sch.running)

    HEALTH_CHECK_STEPS = 256      # steps between two looks at the kernels' fault counters

    def _check_kernels(self, force: bool = False) -> None:
        """Looks at the kernel library's fault counters (bounded waits that gave up) every
        `HEALTH_CHECK_STEPS` steps, and when the engine runs dry: a fault raises `KernelError`
        instead of passing for tokens.  Reading them waits for the device, hence not every step."""
        check = getattr(self.ops, "check_kernels", None)
        if check is None:
            return
        self._steps_since_check += 1
        if force or self._steps_since_check >= self.HEALTH_CHECK_STEPS:
            self._steps_since_check = 0
            check()

    def _resolve(self, flight: _InFlight) -> list[StepOutput]:
        """Reads the tokens of a launched step and lets the scheduler take them in."""
        sampled: dict[int, int] = {}
        if flight.ids is not None:
            if flight.event is not None:
                flight.event.synchronize()
                tokens = flight.host.tolist()
            else:
                tokens = flight.ids.tolist()
            sampled = {seq.seq_id: int(tok) for seq, tok in zip(flight.sampled, tokens)}
        live = [i for i in flight.out.scheduled if not i.seq.is_finished]
        finished = {s.seq_id for s in self.scheduler.resolve(flight.out, sampled)}
        return [StepOutput(i.seq.seq_id, sampled.get(i.seq.seq_id) if i.needs_sampling else None,
                           i.seq.seq_id in finished) for i in live]

    def warm_up(self, max_batch: int | None = None) -> int:
        """Captures the decode graphs of the batch-size buckets up to `max_batch` (default:
        `max_num_seqs`) and the graphs of small mixed steps by running throw-away requests, so that
        no request pays for a capture later (15-150 ms each when a bucket is first seen).  Not in the
        reference.  Returns the number of graphs held afterwards; the cache is as before."""
        if self.has_unfinished_requests:
            raise RuntimeError("warm_up needs an idle engine")
        buckets = [b for b in self.runner.GRAPH_BUCKETS if b <= (max_batch or self.config.max_num_seqs)]
        if not self.runner.use_graphs:
            return 0
        stats, self.stats = self.stats, EngineStats()
        try:
            for b in buckets:
                params = SamplingParams(temperature=0.0, max_tokens=3, ignore_eos=True)
                ids = [self.add_request([0], params) for _ in range(b)]
                while self.has_unfinished_requests:
                    self.step()
                for i in ids:
                    self._seqs.pop(i, None)
            # the graphs of small mixed steps: two prompts that fill a bucket of tokens together, twice each (a
            # graph is captured when its bucket comes the second time), with tokens of their own so that no
            # prefix is found in the cache
            if getattr(self.runner, "mixed_graphs", False) and self.config.max_num_seqs >= 2:
                one = SamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True)
                vocab = self.model_config.vocab_size
                limit = min(self.runner.MIXED_GRAPH_TOKENS, self.config.max_num_batched_tokens,
                            self.config.max_model_len - 2)
                for n, t in enumerate(range(64, limit + 1, 64)):
                    if sum(1 for k in self.runner._graphs if k[0] == "mixed") >= self.runner.MAX_MIXED_GRAPHS:
                        break
                    for again in range(2):
                        tok = (2 * n + again + 1) % vocab
                        ids = [self.add_request([tok] * (t - 1), one), self.add_request([tok], one)]
                        while self.has_unfinished_requests:
                            self.step()
                        for i in ids:
                            self._seqs.pop(i, None)
        finally:
            self.stats = stats
        return len(self.runner._graphs)

    def _to_output(self, seq: Sequence) -> RequestOutput:
        text = ""
        if self.tokenizer is not None:
            text = self.tokenizer.decode(seq.output_token_ids, skip_special_tokens=True)
        return RequestOutput(seq.seq_id, seq.prompt_token_ids, seq.output_token_ids, text,
                             _FINISH[seq.status.name], seq.num_cached_tokens, seq.num_preemptions)

    def generate(self, prompts, sampling_params: SamplingParams | list[SamplingParams] | None = None,
                 use_tqdm: bool = False) -> list[RequestOutput]:
        if not isinstance(sampling_params, list):
            sampling_params = [sampling_params or SamplingParams()] * len(prompts)
        if len(sampling_params) != len(prompts):
            raise ValueError("one SamplingParams per prompt, or one for all")
        ids = [self.add_request(p, sp) for p, sp in zip(prompts, sampling_params)]
        bar = None
        if use_tqdm:
            from tqdm import tqdm
            bar = tqdm(total=len(ids), desc="requests")
        while self.has_unfinished_requests:
            for o in self.step():
                if o.finished and bar is not None:
                    bar.update(1)
        if bar is not None:
            bar.close()
        return [self._to_output(self._seqs.pop(i)) for i in ids]
