"""The step function: a batch of (request, its next tokens) in, logits out.

One step takes any list of (request, number of new tokens): portions of prompts
beside single decoded tokens, cut anywhere.  It runs only those tokens, as one
token-major batch with no padding, against what earlier steps left in the
cache, and returns float32 logits at the places that were asked for
(reference: `ModelRunner.build_inputs` / `run`, pagedllm/engine.py:51-102, which
returns logits only for the last token of requests that sample).

Metadata is gathered on the host into one pinned int32 buffer and reaches the
device in a single copy.  Decode-only steps (every request brings one token) are
replayed from CUDA graphs, one per batch-size bucket, unless `enforce_eager`.
"""

from __future__ import annotations

import gc
import os
from dataclasses import dataclass

import numpy as np
import torch

from ..cache.manager import CacheManager
from ..cache.storage import CacheStorage
from ..config.engine import EngineConfig
from ..kernels.plan import PlanCapacityError
from .context import AttentionPlan, HostBatch, StepContext
from .sequence import Sequence


@dataclass
class StepItem:
    seq: Sequence
    num_new_tokens: int
    want: tuple[int, ...] = ()      # places among this step's tokens whose logits are wanted


def _align(n: int, a: int = 4) -> int:
    return -(-n // a) * a


class _Packer:
    """Lays int32 sections out in one buffer, 16-byte aligned each."""

    def __init__(self):
        self.sections: list[tuple[str, int, np.ndarray]] = []
        self.size = 0

    def add(self, name: str, data: np.ndarray, capacity: int | None = None) -> None:
        data = np.ascontiguousarray(data, dtype=np.int32).reshape(-1)
        cap = max(int(capacity or 0), data.size, 1)
        self.sections.append((name, self.size, data))
        self.size += _align(cap)


class _Graph:
    """A captured step: its metadata buffer on the device, the graph, its output, and the
    packed metadata of the last replay (patched in place while the batch stays the same)."""

    def __init__(self, dev, graph, logits, size, launches, bucket):
        self.dev, self.graph, self.logits, self.size, self.launches, self.bucket = dev, graph, logits, size, launches, bucket
        self.packed = None
        self.offsets = None
        self.seq_ids = None
        self.versions = None
        self.strides = None
        self.plan_tag = None
        self.plan_shapes = None      # per plan key: (sizes of its three sections, max_splits, long_context) as captured
        self.wanted = 0              # rows of `logits` that the last replay asked for (graphs of mixed items)


class _NoMemoryForGraph(RuntimeError):
    """Capturing a graph ran out of device memory."""


class _Staging:
    """One pinned host buffer of the metadata ring, with the event of its last copy."""

    def __init__(self):
        self.tensor = None
        self.array = None
        self.event = None
        self.busy = False


class ModelRunner:
    GRAPH_BUCKETS = (1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128, 192, 256)

    def __init__(self, model, storage: CacheStorage, cache_manager: CacheManager, config: EngineConfig, ops,
                 sampler=None):
        self.model, self.storage, self.cm, self.config, self.ops = model, storage, cache_manager, config, ops
        self.sampler = sampler
        self.device = storage.device
        self.page_size = storage.page_size
        self.plan_keys = sorted({k for k in (getattr(b.mixer, "attention_plan_key", lambda: None)()
                                             for b in model.blocks) if k is not None},
                                key=lambda k: tuple(v or 0 for v in k))
        self._host_ring: list = []
        self._ring_pos = 0
        self._dev_meta = None
        self._graphs: dict[tuple, object] = {}
        self._portion_seen: dict[tuple, int] = {}
        self._no_graph: set[tuple] = set()        # keys whose capture ran out of memory
        self.use_graphs = ((not config.enforce_eager) and self.device.type == "cuda"
                           and getattr(ops, "supports_graphs", False) and getattr(model, "capturable", True))
        self.mixed_graphs = self.use_graphs and os.environ.get("PAGED_LLM_B200_NO_MIXED_GRAPHS") is None
        # request capacity of those graphs: the engine's limit, rounded up to a batch bucket
        self.MIXED_GRAPH_SEQS = next((b for b in self.GRAPH_BUCKETS if b >= config.max_num_seqs), self.GRAPH_BUCKETS[-1])
        self.num_graph_steps = 0
        self.num_eager_steps = 0
        self.graph_launches = 0            # kernels of this package launched by graph replays
        self.h2d_bytes = 0                 # metadata bytes copied host-to-device so far
        # A device tensor of token ids that replaces the next step's input ids on the
        # device (decode loops that never bring sampled tokens to the host).
        self.next_ids_override: torch.Tensor | None = None

    # ------------------------------------------------------------------ metadata
    def _gather(self, items: list[StepItem], pad_to: int | None = None, table_stride: int | None = None,
                pad_mixed: tuple[int, int] | None = None):
        """Host side of a step: numpy sections and the HostBatch.  With `pad_to`
        (replay of a decode graph) token and request counts are padded to the bucket; with
        `pad_mixed` = (tokens, requests) (replay of a graph of mixed items) tokens, requests,
        wanted rows and the attention work lists are padded to the capacity of any such step."""
        S = len(items)
        q_lens = [it.num_new_tokens for it in items]
        starts = [it.seq.num_computed_tokens for it in items]
        T = sum(q_lens)
        limit = self.config.max_model_len         # position tables are prepared for this many positions
        for it, st, n in zip(items, starts, q_lens):
            if st + n > limit:
                raise ValueError(f"request {it.seq.seq_id}: tokens {st}..{st + n} reach past max_model_len={limit}")
        if T == S and all(it.want == (0,) for it in items):
            # every request brings one token and wants its logits: no per-token loops
            for it, st in zip(items, starts):
                if st >= len(it.seq.token_ids):
                    raise ValueError(f"request {it.seq.seq_id} has {len(it.seq.token_ids)} tokens, step asks for {st}")
            ids = np.fromiter((it.seq.token_ids[st] for it, st in zip(items, starts)), np.int32, S)
            pos = np.array(starts, np.int32)
            tseq = np.arange(S, dtype=np.int32)
            want = list(range(S))
        else:
            ids = np.empty(T, np.int32)
            pos = np.empty(T, np.int32)
            tseq = np.empty(T, np.int32)
            want = []
            o = 0
            for s, it in enumerate(items):
                n, st = q_lens[s], starts[s]
                if n < 1:
                    raise ValueError("a step item needs at least one new token")
                toks = it.seq.token_ids[st:st + n]
                if len(toks) != n:
                    raise ValueError(f"request {it.seq.seq_id} has {len(it.seq.token_ids)} tokens, step asks for "
                                     f"{st}..{st + n}")
                ids[o:o + n] = toks
                pos[o:o + n] = np.arange(st, st + n, dtype=np.int32)
                tseq[o:o + n] = s
                for w in it.want:
                    if not 0 <= w < n:
                        raise ValueError(f"wanted place {w} is outside the {n} tokens of this step")
                    want.append(o + w)
                o += n
        S_pad = pad_to or S
        T_pad = pad_to or T
        if pad_mixed is not None:
            T_pad, S_pad = pad_mixed
            if T > T_pad or S > S_pad or len(want) > S_pad:
                raise PlanCapacityError(f"{T} tokens, {S} requests, {len(want)} wanted rows for a graph of "
                                        f"{T_pad} tokens and {S_pad} requests")
        host = HostBatch(q_lens, starts, [(-1 if it.seq.state_slot is None else it.seq.state_slot) for it in items],
                         [it.seq.seq_id for it in items])
        cu = np.zeros(S_pad + 1, np.int32)
        cu[1:S + 1] = np.cumsum(q_lens)
        cu[S + 1:] = T
        klen = np.zeros(S_pad, np.int32)
        klen[:S] = host.k_lens
        slots = np.full(S_pad, -1, np.int32)
        slots[:S] = host.state_slots
        if T_pad > T:
            ids = np.concatenate([ids, np.zeros(T_pad - T, np.int32)])
            pos = np.concatenate([pos, np.zeros(T_pad - T, np.int32)])
            tseq = np.concatenate([tseq, np.full(T_pad - T, -1, np.int32)])
        pk = _Packer()
        pk.add("ids", ids)
        pk.add("pos", pos)
        pk.add("tseq", tseq)
        pk.add("cu", cu)
        pk.add("klen", klen)
        pk.add("slots", slots)
        L_pad = pad_to or (S_pad if pad_mixed is not None else len(want))
        lidx = np.zeros(max(L_pad, 1), np.int32)
        lidx[:len(want)] = want
        pk.add("lidx", lidx)
        strides = []
        for g in range(self.storage.num_groups):
            rows = [self._table_row(it.seq, g) for it in items]
            stride = table_stride or _align(max([len(t) for t in rows] + [1]))
            bt = np.zeros((S_pad, stride), np.int32)
            for s, t in enumerate(rows):
                if len(t) > stride:
                    raise ValueError("block table longer than the captured stride")
                bt[s, :len(t)] = t
            strides.append(stride)
            pk.add(f"bt{g}", bt)
        plans = {}
        for key in self.plan_keys:
            if pad_mixed is not None:
                plan = self.ops.plan_attention(q_lens, host.k_lens, *key, pad_requests=S_pad, fixed_capacity=True,
                                               pad_tokens=T_pad)
            else:
                plan = self.ops.plan_attention(q_lens, host.k_lens, *key, pad_requests=S_pad,
                                               fixed_capacity=pad_to is not None)
            plans[key] = plan
            pk.add(f"small{key}", plan["small"])
            pk.add(f"large{key}", plan["large"])
            pk.add(f"splits{key}", plan["splits"])
        return pk, host, dict(T=T_pad, S=S_pad, L=len(want), L_pad=L_pad, strides=strides, plans=plans,
                              max_q=max(q_lens), padded=pad_mixed is not None,
                              logits_all=(pad_mixed is None and L_pad == T_pad and want == list(range(len(want)))))

    def _table_row(self, seq: Sequence, g: int) -> np.ndarray:
        """The request's block table of group g as an array, rebuilt only when the cache
        manager changed it."""
        cache = seq.__dict__.get("_table_rows")
        if cache is None or cache[0] != seq.table_version:
            cache = (seq.table_version, [np.asarray(t, np.int32) for t in seq.block_tables])
            seq.__dict__["_table_rows"] = cache
        rows = cache[1]
        return rows[g] if g < len(rows) else np.zeros(0, np.int32)

    def _host_buffer(self, n: int) -> "_Staging":
        """A pinned staging buffer that no copy in flight still reads."""
        if not self._host_ring:
            self._host_ring = [_Staging() for _ in range(4)]
        slot = self._host_ring[self._ring_pos % len(self._host_ring)]
        self._ring_pos += 1
        if slot.busy:
            slot.event.synchronize()
            slot.busy = False
        if slot.tensor is None or slot.tensor.numel() < n:
            slot.tensor = torch.empty(max(2 * n, 1 << 14), dtype=torch.int32, pin_memory=self.device.type == "cuda")
            slot.array = slot.tensor.numpy()
        return slot

    def _upload(self, pk: _Packer, dev: torch.Tensor | None = None) -> torch.Tensor:
        slot = self._host_buffer(pk.size)
        hv = slot.array
        for _, off, data in pk.sections:
            hv[off:off + data.size] = data
        if dev is None:
            if self._dev_meta is None or self._dev_meta.numel() < pk.size:
                self._dev_meta = torch.empty(max(pk.size * 2, 1 << 16), dtype=torch.int32, device=self.device)
            dev = self._dev_meta
        self._copy_up(slot, dev, pk.size)
        return dev

    def _context(self, pk: _Packer, dev: torch.Tensor, host: HostBatch, info: dict) -> StepContext:
        off = {name: (o, d.size) for name, o, d in pk.sections}

        def view(name, n=None):
            o, size = off[name]
            return dev[o:o + (size if n is None else n)]

        S, T = info["S"], info["T"]
        tables = [view(f"bt{g}").view(S, info["strides"][g]) for g in range(self.storage.num_groups)]
        plans = {}
        for key, p in info["plans"].items():
            ns = len(p["small"]) // 4
            nl = len(p["large"]) // 4
            plans[key] = AttentionPlan(
                small=view(f"small{key}", ns * 4).view(ns, 4) if ns else None,
                large=view(f"large{key}", nl * 4).view(nl, 4) if nl else None,
                splits=view(f"splits{key}"), n_small=ns, n_large=nl, max_splits=p["max_splits"],
                small_tokens=p["num_small_tokens"], long_context=p.get("long_context", False))
        return StepContext(
            ops=self.ops, num_tokens=T, num_seqs=S, num_logits=info["L_pad"],
            input_ids=view("ids"), positions=view("pos"), token_seq=view("tseq"), cu_seqlens_q=view("cu"),
            seq_lens_k=view("klen"), state_slots=view("slots"), logits_indices=view("lidx", max(info["L_pad"], 1)),
            block_tables=tables, layer_caches=self.storage.layer_caches, page_size=self.page_size,
            max_q_len=info["max_q"], host=host, attention_plans=plans, logits_all=info["logits_all"],
            padded=info.get("padded", False))

    # ------------------------------------------------------------------ the step
    @torch.no_grad()
    def step(self, items: list[StepItem]) -> torch.Tensor | None:
        """Runs the items' tokens as one batch.  Returns float32 logits
        [wanted places, vocab] in the order of the items and of their `want`, or
        None if nothing is wanted.  The caller has made the block tables cover
        the new tokens (`CacheManager.allocate_slots`) and advances the
        watermarks afterwards."""
        if not items:
            return None
        pin = getattr(self.ops, "pin_stream", None)
        if pin is None:
            return self._step(items)
        pin()
        try:
            return self._step(items)
        finally:
            self.ops.unpin_stream()

    def _step(self, items: list[StepItem]) -> torch.Tensor | None:
        self.storage.apply_copies(self.cm.take_pending_copies(), self.ops)
        if self.cm.num_state_slots:
            # state of fixed size: a request that starts (again) begins from zeros, a forked one from its
            # parent's state; both happen on the stream in front of the step, outside any captured graph
            self.storage.zero_state([it.seq.state_slot for it in items
                                     if it.seq.state_slot is not None and it.seq.num_computed_tokens == 0])
            self.storage.copy_state(self.cm.take_pending_state_copies())
        override, self.next_ids_override = self.next_ids_override, None
        key = self._graph_key(items)
        if key is not None:
            try:
                return self._graph_step(items, key, override)
            except PlanCapacityError:
                if key[0] != "mixed":
                    raise                # (a step that does not fit its mixed graph's capacity runs as launches)
            except _NoMemoryForGraph:
                pass                     # (no room to capture this graph: its steps run as launches from now on)
        pk, host, info = self._gather(items)
        dev = self._upload(pk)
        self._override_ids(dev, override)
        ctx = self._context(pk, dev, host, info)
        self.num_eager_steps += 1
        return self.model.forward(ctx)

    # ------------------------------------------------------------------ CUDA graphs for decode
    MAX_PORTION_GRAPHS = 4
    # Steps of mixed items (portions beside decoded tokens, several short prompts) of few tokens take less time
    # on the device than their launches take on the host (about 220 launches, 3 ms), or little more: they replay a
    # graph per 64 tokens, captured with spare capacity for requests, wanted rows and attention work items.
    # (measured beside 63 decoding requests, ms per step as a graph / as launches: 448 tokens 2.46 / 3.43, 768 tokens
    # 2.99 / 3.47, 960 tokens 3.39 / 3.70; beyond that the device takes so much longer than the host that launches do)
    MIXED_GRAPH_TOKENS = 1024
    MIXED_GRAPH_SEQS = 64            # (set per runner from max_num_seqs)
    MAX_MIXED_GRAPHS = 16

    def _graph_key(self, items: list[StepItem]):
        """The captured graph this step can replay, or None.  Decode-only steps (every request
        brings one token) replay a graph per batch-size bucket.  A step that is one portion of
        one request replays a graph per portion length, captured when that length is the token
        budget or comes a second time (a prompt cut by the budget brings the same length again
        and again).  Any other step of up to MIXED_GRAPH_TOKENS tokens replays a graph per 64
        tokens, captured when its bucket comes a second time.  A key whose capture ran out of
        device memory is not offered again."""
        if not self.use_graphs:          # (off too when a part of the model is not capturable)
            return None
        key = self._graph_key_of(items)
        return None if key in self._no_graph else key

    def _graph_key_of(self, items: list[StepItem]):
        if all(it.num_new_tokens == 1 and it.want == (0,) for it in items):
            if len(items) > self.GRAPH_BUCKETS[-1]:
                return None
            bucket = next(b for b in self.GRAPH_BUCKETS if b >= len(items))
            # few requests with long contexts take other attention kernels than the same batch
            # with short ones: a graph of its own
            # (and since the plan keys of a model may differ in kv heads, the class is kept per key)
            classify = getattr(self.ops, "long_context_class", None)
            if classify is not None and self.plan_keys:
                longest = max(it.seq.num_computed_tokens for it in items) + 1
                classes = tuple(bool(not key[2] and classify(bucket, key[1], longest)) for key in self.plan_keys)
                if any(classes):
                    return ("decode", bucket, classes)
            return ("decode", bucket)
        if len(items) == 1:
            n, want = items[0].num_new_tokens, items[0].want
            if n >= 64 and want in ((), (n - 1,)) and items[0].seq.num_computed_tokens + n <= self.config.max_model_len:
                key = ("portion", n, len(want))
                if key in self._graphs:
                    return key
                seen = self._portion_seen.get(key, 0) + 1
                self._portion_seen[key] = seen
                captured = sum(1 for k in self._graphs if k[0] == "portion")
                if captured < self.MAX_PORTION_GRAPHS and (n == self.config.max_num_batched_tokens or seen >= 2):
                    return key
        T = sum(it.num_new_tokens for it in items)
        if (self.mixed_graphs and T <= self.MIXED_GRAPH_TOKENS and len(items) <= self.MIXED_GRAPH_SEQS
                and sum(len(it.want) for it in items) <= self.MIXED_GRAPH_SEQS):
            key = ("mixed", -(-T // 64) * 64)
            if key in self._graphs:
                return key
            seen = self._portion_seen.get(key, 0) + 1
            self._portion_seen[key] = seen
            if seen >= 2 and sum(1 for k in self._graphs if k[0] == "mixed") < self.MAX_MIXED_GRAPHS:
                return key
        return None

    def _table_stride(self) -> int:
        return _align(-(-self.config.max_model_len // self.page_size))

    @staticmethod
    def _override_ids(dev: torch.Tensor, ids: torch.Tensor | None) -> None:
        if ids is not None:
            dev[:ids.numel()].copy_(ids.to(torch.int32), non_blocking=True)     # "ids" is the first section

    def _graph_step(self, items: list[StepItem], key, override: torch.Tensor | None = None):
        entry = self._graphs.get(key)
        if entry is not None and key[0] == "decode" and self._patch_decode(items, entry):
            pass                                        # the packed metadata of the last step was patched in place
        else:
            pad = key[1] if key[0] == "decode" else None
            mixed = (key[1], self.MIXED_GRAPH_SEQS) if key[0] == "mixed" else None
            pk, host, info = self._gather(items, pad_to=pad, table_stride=self._table_stride(), pad_mixed=mixed)
            if entry is None:
                try:
                    entry = self._capture(key, pk, host, info)
                except (torch.OutOfMemoryError, RuntimeError) as err:
                    if not isinstance(err, torch.OutOfMemoryError) and "out of memory" not in str(err).lower():
                        raise
                    # a graph keeps its activations for good; when the device has no room left for them the
                    # step still fits as launches (whose buffers come and go): this key is not tried again
                    self._no_graph.add(key)
                    torch.cuda.empty_cache() if self.device.type == "cuda" else None
                    raise _NoMemoryForGraph(key) from None
                entry.plan_shapes = self._plan_shapes(info["plans"])
            if pk.size != entry.size or self._plan_shapes(info["plans"]) != entry.plan_shapes:
                if mixed is not None:
                    raise PlanCapacityError(f"the plan of this step differs from the one graph {key} was captured with")
                raise RuntimeError("metadata layout or attention plan changed between capture and replay of "
                                   f"graph {key}: the captured kernels would read it wrongly")
            entry.wanted = info["L"]
            packed = np.zeros(pk.size, np.int32)
            for _, off, data in pk.sections:
                packed[off:off + data.size] = data
            entry.packed = packed
            entry.offsets = {name: off for name, off, _ in pk.sections}
            entry.seq_ids = tuple(it.seq.seq_id for it in items)
            entry.versions = [it.seq.table_version for it in items]
            entry.strides = info["strides"]
            entry.plan_tag = None
        slot = self._host_buffer(entry.size)
        slot.array[:entry.size] = entry.packed
        self._copy_up(slot, entry.dev, entry.size)
        self._override_ids(entry.dev, override)
        entry.graph.replay()
        self.num_graph_steps += 1
        self.graph_launches += entry.launches
        if entry.logits is None:
            return None
        if key[0] == "mixed":
            return entry.logits[:entry.wanted] if entry.wanted else None
        return entry.logits[:len(items)] if key[0] == "decode" else entry.logits

    @staticmethod
    def _plan_shapes(plans: dict) -> dict:
        """What a captured graph has baked in of each attention plan: the capacity of its lists,
        the number of splits its kernels were launched for, and its class."""
        return {key: (tuple(int(np.asarray(p[name]).size) for name in ("small", "large", "splits")),
                      int(p["max_splits"]), bool(p.get("long_context", False))) for key, p in plans.items()}

    def _patch_decode(self, items: list[StepItem], entry) -> bool:
        """Steady decoding: the same requests as in the last replay of this graph, one token
        further.  Only what moved is rewritten in the packed metadata: token ids, positions,
        context lengths, block-table rows that the cache manager changed, and the attention
        work lists.  Returns False if the batch is another one (the caller gathers anew)."""
        if entry.packed is None or entry.seq_ids != tuple(it.seq.seq_id for it in items):
            return False
        S = len(items)
        starts = [it.seq.num_computed_tokens for it in items]
        if max(starts) >= self.config.max_model_len:
            raise ValueError(f"a request reaches past max_model_len={self.config.max_model_len}")
        try:
            ids = [it.seq.token_ids[st] for it, st in zip(items, starts)]
        except IndexError:
            raise ValueError("a request has no token at the position this step asks for") from None
        buf, off = entry.packed, entry.offsets
        buf[off["ids"]:off["ids"] + S] = ids
        buf[off["pos"]:off["pos"] + S] = starts
        klen = [st + 1 for st in starts]
        buf[off["klen"]:off["klen"] + S] = klen
        for s, it in enumerate(items):
            if it.seq.table_version != entry.versions[s]:
                entry.versions[s] = it.seq.table_version
                for g, stride in enumerate(entry.strides):
                    row = self._table_row(it.seq, g)
                    if len(row) > stride:
                        raise ValueError("block table longer than the captured stride")
                    o = off[f"bt{g}"] + s * stride
                    buf[o:o + len(row)] = row
                    buf[o + len(row):o + stride] = 0
        # the work lists change only when a context grows past another multiple of the split size
        step_keys = getattr(self.ops, "MIN_SPLIT_KEYS", 128)
        windowed = any(key[2] for key in self.plan_keys)
        tag = None if windowed else tuple(-(-k // step_keys) for k in klen)
        if tag is None or tag != entry.plan_tag:
            entry.plan_tag = tag
            ones = [1] * S
            plans = {key: self.ops.plan_attention(ones, klen, *key, pad_requests=entry.bucket, fixed_capacity=True)
                     for key in self.plan_keys}
            if self._plan_shapes(plans) != entry.plan_shapes:
                # another list capacity, split count or class than the graph was captured with: nothing is
                # patched (a longer list would run over the next section); the caller gathers anew and checks
                entry.packed = None
                return False
            for key, plan in plans.items():
                for name in ("small", "large", "splits"):
                    data = plan[name]
                    o = off[f"{name}{key}"]
                    buf[o:o + data.size] = data
        return True

    def _copy_up(self, slot: "_Staging", dev: torch.Tensor, n: int) -> None:
        if hasattr(self.ops, "copy_h2d"):
            self.ops.copy_h2d(dev, slot.tensor, n * 4)
        else:
            dev[:n].copy_(slot.tensor[:n], non_blocking=True)
        self.h2d_bytes += n * 4
        if self.device.type == "cuda":
            if slot.event is None:
                slot.event = torch.cuda.Event()
            slot.event.record()
            slot.busy = True

    def _capture(self, key, pk: _Packer, host: HostBatch, info: dict) -> "_Graph":
        dev = torch.empty(pk.size, dtype=torch.int32, device=self.device)
        self._upload(pk, dev)
        ctx = self._context(pk, dev, host, info)
        # The trial runs write this step's keys and values (the replay writes the same again) but must
        # leave state of fixed size as it was: a stateful mixer's step is not idempotent.
        saved_state = self.storage.save_state() if self.cm.num_state_slots else None
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        repin = getattr(self.ops, "pin_stream", lambda: None)
        with torch.cuda.stream(side):
            repin()
            for _ in range(2):                       # warm-up: library workspaces, lazy module loads
                self.model.forward(ctx)
        repin()
        torch.cuda.current_stream().wait_stream(side)
        if saved_state is not None:
            self.storage.restore_state(saved_state)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        before = getattr(self.ops, "launches", 0)
        # No garbage collection while the stream captures: collecting an older engine's graphs then
        # (their destructors free device memory) is not permitted during a capture and would invalidate it.
        gc_was_on = gc.isenabled()
        gc.disable()
        try:
            with torch.cuda.graph(graph):
                repin()                              # the capture runs on a stream of its own
                logits = self.model.forward(ctx)
        finally:
            repin()
            if gc_was_on:
                gc.enable()
        launches = getattr(self.ops, "launches", 0) - before
        if hasattr(self.ops, "launches"):
            self.ops.launches = before        # capturing launches nothing; replays are counted in graph_launches
        entry = _Graph(dev, graph, logits, pk.size, launches, key[1] if key[0] == "decode" else None)
        self._graphs[key] = entry
        return entry

    # ------------------------------------------------------------------ scheduler-facing
    @torch.no_grad()
    def run(self, out) -> dict[int, int]:
        """One scheduled step: runs it and samples where a request reached its
        last known token (reference: pagedllm/engine.py:93-102)."""
        sampled, ids = self.launch(out)
        if ids is None:
            return {}
        return {seq.seq_id: int(tok) for seq, tok in zip(sampled, ids.tolist())}

    @torch.no_grad()
    def launch(self, out):
        """The same without waiting for the result: returns the requests that sample in this
        step and their token ids as a device tensor (None if no request samples)."""
        items = [StepItem(s.seq, s.num_new_tokens, (s.num_new_tokens - 1,) if s.needs_sampling else ())
                 for s in out.scheduled]
        logits = self.step(items)
        if logits is None:
            return [], None
        sampled = [s.seq for s in out.scheduled if s.needs_sampling]
        return sampled, self.sampler.sample_on_device(logits, sampled)
