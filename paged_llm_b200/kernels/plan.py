"""Work lists for the attention kernels, made on the host once per step.

A request with nq new tokens and G query heads per kv head has nq*G query rows
per kv head (row r = token r // G, head r % G).  Requests with at most
`small_rows` rows (decoding, or a portion of a very few tokens) go to the
split-context kernel: their keys are cut into `splits` ranges that run in
separate thread blocks and are merged afterwards, so that a few long requests
still fill the machine (the reference runs one program per query tile and never
splits the context: pagedllm/attention/triton_kernel.py:10-12, :120).  The
others are cut into tiles of `large_rows` rows.

An item is four int32: (request, tile or scratch base, split, splits).  For a
fixed request count and fixed lengths the plan is deterministic, so replaying a
step reproduces its logits bit for bit.
"""

from __future__ import annotations

import numpy as np


def wanted_splits(num_small: int, num_kv_heads: int, num_sms: int, max_splits: int) -> int:
    """Splits per request so that requests x kv heads x splits is about one
    thread block per SM (measured: more splits cost more in merging than they win)."""
    if num_small <= 0:
        return 1
    target_items = -(-num_sms // max(num_kv_heads, 1))
    return int(min(max_splits, max(1, -(-target_items // num_small))))


def long_context_splits(num_requests: int, num_kv_heads: int, num_sms: int, max_splits: int) -> int:
    return int(max(1, min(max_splits, (3 * num_sms) // max(1, num_requests * max(num_kv_heads, 1)))))


def is_long_context(num_requests: int, num_kv_heads: int, num_sms: int, max_splits: int, cluster_max: int,
                    long_keys: int, max_context: int) -> bool:
    """Whether a decode step of this shape is in the long-context class: the blocks of a cluster
    (at most `cluster_max` per request and kv head) would each walk more than `long_keys` keys.
    Such a step is split further, through the work list: about three blocks per SM, which is
    what is resident at a time and what it takes to keep memory busy with one block's latencies
    (measured: 16 k context at batch 8, 2.05 ms per step as clusters of 5, 1.50 ms as 13 splits)."""
    if cluster_max <= 0:
        return False
    cluster = min(wanted_splits(num_requests, num_kv_heads, num_sms, max_splits), cluster_max)
    if long_context_splits(num_requests, num_kv_heads, num_sms, max_splits) <= cluster:
        return False                 # so many requests that the work list would not split further either
    return max_context > long_keys * cluster


def _plan_decode(S, S_pad, k_lens, num_kv_heads, min_split_keys, num_sms, max_splits, fixed_capacity,
                 cluster_max=0, long_keys=0) -> dict:
    """The same plan for the common step in which every request brings one token, in array form."""
    n_req = S_pad if fixed_capacity else S
    long_context = is_long_context(n_req, num_kv_heads, num_sms, max_splits, cluster_max, long_keys,
                                   int(max(k_lens)) if len(k_lens) else 0)
    want = long_context_splits(n_req, num_kv_heads, num_sms, max_splits) if long_context \
        else wanted_splits(n_req, num_kv_heads, num_sms, max_splits)
    lk = np.asarray(k_lens, np.int64)
    ns = np.maximum(1, np.minimum(want, -(-lk // min_split_keys))).astype(np.int32)
    splits = np.ones((S_pad, 2), np.int32)
    splits[:, 1] = 0
    splits[:S, 0] = ns
    splits[:S, 1] = np.arange(S, dtype=np.int32)
    total = int(ns.sum())
    seq = np.repeat(np.arange(S, dtype=np.int32), ns)
    first = np.cumsum(ns) - ns
    small = np.empty((total, 4), np.int32)
    small[:, 0] = seq
    small[:, 1] = seq                                   # scratch base: one token per request
    small[:, 2] = np.arange(total, dtype=np.int32) - np.repeat(first, ns).astype(np.int32)
    small[:, 3] = np.repeat(ns, ns)
    if fixed_capacity:
        cap = S_pad * want
        if cap > total:
            small = np.concatenate([small, np.full((cap - total, 4), -1, np.int32)])
    return {"small": small.reshape(-1), "large": np.zeros(0, np.int32), "splits": splits.reshape(-1),
            "max_splits": int(want), "num_small_tokens": int(S_pad if fixed_capacity else S),
            "long_context": long_context}


class PlanCapacityError(ValueError):
    """A step does not fit the fixed capacity its plan was asked for."""


def large_capacity(num_tokens: int, group_size: int, small_rows: int, large_rows: int) -> int:
    """An upper bound of the row tiles of the large items of any step of `num_tokens` tokens: every tile but a
    request's last is full, and a request with a large item has more than `small_rows` rows."""
    rows = num_tokens * group_size
    return rows // large_rows + rows // (small_rows + 1) + 1


def plan_attention(q_lens, k_lens, group_size: int, num_kv_heads: int, window: int | None, *, small_rows: int,
                   large_rows: int, min_split_keys: int, num_sms: int, max_splits: int = 32,
                   pad_requests: int | None = None, fixed_capacity: bool = False, cluster_max: int = 0,
                   long_keys: int = 0, pad_tokens: int | None = None) -> dict:
    """`pad_tokens` (with `fixed_capacity`, for a step of mixed items that replays a captured graph): both lists
    get the capacity of any step of that many tokens and `pad_requests` requests, filled up with items of
    request -1 that the kernels skip."""
    S = len(q_lens)
    S_pad = pad_requests or S
    if pad_tokens is None and S and max(q_lens) == 1 and group_size <= small_rows and not window:
        return _plan_decode(S, S_pad, k_lens, num_kv_heads, min_split_keys, num_sms, max_splits, fixed_capacity,
                            cluster_max, long_keys)
    small_ids = [s for s in range(S) if q_lens[s] * group_size <= small_rows]
    n_small = S_pad if fixed_capacity else len(small_ids)
    want = wanted_splits(n_small, num_kv_heads, num_sms, max_splits)
    splits = np.ones((S_pad, 2), np.int32)
    splits[:, 1] = 0
    small = []
    scratch_base = 0
    for s in small_ids:
        nq, lk = q_lens[s], k_lens[s]
        first_pos = lk - nq
        lo = max(0, first_pos - window + 1) if window else 0
        n_keys = lk - lo
        ns = max(1, min(want, -(-n_keys // min_split_keys)))
        splits[s] = (ns, scratch_base)
        for j in range(ns):
            small.append((s, scratch_base, j, ns))
        scratch_base += nq
    large = []
    for s in range(S):
        rows = q_lens[s] * group_size
        if rows <= small_rows:
            continue
        tiles = -(-rows // large_rows)
        for t in range(tiles):
            last_tok = min(rows - 1, (t + 1) * large_rows - 1) // group_size
            large.append((k_lens[s] - q_lens[s] + last_tok, s, t))
    large.sort(key=lambda x: -x[0])                       # longest first
    small_arr = np.array(small, np.int32).reshape(-1, 4)
    if fixed_capacity:
        cap = S_pad * want
        if len(small_arr) > cap:
            raise PlanCapacityError(f"{len(small_arr)} small items for a capacity of {cap}")
        pad = np.full((cap - len(small_arr), 4), -1, np.int32)
        small_arr = np.concatenate([small_arr, pad]) if len(pad) else small_arr
    large_arr = np.array([(s, t, 0, 1) for _, s, t in large], np.int32).reshape(-1, 4)
    small_tokens = int(scratch_base) if not fixed_capacity else int(S_pad)
    if pad_tokens is not None and fixed_capacity:
        cap = large_capacity(pad_tokens, group_size, small_rows, large_rows)
        if len(large_arr) > cap or sum(q_lens) > pad_tokens:
            raise PlanCapacityError(f"{len(large_arr)} large items for a capacity of {cap}")
        large_arr = np.concatenate([large_arr, np.full((cap - len(large_arr), 4), -1, np.int32)])
        small_tokens = int(S_pad) * max(1, small_rows // group_size)       # a small item may bring several tokens
        if scratch_base > small_tokens:
            raise PlanCapacityError(f"{scratch_base} tokens of small items for {small_tokens} scratch rows")
    return {
        "small": small_arr.reshape(-1),
        "large": large_arr.reshape(-1),
        "splits": splits.reshape(-1),
        "max_splits": int(want),
        "num_small_tokens": small_tokens,
        "long_context": False,
    }
