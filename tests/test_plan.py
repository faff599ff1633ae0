"""Host-side attention work lists: every query row and every key is covered
exactly once, and the array form for decode steps equals the general form."""

import numpy as np
import pytest

from paged_llm_b200.kernels import plan as planning


def general(q_lens, k_lens, G, nkv, window, **kw):
    args = dict(small_rows=16, large_rows=64, min_split_keys=128, num_sms=148, max_splits=32)
    args.update(kw)
    return planning.plan_attention(q_lens, k_lens, G, nkv, window, **args)


@pytest.mark.parametrize("q_lens,k_lens,G", [([1, 1, 1], [5, 700, 2048], 8), ([33, 1, 2, 200], [33, 64, 300, 500], 8),
                                              ([5, 17], [5, 17], 1), ([1], [1], 2)])
def test_items_cover_rows_and_keys(q_lens, k_lens, G):
    plan = general(q_lens, k_lens, G, 4, None)
    small, large = plan["small"].reshape(-1, 4), plan["large"].reshape(-1, 4)
    splits = plan["splits"].reshape(-1, 2)
    for s, (nq, lk) in enumerate(zip(q_lens, k_lens)):
        rows = nq * G
        if rows <= 16:
            mine = small[small[:, 0] == s]
            assert sorted(mine[:, 2].tolist()) == list(range(splits[s, 0])) and (mine[:, 3] == splits[s, 0]).all()
            assert splits[s, 0] <= max(1, -(-lk // 128)) and not (large[:, 0] == s).any()
        else:
            mine = large[large[:, 0] == s]
            assert sorted(mine[:, 1].tolist()) == list(range(-(-rows // 64))) and not (small[:, 0] == s).any()
    bases = [splits[s, 1] for s in range(len(q_lens)) if q_lens[s] * G <= 16]
    sizes = [q_lens[s] for s in range(len(q_lens)) if q_lens[s] * G <= 16]
    assert bases == list(np.cumsum([0] + sizes[:-1])) and plan["num_small_tokens"] == sum(sizes)


@pytest.mark.parametrize("fixed", [False, True])
@pytest.mark.parametrize("k_lens", [[5], [513, 640, 90, 2048, 129], list(range(100, 164))])
def test_decode_fast_path_equals_the_general_plan(k_lens, fixed):
    S = len(k_lens)
    pad = {1: 1, 5: 8, 64: 64}[S] if fixed else None
    fast = general([1] * S, k_lens, 8, 4, None, pad_requests=pad, fixed_capacity=fixed)
    slow = general([1] * S, k_lens, 8, 4, 10 ** 9, pad_requests=pad, fixed_capacity=fixed)   # a window switches it off
    for key in ("small", "large", "splits"):
        assert np.array_equal(fast[key], slow[key]), key
    assert fast["max_splits"] == slow["max_splits"] and fast["num_small_tokens"] == slow["num_small_tokens"]


def test_longest_tiles_first():
    plan = general([300, 40], [300, 900], 8, 4, None)
    large = plan["large"].reshape(-1, 4)
    assert large[0, 0] == 1                     # the request with the longest context leads


def test_long_context_decode_steps_are_split_further():
    """Few long requests: a block of a cluster of at most 8 would walk thousands of keys alone, so
    the plan turns to about three blocks per SM through the work list; short contexts and steps
    with prompt portions stay as they are."""
    from paged_llm_b200.kernels.plan import is_long_context, long_context_splits, plan_attention

    kw = dict(small_rows=16, large_rows=128, min_split_keys=128, num_sms=148, max_splits=32, cluster_max=8, long_keys=600)
    short = plan_attention([1] * 8, [700] * 8, 8, 4, None, **kw)
    assert not short["long_context"] and short["max_splits"] == 5
    long = plan_attention([1] * 8, [16000] * 8, 8, 4, None, **kw)
    assert long["long_context"] and long["max_splits"] == 13 == long_context_splits(8, 4, 148, 32)
    assert len(long["small"]) // 4 == 8 * 13
    one = plan_attention([1], [16000], 8, 4, None, **kw)
    assert one["long_context"] and one["max_splits"] == 32
    assert not plan_attention([1], [4000], 8, 4, None, **kw)["long_context"]           # 8 blocks x 500 keys
    assert not plan_attention([1, 40], [16000, 16000], 8, 4, None, **kw)["long_context"]   # a prompt portion in the step
    assert not plan_attention([1] * 8, [16000] * 8, 8, 4, None, **{**kw, "cluster_max": 0})["long_context"]
    # the class of a padded graph bucket is that of the bucket, whatever the live requests
    assert is_long_context(8, 4, 148, 32, 8, 600, 3001) and not is_long_context(8, 4, 148, 32, 8, 600, 3000)
    # 64 requests x 4 kv heads: one block each either way, so there is no second class (and no second graph)
    assert not is_long_context(64, 4, 148, 32, 8, 600, 100000)
