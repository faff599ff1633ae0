"""Each kernel alone against a plain float32 formulation, at sizes other than
the engine's tiny models: widths and vocabularies that are no power of two,
head sizes in steps of 16, any number of heads and groups, page sizes 8/16/32."""

import math
import types

import numpy as np
import pytest
import torch

from tests import plain_llama

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


@pytest.fixture(scope="module")
def ops():
    from paged_llm_b200.kernels.ops import CudaOps
    return CudaOps("cuda")


def tol(dtype, scale=1.0):
    return (2e-5 if dtype == torch.float32 else 1.6e-2) * scale


def randn(*shape, seed=0, dtype=torch.float32, std=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * std).to(dtype).cuda()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("V,H", [(509, 96), (1000, 2050), (31, 7)])
def test_embedding(ops, dtype, V, H):
    table = randn(V, H, dtype=dtype)
    ids = torch.randint(0, V, (77,), dtype=torch.int32, device="cuda")
    out = ops.embedding(table, ids)
    assert out.dtype == torch.float32 and torch.equal(out, table[ids.long()].float())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("wdtype", DTYPES)
@pytest.mark.parametrize("rows,H,eps", [(5, 96, 1e-6), (3, 2050, 1e-5), (130, 64, 1e-5), (2, 12289, 1e-2)])
def test_rms_norm_and_residual_sum(ops, dtype, wdtype, rows, H, eps):
    ops.set_compute_dtype(dtype)
    x = randn(rows, H, seed=1, std=3.0)
    w = (1 + 0.1 * randn(H, seed=2)).to(wdtype)
    y = ops.rms_norm(x, w, eps)
    want = plain_llama.rms_norm(x.cpu(), w.float().cpu(), eps)
    assert y.dtype == dtype
    torch.testing.assert_close(y.float().cpu(), want, atol=tol(dtype, 4), rtol=tol(dtype))
    branch = randn(rows, H, seed=3).to(dtype)
    x2 = x.clone()
    y2 = ops.add_rms_norm(x2, branch, w, eps)
    summed = x.cpu() + branch.float().cpu()
    torch.testing.assert_close(x2.cpu(), summed, atol=1e-6, rtol=1e-6)       # the sum is float32
    torch.testing.assert_close(y2.float().cpu(), plain_llama.rms_norm(summed, w.float().cpu(), eps),
                               atol=tol(dtype, 4), rtol=tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,I", [(7, 172), (33, 5632), (1, 5)])
def test_silu_mul(ops, dtype, rows, I):
    gu = randn(rows, 2 * I, seed=4, std=2.0).to(dtype)
    out = ops.silu_mul(gu)
    g, u = gu[:, :I].float(), gu[:, I:].float()
    torch.testing.assert_close(out.float(), g * torch.sigmoid(g) * u, atol=tol(dtype, 4), rtol=tol(dtype))


@pytest.mark.parametrize("M,N,K", [(1, 509, 96), (70, 172, 64), (5, 64, 172), (300, 130, 75), (640, 700, 520)])
def test_gemm_f32_is_true_float32_and_batch_independent(ops, M, N, K):
    a, b = randn(M, K, seed=5), randn(N, K, seed=6)
    out = ops.linear(a, b)
    want = (a.double() @ b.double().T).float()
    torch.testing.assert_close(out, want, atol=2e-5 * math.sqrt(K), rtol=2e-6)
    one = ops.linear(a[M // 2:M // 2 + 1].contiguous(), b)
    assert torch.equal(one[0], out[M // 2]), "a row's product must not depend on the rows beside it"


@pytest.mark.parametrize("M,N,K", [(1, 509, 96), (70, 172, 64), (5, 64, 172), (2048, 256, 512)])
def test_linear_bf16(ops, M, N, K):
    a, b = randn(M, K, seed=7, dtype=torch.bfloat16), randn(N, K, seed=8, dtype=torch.bfloat16)
    want = a.float() @ b.float().T
    torch.testing.assert_close(ops.linear(a, b).float(), want, atol=tol(torch.bfloat16, math.sqrt(K)), rtol=1e-2)
    full = ops.linear(a, b, out_float32=True)
    assert full.dtype == torch.float32
    torch.testing.assert_close(full, want, atol=1e-4 * math.sqrt(K), rtol=1e-4)


@pytest.mark.parametrize("dtype", DTYPES)
def test_gather_rows(ops, dtype):
    x = randn(50, 97, seed=9).to(dtype)
    idx = torch.tensor([3, 3, 49, 0], dtype=torch.int32, device="cuda")
    assert torch.equal(ops.gather_rows(x, idx), x[idx.long()])


def test_rope_table_matches_float32_angles(ops):
    inv = plain_llama.inv_frequencies(48, 500000.0, {"rope_type": "llama3", "factor": 8.0,
                                                      "original_max_position_embeddings": 64})
    table = ops.rope_table(inv, 4096).cpu()
    cos, sin = plain_llama.rotary_cos_sin(torch.arange(4096), inv)
    torch.testing.assert_close(table[..., 0], cos[:, :24], atol=2e-6, rtol=0)
    torch.testing.assert_close(table[..., 1], sin[:, :24], atol=2e-6, rtol=0)


@pytest.mark.parametrize("dtype", DTYPES)
def test_fill_normal_on_the_device(ops, dtype):
    """Random weights drawn on the device: N(mean, std) from a counter-based stream that depends
    on (seed, key) alone: the same again on a second call, a prefix of itself at another size,
    other values for another key or seed."""
    n = 1_000_003                                                   # odd: the last pair is half used
    a = ops.fill_normal(torch.empty(n, dtype=dtype, device="cuda"), 7, 11, 0.5, 0.02).float()
    assert abs(float(a.mean()) - 0.5) < 2e-4 and abs(float(a.std()) - 0.02) < 2e-4
    z = (a - 0.5) / 0.02
    assert abs(float((z ** 3).mean())) < 0.02 and abs(float((z ** 4).mean()) - 3.0) < 0.1      # skewness, kurtosis
    assert float(z.abs().max()) < 6.0
    again = ops.fill_normal(torch.empty(n, dtype=dtype, device="cuda"), 7, 11, 0.5, 0.02).float()
    assert torch.equal(a, again)
    shorter = ops.fill_normal(torch.empty(1000, dtype=dtype, device="cuda"), 7, 11, 0.5, 0.02).float()
    assert torch.equal(shorter, a[:1000])
    for seed, key in ((8, 11), (7, 12)):
        other = ops.fill_normal(torch.empty(1000, dtype=dtype, device="cuda"), seed, key, 0.5, 0.02).float()
        assert not torch.equal(other, a[:1000])
        assert abs(float(torch.corrcoef(torch.stack([other, a[:1000]]))[0, 1])) < 0.15


def test_model_from_a_random_stub(ops, tmp_path):
    """A folder without tensors (config.json + random_weights.json): the engine draws the weights on
    the device, the same for the same stub, and generates with them."""
    from paged_llm_b200 import LLMEngine, SamplingParams
    from paged_llm_b200.config import LlamaConfig
    from paged_llm_b200.weights import write_random_stub
    from tests.tiny import TINY_B
    d = write_random_stub(str(tmp_path), LlamaConfig.from_hf_dict(TINY_B), seed=3, std=0.05, norm_std=0.1)
    outs = []
    for _ in range(2):
        eng = LLMEngine(d, dtype="bfloat16", block_size=8, num_gpu_blocks=32, max_model_len=128)
        w = eng.model.blocks[0].mixer.w_qkv.float()
        assert w.dtype == torch.float32 and abs(float(w.std()) - 0.05) < 2e-3 and abs(float(w.mean())) < 2e-3
        assert eng.model.head.weight is eng.model.embedding.weight            # tied, as the configuration says
        nw = eng.model.final_norm.weight
        assert nw.dtype == torch.float32 and abs(float(nw.mean()) - 1.0) < 0.05 and 0.05 < float(nw.std()) < 0.15
        outs.append(eng.generate([[1, 2, 3, 4]], SamplingParams(temperature=0.0, max_tokens=6))[0].token_ids)
    assert outs[0] == outs[1] and len(outs[0]) == 6


# ---------------------------------------------------------------------------- paged pieces

def paged_case(q_lens, k_lens, nh, nkv, d, ps, dtype, seed=0, spare=3):
    """Random pool with pages assigned by a random permutation (as in the
    reference's tests/test_attention_reference.py:10-28), unused slots poisoned."""
    g = torch.Generator().manual_seed(seed)
    S = len(q_lens)
    nblocks = [-(-L // ps) for L in k_lens]
    total = sum(nblocks) + spare
    perm = torch.randperm(total, generator=g)
    stride = max(nblocks) + 2
    bt = torch.full((S, stride), 10 ** 6, dtype=torch.int32)          # padding must never be dereferenced
    kv = torch.full((total, 2, nkv, ps, d), float("nan"))
    keys, vals, o = [], [], 0
    for s, L in enumerate(k_lens):
        bt[s, :nblocks[s]] = perm[o:o + nblocks[s]]
        o += nblocks[s]
        k, v = torch.randn(L, nkv, d, generator=g), torch.randn(L, nkv, d, generator=g)
        keys.append(k.to(dtype).float()); vals.append(v.to(dtype).float())
        for n in range(L):
            kv[bt[s, n // ps], 0, :, n % ps] = keys[-1][n]
            kv[bt[s, n // ps], 1, :, n % ps] = vals[-1][n]
    T = sum(q_lens)
    q = torch.randn(T, nh, d, generator=g).to(dtype)
    return q, kv.to(dtype), bt, keys, vals


def make_ctx(ops, q_lens, k_lens, nh, nkv, window, d=64):
    from paged_llm_b200.engine.context import AttentionPlan, HostBatch
    S = len(q_lens)
    host = HostBatch(list(q_lens), [k - q for q, k in zip(q_lens, k_lens)], [-1] * S)
    plan = ops.plan_attention(q_lens, k_lens, nh // nkv, nkv, window, d)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a, np.int32)).cuda()
    small, large = plan["small"].reshape(-1, 4), plan["large"].reshape(-1, 4)
    ap = AttentionPlan(dev(small) if len(small) else None, dev(large) if len(large) else None, dev(plan["splits"]),
                       len(small), len(large), plan["max_splits"], plan["num_small_tokens"])
    T = sum(q_lens)
    pos = np.concatenate([np.arange(k - q, k) for q, k in zip(q_lens, k_lens)])
    tseq = np.concatenate([np.full(q, s) for s, q in enumerate(q_lens)])
    return types.SimpleNamespace(num_tokens=T, num_seqs=S, host=host, cu_seqlens_q=dev(host.cu),
                                 seq_lens_k=dev(k_lens), positions=dev(pos), token_seq=dev(tseq),
                                 attention_plans={(nh // nkv, nkv, window, d): ap})


ATTN_SHAPES = [(8, 8, 64), (32, 8, 128), (32, 4, 64), (6, 2, 48), (3, 3, 32), (4, 2, 16), (5, 1, 80), (2, 1, 256)]
ATTN_LENGTHS = [
    ([5], [5]),
    ([33, 8, 17], [33, 8, 17]),
    ([1, 1, 1, 1], [1000, 33, 2048, 5]),
    ([37, 1, 12], [500, 64, 77]),
    ([2, 130, 1], [2, 700, 129]),
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("ps", [8, 16, 32])
@pytest.mark.parametrize("nh,nkv,d", ATTN_SHAPES)
@pytest.mark.parametrize("case", range(len(ATTN_LENGTHS)))
def test_paged_attention(ops, dtype, ps, nh, nkv, d, case):
    q_lens, k_lens = ATTN_LENGTHS[case]
    if (ps, case) not in ((8, 0), (16, 1), (16, 2), (32, 3), (8, 4), (16, 3)) and (nh, nkv, d) not in ((32, 4, 64), (32, 8, 128)):
        pytest.skip("full cross product only for the head shapes of the tcgen05 kernel")
    ops.set_compute_dtype(dtype)
    q, kv, bt, keys, vals = paged_case(q_lens, k_lens, nh, nkv, d, ps, dtype, seed=case)
    ctx = make_ctx(ops, q_lens, k_lens, nh, nkv, None, d)
    qkv = torch.cat([q.reshape(-1, nh * d), torch.zeros(q.shape[0], 2 * nkv * d, dtype=dtype)], dim=1).cuda().contiguous()
    out = ops.paged_attention(qkv, nh, nkv, d, kv.cuda(), bt.cuda(), ctx, d ** -0.5, None).float().cpu()
    cu = ctx.host.cu
    for s, (nq, L) in enumerate(zip(q_lens, k_lens)):
        qs = torch.zeros(L, nh, d)
        qs[L - nq:] = q[cu[s]:cu[s + 1]].float()
        want = plain_llama.causal_attention(qs, keys[s], vals[s], d ** -0.5)[L - nq:].reshape(nq, nh * d)
        torch.testing.assert_close(out[cu[s]:cu[s + 1]], want, atol=tol(dtype), rtol=tol(dtype), msg=f"request {s}")


@pytest.mark.parametrize("ps", [4, 2])
def test_prefill_attention_with_pages_too_small_for_tma_boxes(ops, ps):
    """Pages of fewer than 8 tokens: the tcgen05 kernel that copies keys through the block table
    with cp.async takes over from the one that brings whole pages in with TMA."""
    dtype, nh, nkv, d = torch.bfloat16, 32, 4, 64
    ops.set_compute_dtype(dtype)
    q_lens, k_lens = [130, 1, 40], [300, 90, 40]
    q, kv, bt, keys, vals = paged_case(q_lens, k_lens, nh, nkv, d, ps, dtype, seed=ps)
    ctx = make_ctx(ops, q_lens, k_lens, nh, nkv, None, d)
    qkv = torch.cat([q.reshape(-1, nh * d), torch.zeros(q.shape[0], 2 * nkv * d, dtype=dtype)], dim=1).cuda().contiguous()
    out = ops.paged_attention(qkv, nh, nkv, d, kv.cuda(), bt.cuda(), ctx, d ** -0.5, None).float().cpu()
    cu = ctx.host.cu
    for s, (nq, L) in enumerate(zip(q_lens, k_lens)):
        qs = torch.zeros(L, nh, d)
        qs[L - nq:] = q[cu[s]:cu[s + 1]].float()
        want = plain_llama.causal_attention(qs, keys[s], vals[s], d ** -0.5)[L - nq:].reshape(nq, nh * d)
        torch.testing.assert_close(out[cu[s]:cu[s + 1]], want, atol=tol(dtype), rtol=tol(dtype), msg=f"request {s}")
    assert ops._attention_bf16(d)[0].pl_attention_tc_timeouts() == 0


@pytest.mark.parametrize("cluster", [True, False])
@pytest.mark.parametrize("window", [None, 50])
@pytest.mark.parametrize("nh,nkv,d", [(32, 4, 64), (4, 2, 16), (6, 6, 128)])
@pytest.mark.parametrize("q_lens,k_lens", [([1, 1, 1], [700, 64, 5]), ([2, 1, 2, 1, 1], [300, 2, 129, 1000, 33]), ([1], [4000])])
def test_decode_attention_as_clusters_and_from_the_work_list(ops, cluster, window, nh, nkv, d, q_lens, k_lens):
    """Steps in which every request brings a token or two: the splits of a request merged through
    distributed shared memory by a thread-block cluster, or through global memory by the block
    that finishes last."""
    if max(q_lens) * (nh // nkv) > 16:
        pytest.skip("more than 16 rows per request: not a decode step for this shape")
    dtype, ps = torch.bfloat16, 16
    ops.set_compute_dtype(dtype)
    q, kv, bt, keys, vals = paged_case(q_lens, k_lens, nh, nkv, d, ps, dtype, seed=len(q_lens))
    ctx = make_ctx(ops, q_lens, k_lens, nh, nkv, window, d)
    qkv = torch.cat([q.reshape(-1, nh * d), torch.zeros(q.shape[0], 2 * nkv * d, dtype=dtype)], dim=1).cuda().contiguous()
    before, ops.cluster_attention = ops.cluster_attention, cluster
    try:
        out = ops.paged_attention(qkv, nh, nkv, d, kv.cuda(), bt.cuda(), ctx, d ** -0.5, window).float().cpu()
    finally:
        ops.cluster_attention = before
    cu = ctx.host.cu
    for s, (nq, L) in enumerate(zip(q_lens, k_lens)):
        qs = torch.zeros(L, nh, d)
        qs[L - nq:] = q[cu[s]:cu[s + 1]].float()
        want = plain_llama.causal_attention(qs, keys[s], vals[s], d ** -0.5, window=window)[L - nq:].reshape(nq, nh * d)
        torch.testing.assert_close(out[cu[s]:cu[s + 1]], want, atol=tol(dtype), rtol=tol(dtype), msg=f"request {s}")


@pytest.mark.parametrize("nh,nkv,d,H", [(32, 4, 64, 256), (32, 8, 128, 512), (6, 2, 48, 96), (4, 4, 16, 64)])
@pytest.mark.parametrize("q_lens,k_lens,window", [([1] * 20, [5, 17, 600, 64, 1, 129, 1023, 48, 300, 2, 33, 16, 700, 90, 250, 31, 32, 128, 257, 400], None),
                                                  ([1] * 64, [520] * 64, None), ([2, 1, 2] * 7, [300, 2, 129] * 7, None),
                                                  # two new tokens whose keys fall on both sides of a cluster rank's edge
                                                  ([2] * 18, [65, 33, 97, 129, 2, 3, 64, 66, 34, 200, 161, 95, 96, 31, 32, 1000, 500, 193], None),
                                                  ([1] * 17, [90, 400, 3] * 5 + [1000, 7], 50)])
def test_decode_step_with_rotation_inside_the_attention_kernel(ops, nh, nkv, d, H, q_lens, k_lens, window):
    """A decode step of more than 16 tokens: the projection is a library product, and rotary
    positions and the cache write happen inside the attention kernel (`qkv_attention`).  Held to
    the plain formulation: float32 projection, rotate-half, attention over the rotated keys; and
    the cache must hold the step's rotated keys and values afterwards, and nothing else new."""
    from paged_llm_b200.parts.rope import RotaryEncoding
    if max(q_lens) * (nh // nkv) > 16:
        q_lens = [1] * len(q_lens)
    dtype, ps, theta = torch.bfloat16, 16, 10000.0
    ops.set_compute_dtype(dtype)
    rope = RotaryEncoding({}, head_dim=d, theta=theta)
    rope.prepare(1024, "cuda", ops)
    _, kv, bt, keys, vals = paged_case(q_lens, k_lens, nh, nkv, d, ps, dtype, seed=3)
    T = sum(q_lens)
    h = randn(T, H, seed=41, dtype=dtype)
    w = randn((nh + 2 * nkv) * d, H, seed=42, dtype=dtype, std=H ** -0.5)
    y = (h.float().cpu() @ w.float().cpu().T).to(dtype).float()           # the projection rounds to bfloat16
    pos = torch.cat([torch.arange(k - q, k) for q, k in zip(q_lens, k_lens)])
    cos, sin = plain_llama.rotary_cos_sin(pos, plain_llama.inv_frequencies(d, theta, None))
    q_rot = plain_llama.apply_rotary(y[:, :nh * d].view(T, nh, d), cos, sin).to(dtype).float()
    k_rot = plain_llama.apply_rotary(y[:, nh * d:(nh + nkv) * d].view(T, nkv, d), cos, sin).to(dtype).float()
    v_new = y[:, (nh + nkv) * d:].view(T, nkv, d)
    # the slots of the step's own tokens hold poison until the step writes them
    kv = kv.clone()
    t = 0
    for s, (nq, L) in enumerate(zip(q_lens, k_lens)):
        for n in range(L - nq, L):
            kv[bt[s, n // ps], :, :, n % ps] = float("nan")
            keys[s][n], vals[s][n] = k_rot[t], v_new[t]
            t += 1
    ctx = make_ctx(ops, q_lens, k_lens, nh, nkv, window, d)
    plan = ctx.attention_plans[(nh // nkv, nkv, window, d)]
    assert ops._runs_as_clusters(plan, ctx, nh, nkv, True), "this test is about the cluster form"
    kv_dev = kv.cuda()
    before = ops.launches
    out = ops.qkv_attention(h, w, nh, nkv, d, rope, ctx, kv_dev, bt.cuda(), d ** -0.5, window).float().cpu()
    assert ops.launches - before == 1, "one kernel of this package beside the library product"
    cu = ctx.host.cu
    for s, (nq, L) in enumerate(zip(q_lens, k_lens)):
        qs = torch.zeros(L, nh, d)
        qs[L - nq:] = q_rot[cu[s]:cu[s + 1]]
        want = plain_llama.causal_attention(qs, keys[s], vals[s], d ** -0.5, window=window)[L - nq:].reshape(nq, nh * d)
        torch.testing.assert_close(out[cu[s]:cu[s + 1]], want, atol=tol(dtype), rtol=tol(dtype), msg=f"request {s}")
    got_kv = kv_dev.float().cpu()
    for s, (nq, L) in enumerate(zip(q_lens, k_lens)):
        for n in range(L - nq, L):
            torch.testing.assert_close(got_kv[bt[s, n // ps], 0, :, n % ps], keys[s][n], atol=tol(dtype), rtol=tol(dtype))
            torch.testing.assert_close(got_kv[bt[s, n // ps], 1, :, n % ps], vals[s][n], atol=tol(dtype), rtol=tol(dtype))
    same = torch.isnan(kv.float()) | (got_kv == kv.float())
    assert same.all(), "only the slots of the step's own tokens may change"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [1, 7, 16, 100])
@pytest.mark.parametrize("nh,nkv,d", [(4, 2, 32), (8, 2, 64), (6, 3, 128)])
def test_paged_attention_window(ops, dtype, window, nh, nkv, d):
    ops.set_compute_dtype(dtype)
    ps = 16
    q_lens, k_lens = [40, 1, 3, 90], [40, 300, 19, 200]
    q, kv, bt, keys, vals = paged_case(q_lens, k_lens, nh, nkv, d, ps, dtype, seed=window)
    # pages wholly behind the window are given back by the cache manager: poison their table entries
    for s, (nq, L) in enumerate(zip(q_lens, k_lens)):
        first_needed = (L - nq) - window + 1
        for j in range(bt.shape[1]):
            if (j + 1) * ps <= first_needed:
                bt[s, j] = -1
    ctx = make_ctx(ops, q_lens, k_lens, nh, nkv, window, d)
    qkv = torch.cat([q.reshape(-1, nh * d), torch.zeros(q.shape[0], 2 * nkv * d, dtype=dtype)], dim=1).cuda().contiguous()
    out = ops.paged_attention(qkv, nh, nkv, d, kv.cuda(), bt.cuda(), ctx, 0.3, window).float().cpu()
    cu = ctx.host.cu
    for s, (nq, L) in enumerate(zip(q_lens, k_lens)):
        qs = torch.zeros(L, nh, d)
        qs[L - nq:] = q[cu[s]:cu[s + 1]].float()
        want = plain_llama.causal_attention(qs, keys[s], vals[s], 0.3, window=window)[L - nq:].reshape(nq, nh * d)
        torch.testing.assert_close(out[cu[s]:cu[s + 1]], want, atol=tol(dtype), rtol=tol(dtype), msg=f"request {s}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,d", [(32, 4, 64), (6, 3, 128), (4, 2, 16)])
@pytest.mark.parametrize("softcap,sloped", [(None, True), (1.5, False), (0.7, True)])
def test_paged_attention_with_score_modifiers(ops, dtype, nh, nkv, d, softcap, sloped):
    """The two score modifiers of the attention part (a cap c * tanh(s / c) and a per-head bias
    slope * (key position - query position)) against the plain formulation, for prompt portions
    (head sizes 64 and 128 leave the tcgen05 kernel for them), decode clusters and work-list splits."""
    ops.set_compute_dtype(dtype)
    ps = 16
    q_lens, k_lens = [150, 1, 2, 1, 40], [400, 700, 19, 3000, 40]
    if max(q for q in q_lens if q <= 2) * (nh // nkv) > 16:
        q_lens[2] = 1
    q, kv, bt, keys, vals = paged_case(q_lens, k_lens, nh, nkv, d, ps, dtype, seed=11)
    slopes = [2.0 ** -(1 + 8.0 * h / nh) for h in range(nh)] if sloped else None
    dev_slopes = torch.tensor(slopes, dtype=torch.float32, device="cuda") if sloped else None
    cu = [0]
    for n in q_lens:
        cu.append(cu[-1] + n)
    qkv = torch.cat([q.reshape(-1, nh * d), torch.zeros(q.shape[0], 2 * nkv * d, dtype=dtype)], dim=1).cuda().contiguous()
    # the whole mixed batch, then the decoding requests alone (so that they run as clusters in bfloat16)
    for pick in (list(range(len(q_lens))), [1, 3]):
        ql, kl = [q_lens[s] for s in pick], [k_lens[s] for s in pick]
        ctx = make_ctx(ops, ql, kl, nh, nkv, None, d)
        rows = torch.cat([torch.arange(cu[s], cu[s + 1]) for s in pick])
        out = ops.paged_attention(qkv[rows.cuda()].contiguous(), nh, nkv, d, kv.cuda(), bt[pick].contiguous().cuda(), ctx,
                                  d ** -0.5, None, softcap=softcap, slopes=dev_slopes).float().cpu()
        o = 0
        for s in pick:
            nq, L = q_lens[s], k_lens[s]
            qs = torch.zeros(L, nh, d)
            qs[L - nq:] = q[cu[s]:cu[s + 1]].float()
            want = plain_llama.causal_attention(qs, keys[s], vals[s], d ** -0.5, softcap=softcap,
                                                slopes=slopes)[L - nq:].reshape(nq, nh * d)
            torch.testing.assert_close(out[o:o + nq], want, atol=tol(dtype), rtol=tol(dtype), msg=f"request {s}")
            o += nq


@pytest.mark.parametrize("dtype", DTYPES)
def test_one_far_key_among_hundreds(ops, dtype):
    """Random scores would hide a key that is skipped: make one query-key pair
    stand out so that the output is that key's value, for keys on page edges, in
    the first and last split, and right at the causal edge."""
    ops.set_compute_dtype(dtype)
    nh, nkv, d, ps, L = 8, 2, 64, 16, 1500
    for target in (0, 15, 16, 255, 256, 767, 1024, L - 2, L - 1):
        q, kv, bt, keys, vals = paged_case([1], [L], nh, nkv, d, ps, dtype, seed=target)
        direction = torch.randn(d, generator=torch.Generator().manual_seed(1))
        direction = direction / direction.norm()
        q[:] = (direction * 40).to(dtype)
        for h in range(nkv):
            keys[0][target, h] = (direction * 40).to(dtype).float()
            kv[bt[0, target // ps], 0, h, target % ps] = keys[0][target, h].to(dtype)
        ctx = make_ctx(ops, [1], [L], nh, nkv, None, d)
        qkv = torch.cat([q.reshape(-1, nh * d), torch.zeros(1, 2 * nkv * d, dtype=dtype)], dim=1).cuda().contiguous()
        out = ops.paged_attention(qkv, nh, nkv, d, kv.cuda(), bt.cuda(), ctx, d ** -0.5, None).float().cpu()
        want = vals[0][target].repeat_interleave(nh // nkv, dim=0).reshape(1, nh * d)
        torch.testing.assert_close(out, want, atol=2e-2, rtol=2e-2, msg=f"key {target}")


@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("nq,L,targets", [
    (200, 1500, (0, 15, 16, 63, 64, 1023, 1024, 1299, 1300, 1498, 1499)),      # a prompt portion: 128-row tiles, TMA page boxes
    (1, 6000, (0, 127, 128, 191, 192, 2999, 5998, 5999)),                      # one long request: the long-context class
])
def test_one_far_key_in_a_portion_and_in_a_long_context(ops, nq, L, targets, d):
    """The same for the other two attention paths of bfloat16 at head sizes 64 and 128: the last
    row of a prompt portion (tcgen05 kernel, keys brought in page by page with TMA) and a single
    decoding request whose context is long enough for the work-list splits."""
    dtype = torch.bfloat16
    ops.set_compute_dtype(dtype)
    if nq == 1 and not ops.cluster_attention:
        pytest.skip("without clusters there is one decode class only")
    nh, nkv, ps = 8, 2, 16
    for target in targets:
        q, kv, bt, keys, vals = paged_case([nq], [L], nh, nkv, d, ps, dtype, seed=target)
        direction = torch.randn(d, generator=torch.Generator().manual_seed(2))
        direction = direction / direction.norm()
        q[-1] = (direction * 40).to(dtype)                 # the last row looks for the target key
        for h in range(nkv):
            keys[0][target, h] = (direction * 40).to(dtype).float()
            kv[bt[0, target // ps], 0, h, target % ps] = keys[0][target, h].to(dtype)
        ctx = make_ctx(ops, [nq], [L], nh, nkv, None, d)
        if nq == 1:
            assert ops.long_context_class(1, nkv, L), "this case is meant for the long-context class"
        qkv = torch.cat([q.reshape(-1, nh * d), torch.zeros(nq, 2 * nkv * d, dtype=dtype)], dim=1).cuda().contiguous()
        out = ops.paged_attention(qkv, nh, nkv, d, kv.cuda(), bt.cuda(), ctx, d ** -0.5, None).float().cpu()
        want = vals[0][target].repeat_interleave(nh // nkv, dim=0).reshape(1, nh * d)
        torch.testing.assert_close(out[-1:], want, atol=2e-2, rtol=2e-2, msg=f"key {target}")
    if nq > 1:
        assert ops._attention_bf16(d)[0].pl_attention_tc_timeouts() == 0


def padded_ctx(ops, k_lens, pad_to, nh, nkv, d):
    """A decode step of len(k_lens) requests padded to `pad_to` request slots, as the runner packs it for a
    captured graph: empty slots have no token (cu stays), no keys, and -1 as their token's request."""
    from paged_llm_b200.engine.context import AttentionPlan, HostBatch
    S = len(k_lens)
    q_lens = [1] * S
    host = HostBatch(q_lens, [k - 1 for k in k_lens], [-1] * S)
    plan = ops.plan_attention(q_lens, k_lens, nh // nkv, nkv, None, d, pad_requests=pad_to, fixed_capacity=True)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a, np.int32)).cuda()
    small = plan["small"].reshape(-1, 4)
    ap = AttentionPlan(dev(small), None, dev(plan["splits"]), len(small), 0, plan["max_splits"],
                       plan["num_small_tokens"], plan.get("long_context", False))
    cu = np.full(pad_to + 1, S, np.int32)
    cu[:S + 1] = np.arange(S + 1)
    klen = np.zeros(pad_to, np.int32)
    klen[:S] = k_lens
    pos = np.zeros(pad_to, np.int32)
    pos[:S] = [k - 1 for k in k_lens]
    tseq = np.full(pad_to, -1, np.int32)
    tseq[:S] = np.arange(S)
    return types.SimpleNamespace(num_tokens=pad_to, num_seqs=pad_to, host=host, cu_seqlens_q=dev(cu),
                                 seq_lens_k=dev(klen), positions=dev(pos), token_seq=dev(tseq),
                                 attention_plans={(nh // nkv, nkv, None, d): ap})


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("k_lens,pad_to", [([300, 5, 77], 8), ([40] * 5, 8), ([6000, 5200], 4), ([33], 2)])
def test_rows_that_pad_a_decode_step_come_back_zero(ops, dtype, k_lens, pad_to):
    """A step padded to the size of its graph: the rows of the requests are what the unpadded step gives, the
    rows behind them are zero although the buffer held NaN before (no fill kernel runs: the attention
    kernel's first block zeroes them), for the cluster form, the work list (long contexts) and float32."""
    nh, nkv, d, ps = 32, 4, 64, 16
    ops.set_compute_dtype(dtype)
    S = len(k_lens)
    q, kv, bt, _, _ = paged_case([1] * S, k_lens, nh, nkv, d, ps, dtype, seed=len(k_lens))
    kv, bt = kv.cuda(), bt.cuda()
    bt_pad = torch.zeros((pad_to, bt.shape[1]), dtype=torch.int32, device="cuda")
    bt_pad[:S] = bt
    qkv = torch.full((pad_to, (nh + 2 * nkv) * d), float("nan"), dtype=dtype, device="cuda")
    qkv[:S, :nh * d] = q.reshape(S, nh * d).cuda()
    qkv[:S, nh * d:] = 0
    want = ops.paged_attention(qkv[:S].contiguous(), nh, nkv, d, kv, bt, make_ctx(ops, [1] * S, k_lens, nh, nkv, None, d),
                               d ** -0.5, None)
    ctx = padded_ctx(ops, k_lens, pad_to, nh, nkv, d)
    for _ in range(3):
        poison = torch.full((pad_to, nh * d), float("nan"), dtype=dtype, device="cuda")
        del poison                                        # the allocator hands this block to the kernel's output
        out = ops.paged_attention(qkv, nh, nkv, d, kv, bt_pad, ctx, d ** -0.5, None)
        assert torch.equal(out[S:], torch.zeros_like(out[S:])), "rows that pad the step are not zero"
        torch.testing.assert_close(out[:S].float(), want.float(), atol=tol(dtype, 4), rtol=tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("pairing", ["half", "interleaved"])
@pytest.mark.parametrize("nh,nkv,d,rd", [(4, 2, 16, 16), (3, 3, 32, 32), (6, 2, 48, 24), (32, 4, 64, 64)])
def test_rope_and_kv_write(ops, dtype, pairing, nh, nkv, d, rd):
    from paged_llm_b200.parts.rope import RotaryEncoding
    ops.set_compute_dtype(dtype)
    rope = RotaryEncoding({}, head_dim=d, theta=10000.0, rotary_dim=rd, pairing=pairing)
    rope.prepare(512, "cuda", ops)
    ps, q_lens, k_lens = 8, [5, 1, 20], [5, 300, 31]
    ctx = make_ctx(ops, q_lens, k_lens, nh, nkv, None, d)
    T = sum(q_lens)
    qkv = randn(T, (nh + 2 * nkv) * d, seed=11).to(dtype)
    before = qkv.clone()
    pages = 64
    bt = torch.stack([torch.randperm(pages, generator=torch.Generator().manual_seed(s))[:40] for s in range(3)]).int().cuda()
    kv = torch.full((pages, 2, nkv, ps, d), 7.0, dtype=dtype, device="cuda")
    ops.rope_kv_write(qkv, nh, nkv, d, rope, ctx, kv, bt, write=True)
    pos = ctx.positions.cpu().long()
    inv = rope.inv_freq()
    ang = torch.outer(pos.float(), inv)
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]

    def rotate(x):
        x = x.float().cpu().clone()
        r = x[..., :rd]
        if pairing == "half":
            a, b = r[..., :rd // 2], r[..., rd // 2:]
            x[..., :rd] = torch.cat([a * cos - b * sin, b * cos + a * sin], -1)
        else:
            a, b = r[..., 0::2], r[..., 1::2]
            x[..., :rd] = torch.stack([a * cos - b * sin, b * cos + a * sin], -1).flatten(-2)
        return x

    want_q = rotate(before[:, :nh * d].view(T, nh, d))
    want_k = rotate(before[:, nh * d:(nh + nkv) * d].view(T, nkv, d))
    want_v = before[:, (nh + nkv) * d:].view(T, nkv, d).float().cpu()
    torch.testing.assert_close(qkv[:, :nh * d].view(T, nh, d).float().cpu(), want_q, atol=tol(dtype, 4), rtol=tol(dtype))
    seq = ctx.token_seq.cpu()
    written = torch.zeros(pages, ps, dtype=torch.bool)
    for t in range(T):
        page, off = int(bt[seq[t], pos[t] // ps]), int(pos[t] % ps)
        written[page, off] = True
        torch.testing.assert_close(kv[page, 0, :, off].float().cpu(), want_k[t], atol=tol(dtype, 4), rtol=tol(dtype))
        assert torch.equal(kv[page, 1, :, off].float().cpu(), want_v[t])
    untouched = kv.float().cpu().permute(0, 3, 1, 2, 4)[~written]
    assert (untouched == 7.0).all(), "slots of other tokens were written"
    again = before.clone()
    kv2 = torch.full_like(kv, 7.0)
    ops.rope_kv_write(again, nh, nkv, d, rope, ctx, kv2, bt, write=False)     # a run that reads another run's cache
    assert (kv2 == 7.0).all() and torch.equal(again[:, :nh * d], qkv[:, :nh * d])


@pytest.mark.parametrize("dtype", DTYPES)
def test_copy_pages(ops, dtype):
    pool = randn(3, 10, 2, 2, 8, 16, seed=12).to(dtype)
    want = pool.clone()
    want[:, 7] = want[:, 2]
    want[:, 0] = want[:, 9]
    ops.copy_pages(pool, [(2, 7), (9, 0)])
    assert torch.equal(pool, want)


# ---------------------------------------------------------------------------- sampling

@pytest.mark.parametrize("V", [509, 32000, 7])
def test_argmax(ops, V):
    logits = randn(9, V, seed=13)
    logits[3, V // 2] = logits[3, 0] = 50.0                  # a tie goes to the first index
    assert ops.argmax(logits).tolist() == logits.argmax(-1).tolist()
    assert int(ops.argmax(logits)[3]) == 0


def test_sampling_matches_the_plain_draw(ops):
    from tests.plain_sampling import sample_rows
    V, rows = 509, 64
    logits = randn(rows, V, seed=14, std=2.0)
    temps = np.array([0.7, 1.0, 0.0, 1.3] * 16, np.float32)
    top_k = np.array([0, 5, 0, 50] * 16, np.int32)
    top_p = np.array([1.0, 1.0, 1.0, 0.8] * 16, np.float32)
    seeds = np.arange(rows, dtype=np.uint64) * 977 + 3
    counters = np.arange(rows, dtype=np.uint64) + 10
    got = ops.sample(logits, temps, top_k, top_p, seeds, counters).tolist()
    want = sample_rows(logits.cpu().numpy(), temps, top_k, top_p, seeds, counters)
    assert sum(g == w for g, w in zip(got, want)) >= rows - 1      # a near-tie may round differently
    again = ops.sample(logits, temps, top_k, top_p, seeds, counters).tolist()
    assert again == got


@pytest.mark.parametrize("V", [32000, 128256, 1031])
def test_sampling_filters_of_a_large_vocabulary(ops, V):
    """top-k and top-p over vocabularies of real size (the thresholds come from a radix search over the
    row): every draw of many falls into the set the plain filter keeps, the most likely kept tokens are
    all drawn, and the draws equal the plain draws but for near-ties."""
    from tests.plain_sampling import sample_rows
    n = 256
    row = randn(1, V, seed=16, std=2.5)
    row[0, 7] = row[0, 11]                                   # a tie inside the kept set
    logits = row.expand(n, V).contiguous()
    for temp, k, p in ((0.8, 50, 1.0), (1.0, 0, 0.9), (0.7, 40, 0.95), (1.5, 1000, 0.5), (1.0, 1, 1.0), (1.0, 0, 1e-6)):
        kept = torch.isfinite(plain_llama.filter_logits(row[0].float().cpu(), temp, k if k else -1, p)).numpy()
        temps, ks, ps = np.full(n, temp, np.float32), np.full(n, k, np.int32), np.full(n, p, np.float32)
        seeds, counters = np.full(n, 9, np.uint64), np.arange(n, dtype=np.uint64)
        got = ops.sample(logits, temps, ks, ps, seeds, counters).cpu().numpy()
        assert kept[got].all(), f"T={temp} k={k} p={p}: a filtered token was drawn"
        want = sample_rows(logits.cpu().numpy()[:32], temps, ks, ps, seeds, counters)
        assert sum(int(g) == w for g, w in zip(got[:32], want)) >= 31, f"T={temp} k={k} p={p}"
        if kept.sum() == 1:
            assert (got == int(np.flatnonzero(kept)[0])).all()
    # mixed rows: each row its own filter
    temps = np.array([0.7, 1.0, 0.0, 1.3] * 64, np.float32)
    ks = np.array([0, 5, 0, 50] * 64, np.int32)
    ps = np.array([1.0, 0.3, 1.0, 0.8] * 64, np.float32)
    seeds, counters = np.arange(n, dtype=np.uint64) * 31 + 1, np.arange(n, dtype=np.uint64) + 5
    got = ops.sample(logits, temps, ks, ps, seeds, counters).tolist()
    want = sample_rows(logits.cpu().numpy()[:64], temps, ks, ps, seeds, counters)
    assert sum(g == w for g, w in zip(got[:64], want)) >= 63
    assert ops.sample(logits, temps, ks, ps, seeds, counters).tolist() == got


def test_sampling_distribution(ops):
    """Many draws with different counters follow the filtered softmax."""
    V, n = 40, 20000
    row = randn(1, V, seed=15, std=1.5)
    logits = row.expand(n, V).contiguous()
    for temp, k, p in ((0.7, 0, 1.0), (1.0, 5, 1.0), (1.2, 0, 0.7)):
        got = ops.sample(logits, np.full(n, temp, np.float32), np.full(n, k, np.int32), np.full(n, p, np.float32),
                         np.full(n, 42, np.uint64), np.arange(n, dtype=np.uint64)).cpu().numpy()
        freq = np.bincount(got, minlength=V) / n
        want = plain_llama.sampling_distribution(row[0].cpu(), temp, k if k else -1, p).numpy()
        assert (freq[want == 0] == 0).all(), "a filtered token was drawn"
        assert np.abs(freq - want).max() < 0.015


# ---------------------------------------------------------------------------- few-token products

@pytest.mark.parametrize("M", [1, 3, 8, 9, 16])
@pytest.mark.parametrize("N,K", [(2560, 2048), (509, 96), (100, 64), (2048, 5632), (37, 160), (130, 8192), (64, 14336)])
def test_skinny_linear(ops, M, N, K):
    a, b = randn(M, K, seed=20, dtype=torch.bfloat16), randn(N, K, seed=21, dtype=torch.bfloat16, std=0.1)
    want = a.float() @ b.float().T
    got = ops.linear(a, b)
    assert got.dtype == torch.bfloat16
    torch.testing.assert_close(got.float(), want, atol=2e-2 * math.sqrt(K) * 0.1, rtol=1e-2)
    full = ops.linear(a, b, out_float32=True)
    torch.testing.assert_close(full, want, atol=1e-4 * math.sqrt(K), rtol=1e-4)
    one = ops.linear(a[M // 2:M // 2 + 1].contiguous(), b, out_float32=True)
    assert torch.equal(one[0], full[M // 2]), "a token's product must not depend on the tokens beside it"
    assert ops.core.pl_gemm_skinny_timeouts() == 0, "a bounded wait inside the kernel gave up"


@pytest.mark.parametrize("M", [1, 8, 13])
@pytest.mark.parametrize("I,K", [(5632, 2048), (172, 64), (100, 96), (7, 32)])
def test_skinny_gated_silu(ops, M, I, K):
    h, w = randn(M, K, seed=22, dtype=torch.bfloat16), randn(2 * I, K, seed=23, dtype=torch.bfloat16, std=0.1)
    got = ops.gated_silu_linear(h, w)
    ops.use_skinny = False
    try:
        want = ops.gated_silu_linear(h, w)
    finally:
        ops.use_skinny = True
    g, u = (h.float() @ w[:I].float().T), (h.float() @ w[I:].float().T)
    torch.testing.assert_close(got.float(), g * torch.sigmoid(g) * u, atol=3e-2, rtol=3e-2)
    torch.testing.assert_close(got.float(), want.float(), atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("M", [129, 256, 300, 2048, 2500])
@pytest.mark.parametrize("N,K", [(2048, 2048), (2560, 2048), (520, 128), (2048, 5632), (1000, 64), (11264, 2048)])
def test_gemm_tc_product(ops, M, N, K):
    """More than 128 tokens: the tcgen05 product (two blocks on one 256 x 256 tile) and its epilogues against
    float32 arithmetic on the same bfloat16 inputs."""
    if M == 2048 and K != 2048:
        pytest.skip("2,048 tokens only at the benchmark's K")
    if M == 2500 and (N, K) not in ((520, 128), (2560, 2048)):
        pytest.skip("more than eight pairs of token tiles (two bands of the tile order) at two shapes only")
    ops.set_compute_dtype(torch.bfloat16)
    h = randn(M, K, seed=50 + M % 97, dtype=torch.bfloat16)
    w = randn(N, K, seed=51 + N % 89, dtype=torch.bfloat16, std=K ** -0.5)
    want = h.float() @ w.float().T
    was, ops.gemm_tc_for = ops.gemm_tc_for, {"silu", "add", "plain"}
    was_min, ops.gemm_tc_min_tokens = ops.gemm_tc_min_tokens, 129
    try:
        before = ops.launches
        got = ops.linear(h, w)
        assert ops.launches == before + 1, "the product did not run on this package's kernel"
        torch.testing.assert_close(got.float(), want, atol=2e-2, rtol=2e-2)
        got32 = ops.linear(h, w, out_float32=True)
        torch.testing.assert_close(got32, want, atol=2e-3, rtol=2e-3)
        x = randn(M, N, seed=52, dtype=torch.float32)
        norm_w = randn(N, seed=53, dtype=torch.float32, std=0.1) + 1.0
        x_new = x.clone()
        normed = ops.linear_add_rms_norm(h, w, x_new, norm_w, 1e-5)
        torch.testing.assert_close(x_new, x + want.bfloat16().float(), atol=2e-2, rtol=2e-2)
        ref = x_new * torch.rsqrt(x_new.pow(2).mean(-1, keepdim=True) + 1e-5) * norm_w
        torch.testing.assert_close(normed.float(), ref, atol=3e-2, rtol=3e-2)
        I = N // 2
        if I % 8 == 0:
            act = ops.gated_silu_linear(h, w)
            g, u = want[:, :I].bfloat16().float(), want[:, I:].bfloat16().float()
            torch.testing.assert_close(act.float(), g * torch.sigmoid(g) * u, atol=3e-2, rtol=3e-2)
        assert ops.core.pl_gemm_tc_timeouts() == 0
    finally:
        ops.gemm_tc_for, ops.gemm_tc_min_tokens = was, was_min


@pytest.mark.parametrize("nh,nkv,d", [(32, 4, 64), (4, 2, 16), (3, 3, 32), (6, 2, 48)])
@pytest.mark.parametrize("q_lens,k_lens", [([1, 1, 1], [5, 300, 31]), ([5, 1, 7], [5, 300, 31]), ([1], [1])])
def test_skinny_qkv_rope_write_equals_the_separate_kernels(ops, nh, nkv, d, q_lens, k_lens):
    from paged_llm_b200.parts.rope import RotaryEncoding
    ops.set_compute_dtype(torch.bfloat16)
    rope = RotaryEncoding({}, head_dim=d, theta=10000.0)
    rope.prepare(512, "cuda", ops)
    H, ps, pages = 96, 8, 64
    ctx = make_ctx(ops, q_lens, k_lens, nh, nkv, None, d)
    T = sum(q_lens)
    h = randn(T, H, seed=24, dtype=torch.bfloat16)
    w = randn((nh + 2 * nkv) * d, H, seed=25, dtype=torch.bfloat16, std=0.2)
    bt = torch.stack([torch.randperm(pages, generator=torch.Generator().manual_seed(s))[:40] for s in range(len(q_lens))]).int().cuda()
    kv_a = torch.full((pages, 2, nkv, ps, d), 7.0, dtype=torch.bfloat16, device="cuda")
    kv_b = kv_a.clone()
    fused = ops.qkv_rope_write(h, w, nh, nkv, d, rope, ctx, kv_a, bt, write=True)
    ops.use_skinny = False
    try:
        plain = ops.qkv_rope_write(h, w, nh, nkv, d, rope, ctx, kv_b, bt, write=True)
    finally:
        ops.use_skinny = True
    torch.testing.assert_close(fused[:, :nh * d].float(), plain[:, :nh * d].float(), atol=3e-2, rtol=3e-2)
    torch.testing.assert_close(kv_a.float(), kv_b.float(), atol=3e-2, rtol=3e-2)
    assert ((kv_a == 7.0) == (kv_b == 7.0)).all(), "the fused kernel must write exactly the same slots"


@pytest.mark.parametrize("nh,nkv,d,H", [(32, 4, 64, 2048), (32, 8, 128, 4096)])
@pytest.mark.parametrize("q_lens,k_lens", [([1], [300]), ([1] * 8, [5, 17, 600, 64, 1, 129, 1023, 48]), ([3, 2, 6], [40, 2, 300])])
def test_skinny_qkv_rope_write_against_the_plain_rotation(ops, nh, nkv, d, H, q_lens, k_lens):
    """The product with the rotary epilogue and the page write at the widths of the benchmarks,
    held to the plain formulation (tests/plain_llama.py: projection in float32, rotate-half with
    float32 angles), not to another path of the engine: the rotated queries it returns and the
    keys and values it leaves in the cache, slot by slot."""
    from paged_llm_b200.parts.rope import RotaryEncoding
    ops.set_compute_dtype(torch.bfloat16)
    theta, ps = 500000.0, 16
    rope = RotaryEncoding({}, head_dim=d, theta=theta)
    rope.prepare(1024, "cuda", ops)
    ctx = make_ctx(ops, q_lens, k_lens, nh, nkv, None, d)
    T = sum(q_lens)
    h = randn(T, H, seed=31, dtype=torch.bfloat16)
    w = randn((nh + 2 * nkv) * d, H, seed=32, dtype=torch.bfloat16, std=0.03)
    pages = sum(-(-k // ps) for k in k_lens) + 3
    g = torch.Generator().manual_seed(5)
    perm = torch.randperm(pages, generator=g)
    bt = torch.full((len(q_lens), max(-(-k // ps) for k in k_lens) + 1), -1, dtype=torch.int32)
    o = 0
    for s, k in enumerate(k_lens):
        n = -(-k // ps)
        bt[s, :n] = perm[o:o + n]
        o += n
    kv = torch.full((pages, 2, nkv, ps, d), 7.0, dtype=torch.bfloat16, device="cuda")
    got = ops.qkv_rope_write(h, w, nh, nkv, d, rope, ctx, kv, bt.cuda(), write=True)
    assert ops.core.pl_gemm_skinny_timeouts() == 0
    # plain: q, k, v = h W^T in float32; q and k rotated at each token's position
    y = h.float().cpu() @ w.float().cpu().T
    pos = torch.cat([torch.arange(k - q, k) for q, k in zip(q_lens, k_lens)])
    cos, sin = plain_llama.rotary_cos_sin(pos, plain_llama.inv_frequencies(d, theta, None))
    q_want = plain_llama.apply_rotary(y[:, :nh * d].view(T, nh, d), cos, sin)
    k_want = plain_llama.apply_rotary(y[:, nh * d:(nh + nkv) * d].view(T, nkv, d), cos, sin)
    v_want = y[:, (nh + nkv) * d:].view(T, nkv, d)
    scale = float(y.abs().max())
    torch.testing.assert_close(got[:, :nh * d].float().cpu().view(T, nh, d), q_want, atol=1e-2 * scale, rtol=1.6e-2)
    kv_cpu = kv.float().cpu()
    written = torch.zeros(pages, ps, dtype=torch.bool)
    t = 0
    for s, (nq, lk) in enumerate(zip(q_lens, k_lens)):
        for p_ in range(lk - nq, lk):
            page, slot = int(bt[s, p_ // ps]), p_ % ps
            torch.testing.assert_close(kv_cpu[page, 0, :, slot], k_want[t], atol=1e-2 * scale, rtol=1.6e-2)
            torch.testing.assert_close(kv_cpu[page, 1, :, slot], v_want[t], atol=1e-2 * scale, rtol=1.6e-2)
            written[page, slot] = True
            t += 1
    untouched = kv_cpu[:, 0, 0, :, 0] == 7.0
    assert (untouched == ~written).all(), "exactly the slots of the step's tokens are written"


@pytest.mark.parametrize("M", [1, 8, 11])
@pytest.mark.parametrize("N,K,wdtype", [(2048, 2048, torch.bfloat16), (2048, 5632, torch.bfloat16), (96, 256, torch.float32),
                                        (128, 64, torch.float32)])
def test_skinny_add_then_normalising_products(ops, M, N, K, wdtype):
    """Projection + residual sum in one kernel, the norm carried out by the products that
    follow while they load; three rounds in a row on the same workspace."""
    from paged_llm_b200.kernels.ops import LazyNorm
    ops.set_compute_dtype(torch.bfloat16)
    for rep in range(3):
        h, w = randn(M, K, seed=30 + rep, dtype=torch.bfloat16), randn(N, K, seed=31, dtype=torch.bfloat16, std=0.05)
        x = randn(M, N, seed=32 + rep, std=2.0)
        nw = (1 + 0.1 * randn(N, seed=33)).to(wdtype)
        x_fused = x.clone()
        lazy = ops.linear_add_rms_norm(h, w, x_fused, nw, 1e-5)
        assert isinstance(lazy, LazyNorm)
        branch = (h.float() @ w.float().T).to(torch.bfloat16).float()
        torch.testing.assert_close(x_fused, x + branch, atol=2e-2, rtol=1e-2)
        normed = plain_llama.rms_norm(x_fused.cpu(), nw.float().cpu(), 1e-5)
        torch.testing.assert_close(ops.materialize(lazy).float().cpu(), normed, atol=4e-2, rtol=1.6e-2)
        w2 = randn(176, N, seed=34, dtype=torch.bfloat16, std=0.05)
        want = normed.to(torch.bfloat16).float() @ w2.float().cpu().T
        torch.testing.assert_close(ops.linear(lazy, w2, out_float32=True).cpu(), want, atol=3e-2, rtol=2e-2)
        g, u = want[:, :88], want[:, 88:]
        torch.testing.assert_close(ops.gated_silu_linear(lazy, w2).float().cpu(), g * torch.sigmoid(g) * u, atol=4e-2, rtol=4e-2)
    assert ops.core.pl_gemm_skinny_timeouts() == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d", [32, 64, 128])
def test_window_edge_is_exact(ops, dtype, d):
    """Random scores would hide an off-by-one at the window's edge: put a key with an
    overwhelming score just outside the window (it must change nothing) and one just inside
    (it must take all the weight), for a decoded token and for rows of a prompt portion."""
    ops.set_compute_dtype(dtype)
    nh, nkv, ps, L, window = 4, 2, 16, 300, 37
    for nq in (1, 40):
        q, kv, bt, keys, vals = paged_case([nq], [L], nh, nkv, d, ps, dtype, seed=nq)
        direction = torch.randn(d, generator=torch.Generator().manual_seed(2))
        direction = (direction / direction.norm() * 40).to(dtype)
        q[:] = direction
        last = L - 1                               # position of the last query row
        outside, inside = last - window, last - window + 1
        for n, kdir in ((outside, direction * 2), (inside, direction)):
            for h in range(nkv):
                keys[0][n, h] = kdir.float()
                kv[bt[0, n // ps], 0, h, n % ps] = kdir
        ctx = make_ctx(ops, [nq], [L], nh, nkv, window, d)
        qkv = torch.cat([q.reshape(-1, nh * d), torch.zeros(nq, 2 * nkv * d, dtype=dtype)], dim=1).cuda().contiguous()
        out = ops.paged_attention(qkv, nh, nkv, d, kv.cuda(), bt.cuda(), ctx, d ** -0.5, window).float().cpu()
        want_last = vals[0][inside].repeat_interleave(nh // nkv, dim=0).reshape(nh * d)
        torch.testing.assert_close(out[-1], want_last, atol=2e-2, rtol=2e-2, msg=f"nq={nq}: the key at the edge")
        qs = torch.zeros(L, nh, d)
        qs[L - nq:] = q.float()
        full = plain_llama.causal_attention(qs, keys[0], vals[0], d ** -0.5, window=window)[L - nq:].reshape(nq, nh * d)
        torch.testing.assert_close(out, full, atol=2e-2, rtol=2e-2, msg=f"nq={nq}")
