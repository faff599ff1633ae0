"""The decode-attention entry point that allocates nothing
(csrc/attention_decode_static.h), called through its exported C symbol.

Callers that may not allocate device memory when they call (a host with a fixed
arena, code inside somebody else's capture, a plug-in that must stay out of the
allocator) get the split-context decode attention with its scratch inside the
library.  This test drives it with ctypes exactly as such a caller would, twice
in a row with different inputs (the built-in scratch keeps the first call's
contents), on a stream of its own, and holds the results to the regular entry
point's and to the plain float32 attention of tests/plain_llama.py.

It is collected last so that a run that stops at the first failure has already
run every other test; it needs nothing from them and also passes alone.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _load():
    from paged_llm_b200.csrc import build
    lib = ctypes.CDLL(build.build_module("attn_static"))
    lib.pl_last_error.restype = ctypes.c_char_p
    lib.pl_attention_decode_static_capacity.restype = ctypes.c_longlong
    return lib


def _call(lib, qkv, kv, out, bt, ctx, plan, nh, nkv, d, window, scale):
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    return lib.pl_attention_decode_static(
        p(qkv), qkv.shape[1], p(kv), p(out), nh * d, p(bt), bt.shape[1], p(ctx.cu_seqlens_q), p(ctx.seq_lens_k),
        p(plan.small), plan.n_small, plan.max_splits, max(plan.small_tokens, 1), nh, nkv, d, kv.shape[3],
        int(window or 0), ctypes.c_float(scale), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


def _plain_attention(q, keys, vals, q_lens, k_lens, nh, nkv, d, window):
    """The same attention by the plain float32 formulation on the CPU (tests/plain_llama.py),
    request by request: the new tokens are the last rows of the request's whole sequence."""
    from tests import plain_llama
    rows, o = [], 0
    for s, (nq, lk) in enumerate(zip(q_lens, k_lens)):
        full_q = torch.zeros(lk, nh, d)
        full_q[lk - nq:] = q[o:o + nq].float()
        out = plain_llama.causal_attention(full_q, keys[s], vals[s], d ** -0.5, window)
        rows.append(out[lk - nq:].reshape(nq, nh * d))
        o += nq
    return torch.cat(rows)


@pytest.mark.parametrize("nh,nkv,d,ps,window", [(32, 4, 64, 16, None), (6, 2, 48, 8, None), (8, 8, 128, 32, None),
                                                (32, 4, 64, 16, 50)])
def test_static_scratch_entry_point_matches_the_regular_one(nh, nkv, d, ps, window):
    from paged_llm_b200.kernels.ops import CudaOps
    from tests.test_kernels_gpu import make_ctx, paged_case

    ops = CudaOps("cuda")
    ops.set_compute_dtype(torch.bfloat16)
    lib = _load()
    assert lib.pl_attention_decode_static_capacity() == 8 << 20
    side = torch.cuda.Stream()                       # a caller's own stream, not the default one
    cases = [([1, 1, 1], [700, 33, 1500]), ([1, 2, 1, 1], [90, 400, 2048, 5])]
    for call, (q_lens, k_lens) in enumerate(cases):                     # two calls in a row
        if nh // nkv * max(q_lens) > 16:
            q_lens = [1] * len(q_lens)
        q, kv, bt, keys, vals = paged_case(q_lens, k_lens, nh, nkv, d, ps, torch.bfloat16, seed=40 + call)
        ctx = make_ctx(ops, q_lens, k_lens, nh, nkv, window, d)
        plan = ctx.attention_plans[(nh // nkv, nkv, window, d)]
        assert plan.n_small and not plan.n_large and (plan.max_splits > 1 or window)
        qkv = torch.cat([q.reshape(-1, nh * d), torch.zeros(q.shape[0], 2 * nkv * d, dtype=torch.bfloat16)], 1).cuda().contiguous()
        kv, bt = kv.cuda(), bt.cuda()
        want = ops.paged_attention(qkv, nh, nkv, d, kv, bt, ctx, d ** -0.5, window)
        out = torch.full_like(want, float("nan"))
        torch.cuda.synchronize()
        # the driver's own count of free device memory: an allocation by any route would move it
        free_before, _ = torch.cuda.mem_get_info()
        with torch.cuda.stream(side):
            rc = _call(lib, qkv, kv, out, bt, ctx, plan, nh, nkv, d, window, d ** -0.5)
        torch.cuda.synchronize()
        assert rc == 0, lib.pl_last_error().decode()
        if call > 0:                                 # the first call on a device sets the entry point up
            assert torch.cuda.mem_get_info()[0] == free_before, "the call changed the device's free memory"
        torch.testing.assert_close(out.float(), want.float(), atol=1.6e-2, rtol=1.6e-2, msg=f"call {call}")
        plain = _plain_attention(q, keys, vals, q_lens, k_lens, nh, nkv, d, window)
        torch.testing.assert_close(out.float().cpu(), plain, atol=1.6e-2, rtol=1.6e-2, msg=f"call {call} against plain")


def test_static_scratch_entry_point_takes_the_last_row_that_fits():
    """A work list whose request sits on the last scratch row the caller declared, with as many
    rows declared as the array holds for this shape: partials go to the very end of the array."""
    from paged_llm_b200.kernels.ops import CudaOps
    from tests.test_kernels_gpu import make_ctx, paged_case

    nh, nkv, d, ps = 32, 4, 64, 16
    ops = CudaOps("cuda")
    ops.set_compute_dtype(torch.bfloat16)
    lib = _load()
    q_lens, k_lens = [1, 1], [900, 300]
    q, kv, bt, keys, vals = paged_case(q_lens, k_lens, nh, nkv, d, ps, torch.bfloat16, seed=7)
    ctx = make_ctx(ops, q_lens, k_lens, nh, nkv, None, d)
    plan = ctx.attention_plans[(nh // nkv, nkv, None, d)]
    assert plan.max_splits > 1
    rows = (8 << 20) // (4 * nh * plan.max_splits * (d + 2))            # scratch rows that fit the array
    work = plan.small.cpu().clone()
    work[work[:, 0] == 1, 1] = rows - 1                                  # request 1 on the last row
    plan.small = work.cuda()
    plan.small_tokens = rows
    qkv = torch.cat([q.reshape(-1, nh * d), torch.zeros(q.shape[0], 2 * nkv * d, dtype=torch.bfloat16)], 1).cuda().contiguous()
    kv, bt = kv.cuda(), bt.cuda()
    out = torch.full((2, nh * d), float("nan"), dtype=torch.bfloat16, device="cuda")
    rc = _call(lib, qkv, kv, out, bt, ctx, plan, nh, nkv, d, None, d ** -0.5)
    torch.cuda.synchronize()
    assert rc == 0, lib.pl_last_error().decode()
    plain = _plain_attention(q, keys, vals, q_lens, k_lens, nh, nkv, d, None)
    torch.testing.assert_close(out.float().cpu(), plain, atol=1.6e-2, rtol=1.6e-2)


def test_static_scratch_entry_point_rejects_what_does_not_fit():
    lib = _load()
    z = ctypes.c_void_p(0)
    # 4096 rows x 32 heads x 32 splits x 66 floats is far beyond 8 MiB: refused before anything is launched
    rc = lib.pl_attention_decode_static(z, 2560, z, z, 2048, z, 8, z, z, z, 4096 * 32, 32, 4096, 32, 4, 64, 16, 0,
                                        ctypes.c_float(0.125), z)
    assert rc != 0 and "built-in scratch" in lib.pl_last_error().decode()
    rc = lib.pl_attention_decode_static(z, 2560, z, z, 2048, z, 8, z, z, z, 4, 2, 4, 32, 4, 144, 16, 0,
                                        ctypes.c_float(0.125), z)
    assert rc != 0 and "head_dim" in lib.pl_last_error().decode()
