"""The decode-attention entry point that allocates nothing
(csrc/attention_decode_static.h), called through its exported C symbol.

Callers that may not allocate device memory when they call (a host with a fixed
arena, code inside somebody else's capture, a plug-in that must stay out of the
allocator) get the split-context decode attention with its scratch inside the
library.  This test drives it with ctypes exactly as such a caller would, twice
in a row with different inputs (the built-in scratch keeps the first call's
contents), and holds the results to the regular entry point's.

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


@pytest.mark.parametrize("nh,nkv,d,ps", [(32, 4, 64, 16), (6, 2, 48, 8), (8, 8, 128, 32)])
def test_static_scratch_entry_point_matches_the_regular_one(nh, nkv, d, ps):
    from paged_llm_b200.kernels.ops import CudaOps
    from tests.test_kernels_gpu import make_ctx, paged_case

    ops = CudaOps("cuda")
    ops.set_compute_dtype(torch.bfloat16)
    lib = _load()
    assert lib.pl_attention_decode_static_capacity() == 8 << 20
    cases = [([1, 1, 1], [700, 33, 1500]), ([1, 2, 1, 1], [90, 400, 2048, 5])]
    for call, (q_lens, k_lens) in enumerate(cases):                     # two calls in a row
        if nh // nkv * max(q_lens) > 16:
            q_lens = [1] * len(q_lens)
        q, kv, bt, _, _ = paged_case(q_lens, k_lens, nh, nkv, d, ps, torch.bfloat16, seed=40 + call)
        ctx = make_ctx(ops, q_lens, k_lens, nh, nkv, None, d)
        plan = ctx.attention_plans[(nh // nkv, nkv, None, d)]
        assert plan.n_small and not plan.n_large and plan.max_splits > 1
        qkv = torch.cat([q.reshape(-1, nh * d), torch.zeros(q.shape[0], 2 * nkv * d, dtype=torch.bfloat16)], 1).cuda().contiguous()
        kv, bt = kv.cuda(), bt.cuda()
        want = ops.paged_attention(qkv, nh, nkv, d, kv, bt, ctx, d ** -0.5, None)
        out = torch.full_like(want, float("nan"))
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        rc = _call(lib, qkv, kv, out, bt, ctx, plan, nh, nkv, d, None, d ** -0.5)
        torch.cuda.synchronize()
        assert rc == 0, lib.pl_last_error().decode()
        assert torch.cuda.memory_allocated() == before
        torch.testing.assert_close(out.float(), want.float(), atol=1.6e-2, rtol=1.6e-2, msg=f"call {call}")


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
