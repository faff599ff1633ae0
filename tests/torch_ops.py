"""A stand-in for the kernel library, in plain tensor code, for tests only.

It has the interface of `paged_llm_b200.kernels.ops.CudaOps` so that the engine's
host logic (runner, cache, scheduler, replay) can be exercised on a machine
without a GPU.  The product never imports it; on the product path a missing
extension is an error.
"""

from __future__ import annotations

import numpy as np
import torch

from paged_llm_b200.kernels.plan import plan_attention


class TorchOps:
    supports_graphs = False

    def __init__(self, device="cpu"):
        self.device = torch.device(device)
        self.compute_dtype = torch.float32
        self.calls: dict[str, int] = {}

    def _count(self, name):
        self.calls[name] = self.calls.get(name, 0) + 1

    def set_compute_dtype(self, dtype):
        self.compute_dtype = dtype

    # ---- elementwise / norms ---------------------------------------------------
    def embedding(self, table, ids):
        self._count("embedding")
        return table[ids.long()].float()

    def rms_norm(self, x, w, eps):
        self._count("rms_norm")
        xf = x.float()
        y = xf * torch.rsqrt((xf * xf).mean(-1, keepdim=True) + eps) * w.float()
        return y.to(self.compute_dtype)

    def add_rms_norm(self, x, branch, w, eps):
        x += branch.float()
        return self.rms_norm(x, w, eps)

    def linear(self, h, w, out_float32=False):
        self._count("linear")
        y = h.float() @ w.float().T
        return y if out_float32 else y.to(self.compute_dtype)

    def silu_mul(self, gate_up):
        self._count("silu_mul")
        i = gate_up.shape[1] // 2
        g, u = gate_up[:, :i].float(), gate_up[:, i:].float()
        return (g * torch.sigmoid(g) * u).to(self.compute_dtype)

    def materialize(self, h):
        return h

    def linear_add_rms_norm(self, h, w, x, norm_w, eps):
        return self.add_rms_norm(x, self.linear(h, w), norm_w, eps)

    def gated_silu_linear(self, h, w_gate_up):
        return self.silu_mul(self.linear(h, w_gate_up))

    def qkv_rope_write(self, h, w_qkv, nh, nkv, d, position, ctx, kv, block_table, write=True):
        qkv = self.linear(h, w_qkv)
        self.rope_kv_write(qkv, nh, nkv, d, position, ctx, kv, block_table, write=write)
        return qkv

    def qkv_attention(self, h, w_qkv, nh, nkv, d, position, ctx, kv, block_table, scale, window, write=True,
                      softcap=None, slopes=None):
        qkv = self.qkv_rope_write(h, w_qkv, nh, nkv, d, position, ctx, kv, block_table, write=write)
        return self.paged_attention(qkv, nh, nkv, d, kv, block_table, ctx, scale, window, softcap=softcap, slopes=slopes)

    def gather_rows(self, x, idx):
        return x[idx.long()].clone()

    # ---- positions -------------------------------------------------------------
    def rope_table(self, inv_freq, max_positions):
        ang = torch.outer(torch.arange(max_positions, dtype=torch.float32), inv_freq.float().cpu())
        return torch.stack([ang.cos(), ang.sin()], dim=-1).to(self.device)

    def rope_kv_write(self, qkv, nh, nkv, d, position, ctx, kv, block_table, write=True):
        self._count("rope_kv_write")
        T = ctx.num_tokens
        q = qkv[:, :nh * d].view(T, nh, d)
        k = qkv[:, nh * d:(nh + nkv) * d].view(T, nkv, d)
        v = qkv[:, (nh + nkv) * d:].view(T, nkv, d)
        pos = ctx.positions.long()
        if position is not None:
            rd = position.rotary_dim
            cs = position.table[pos]                 # [T, rd/2, 2]
            cos, sin = cs[..., 0][:, None, :], cs[..., 1][:, None, :]
            for x in (q, k):
                xf = x[..., :rd].float()
                if position.pairing == "half":
                    a, b = xf[..., :rd // 2], xf[..., rd // 2:]
                    out = torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1)
                else:
                    a, b = xf[..., 0::2], xf[..., 1::2]
                    out = torch.stack([a * cos - b * sin, b * cos + a * sin], dim=-1).flatten(-2)
                x[..., :rd] = out.to(x.dtype)
        if write:
            ps = kv.shape[3]
            seq = ctx.token_seq.long()
            for t in range(T):
                if seq[t] < 0:
                    continue
                p = int(pos[t])
                page = int(block_table[seq[t], p // ps])
                assert page >= 0, "write into a page that was given back"
                kv[page, 0, :, p % ps, :] = k[t].to(kv.dtype)
                kv[page, 1, :, p % ps, :] = v[t].to(kv.dtype)

    # ---- attention -------------------------------------------------------------
    def plan_attention(self, q_lens, k_lens, group_size, num_kv_heads, window, head_dim, pad_requests=None,
                       fixed_capacity=False, pad_tokens=None):
        return plan_attention(q_lens, k_lens, group_size, num_kv_heads, window, small_rows=16, large_rows=64,
                              min_split_keys=128, num_sms=4, pad_requests=pad_requests, fixed_capacity=fixed_capacity,
                              pad_tokens=pad_tokens)

    def paged_attention(self, qkv, nh, nkv, d, kv, block_table, ctx, scale, window, softcap=None, slopes=None):
        self._count("paged_attention")
        T = ctx.num_tokens
        q = qkv[:, :nh * d].view(T, nh, d).float()
        out = torch.zeros(T, nh * d, dtype=self.compute_dtype, device=qkv.device)
        ps = kv.shape[3]
        g = nh // nkv
        cu = ctx.host.cu
        for s, (nq, lk) in enumerate(zip(ctx.host.q_lens, ctx.host.k_lens)):
            first = lk - nq
            lo = max(0, first - window + 1) if window else 0
            idx = torch.arange(lo, lk)
            pages = block_table[s, (idx // ps)].long()
            assert (pages >= 0).all(), "read of a page that was given back"
            k = kv[pages, 0, :, idx % ps, :].float()       # [n, nkv, d]
            v = kv[pages, 1, :, idx % ps, :].float()
            k = k.repeat_interleave(g, dim=1)
            v = v.repeat_interleave(g, dim=1)
            qs = q[cu[s]:cu[s + 1]]
            scores = torch.einsum("qhd,khd->hqk", qs, k) * scale
            qpos = torch.arange(first, lk)
            if softcap:
                scores = softcap * torch.tanh(scores / softcap)
            if slopes is not None:
                scores = scores + slopes.float().cpu()[:, None, None] * (idx[None, None, :] - qpos[None, :, None])
            hidden = idx[None, :] > qpos[:, None]
            if window:
                hidden |= idx[None, :] <= qpos[:, None] - window
            scores = scores.masked_fill(hidden[None], float("-inf"))
            o = torch.einsum("hqk,khd->qhd", scores.softmax(-1), v)
            out[cu[s]:cu[s + 1]] = o.reshape(nq, nh * d).to(self.compute_dtype)
        return out

    def copy_pages(self, pool, pairs):
        self._count("copy_pages")
        for src, dst in pairs:
            pool[:, dst] = pool[:, src]

    # ---- sampling --------------------------------------------------------------
    def argmax(self, logits):
        return logits.argmax(-1)

    def sample(self, logits, temps, top_k, top_p, seeds, counters):
        from tests.plain_sampling import sample_rows
        return torch.tensor(sample_rows(logits.float().cpu().numpy(), temps, top_k, top_p, seeds, counters))
