"""The kernel library as the parts see it: `CudaOps`.

Every method launches hand-written CUDA kernels of `csrc/` (compiled for
sm_100a at first use, called through ctypes on the current stream) on torch
tensors.  There is no CPU fallback: without a CUDA device or without nvcc the
constructor raises.  The only library calls are the bfloat16 matrix products
(cuBLAS through torch), where the reference's engine also calls a library
(`nn.Linear`, pagedllm/model/llama.py:141-144); float32 products use this
package's own CUDA-core kernel so that no reduced-precision mode can slip in.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_void_p

import numpy as np
import torch

from ..csrc import build
from . import plan as planning
from .errors import KernelError

PL_F32, PL_BF16 = 0, 1
_DTYPE_CODE = {torch.float32: PL_F32, torch.bfloat16: PL_BF16}


class LazyNorm:
    """RMSNorm(x) * weight that no kernel has formed yet: the product that comes next
    normalises while it loads.  `part` holds the sums of squares of x that the product
    in front left (per 16 columns and token)."""

    def __init__(self, x: torch.Tensor, part: torch.Tensor, weight: torch.Tensor, eps: float):
        self.x, self.part, self.weight, self.eps = x, part, weight, eps
        self.shape = x.shape
        self.dtype = torch.bfloat16


class AttnParams(ctypes.Structure):
    _fields_ = [
        ("q", c_void_p), ("kv", c_void_p), ("out", c_void_p), ("block_table", c_void_p), ("cu_q", c_void_p),
        ("k_lens", c_void_p), ("work", c_void_p), ("scratch", c_void_p), ("scratch_floats", c_longlong),
        ("q_stride", c_int), ("out_stride", c_int), ("bt_stride", c_int), ("n_work", c_int), ("max_splits", c_int),
        ("nh", c_int), ("nkv", c_int), ("d", c_int), ("ps", c_int), ("window", c_int), ("is_small", c_int),
        ("scale", c_float), ("ps_shift", c_int), ("counters", c_void_p), ("num_pages", c_int), ("cluster", c_int),
        ("softcap", c_float), ("slopes", c_void_p), ("rope_table", c_void_p), ("rope_len", c_int),
        ("pad_seqs", c_int), ("pad_to", c_int),
    ]


_LIBS: dict[str, ctypes.CDLL] = {}


def load_module(name: str) -> ctypes.CDLL:
    """The compiled module `name`, built first if need be."""
    lib = _LIBS.get(name)
    if lib is None:
        path = build.build_module(name)
        lib = ctypes.CDLL(path)
        lib.pl_last_error.restype = ctypes.c_char_p
        _LIBS[name] = lib
    return lib


# Every wait inside a kernel (on an mbarrier of a TMA ring or of tcgen05) is bounded; a wait that
# gives up adds one to a counter of its module, which these exports read.
_TIMEOUT_EXPORTS = ("pl_gemm_skinny_timeouts", "pl_gemm_tc_timeouts", "pl_attention_tc_timeouts")


def _check(lib, rc: int) -> None:
    if rc != 0:
        raise KernelError(lib.pl_last_error().decode())


def head_dim_build(d: int) -> int:
    if d % 16 or d <= 0:
        raise KernelError(f"head_dim={d}: the attention kernels take head sizes in steps of 16")
    for b in build.HEAD_DIM_BUILDS:
        if d <= b:
            return b
    raise KernelError(f"head_dim={d} is larger than the largest attention build ({build.HEAD_DIM_BUILDS[-1]})")


class CudaOps:
    supports_graphs = True
    SMALL_ROWS = 16
    MIN_SPLIT_KEYS = 128
    MAX_CLUSTER = int(os.environ.get("PAGED_LLM_B200_MAX_CLUSTER", "8"))     # blocks of a decode-attention cluster
    MAX_SPLITS = 32

    def __init__(self, device="cuda"):
        self.device = torch.device(device)
        if self.device.type != "cuda" or not torch.cuda.is_available():
            raise KernelError("paged_llm_b200 runs on a CUDA device only (no CPU path); none is available")
        major, minor = torch.cuda.get_device_capability(self.device)
        if major < 10:
            raise KernelError(f"the kernels are built for sm_100a (B200); this device is sm_{major}{minor}")
        self.core = load_module("core")
        self.compute_dtype = torch.bfloat16
        self.num_sms = torch.cuda.get_device_properties(self.device).multi_processor_count
        self._scratch: list[torch.Tensor] = []
        self._pinned_stream = None
        self._attn_lib = None
        self._attn_fn = None
        self.launches = 0                 # kernels of this package launched so far
        self.use_skinny = True            # few-token products on this package's weight-streaming kernel
        # Many tokens: this package's tcgen05 kernel (pairs of blocks on 256 x 256 tiles, fused epilogues) where it is at least
        # as fast as the library product followed by the elementwise kernel.  Measured: the gate/up product
        # with SiLU-mul from 2,048 tokens on (77 us against 87 us, timed alone); the narrower products and fewer
        # tokens are faster through the library.  PAGED_LLM_B200_GEMM_TC lists the kinds ("silu", "add", "plain", "all",
        # "" for none) to run on it from 129 tokens on instead.
        tc_for = os.environ.get("PAGED_LLM_B200_GEMM_TC")
        self.gemm_tc_min_tokens = 2048 if tc_for is None else 129
        tc_for = "silu" if tc_for is None else tc_for
        self.gemm_tc_for = {"silu", "add", "plain"} if tc_for == "all" else {t for t in tc_for.split(",") if t}
        self.cluster_attention = os.environ.get("PAGED_LLM_B200_NO_CLUSTER") is None   # decode attention as clusters
        # decode steps of more than 16 tokens: rotary positions and the cache write inside the attention kernel
        self.rope_in_attention = os.environ.get("PAGED_LLM_B200_NO_ROPE_IN_ATTENTION") is None
        # long work-list ranges of decode attention in a ring of three 64-key tiles (head sizes up to 64)
        self.deep_list = os.environ.get("PAGED_LLM_B200_NO_DEEP_LIST") is None
        self._argmax_ws = None            # (packed winners, arrival counters) of the multi-block argmax
        self._sample_dev = None           # the sampling parameters of a step on the device, and their pinned ring
        self._sample_ring: list = []
        self._sample_keep: list = []
        self._sample_pos = 0
        self._argmax_keep: list = []
        self._attn_counters = None        # arrival counters of the split merge inside the attention kernel
        self._attn_counters_keep: list = []
        self._norm_part = None            # sums of squares that an adding product leaves for the next one
        self._norm_part_keep: list = []
        # the library matrix products must not reduce in bfloat16
        torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False

    def set_compute_dtype(self, dtype: torch.dtype) -> None:
        if dtype not in _DTYPE_CODE:
            raise KernelError(f"compute dtype {dtype} is not supported (bfloat16 or float32)")
        self.compute_dtype = dtype

    @property
    def _stream(self):
        if self._pinned_stream is not None:
            return self._pinned_stream
        return c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    def pin_stream(self) -> None:
        """Looks the current stream up once and launches on it until `unpin_stream` (asking torch for the
        current stream costs more than the rest of a launch; the step function pins it for the length of a
        step and again wherever it changes the stream itself)."""
        self._pinned_stream = c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    def unpin_stream(self) -> None:
        self._pinned_stream = None

    @staticmethod
    def _p(t: torch.Tensor | None):
        return c_void_p(t.data_ptr()) if t is not None else c_void_p(0)

    def _code(self, t: torch.Tensor) -> int:
        try:
            return _DTYPE_CODE[t.dtype]
        except KeyError:
            raise KernelError(f"tensor of dtype {t.dtype} where float32 or bfloat16 is expected") from None

    def kernel_timeouts(self) -> int:
        """Bounded waits inside kernels that gave up since the process started, over all loaded
        modules.  Reading the counters waits for the device."""
        total = 0
        for lib in list(_LIBS.values()):
            for name in _TIMEOUT_EXPORTS:
                try:
                    fn = getattr(lib, name)
                except AttributeError:
                    continue
                n = int(fn())
                if n < 0:
                    raise KernelError(f"{name}: the counter could not be read")
                total += n
        return total

    def check_kernels(self) -> None:
        """Raises if a kernel gave up on a wait: what it computed afterwards is not to be trusted."""
        n = self.kernel_timeouts()
        if n:
            raise KernelError(f"{n} bounded wait(s) inside kernels gave up (a TMA copy or a tensor-core product "
                              "never signalled its barrier); results since the last check may be wrong")

    def copy_h2d(self, dst: torch.Tensor, src: torch.Tensor, nbytes: int) -> None:
        """Asynchronous copy of `nbytes` from pinned host memory to the device on the current stream."""
        _check(self.core, self.core.pl_copy_h2d(self._p(dst), self._p(src), c_longlong(nbytes), self._stream))

    def fill_normal(self, out: torch.Tensor, seed: int, key: int, mean: float = 0.0, std: float = 1.0) -> torch.Tensor:
        """out[...] = mean + std * N(0, 1) from the counter-based stream (seed, key): the values depend
        on nothing else.  For random weights drawn on the device."""
        assert out.is_contiguous() and out.is_cuda
        _check(self.core, self.core.pl_fill_normal(self._p(out), self._code(out), c_longlong(out.numel()),
                                                   ctypes.c_ulonglong(seed & (2 ** 64 - 1)),
                                                   ctypes.c_ulonglong(key & (2 ** 64 - 1)), c_float(mean), c_float(std),
                                                   self._stream))
        self.launches += 1
        return out

    # ---- embedding, norms, activation ------------------------------------------
    def embedding(self, table: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
        T, (V, H) = ids.numel(), table.shape
        out = torch.empty((T, H), dtype=torch.float32, device=self.device)
        _check(self.core, self.core.pl_embedding(self._p(table), self._code(table), self._p(ids), self._p(out),
                                                 T, H, V, self._stream))
        self.launches += 1
        return out

    def rms_norm(self, x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
        return self._norm(x, None, w, eps)

    def add_rms_norm(self, x: torch.Tensor, branch: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
        return self._norm(x, branch, w, eps)

    def _norm(self, x, branch, w, eps):
        assert x.dtype == torch.float32 and x.is_contiguous(), "the residual stream is contiguous float32"
        rows, H = x.shape
        y = torch.empty((rows, H), dtype=self.compute_dtype, device=self.device)
        if branch is not None:
            assert branch.shape == x.shape and branch.is_contiguous()
        bcode = self._code(branch) if branch is not None else PL_F32
        _check(self.core, self.core.pl_rmsnorm(self._p(x), self._p(branch), bcode, self._p(w), self._code(w),
                                               self._p(y), self._code(y), rows, H, c_float(eps), self._stream))
        self.launches += 1
        return y

    def silu_mul(self, gate_up: torch.Tensor) -> torch.Tensor:
        rows, two_i = gate_up.shape
        assert gate_up.is_contiguous() and two_i % 2 == 0
        out = torch.empty((rows, two_i // 2), dtype=gate_up.dtype, device=self.device)
        _check(self.core, self.core.pl_silu_mul(self._p(gate_up), self._p(out), self._code(gate_up), rows, two_i // 2,
                                                self._stream))
        self.launches += 1
        return out

    def gather_rows(self, x: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
        n, H = idx.numel(), x.shape[1]
        assert x.is_contiguous()
        out = torch.empty((n, H), dtype=x.dtype, device=self.device)
        _check(self.core, self.core.pl_gather_rows(self._p(x), self._p(idx), self._p(out), self._code(x), n, H,
                                                   x.shape[0], self._stream))
        self.launches += 1
        return out

    # ---- matrix products ---------------------------------------------------------
    def materialize(self, h):
        """A tensor for `h`, which may be a `LazyNorm`."""
        if isinstance(h, LazyNorm):
            return self.rms_norm(h.x, h.weight, h.eps)
        return h

    def _norm_args(self, h):
        """(X pointer, row stride, partial sums, norm weight, its dtype code, eps) for a product."""
        if isinstance(h, LazyNorm):
            return (self._p(h.x), h.x.shape[1], self._p(h.part), self._p(h.weight), self._code(h.weight), c_float(h.eps))
        return (self._p(h), h.shape[1], c_void_p(0), c_void_p(0), 0, c_float(0.0))

    def _skinny_ok(self, h, N: int) -> bool:
        """Few tokens: the weight-streaming kernel of this package instead of the library."""
        M, K = h.shape
        return self.use_skinny and h.dtype == torch.bfloat16 and 1 <= M <= 16 and K >= 32 and K % 32 == 0

    def _gemm_tc_ok(self, h, w: torch.Tensor, kind: str) -> bool:
        M, K = h.shape
        return (kind in self.gemm_tc_for and h.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
                and M >= self.gemm_tc_min_tokens
                and K >= 64 and K % 64 == 0 and w.is_contiguous())

    def _gemm_tc(self, h: torch.Tensor, w: torch.Tensor, out, resid, N: int, epi: int) -> None:
        M, K = h.shape
        assert h.stride(1) == 1 and h.stride(0) % 8 == 0
        lib, fn = self.core, self.core.pl_gemm_tc
        _check(lib, fn(self._p(h), h.stride(0), self._p(w), self._p(out), out.shape[1] if out is not None else 0,
                       self._p(resid), M, N, K, epi, self._stream))
        self.launches += 1

    def linear(self, h, w: torch.Tensor, out_float32: bool = False) -> torch.Tensor:
        """h [M, K] @ w[N, K]^T.  float32: this package's CUDA-core kernel; bfloat16 with few
        tokens: this package's weight-streaming kernel; else the library product with
        float32 accumulation.  `h` may be a `LazyNorm`."""
        M, K = h.shape
        N = w.shape[0]
        assert w.shape[1] == K and w.is_contiguous()
        if self._skinny_ok(h, N) and w.dtype == torch.bfloat16:
            x, ldx, part, nw, nwc, eps = self._norm_args(h)
            out = torch.empty((M, N), dtype=torch.float32 if out_float32 else torch.bfloat16, device=self.device)
            _check(self.core, self.core.pl_gemm_skinny(x, ldx, self._p(w), self._p(out), N, M, N, K,
                                                       1 if out_float32 else 0, part, nw, nwc, eps, self._stream))
            self.launches += 1
            return out
        h = self.materialize(h)
        assert h.is_contiguous()
        if self._gemm_tc_ok(h, w, "plain") and N % 8 == 0:
            out = torch.empty((M, N), dtype=torch.float32 if out_float32 else torch.bfloat16, device=self.device)
            self._gemm_tc(h, w, out, None, N, 1 if out_float32 else 0)
            return out
        if h.dtype == torch.float32:
            assert w.dtype == torch.float32
            out = torch.empty((M, N), dtype=torch.float32, device=self.device)
            _check(self.core, self.core.pl_gemm_f32(self._p(h), self._p(w), self._p(out), M, N, K, K, K, N,
                                                    self._stream))
            self.launches += 1
            return out
        assert h.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
        if out_float32:
            return torch.mm(h, w.t(), out_dtype=torch.float32)
        return torch.nn.functional.linear(h, w)

    def linear_add_rms_norm(self, h, w, x, norm_w, eps):
        """x += h @ w^T (float32 stream, in place), then RMSNorm(x) * norm_w.  With few tokens
        the product's epilogue adds and the result is a `LazyNorm` that the next product
        forms while loading; else the product is followed by the fused sum+norm kernel."""
        M, K = h.shape
        N = w.shape[0]
        if not isinstance(h, LazyNorm) and self._skinny_ok(h, N) and N % 16 == 0 and N % 32 == 0:
            assert x.dtype == torch.float32 and x.is_contiguous() and x.shape == (M, N) and h.is_contiguous()
            if self._norm_part is None or self._norm_part.numel() < N:
                self._norm_part_keep.append(self._norm_part)        # captured graphs hold the old address
                self._norm_part = torch.zeros(max(N, 1 << 16), dtype=torch.float32, device=self.device)
            _check(self.core, self.core.pl_gemm_skinny_add(self._p(h), K, self._p(w), self._p(x), M, N, K,
                                                           self._p(self._norm_part), self._stream))
            self.launches += 1
            return LazyNorm(x, self._norm_part, norm_w, eps)
        if (not isinstance(h, LazyNorm) and self._gemm_tc_ok(h, w, "add") and x.dtype == torch.float32
                and x.is_contiguous() and N % 4 == 0):
            self._gemm_tc(h, w, None, x, N, 3)
            return self.rms_norm(x, norm_w, eps)
        return self.add_rms_norm(x, self.linear(h, w), norm_w, eps)

    def gated_silu_linear(self, h, w_gate_up: torch.Tensor) -> torch.Tensor:
        """silu(h Wg^T) * (h Wu^T) for W = [Wg; Wu]: one kernel for few tokens, else the
        product followed by the activation kernel."""
        M, K = h.shape
        I = w_gate_up.shape[0] // 2
        if self._skinny_ok(h, 2 * I):
            x, ldx, part, nw, nwc, eps = self._norm_args(h)
            out = torch.empty((M, I), dtype=torch.bfloat16, device=self.device)
            _check(self.core, self.core.pl_gemm_skinny_silu(x, ldx, self._p(w_gate_up), self._p(out), I, M, I, K,
                                                            part, nw, nwc, eps, self._stream))
            self.launches += 1
            return out
        h = self.materialize(h)
        if self._gemm_tc_ok(h, w_gate_up, "silu") and h.is_contiguous() and I % 8 == 0:
            out = torch.empty((M, I), dtype=torch.bfloat16, device=self.device)
            self._gemm_tc(h, w_gate_up, out, None, I, 2)
            return out
        return self.silu_mul(self.linear(h, w_gate_up))

    def qkv_rope_write(self, h, w_qkv, nh, nkv, d, position, ctx, kv, block_table, write=True) -> torch.Tensor:
        """The fused q/k/v projection with rotary positions applied to q and k and k, v
        written to the cache.  Returns the [T, (nh + 2 nkv) d] buffer whose first nh*d
        columns are the rotated queries."""
        M, K = h.shape
        N = (nh + 2 * nkv) * d
        fusable = (self._skinny_ok(h, N) and position is not None and position.pairing == "half"
                   and position.rotary_dim == d and M == ctx.num_tokens)
        if not fusable:
            qkv = self.linear(h, w_qkv)
            self.rope_kv_write(qkv, nh, nkv, d, position, ctx, kv, block_table, write=write)
            return qkv
        x, ldx, part, nw, nwc, eps = self._norm_args(h)
        qkv = torch.empty((M, N), dtype=torch.bfloat16, device=self.device)
        assert kv.dtype == torch.bfloat16 and kv.is_contiguous()
        _check(self.core, self.core.pl_gemm_skinny_rope(
            x, ldx, self._p(w_qkv), self._p(qkv), N, M, K, nh, nkv, d, self._p(position.table),
            position.table.shape[0], self._p(ctx.positions), self._p(ctx.token_seq), self._p(block_table),
            block_table.shape[1], self._p(kv), kv.shape[0], kv.shape[3], 1 if write else 0, part, nw, nwc, eps,
            self._stream))
        self.launches += 1
        return qkv

    # ---- positions ---------------------------------------------------------------
    def rope_table(self, inv_freq: torch.Tensor, max_positions: int) -> torch.Tensor:
        inv_freq = inv_freq.to(device=self.device, dtype=torch.float32).contiguous()
        half = inv_freq.numel()
        table = torch.empty((max_positions, half, 2), dtype=torch.float32, device=self.device)
        _check(self.core, self.core.pl_rope_table(self._p(inv_freq), self._p(table), max_positions, half, self._stream))
        self.launches += 1
        return table

    def rope_kv_write(self, qkv, nh, nkv, d, position, ctx, kv, block_table, write=True):
        T = ctx.num_tokens
        assert qkv.is_contiguous() and qkv.shape[0] == T
        if position is not None:
            table, table_len, rd = position.table, position.table.shape[0], position.rotary_dim
            inter = 1 if position.pairing == "interleaved" else 0
        else:
            table, table_len, rd, inter = None, 0, 0, 0
        num_pages, ps = kv.shape[0], kv.shape[3]
        assert kv.dtype == qkv.dtype and kv.is_contiguous()
        _check(self.core, self.core.pl_rope_kv_write(
            self._p(qkv), self._code(qkv), T, qkv.shape[1], self._p(table), table_len, rd, inter,
            self._p(ctx.positions), self._p(ctx.token_seq), self._p(block_table), block_table.shape[1],
            self._p(kv), num_pages, nh, nkv, d, ps, 1 if write else 0, self._stream))
        self.launches += 1

    # ---- attention ---------------------------------------------------------------
    def _large_rows(self, head_dim: int) -> int:
        """Query rows of a prefill tile: what the kernel that will run was built with."""
        if self.compute_dtype != torch.bfloat16:
            return 16
        b = head_dim_build(head_dim)
        lib = load_module(f"attn_bf16_d{b}")
        return int(getattr(lib, f"pl_attention_bf16_rows_d{b}")(0))

    CLUSTER_KEYS = 600      # keys a block of a decode-attention cluster may have to walk before more splits pay

    def long_context_class(self, num_requests: int, num_kv_heads: int, max_context: int) -> bool:
        """True if a decode step of this shape is planned as a long-context step (see
        plan.is_long_context).  A step replayed from a graph must stay in the class it was
        captured in, so the runner keeps a graph per class."""
        return planning.is_long_context(num_requests, num_kv_heads, self.num_sms, self.MAX_SPLITS,
                                        self.MAX_CLUSTER if self.cluster_attention else 0, self.CLUSTER_KEYS, max_context)

    def plan_attention(self, q_lens, k_lens, group_size, num_kv_heads, window, head_dim, pad_requests=None,
                       fixed_capacity=False, pad_tokens=None) -> dict:
        return planning.plan_attention(
            q_lens, k_lens, group_size, num_kv_heads, window, small_rows=self.SMALL_ROWS,
            large_rows=self._large_rows(head_dim), min_split_keys=self.MIN_SPLIT_KEYS, num_sms=self.num_sms,
            max_splits=self.MAX_SPLITS, pad_requests=pad_requests, fixed_capacity=fixed_capacity,
            cluster_max=self.MAX_CLUSTER if self.cluster_attention else 0, long_keys=self.CLUSTER_KEYS,
            pad_tokens=pad_tokens)

    def _scratch_for(self, floats: int) -> torch.Tensor:
        """Scratch for split partials.  Grown by allocating anew and keeping the
        old buffers, since captured graphs hold their addresses."""
        if not self._scratch or self._scratch[-1].numel() < floats:
            self._scratch.append(torch.empty(max(floats, 1 << 20), dtype=torch.float32, device=self.device))
        return self._scratch[-1]

    def _attention_bf16(self, d: int):
        b = head_dim_build(d)
        lib = load_module(f"attn_bf16_d{b}")
        return lib, getattr(lib, f"pl_attention_bf16_d{b}")

    def _runs_as_clusters(self, plan, ctx, nh: int, nkv: int, bf16: bool) -> bool:
        """Whether this step's attention takes the cluster form of the decode kernel: every request
        is a small item (a decode step), in bfloat16, with contexts short enough."""
        return bool(bf16 and self.cluster_attention and plan.n_small and not plan.n_large
                    and max(ctx.host.q_lens) * (nh // nkv) <= self.SMALL_ROWS and not plan.long_context)

    def qkv_attention(self, h, w_qkv, nh, nkv, d, position, ctx, kv, block_table, scale, window, write=True,
                      softcap=None, slopes=None) -> torch.Tensor:
        """The mixer's whole front: fused q/k/v projection, rotary positions on q and k, k and v written
        to the cache, attention over the pages.  Returns [T, nh * d].  It is `qkv_rope_write` followed by
        `paged_attention`, but for a decode step of more than 16 tokens (the projection is a library
        product then, without an epilogue) rotation and cache write happen inside the attention
        kernel instead of in a kernel of their own."""
        M = h.shape[0]
        plan = ctx.attention_plans.get((nh // nkv, nkv, window, d))
        inside = (plan is not None and write and softcap is None and slopes is None and position is not None
                  and position.pairing == "half" and position.rotary_dim == d and M == ctx.num_tokens
                  and not self._skinny_ok(h, (nh + 2 * nkv) * d) and self.compute_dtype == torch.bfloat16
                  and kv.dtype == torch.bfloat16 and self._runs_as_clusters(plan, ctx, nh, nkv, True)
                  and self.rope_in_attention)
        if inside:
            qkv = self.linear(h, w_qkv)
            return self.paged_attention(qkv, nh, nkv, d, kv, block_table, ctx, scale, window, rope=position)
        qkv = self.qkv_rope_write(h, w_qkv, nh, nkv, d, position, ctx, kv, block_table, write=write)
        return self.paged_attention(qkv, nh, nkv, d, kv, block_table, ctx, scale, window, softcap=softcap, slopes=slopes)

    def paged_attention(self, qkv, nh, nkv, d, kv, block_table, ctx, scale, window, softcap=None, slopes=None,
                        rope=None):
        """Attention of the step's tokens over the paged cache.  `softcap` (scores become
        softcap * tanh(score / softcap)) and `slopes` (a float32 tensor [nh]: head h adds
        slopes[h] * (key position - query position) to its scores) modify the scores; both off
        by default.  `rope` (a prepared rotary encoding; only where the step runs as clusters, see
        `qkv_attention`): qkv is the unrotated projection, and the kernel rotates q and the step's own
        keys and writes those keys and values to the cache itself."""
        T = ctx.num_tokens
        plan = ctx.attention_plans[(nh // nkv, nkv, window, d)]
        out = torch.empty((T, nh * d), dtype=qkv.dtype, device=self.device)
        p = AttnParams()
        real = sum(ctx.host.q_lens)
        if T > real or getattr(ctx, "padded", False):
            # Rows that pad the step to the size of its graph.  The split-context kernels zero them themselves
            # (a fill kernel between two kernels of a layer would keep them from overlapping: 0.97 against 0.92 ms
            # per step at 12 requests); a step with large items too is not padded in practice and gets the fill.
            if plan.n_large:
                out.zero_()
            else:
                p.pad_seqs, p.pad_to = ctx.num_seqs, T
        p.q, p.kv, p.out = qkv.data_ptr(), kv.data_ptr(), out.data_ptr()
        p.block_table, p.cu_q, p.k_lens = block_table.data_ptr(), ctx.cu_seqlens_q.data_ptr(), ctx.seq_lens_k.data_ptr()
        p.q_stride, p.out_stride, p.bt_stride = qkv.shape[1], nh * d, block_table.shape[1]
        p.nh, p.nkv, p.d, p.ps, p.num_pages = nh, nkv, d, kv.shape[3], kv.shape[0]
        p.window, p.scale, p.max_splits = int(window or 0), float(scale), plan.max_splits
        p.softcap = float(softcap or 0.0)
        if slopes is not None:
            assert slopes.dtype == torch.float32 and slopes.numel() == nh and slopes.is_contiguous() and slopes.is_cuda
            p.slopes = slopes.data_ptr()
        ps = kv.shape[3]
        p.ps_shift = ps.bit_length() - 1 if ps & (ps - 1) == 0 else -1
        p.counters = 0
        bf16 = qkv.dtype == torch.bfloat16
        if bf16:
            lib, fn = self._attention_bf16(d)
        else:
            lib, fn = self.core, self.core.pl_attention_f32
        p.cluster = 0
        if rope is not None:
            if not self._runs_as_clusters(plan, ctx, nh, nkv, bf16) or softcap or slopes is not None:
                raise KernelError("rotary positions inside the attention kernel: only for decode steps that run as "
                                  "clusters, without score modifiers")
            assert qkv.shape[1] == (nh + 2 * nkv) * d and rope.table.is_contiguous() and rope.rotary_dim == d
            p.rope_table, p.rope_len = rope.table.data_ptr(), rope.table.shape[0]
        if self._runs_as_clusters(plan, ctx, nh, nkv, bf16):
            # every request is a small item: the splits of a (request, kv head) are the blocks of
            # a thread-block cluster that merge through distributed shared memory
            p.work, p.n_work, p.is_small, p.cluster = 0, ctx.num_seqs, 1, min(plan.max_splits, self.MAX_CLUSTER)
            p.scratch, p.scratch_floats = 0, 0
            _check(lib, fn(ctypes.byref(p), self._stream))
            self.launches += 1
            return out
        if plan.n_small:
            floats = max(plan.small_tokens, 1) * nh * plan.max_splits * (d + 2)
            scratch = self._scratch_for(floats)
            p.scratch, p.scratch_floats = scratch.data_ptr(), scratch.numel()
            # long ranges and blocks in plenty (two per SM or more): the ring of three 64-key tiles; with fewer
            # blocks eight warps per block do better (one request x 16,384 keys: 1.00 against 1.10 ms per step)
            deep = plan.long_context and self.deep_list and plan.n_small * nkv >= 2 * self.num_sms
            p.work, p.n_work, p.is_small = plan.small.data_ptr(), plan.n_small, 2 if deep else 1
            fused_merge = bf16 and plan.max_splits > 1
            if fused_merge:
                need = ctx.num_seqs * nkv
                if self._attn_counters is None or self._attn_counters.numel() < need:
                    self._attn_counters_keep.append(self._attn_counters)    # captured graphs hold the old address
                    self._attn_counters = torch.zeros(max(need, 4096), dtype=torch.int32, device=self.device)
                p.counters = self._attn_counters.data_ptr()
            _check(lib, fn(ctypes.byref(p), self._stream))
            self.launches += 1
            p.counters = 0
            if plan.max_splits > 1 and not fused_merge:
                _check(self.core, self.core.pl_attention_combine(ctypes.byref(p), self._code(out), self._stream))
                self.launches += 1
        if plan.n_large:
            p.scratch, p.scratch_floats = 0, 0
            p.work, p.n_work, p.is_small = plan.large.data_ptr(), plan.n_large, 0
            p.max_splits = 1
            _check(lib, fn(ctypes.byref(p), self._stream))
            self.launches += 1
        return out

    # ---- cache -------------------------------------------------------------------
    def copy_pages(self, pool: torch.Tensor, pairs) -> None:
        layers, pages = pool.shape[0], pool.shape[1]
        page_bytes = pool[0, 0].numel() * pool.element_size()
        for src, dst in pairs:
            _check(self.core, self.core.pl_copy_page(self._p(pool), layers, c_longlong(pages), c_longlong(page_bytes),
                                                     int(src), int(dst), self._stream))
            self.launches += 1

    # ---- sampling ----------------------------------------------------------------
    def argmax(self, logits: torch.Tensor) -> torch.Tensor:
        rows, V = logits.shape
        assert logits.dtype == torch.float32 and logits.stride(1) == 1
        out = torch.empty(rows, dtype=torch.int32, device=self.device)
        if self._argmax_ws is None or self._argmax_ws[0].numel() < rows:
            self._argmax_keep.append(self._argmax_ws)               # captured graphs hold the old addresses
            self._argmax_ws = (torch.zeros(max(rows, 1024), dtype=torch.int64, device=self.device),
                               torch.zeros(max(rows, 1024), dtype=torch.int32, device=self.device))
        cells, counters = self._argmax_ws
        _check(self.core, self.core.pl_argmax(self._p(logits), self._p(out), rows, V, c_longlong(logits.stride(0)),
                                              self._p(cells), self._p(counters), self._stream))
        self.launches += 1
        return out

    def sample(self, logits, temps, top_k, top_p, seeds, counters) -> torch.Tensor:
        rows, V = logits.shape
        assert logits.dtype == torch.float32 and logits.stride(1) == 1
        dev = self.device
        # The five per-row arrays go up as one copy from pinned memory that does not wait for the step in front
        # of it (five copies from pageable memory each waited for the device: 1.01 against 0.81 ms per step at
        # batch 8).  Layout in 8-byte words: seeds [rows], counters [rows], then temps, top_p, top_k as 4-byte
        # values.
        words = 2 * rows + (3 * rows + 1) // 2
        if self._sample_dev is None or self._sample_dev.numel() < words:
            self._sample_keep.append(self._sample_dev)              # a kernel in flight may still read the old one
            self._sample_dev = torch.empty(max(2 * words, 1024), dtype=torch.int64, device=dev)
            self._sample_ring = [[torch.empty(max(2 * words, 1024), dtype=torch.int64, pin_memory=True), None]
                                 for _ in range(4)]
        slot = self._sample_ring[self._sample_pos % len(self._sample_ring)]
        self._sample_pos += 1
        if slot[1] is not None:
            slot[1].synchronize()                                   # its last copy has left the buffer
        host = slot[0].numpy()
        host[:rows] = np.ascontiguousarray(seeds, np.uint64).view(np.int64)
        host[rows:2 * rows] = np.ascontiguousarray(counters, np.uint64).view(np.int64)
        tail = host[2 * rows:words].view(np.float32)
        tail[:rows] = temps
        tail[rows:2 * rows] = top_p
        tail[2 * rows:3 * rows].view(np.int32)[:] = top_k
        self.copy_h2d(self._sample_dev, slot[0], words * 8)
        slot[1] = torch.cuda.Event()
        slot[1].record()
        s, c = self._sample_dev[:rows], self._sample_dev[rows:2 * rows]
        tail_dev = self._sample_dev[2 * rows:words].view(torch.float32)
        t, pp, k = tail_dev[:rows], tail_dev[rows:2 * rows], tail_dev[2 * rows:3 * rows].view(torch.int32)
        out = torch.empty(rows, dtype=torch.int32, device=dev)
        _check(self.core, self.core.pl_sample(self._p(logits), self._p(out), rows, V, c_longlong(logits.stride(0)),
                                              self._p(t), self._p(k), self._p(pp), self._p(s), self._p(c),
                                              self._stream))
        self.launches += 1
        return out
