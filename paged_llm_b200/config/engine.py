"""Engine-wide options.

Names and defaults follow the reference's `EngineConfig` (pagedllm/config.py:4-28)
so that a call written for it reads the same here.  What differs:

* there is one attention implementation, so `attention_backend` is accepted for
  compatibility and must be "auto" or "cuda";
* `dtype` is "auto", "bfloat16" or "float32" ("auto" reads the checkpoint's
  `torch_dtype`/`dtype` key; float16 checkpoints run in bfloat16);
* `enforce_eager` switches CUDA-graph replay of decode steps off;
* `overlap_decode` (not in the reference): while requests only decode, the engine launches
  the next step before it has read the tokens of the last one (see `LLMEngine.step`).
"""

from __future__ import annotations

from dataclasses import dataclass

SUPPORTED_DTYPES = ("auto", "bfloat16", "float32")


@dataclass
class EngineConfig:
    block_size: int = 16
    num_gpu_blocks: int | None = None          # None: sized from free memory at start
    gpu_memory_utilization: float = 0.9
    max_num_seqs: int = 256
    max_num_batched_tokens: int = 2048         # token budget of one step
    max_model_len: int = 4096
    enable_prefix_caching: bool = True
    enable_chunked_prefill: bool = True
    attention_backend: str = "auto"
    dtype: str = "auto"
    device: str = "cuda"
    seed: int = 0
    enforce_eager: bool = False
    overlap_decode: bool = True

    def __post_init__(self) -> None:
        if self.block_size <= 0 or self.block_size & (self.block_size - 1):
            raise ValueError(f"block_size must be a power of two, got {self.block_size}")
        if self.max_num_batched_tokens < self.block_size:
            raise ValueError("max_num_batched_tokens must be >= block_size")
        if self.max_num_seqs < 1:
            raise ValueError("max_num_seqs must be >= 1")
        if self.max_model_len < 2:
            raise ValueError("max_model_len must be >= 2")
        if not 0.0 < self.gpu_memory_utilization <= 1.0:
            raise ValueError("gpu_memory_utilization must be in (0, 1]")
        if self.num_gpu_blocks is not None and self.num_gpu_blocks < 1:
            raise ValueError("num_gpu_blocks must be positive")
        if self.attention_backend not in ("auto", "cuda"):
            raise ValueError(
                f"attention_backend={self.attention_backend!r}: this engine has one attention "
                "implementation (hand-written CUDA); use 'auto'")
        if self.dtype not in SUPPORTED_DTYPES and self.dtype != "float16":
            raise ValueError(f"dtype must be one of {SUPPORTED_DTYPES}, got {self.dtype!r}")
