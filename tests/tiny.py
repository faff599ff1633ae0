"""The two tiny Llama configurations the tests run, which differ in every size
and option, and helpers to write and read their model folders."""

from __future__ import annotations

import json
import os

import torch

from paged_llm_b200.config import LlamaConfig
from paged_llm_b200.weights import write_model_folder

TINY_A = {
    "architectures": ["LlamaForCausalLM"], "vocab_size": 256, "hidden_size": 64, "intermediate_size": 172,
    "num_hidden_layers": 2, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16,
    "rms_norm_eps": 1e-5, "rope_theta": 10000.0, "max_position_embeddings": 128, "tie_word_embeddings": False,
    "hidden_act": "silu", "torch_dtype": "float32",
}
TINY_A_INIT = dict(seed=0, std=0.02, norm_std=0.0)

TINY_B = {
    "architectures": ["LlamaForCausalLM"], "vocab_size": 509, "hidden_size": 96, "intermediate_size": 256,
    "num_hidden_layers": 3, "num_attention_heads": 3, "num_key_value_heads": 3, "head_dim": 32,
    "rms_norm_eps": 1e-6, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 64},
    "max_position_embeddings": 256, "tie_word_embeddings": True, "hidden_act": "silu", "torch_dtype": "float32",
}
TINY_B_INIT = dict(seed=1, std=0.05, norm_std=0.1)

# A third shape for kernels: head_dim 48 (a multiple of 16 that is no power of two), 6 query heads on 2 kv heads.
TINY_C = {
    "architectures": ["LlamaForCausalLM"], "vocab_size": 131, "hidden_size": 72, "intermediate_size": 100,
    "num_hidden_layers": 2, "num_attention_heads": 6, "num_key_value_heads": 2, "head_dim": 48,
    "rms_norm_eps": 1e-5, "rope_theta": 1000.0, "max_position_embeddings": 512, "tie_word_embeddings": False,
    "hidden_act": "silu", "torch_dtype": "float32",
}
TINY_C_INIT = dict(seed=2, std=0.08, norm_std=0.05)

TINIES = {"A": (TINY_A, TINY_A_INIT), "B": (TINY_B, TINY_B_INIT), "C": (TINY_C, TINY_C_INIT)}


def make_folder(path, hf_cfg: dict, init: dict, dtype: str = "float32") -> str:
    cfg = LlamaConfig.from_hf_dict(hf_cfg)
    return write_model_folder(str(path), cfg, dtype=dtype, **init)


def read_folder(path) -> tuple[dict, dict]:
    """(config.json dict, tensors by name) read without the product's loader."""
    from safetensors import safe_open

    with open(os.path.join(path, "config.json")) as f:
        cfg = json.load(f)
    tensors = {}
    with safe_open(os.path.join(path, "model.safetensors"), framework="pt", device="cpu") as f:
        for k in f.keys():
            tensors[k] = f.get_tensor(k)
    return cfg, tensors


def random_tokens(vocab: int, n: int, seed: int) -> list[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()
