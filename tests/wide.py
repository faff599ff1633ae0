"""Models with the layer widths of the benchmarks, for the GPU tests that check logits where
the published numbers are measured.  Two layers each (of the 22 and 32 the full models have),
so that a test runs in seconds; every other size of a layer is the full model's.

The folders are written in bfloat16: the float32 engine, the bfloat16 engine and the plain
implementation then all compute with the same weight values, and what remains between them is
the rounding of activations."""

from __future__ import annotations

from tests.tiny import make_folder

# TinyLlama 1.1B widths (2 of 22 layers).  max_position_embeddings is 4096 instead of the
# model's 2048 because the traces run 2,048-token portions followed by decoded tokens.
WIDE_T = {
    "architectures": ["LlamaForCausalLM"], "vocab_size": 32000, "hidden_size": 2048, "intermediate_size": 5632,
    "num_hidden_layers": 2, "num_attention_heads": 32, "num_key_value_heads": 4, "head_dim": 64,
    "rms_norm_eps": 1e-5, "rope_theta": 10000.0, "max_position_embeddings": 4096, "tie_word_embeddings": False,
    "hidden_act": "silu", "torch_dtype": "bfloat16",
}
WIDE_T_INIT = dict(seed=0, std=0.02, norm_std=0.1)

# Llama-3-8B widths (2 of 32 layers; head size 128, 32 query heads on 8 kv heads).  The
# vocabulary is cut to 8,209 rows (no multiple of 8; the model has 128,256) to keep the folder small.
WIDE_8B = {
    "architectures": ["LlamaForCausalLM"], "vocab_size": 8209, "hidden_size": 4096, "intermediate_size": 14336,
    "num_hidden_layers": 2, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128,
    "rms_norm_eps": 1e-5, "rope_theta": 500000.0, "max_position_embeddings": 8192, "tie_word_embeddings": False,
    "hidden_act": "silu", "torch_dtype": "bfloat16",
}
WIDE_8B_INIT = dict(seed=1, std=0.02, norm_std=0.1)

WIDES = {"T": (WIDE_T, WIDE_T_INIT), "8B": (WIDE_8B, WIDE_8B_INIT)}


def wide_folder(tmp_path_factory, name: str) -> str:
    hf, init = WIDES[name]
    d = tmp_path_factory.mktemp(f"wide{name}")
    make_folder(d, hf, init, dtype="bfloat16")
    return str(d)
