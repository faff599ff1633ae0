"""Makes tests/golden/reference_logits.npz: logits of the REFERENCE's own model
code (xiyiji/paged-llm, imported from a checkout given by --reference) on the
tiny random models of tests/tiny.py, on the CPU in float32.

    python tests/golden/make_golden.py --reference /path/to/paged-llm

The reference is loaded through its own `load_model` with its pure-PyTorch
attention (pagedllm/model/loader.py:39-69, pagedllm/attention/reference.py:23-55)
from folders that this package's random-weights mode wrote, so the same file
also checks that the folders are readable by it.  The committed .npz lets
tests/test_plain_reference.py hold the plain implementation (tests/plain_llama.py)
to the reference without the reference being present.
"""

from __future__ import annotations

import argparse
import os
import sys
import tempfile

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from tests.tiny import TINIES, make_folder, random_tokens  # noqa: E402

NUM_TOKENS = 48


def reference_logits(folder: str, tokens: list[int]) -> np.ndarray:
    from pagedllm.attention.reference import paged_attention_reference
    from pagedllm.kv_cache import KVCache
    from pagedllm.model.llama import AttentionMetadata
    from pagedllm.model.loader import load_model

    model = load_model(folder, paged_attention_reference, torch.device("cpu"), torch.float32)
    c = model.config
    n, bs = len(tokens), 8
    nb = (n + bs - 1) // bs
    cache = KVCache(c.num_hidden_layers, nb, bs, c.num_key_value_heads, c.head_dim, torch.float32, "cpu")
    meta = AttentionMetadata(torch.arange(n), torch.arange(nb, dtype=torch.int32)[None],
                             torch.tensor([0, n], dtype=torch.int32), torch.tensor([n], dtype=torch.int32), n)
    with torch.no_grad():
        return model(torch.tensor(tokens), torch.arange(n), cache, meta, torch.arange(n)).numpy()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of xiyiji/paged-llm")
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    out = {}
    for name, (hf, init) in TINIES.items():
        with tempfile.TemporaryDirectory() as d:
            make_folder(d, hf, init)
            tokens = random_tokens(hf["vocab_size"], NUM_TOKENS, seed=11)
            out[f"{name}_tokens"] = np.array(tokens, np.int32)
            out[f"{name}_logits"] = reference_logits(d, tokens).astype(np.float32)
    np.savez_compressed(os.path.join(HERE, "reference_logits.npz"), **out)
    print({k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
