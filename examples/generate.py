"""Minimal usage, in the manner of the reference's examples/generate.py:

    python examples/generate.py --model /path/to/model --max-tokens 64 --temperature 0.0

`--model` is a folder with config.json and *.safetensors (and tokenizer files,
if text prompts are wanted).  Without tokenizer files pass token ids with
`--prompt-ids 5,17,3` (repeatable).  `--random-weights NAME` writes a folder of
random weights of a named size first (tiny-a, tiny-b, tinyllama-1.1b) and runs
that.  The other options are the engine's (`EngineConfig`).
"""
import argparse
import logging
import os
import sys
import tempfile

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from paged_llm_b200 import EngineConfig, LLMEngine, SamplingParams  # noqa: E402

NAMED_SIZES = {
    "tiny-a": dict(vocab_size=256, hidden_size=64, intermediate_size=172, num_hidden_layers=2, num_attention_heads=4,
                   num_key_value_heads=2, head_dim=16, max_position_embeddings=128),
    "tiny-b": dict(vocab_size=509, hidden_size=96, intermediate_size=256, num_hidden_layers=3, num_attention_heads=3,
                   num_key_value_heads=3, head_dim=32, rms_norm_eps=1e-6, rope_theta=500000.0,
                   rope_scaling={"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                                 "original_max_position_embeddings": 64},
                   max_position_embeddings=256, tie_word_embeddings=True),
    "tinyllama-1.1b": dict(vocab_size=32000, hidden_size=2048, intermediate_size=5632, num_hidden_layers=22,
                           num_attention_heads=32, num_key_value_heads=4, head_dim=64, max_position_embeddings=2048),
}


def main() -> None:
    logging.basicConfig(level=logging.INFO, format="%(message)s")
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", default=None)
    ap.add_argument("--backend", default="auto", help="kept for compatibility; there is one attention implementation")
    ap.add_argument("--max-tokens", type=int, default=64)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--top-k", type=int, default=-1)
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--prompt-ids", action="append", default=[], help="comma-separated token ids; repeatable")
    ap.add_argument("--random-weights", choices=sorted(NAMED_SIZES), default=None)
    ap.add_argument("--dtype", default="auto")
    ap.add_argument("--block-size", type=int, default=16)
    ap.add_argument("--num-blocks", type=int, default=None)
    ap.add_argument("--max-num-batched-tokens", type=int, default=2048)
    ap.add_argument("--max-model-len", type=int, default=4096)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--enforce-eager", action="store_true")
    args = ap.parse_args()

    tmp = None
    model = args.model
    if args.random_weights:
        from paged_llm_b200.config.registry import parse_model_config
        from paged_llm_b200.weights import write_model_folder
        tmp = tempfile.TemporaryDirectory()
        # the architecture named in the configuration decides the config class, as for a checkpoint
        _, cfg = parse_model_config({"architectures": ["LlamaForCausalLM"], **NAMED_SIZES[args.random_weights]})
        model = write_model_folder(tmp.name, cfg, seed=args.seed, dtype="bfloat16" if args.dtype == "auto" else args.dtype)
    if model is None:
        ap.error("--model or --random-weights is required")

    engine = LLMEngine(model, EngineConfig(
        attention_backend=args.backend, dtype=args.dtype, block_size=args.block_size, num_gpu_blocks=args.num_blocks,
        max_num_batched_tokens=args.max_num_batched_tokens, max_model_len=args.max_model_len, seed=args.seed,
        enforce_eager=args.enforce_eager))
    if args.prompt_ids:
        prompts = [[int(t) for t in p.split(",") if t.strip()] for p in args.prompt_ids]
    elif engine.tokenizer is not None:
        prompts = [
            "The three laws of robotics are",
            "Explain why paged attention reduces GPU memory fragmentation in one paragraph.",
            "Explain why paged attention reduces GPU memory fragmentation in two sentences.",
        ]
    else:
        vocab = engine.model_config.vocab_size
        prompts = [[(7 * i + 3) % vocab for i in range(n)] for n in (6, 24, 26)]
    sp = SamplingParams(temperature=args.temperature, top_k=args.top_k, top_p=args.top_p, max_tokens=args.max_tokens)
    for out in engine.generate(prompts, sp):
        shown = out.text if engine.tokenizer is not None else str(out.token_ids)
        print(f"--- [{out.finish_reason}] cached_prefix_tokens={out.num_cached_tokens}\n{shown}\n")
    s = engine.stats
    print(f"steps={s.num_steps} prefill_tokens={s.num_prefill_tokens} decode_tokens={s.num_decode_tokens} "
          f"preemptions={s.num_preemptions} attention=cuda")
    if tmp is not None:
        tmp.cleanup()


if __name__ == "__main__":
    main()
