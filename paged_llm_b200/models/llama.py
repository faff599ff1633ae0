"""The Llama dense decoder as data: `LlamaConfig` -> `ModelSpec`.

Tensor names are the checkpoint's own (reference: pagedllm/model/llama.py:1-7,
:141-144, :166-168, :179-180, :191-193, :208).  Every layer is a pre-norm block
of grouped-query attention with rotary positions and a SiLU-gated feed-forward;
the schedule runs the layers once each, in order.
"""

from __future__ import annotations

from ..config.llama import LlamaConfig
from ..parts.base import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def llama_spec(cfg: LlamaConfig) -> ModelSpec:
    h, d = cfg.hidden_size, cfg.head_dim
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        mixer = PartSpec(
            "paged_attention",
            dict(hidden_size=h, num_heads=cfg.num_attention_heads, num_kv_heads=cfg.num_key_value_heads,
                 head_dim=d, scale=d ** -0.5, window=None, position="rotary"),
            {k: f"{p}self_attn.{k}.weight" for k in ("q_proj", "k_proj", "v_proj", "o_proj")},
        )
        ffn = PartSpec(
            "gated_mlp",
            dict(hidden_size=h, intermediate_size=cfg.intermediate_size, activation=cfg.hidden_act),
            {k: f"{p}mlp.{k}.weight" for k in ("gate_proj", "up_proj", "down_proj")},
        )
        norms = {
            "input": PartSpec("rms_norm", dict(dim=h, eps=cfg.rms_norm_eps), {"weight": p + "input_layernorm.weight"}),
            "post_mixer": PartSpec("rms_norm", dict(dim=h, eps=cfg.rms_norm_eps),
                                   {"weight": p + "post_attention_layernorm.weight"}),
        }
        layers.append(LayerSpec("pre_norm", mixer, ffn, norms))
    rotary = PartSpec("rotary", dict(
        head_dim=d, theta=cfg.rope_theta, pairing="half", rotary_dim=d,
        scaling=cfg.rope_scaling.to_dict() if cfg.rope_scaling else None))
    return ModelSpec(
        hidden_size=h,
        vocab_size=cfg.vocab_size,
        embedding=PartSpec("embedding", dict(vocab_size=cfg.vocab_size, hidden_size=h),
                           {"weight": "model.embed_tokens.weight"}),
        layers=layers,
        schedule=[ScheduleEntry(i) for i in range(cfg.num_hidden_layers)],
        final_norm=PartSpec("rms_norm", dict(dim=h, eps=cfg.rms_norm_eps), {"weight": "model.norm.weight"}),
        head=PartSpec("lm_head", dict(vocab_size=cfg.vocab_size, hidden_size=h,
                                      tied_to="model.embed_tokens.weight" if cfg.tie_word_embeddings else None),
                      {"weight": "lm_head.weight"}),
        positions={"rotary": rotary},
        ignored_tensors=("rotary_emb.inv_freq",),
    )
