"""Weights: loading by name, storage dtypes, the one error that lists all that
is wrong, tied heads, and the random-weights mode."""

import json
import os

import pytest
import torch
from safetensors.torch import load_file, save_file

from paged_llm_b200.config import LlamaConfig
from paged_llm_b200.weights import WeightError, load_model, random_tensors, resolve_dtype, write_model_folder
from tests.tiny import TINY_A, TINY_B, make_folder, TINY_A_INIT, TINY_B_INIT


def test_random_weights_are_reproducible_and_shared_between_dtypes(tmp_path):
    cfg = LlamaConfig.from_hf_dict(TINY_B)
    a = random_tensors(cfg, seed=1, std=0.05, norm_std=0.1)
    b = random_tensors(cfg, seed=1, std=0.05, norm_std=0.1)
    c = random_tensors(cfg, seed=2, std=0.05, norm_std=0.1)
    h = random_tensors(cfg, seed=1, std=0.05, norm_std=0.1, dtype="bfloat16")
    assert a.keys() == b.keys() and all(torch.equal(a[k], b[k]) for k in a)
    assert any(not torch.equal(a[k], c[k]) for k in a)
    assert all(torch.equal(a[k].to(torch.bfloat16), h[k]) for k in a)
    assert "lm_head.weight" not in a                       # tied: the embedding is the head
    w = a["model.layers.0.self_attn.q_proj.weight"]
    assert abs(float(w.std()) - 0.05) < 0.005
    n = a["model.layers.1.input_layernorm.weight"]
    assert abs(float(n.mean()) - 1.0) < 0.05 and 0.05 < float(n.std()) < 0.15
    assert sum(t.numel() for t in a.values()) == cfg.num_parameters == 381312


def test_folder_round_trip(tmp_path):
    d = make_folder(tmp_path / "a", TINY_A, TINY_A_INIT)
    assert sorted(os.listdir(d)) == ["config.json", "model.safetensors"]
    with open(os.path.join(d, "config.json")) as f:
        assert json.load(f)["architectures"] == ["LlamaForCausalLM"]
    model, cfg, dtype = load_model(d, "auto", "cpu")
    assert dtype == torch.float32 and cfg.num_parameters == 123712
    stored = load_file(os.path.join(d, "model.safetensors"))
    attn = model.blocks[0].mixer
    q = stored["model.layers.0.self_attn.q_proj.weight"]
    assert torch.equal(attn.w_qkv[:q.shape[0]], q)         # stacked q, k, v
    assert attn.w_qkv.shape == (4 * 16 + 2 * 2 * 16, 64)
    assert model.blocks[1].feed_forward.w_gate_up.shape == (2 * 172, 64)


def test_storage_dtypes(tmp_path):
    d = make_folder(tmp_path / "b", TINY_B, TINY_B_INIT)              # stored in float32
    model, _, dtype = load_model(d, "bfloat16", "cpu")
    assert dtype == torch.bfloat16
    assert model.blocks[0].mixer.w_qkv.dtype == torch.bfloat16        # matrices: compute dtype
    assert model.blocks[0].norms["input"].weight.dtype == torch.float32  # a 32-bit vector stays 32-bit
    assert model.head.weight is model.embedding.weight                 # tied: one buffer
    d16 = make_folder(tmp_path / "b16", TINY_B, TINY_B_INIT, dtype="bfloat16")
    model16, _, dtype16 = load_model(d16, "auto", "cpu")
    assert dtype16 == torch.bfloat16 and model16.blocks[0].norms["input"].weight.dtype == torch.bfloat16
    model32, _, _ = load_model(d16, "float32", "cpu")
    assert model32.blocks[0].mixer.w_qkv.dtype == torch.float32


def test_resolve_dtype():
    assert resolve_dtype("auto", {"torch_dtype": "bfloat16"}) == torch.bfloat16
    assert resolve_dtype("auto", {"dtype": "float32"}) == torch.float32
    assert resolve_dtype("auto", {}) == torch.bfloat16               # half-precision default runs in bfloat16
    assert resolve_dtype("float32", {"torch_dtype": "bfloat16"}) == torch.float32
    with pytest.raises(ValueError):
        resolve_dtype("int8", {})


def test_one_error_lists_everything(tmp_path):
    d = make_folder(tmp_path / "bad", TINY_A, TINY_A_INIT)
    path = os.path.join(d, "model.safetensors")
    t = load_file(path)
    del t["model.layers.1.mlp.up_proj.weight"]
    del t["model.norm.weight"]
    t["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(64)
    t["model.layers.0.mlp.down_proj.weight"] = torch.zeros(64, 171)
    t["model.layers.1.self_attn.o_proj.weight"] = torch.zeros(64, 64, dtype=torch.int8)     # a quantized matrix
    t["model.layers.1.input_layernorm.weight"] = torch.ones(64, dtype=torch.int32)
    save_file(t, path)
    with pytest.raises(WeightError) as info:
        load_model(d, "float32", "cpu")
    e = info.value
    assert e.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert e.unexpected == ["model.layers.0.self_attn.q_proj.bias"]
    assert [w[0] for w in e.wrong_shape] == ["model.layers.0.mlp.down_proj.weight"]
    assert [w[0] for w in e.wrong_dtype] == ["model.layers.1.input_layernorm.weight",
                                             "model.layers.1.self_attn.o_proj.weight"]
    msg = str(e)
    for needle in ("missing tensors (2)", "unexpected tensors (1)", "wrong shapes (1)", "(64, 171)", "(64, 172)",
                   "wrong dtypes (2)", "file stores int8"):
        assert needle in msg, msg


def test_tied_head_in_file_and_ignored_buffers(tmp_path):
    d = make_folder(tmp_path / "tied", TINY_B, TINY_B_INIT)
    path = os.path.join(d, "model.safetensors")
    t = load_file(path)
    t["lm_head.weight"] = t["model.embed_tokens.weight"].clone()      # some exporters write the tied head too
    t["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(16)
    save_file(t, path)
    model, _, _ = load_model(d, "float32", "cpu")
    assert model.head.weight is model.embedding.weight


def test_untied_head_is_required(tmp_path):
    d = make_folder(tmp_path / "untied", TINY_A, TINY_A_INIT)
    path = os.path.join(d, "model.safetensors")
    t = load_file(path)
    del t["lm_head.weight"]
    save_file(t, path)
    with pytest.raises(WeightError, match="lm_head.weight"):
        load_model(d, "float32", "cpu")


def test_tensor_in_two_files_is_an_error(tmp_path):
    d = make_folder(tmp_path / "dup", TINY_A, TINY_A_INIT)
    t = load_file(os.path.join(d, "model.safetensors"))
    save_file({"model.norm.weight": t["model.norm.weight"]}, os.path.join(d, "extra.safetensors"))
    with pytest.raises(WeightError, match="more than one file"):
        load_model(d, "float32", "cpu")


def test_missing_files(tmp_path):
    with pytest.raises(FileNotFoundError, match="config.json"):
        load_model(str(tmp_path), "float32", "cpu")
    cfg = LlamaConfig.from_hf_dict(TINY_A)
    with open(tmp_path / "config.json", "w") as f:
        json.dump(cfg.to_hf_dict(), f)
    with pytest.raises(FileNotFoundError, match="safetensors"):
        load_model(str(tmp_path), "float32", "cpu")


def test_random_stub_needs_the_kernel_library_and_no_tensors_beside_it(tmp_path):
    """A folder of config.json + random_weights.json (weights drawn on the device): refused
    without the kernel library, with tensor files beside it, or with unknown keys."""
    from paged_llm_b200.weights import write_random_stub
    from paged_llm_b200.weights.random_init import read_random_stub, tensor_key
    cfg = LlamaConfig.from_hf_dict(TINY_A)
    d = write_random_stub(str(tmp_path / "stub"), cfg, seed=5, std=0.03)
    assert read_random_stub(d) == {"seed": 5, "std": 0.03, "norm_std": 0.0}
    assert read_random_stub(make_folder(tmp_path / "plain", TINY_A, TINY_A_INIT)) is None
    with pytest.raises(ValueError, match="kernel library"):
        load_model(d, "float32", "cpu")
    save_file({"model.norm.weight": torch.ones(64)}, os.path.join(d, "model.safetensors"))
    with pytest.raises(ValueError, match="both"):
        load_model(d, "float32", "cpu")
    with open(os.path.join(d, "random_weights.json"), "w") as f:
        json.dump({"seed": 1, "sigma": 2}, f)
    with pytest.raises(ValueError, match="expected the keys"):
        read_random_stub(d)
    assert tensor_key("a.weight") != tensor_key("b.weight") and 0 <= tensor_key("a.weight") < 2 ** 64
