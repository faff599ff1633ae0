"""Each part alone on the GPU against the plain formulation, the toy
architecture with a stateful mixer, and layers that differ within one model."""

import numpy as np
import pytest
import torch

from tests import plain_llama, schedules
from tests.helpers import assert_logits_close
from tests.test_kernels_gpu import make_ctx, randn
from tests.tiny import random_tokens, read_folder

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


@pytest.fixture(scope="module")
def ops():
    from paged_llm_b200.kernels.ops import CudaOps
    return CudaOps("cuda")


def names(*keys, prefix="p."):
    return {k: prefix + k for k in keys}


@pytest.mark.parametrize("dtype", DTYPES)
def test_norm_part(ops, dtype):
    from paged_llm_b200.parts import NORMS
    ops.set_compute_dtype(dtype)
    norm = NORMS["rms_norm"](weights={"weight": "n.w"}, dim=200, eps=3e-4)
    assert list(norm.tensor_specs()) == ["n.w"] and norm.tensor_specs()["n.w"].role == "vector"
    w = 1 + 0.2 * randn(200, seed=1)
    norm.load({"n.w": w})
    ctx = type("C", (), {"ops": ops})()
    x = randn(9, 200, seed=2, std=2.0)
    got = norm.forward(x, ctx).float().cpu()
    want = plain_llama.rms_norm(x.cpu(), w.cpu(), 3e-4)
    torch.testing.assert_close(got, want, atol=5e-2 if dtype == torch.bfloat16 else 1e-5, rtol=1e-2 if dtype == torch.bfloat16 else 1e-5)
    branch = randn(9, 200, seed=3).to(dtype)
    x2 = x.clone()
    norm.add_forward(x2, branch, ctx)
    torch.testing.assert_close(x2, x + branch.float())


@pytest.mark.parametrize("dtype", DTYPES)
def test_feed_forward_part(ops, dtype):
    from paged_llm_b200.parts import FEED_FORWARDS
    ops.set_compute_dtype(dtype)
    ffn = FEED_FORWARDS["gated_mlp"](weights=names("gate_proj", "up_proj", "down_proj"), hidden_size=72,
                                     intermediate_size=100)
    ws = {"p.gate_proj": randn(100, 72, seed=4, std=0.2).to(dtype), "p.up_proj": randn(100, 72, seed=5, std=0.2).to(dtype),
          "p.down_proj": randn(72, 100, seed=6, std=0.2).to(dtype)}
    assert {k: v.shape for k, v in ffn.tensor_specs().items()} == {k: tuple(v.shape) for k, v in ws.items()}
    ffn.load(ws)
    h = randn(13, 72, seed=7).to(dtype)
    from paged_llm_b200.parts import materialize
    got = materialize(ffn.forward(h, type("C", (), {"ops": ops})()), ops).float().cpu()
    want = plain_llama.gated_mlp(h.float().cpu(), *(ws[k].float().cpu() for k in ("p.gate_proj", "p.up_proj", "p.down_proj")))
    torch.testing.assert_close(got, want, atol=3e-2 if dtype == torch.bfloat16 else 1e-5, rtol=3e-2 if dtype == torch.bfloat16 else 1e-5)
    with pytest.raises(ValueError, match="silu"):
        FEED_FORWARDS["gated_mlp"](weights={}, hidden_size=8, intermediate_size=8, activation="gelu")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [None, 9])
def test_attention_part(ops, dtype, window):
    """Projections + rotary + cache write + attention + output projection for a
    prompt portion and a decoded token, against the plain block on the whole
    sequences."""
    from paged_llm_b200.cache.storage import LayerCache
    from paged_llm_b200.parts import MIXERS
    from paged_llm_b200.parts.rope import RotaryEncoding
    ops.set_compute_dtype(dtype)
    H, nh, nkv, d, ps = 72, 6, 2, 48, 8
    rope = RotaryEncoding({}, head_dim=d, theta=1000.0)
    rope.prepare(256, "cuda", ops)
    mixer = MIXERS["paged_attention"](weights=names("q_proj", "k_proj", "v_proj", "o_proj"), hidden_size=H,
                                      num_heads=nh, num_kv_heads=nkv, head_dim=d, scale=0.2, window=window,
                                      position=rope)
    assert mixer.cache_requirement().window == window
    ws = {"p.q_proj": randn(nh * d, H, seed=1, std=0.15), "p.k_proj": randn(nkv * d, H, seed=2, std=0.15),
          "p.v_proj": randn(nkv * d, H, seed=3, std=0.15), "p.o_proj": randn(H, nh * d, seed=4, std=0.15)}
    ws = {k: v.to(dtype) for k, v in ws.items()}
    mixer.load(ws)
    lens = [30, 21]
    hs = [randn(L, H, seed=10 + i).to(dtype) for i, L in enumerate(lens)]
    kv = torch.full((16, 2, nkv, ps, d), float("nan"), dtype=dtype, device="cuda")
    bt = torch.tensor([[5, 2, 9, 11, 0, 0], [7, 1, 3, 0, 0, 0]], dtype=torch.int32, device="cuda")
    cache = LayerCache("paged_kv", 0, True, kv=kv, window=window)
    outs = [[], []]
    # three steps: first portions, then a portion beside a single token, then two single tokens
    cuts = [([0, 0], [17, 20]), ([17, 20], [29, 21]), ([29, 21], [30, 21])]
    for starts, ends in cuts:
        active = [s for s in range(2) if ends[s] > starts[s]]
        q_lens = [ends[s] - starts[s] for s in active]
        ctx = make_ctx(ops, q_lens, [ends[s] for s in active], nh, nkv, window, d)
        ctx.ops = ops
        ctx.block_tables = [bt[active].contiguous()]
        h = torch.cat([hs[s][starts[s]:ends[s]] for s in active]).contiguous()
        from paged_llm_b200.parts import materialize
        out = materialize(mixer.forward(h, ctx, cache), ops).float().cpu()
        o = 0
        for s, n in zip(active, q_lens):
            outs[s].append(out[o:o + n])
            o += n
    w = {k.replace("p.", "") + ".weight": v.float().cpu() for k, v in ws.items()}
    for s, L in enumerate(lens):
        cos, sin = plain_llama.rotary_cos_sin(torch.arange(L), plain_llama.inv_frequencies(d, 1000.0, None))
        x = hs[s].float().cpu()
        q = plain_llama.apply_rotary((x @ w["q_proj.weight"].T).view(L, nh, d), cos, sin)
        k = plain_llama.apply_rotary((x @ w["k_proj.weight"].T).view(L, nkv, d), cos, sin)
        v = (x @ w["v_proj.weight"].T).view(L, nkv, d)
        want = plain_llama.causal_attention(q, k, v, 0.2, window).reshape(L, -1) @ w["o_proj.weight"].T
        tol = 4e-2 if dtype == torch.bfloat16 else 2e-5
        torch.testing.assert_close(torch.cat(outs[s]), want, atol=tol * float(want.abs().max()), rtol=tol)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_architecture_with_state(tmp_path, dtype):
    """A mixer with state of its own, registered by the test, runs through the
    real loader, cache manager, step function and kernels."""
    from paged_llm_b200.engine.replay import TraceReplayer
    from paged_llm_b200.weights import write_model_folder
    from tests.toy_parts import TOY, ToyConfig, plain_toy_logits

    write_model_folder(str(tmp_path), ToyConfig.from_hf_dict(TOY), seed=4, std=0.1, norm_std=0.05)
    cfg, w = read_folder(tmp_path)
    reqs = {"a": random_tokens(61, 50, 1), "b": random_tokens(61, 37, 2), "c": random_tokens(61, 64, 3)}
    steps, max_tokens = schedules.mixed(reqs, live=2, seed=4)
    rp = TraceReplayer(str(tmp_path), dtype, max_tokens, poison=float("nan"))
    outputs = {rec["step"]: out for rec in steps if (out := rp.step(rec)) is not None}
    got = schedules.collect(steps, outputs)
    for rid, toks in reqs.items():
        assert_logits_close(got[rid], plain_toy_logits(cfg, w, toks).numpy(), dtype, f"toy/{rid}")
    assert rp.cm.num_free_state_slots == rp.cm.num_state_slots and rp.runner.num_graph_steps == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_stateful_toy_that_replays_graphs(tmp_path, dtype):
    """The same toy with its running mean written on the device's metadata alone (`capturable`):
    decode steps replay CUDA graphs, the engine launches steps ahead, and a forked request starts
    from a copy of its parent's state.  Nothing in the package knows the mixer."""
    from paged_llm_b200 import LLMEngine, SamplingParams
    from paged_llm_b200.engine.replay import TraceReplayer
    from paged_llm_b200.engine.sequence import Sequence
    from paged_llm_b200.weights import write_model_folder
    from tests.toy_parts import TOY, ToyConfig, plain_toy_logits

    hf = {**TOY, "architectures": ["DeviceToyForCausalLM"]}
    write_model_folder(str(tmp_path), ToyConfig.from_hf_dict(hf, architecture="DeviceToyForCausalLM"), seed=4, std=0.1,
                       norm_std=0.05)
    cfg, w = read_folder(tmp_path)
    reqs = {"a": random_tokens(61, 50, 1), "b": random_tokens(61, 37, 2), "c": random_tokens(61, 64, 3)}
    plain = {rid: plain_toy_logits(cfg, w, toks).numpy() for rid, toks in reqs.items()}
    for make in (schedules.tail, lambda r: schedules.mixed(r, live=2, seed=4)):
        steps, max_tokens = make(reqs)
        rp = TraceReplayer(str(tmp_path), dtype, max_tokens, poison=float("nan"))
        outputs = {rec["step"]: out for rec in steps if (out := rp.step(rec)) is not None}
        got = schedules.collect(steps, outputs)
        for rid in reqs:
            assert_logits_close(got[rid], plain[rid], dtype, f"device toy/{rid}")
        assert rp.cm.num_free_state_slots == rp.cm.num_state_slots
        assert rp.runner.num_graph_steps > 0, "decode steps of a capturable stateful model replay graphs"

    # through the engine: steps run ahead; greedy tokens follow the plain model
    eng = LLMEngine(str(tmp_path), dtype=dtype, block_size=16, num_gpu_blocks=32, max_model_len=128, max_num_seqs=4)
    prompts = [reqs["a"][:9], reqs["b"][:20]]
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True))
    assert eng.stats.num_steps_ahead > 0 and eng.runner.num_graph_steps > 0
    for p, o in zip(prompts, outs):
        seq = list(p)
        for tok in o.token_ids:
            ref = plain_toy_logits(cfg, w, seq)[-1].numpy()
            assert ref.max() - ref[tok] <= (1e-4 if dtype == "float32" else 3e-2 * np.abs(ref).max())
            seq.append(tok)

    # fork: the child continues from a copy of the parent's state and pages
    sched, cm, runner = eng.scheduler, eng.block_manager, eng.runner
    base = reqs["c"][:21]
    root = Sequence(base, SamplingParams(temperature=0.0, max_tokens=50, ignore_eos=True))
    sched.add(root)
    out = sched.schedule()
    sched.update(out, runner.run(out))
    child = Sequence(base, SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True))
    cm.fork(root, child)
    assert child.state_slot is not None and child.state_slot != root.state_slot
    child.token_ids = base + [7]
    child.status = root.status
    sched.running.append(child)
    sched.abort(root.seq_id)
    while sched.has_unfinished:
        out = sched.schedule()
        sched.update(out, runner.run(out))
    seq = base + [7]
    for tok in child.output_token_ids[1:]:
        ref = plain_toy_logits(cfg, w, seq)[-1].numpy()
        assert ref.max() - ref[tok] <= (1e-4 if dtype == "float32" else 3e-2 * np.abs(ref).max())
        seq.append(tok)
    assert len(child.output_token_ids) == 5 and cm.num_free_state_slots == cm.num_state_slots


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_with_a_bias_by_distance_instead_of_rotation(tmp_path, dtype):
    """A Llama whose attention rotates nothing and instead adds, per head, a slope times the
    distance to the key, with a cap on the scores of its second layer: two parameters of the
    attention part chosen by a spec of the test's own, against the plain formulation."""
    from paged_llm_b200.engine.replay import TraceReplayer
    from tests.toy_parts import biased_llama_case

    hf, w, reqs, plain = biased_llama_case(tmp_path, dtype)
    for make in (schedules.tail, lambda r: schedules.mixed(r, live=3, seed=6)):
        steps, max_tokens = make(reqs)
        rp = TraceReplayer(str(tmp_path), dtype, max_tokens, poison=float("nan"))
        outputs = {rec["step"]: out for rec in steps if (out := rp.step(rec)) is not None}
        got = schedules.collect(steps, outputs)
        for rid, toks in reqs.items():
            assert_logits_close(got[rid], plain(toks), dtype, f"biased/{rid}")
    without = plain_llama.forward_logits(hf, w, reqs["a"]).numpy()
    assert np.abs(without - plain(reqs["a"])).max() > 0.05 * np.abs(without).max(), "the modifiers must matter here"


@pytest.mark.parametrize("which,dtype", [("A", "float32"), ("B", "float32"), ("B", "bfloat16")])
def test_routed_toy_architecture(tmp_path, which, dtype):
    """A learned table of positions added by an embedding of the test's own, attention that
    rotates nothing, and a feed-forward that routes tokens to experts: registered by the test,
    run through the real loader, cache manager, step function and kernels."""
    from paged_llm_b200.engine.replay import TraceReplayer
    from paged_llm_b200.weights import write_model_folder
    from tests.toy_parts import ROUTED_TOY_A, ROUTED_TOY_B, RoutedToyConfig, plain_routed_toy_logits

    hf = {"A": ROUTED_TOY_A, "B": ROUTED_TOY_B}[which]
    # the folder holds the weights in the dtype under test, so both sides read the same values
    write_model_folder(str(tmp_path), RoutedToyConfig.from_hf_dict(hf), seed=6, std=0.1, norm_std=0.05, dtype=dtype)
    cfg, w = read_folder(tmp_path)
    V = hf["vocab_size"]
    reqs = {"a": random_tokens(V, 45, 1), "b": random_tokens(V, 70, 2), "c": random_tokens(V, 33, 3)}
    steps, max_tokens = schedules.mixed(reqs, live=2, seed=5)
    rp = TraceReplayer(str(tmp_path), dtype, max_tokens, poison=float("nan"))
    outputs = {rec["step"]: out for rec in steps if (out := rp.step(rec)) is not None}
    got = schedules.collect(steps, outputs)
    for rid, toks in reqs.items():
        assert_logits_close(got[rid], plain_routed_toy_logits(cfg, w, toks).numpy(), dtype, f"routed toy/{rid}")
    assert rp.runner.num_graph_steps == 0, "a model with a part that is not capturable steps eagerly"


def test_layers_of_one_model_may_differ(tmp_path):
    """Per-layer choice of parts: a Llama whose second layer has a window and
    other head counts gets two cache groups and still matches the plain model."""
    import json
    from paged_llm_b200.config.registry import ARCHITECTURES, register_architecture
    from paged_llm_b200.config import LlamaConfig
    from paged_llm_b200.engine.replay import TraceReplayer
    from paged_llm_b200.models.llama import llama_spec
    from paged_llm_b200.weights import write_model_folder
    from tests.tiny import TINY_A

    def spec(cfg):
        s = llama_spec(cfg)
        s.layers[1].mixer.params["window"] = 10
        return s
    if "WindowedLlama" not in ARCHITECTURES:
        register_architecture("WindowedLlama", LlamaConfig, spec)
    cfg = LlamaConfig.from_hf_dict({**TINY_A, "architectures": ["WindowedLlama"]}, architecture="WindowedLlama")
    write_model_folder(str(tmp_path), cfg, seed=5, std=0.1)
    hf, w = read_folder(tmp_path)
    toks = random_tokens(256, 90, 9)
    # plain: layer 0 sees all keys, layer 1 a window of 10
    c = plain_llama.read_config(hf)
    x = w["model.embed_tokens.weight"][torch.tensor(toks)]
    cos, sin = plain_llama.rotary_cos_sin(torch.arange(90), plain_llama.inv_frequencies(16, 10000.0, None))
    for i, win in enumerate((None, 10)):
        p = f"model.layers.{i}."
        h = plain_llama.rms_norm(x, w[p + "input_layernorm.weight"], c["eps"])
        x = x + plain_llama.attention_block(h, w, p + "self_attn.", c, cos, sin, window=win)
        h = plain_llama.rms_norm(x, w[p + "post_attention_layernorm.weight"], c["eps"])
        x = x + plain_llama.gated_mlp(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    want = (plain_llama.rms_norm(x, w["model.norm.weight"], c["eps"]) @ w["lm_head.weight"].T).numpy()
    steps, max_tokens = schedules.portions({"a": toks})
    rp = TraceReplayer(str(tmp_path), "float32", max_tokens, poison=float("nan"))
    assert rp.storage.num_groups == 2 and [g.window for g in rp.cm.group_specs] == [None, 10]
    outputs = {}
    held = []
    for rec in steps:
        out = rp.step(rec)
        outputs[rec["step"]] = out
        if rp.live:
            held.append(sum(1 for b in rp.live["a"].block_tables[1] if b >= 0))
    got = schedules.collect(steps, outputs)["a"]
    assert_logits_close(got, want, "float32", "windowed layer")
    assert max(held) <= 10 // 16 + 2 + 64 // 16, "the windowed group must give pages back as the window passes"
