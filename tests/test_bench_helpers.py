"""The benchmark script's host-side helpers: peaks file, flop counts, sizes, and the
one-GPU contract (no GPU needed)."""

import json
import subprocess
import sys

import pytest

import bench
from paged_llm_b200.config import LlamaConfig


def test_peaks_come_from_the_measured_file_when_it_is_there(tmp_path, monkeypatch):
    monkeypatch.setattr(bench, "ROOT", str(tmp_path))
    assert bench.load_peaks() == bench.FALLBACK_PEAKS
    (tmp_path / "MEASURED_PEAKS.json").write_text(json.dumps(
        {"gpu": "B200", "copy": {"hbm_gbs": 6900.5}, "gemm": {"bf16_tflops": 1610.0, "bf16_tflops_sustained": 1405.0}}))
    peaks = bench.load_peaks()
    assert peaks == {"source": "measured", "hbm_gbs": 6900.5, "bf16_tflops": 1610.0, "bf16_tflops_sustained": 1405.0}
    (tmp_path / "MEASURED_PEAKS.json").write_text("{not json")
    assert bench.load_peaks() == bench.FALLBACK_PEAKS


def test_flops_of_a_prefill_step_at_the_benchmark_sizes():
    cfg = LlamaConfig.from_hf_dict({"architectures": ["LlamaForCausalLM"], **bench.SIZES["tinyllama-1.1b"]})
    per_layer = 5_242_880 + 4_194_304 + 23_068_672 + 11_534_336          # q/k/v, o, gate/up, down
    products = 2 * 2048 * per_layer * 22 + 2 * 32000 * 2048               # the head runs on one row
    attention = 4 * 32 * 64 * (2048 * 2049 // 2) * 22
    assert bench.step_flops(cfg, 2048) == pytest.approx(products + attention, rel=1e-12)
    assert products == pytest.approx(3.969e12, rel=1e-3) and attention == pytest.approx(0.378e12, rel=2e-3)
    # a decoded token at context c reads c + 1 keys
    one = bench.step_flops(cfg, 1, context_start=640)
    assert one == pytest.approx(2 * per_layer * 22 + 2 * 32000 * 2048 + 4 * 32 * 64 * 641 * 22, rel=1e-12)


@pytest.mark.parametrize("size", sorted(bench.SIZES))
def test_every_named_size_is_a_valid_configuration(size):
    cfg = LlamaConfig.from_hf_dict({"architectures": ["LlamaForCausalLM"], **bench.SIZES[size]})
    assert cfg.num_attention_heads % cfg.num_key_value_heads == 0 and cfg.head_dim % 16 == 0


def test_more_than_one_gpu_is_refused_with_one_line_and_exit_code_2():
    r = subprocess.run([sys.executable, bench.__file__, "--gpus", "2"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 2
    lines = [ln for ln in r.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1 and json.loads(lines[0])["n_gpus"] == 2
