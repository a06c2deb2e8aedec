"""The denominators of bench.py's roofline figures, from the sizes alone (no GPU)."""
import json
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
import bench  # noqa: E402


@pytest.mark.parametrize("size,weights_gb,kv_per_token,prefill_flops", [
    ("8b", 15.137, 147456, 2.97e13), ("14b", 27.98, 163840, 5.584e13), ("32b", 63.97, 262144, 1.322e14)])
def test_bytes_a_decode_step_reads_and_flops_of_the_prefill(size, weights_gb, kv_per_token, prefill_flops):
    """Every matrix of the layers and the vocabulary head once, in bfloat16 (the embedding is a row
    gather); keys and values of all layers per cached token; 2 flops per matrix element and token plus
    the causal half of the attention products."""
    layers, hidden, heads, inter = bench.SIZES[size]
    cfg = dict(bench.QWEN3_8B, num_hidden_layers=layers, hidden_size=hidden, num_attention_heads=heads,
               intermediate_size=inter)
    w, kv, flops = bench.model_bytes_and_flops(cfg, layers)
    assert abs(w / 1e9 - weights_gb) < 0.01
    assert kv == kv_per_token
    assert abs(flops / prefill_flops - 1) < 0.005
    half, _, _ = bench.model_bytes_and_flops(cfg, layers // 2)
    vocab_head = 2 * cfg["vocab_size"] * hidden
    assert abs((w - vocab_head) / (half - vocab_head) - 2) < 1e-3        # fewer layers: the layers' share shrinks, the head stays


def test_contract_edges_need_no_gpu():
    two = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--gpus", "2"], capture_output=True, text=True)
    assert two.returncode == 2 and len(two.stdout.strip().splitlines()) == 1
    ref = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference"], capture_output=True, text=True)
    line = json.loads(ref.stdout)
    assert ref.returncode == 0 and line["impl"] == "reference" and "unavailable" in line
