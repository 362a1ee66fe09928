"""bench.py's command line without a GPU: what it prints for more than one GPU and for the
reference arm, and the arithmetic behind its roofline figures."""
import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def _run(*args):
    return subprocess.run([sys.executable, str(ROOT / "bench.py"), *args], capture_output=True, text=True, timeout=120)


def test_more_than_one_gpu_is_refused_with_one_line_and_exit_code_2():
    r = _run("--gpus", "2", "--steps", "1", "--warmup", "1")
    assert r.returncode == 2
    lines = [l for l in r.stdout.splitlines() if l.strip()]
    assert len(lines) == 1 and "one GPU" in lines[0]


def test_reference_arm_says_why_it_is_unavailable():
    r = _run("--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1")
    assert r.returncode == 0
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and isinstance(line["unavailable"], str) and line["unavailable"]


def test_prefill_flops_count_every_product_once():
    sys.path.insert(0, str(ROOT))
    import bench
    cfg = dict(hidden_size=8, intermediate_size=24, vocab_size=50, num_attention_heads=2, num_key_value_heads=1, head_dim=4)
    T, L = 6, 3
    per_layer = 2 * T * (8 * (2 + 2 * 1) * 4 + 2 * 4 * 8 + 3 * 8 * 24)      # qkv, o, gate + up + down
    attn = 4 * 2 * 4 * T * (T + 1) / 2                                        # causal q.k and p.v
    assert bench.prefill_flops(cfg, L, T) == L * (per_layer + attn) + 2 * 8 * 50   # + the head for one row
    assert set(bench.MODEL) >= {"hidden_size", "num_hidden_layers", "num_attention_heads", "vocab_size"}
    assert len(bench.WORKLOADS) >= 2
