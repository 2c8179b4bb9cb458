"""What ``bench.py`` does before it touches a GPU: the arms it refuses, and the figures it computes on the host."""

import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def _run(*args):
    return subprocess.run([sys.executable, str(ROOT / "bench.py"), *args], capture_output=True, text=True, timeout=120)


def test_more_than_one_gpu_is_refused_with_one_line_and_exit_code_2():
    r = _run("--gpus", "2", "--steps", "2", "--warmup", "1")
    assert r.returncode == 2
    assert len(r.stdout.strip().splitlines()) == 1 and "one GPU" in r.stdout


def test_reference_arm_says_why_it_is_unavailable():
    r = _run("--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1")
    assert r.returncode == 0
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and isinstance(line["unavailable"], str) and line["unavailable"]


def test_a_context_too_short_for_the_steps_is_refused_before_anything_is_built():
    r = _run("--prompt-len", "4000", "--context", "4096", "--steps", "256")
    assert r.returncode == 2 and "too short" in r.stderr


def test_byte_and_flop_counts_of_the_default_sizes():
    sys.path.insert(0, str(ROOT))
    import bench
    c = bench.SIZES
    # one layer: attention weights 88.1 MB, router 3.1 MB, one expert 28.3 MB; the head 1.229 GB
    one_expert = bench.decode_bytes(None, c, 1, [], [1]) - bench.decode_bytes(None, c, 1, [], [0])
    assert abs(one_expert - 28.31e6) < 0.01e6
    fixed = bench.decode_bytes(None, c, 1, [], [0]) - 2 * c["hidden_size"] * c["vocab_size"]
    assert abs(fixed - (88.08e6 + 3.146e6)) < 0.02e6
    # keys and values: 4,096 bytes a token and layer
    assert bench.decode_bytes(None, c, 3, [100, 50], [0, 0, 0]) - bench.decode_bytes(None, c, 3, [], [0, 0, 0]) == 3 * 150 * 4096
    # prefill of 2,048 tokens on 16 layers: about 11.2 TFLOP
    assert abs(bench.prefill_flops(c, 16, 2048) / 1e12 - 11.2) < 0.2
    peaks, source = bench.peaks()
    assert source in ("measured", "fallback") and peaks["hbm_gbs"] > 1000 and peaks["bf16_tflops"] > 100
