"""Host-side checks of bench.py's contract: the reference arm runs on CPU and prints one
JSON line with the agreed keys, both arms describe the workload with the same `config`
object, and the byte accounting is the algorithmic-bytes formula."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import bench  # noqa: E402


def test_algorithmic_bytes_formula():
    # one layer, 2 sequences of 10 and 30 tokens, 8 q / 2 kv heads, bf16: K and V read once, Q read + O written
    attn, app = bench.algorithmic_bytes([10, 30], 1, 8, 2, 2)
    assert attn == 40 * 2 * 2 * 128 * 2 + 2 * 2 * 8 * 128 * 2
    assert app == 2 * 2 * 2 * 128 * (2 + 2)
    attn8, app8 = bench.algorithmic_bytes([10, 30], 3, 8, 2, 1)          # fp8 cache, 3 layers
    assert attn8 == 3 * (40 * 2 * 2 * 128 * 1 + 2 * 2 * 8 * 128 * 2) and app8 == 3 * (2 * 2 * 2 * 128 * 3)


def test_context_lengths_are_seeded_and_in_range():
    a, b = bench.context_lens(0, 64, 1024, 4096), bench.context_lens(0, 64, 1024, 4096)
    assert a == b and len(a) == 64 and min(a) >= 1024 and max(a) <= 4096
    assert bench.context_lens(1, 64, 1024, 4096) != a


def test_both_arms_share_one_config_object():
    for name, world in (("7b", 1), ("70b", 8), ("op1", 1)):
        cfg = bench.shared_config(name, world, 0)
        assert cfg["name"] == name and cfg["workload"] == bench.WORKLOAD_TEXT[name]
        assert {"layers", "batch", "q_heads", "kv_heads", "head_dim", "context", "kv_dtype", "parallelism", "l2"} <= set(cfg)
        assert "model" not in cfg
    assert "all-reduces" in bench.shared_config("70b", 8, 0)["parallelism"]


def test_reference_arm_prints_the_contract_line():
    from oracle import oracle as O
    if O.load_ref() is None:
        pytest.skip("the compiled reference CPU kernels do not load on this host")
    env = dict(os.environ, OMP_NUM_THREADS="1")        # what torchrun exports; the arm must override it
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--workload", "op1",
                          "--steps", "3", "--warmup", "1"], capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l for l in out.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == bench.METRIC and d["unit"] == "GB/s"
    assert d["steps"] == 3 and d["warmup"] == 1 and d["higher_is_better"] is True and d["gpu_launches"] == 0
    assert d["config"] == bench.shared_config("op1", 1, 0)
    assert d["cpu_baseline"]["kind"] == "reference" and d["cpu_baseline"]["cores"] == (os.cpu_count() or 1)
    assert d["cpu_baseline"]["value"] == d["value"] == d["e2e"]["value"] > 0
    assert d["e2e"]["h2d_bytes_per_step"] == 0 and d["e2e"]["d2h_bytes_per_step"] == 0
    assert d["ms_per_step"] > 0
