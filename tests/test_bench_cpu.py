"""bench.py on a machine without a GPU: the reference arm (CPU oracle) prints the contract's JSON line,
and the byte accounting of the roofline matches the cache layout."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_the_contract_line():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--workload", "c1",
                          "--steps", "2", "--warmup", "1"], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["metric"] == "decode_tokens_per_s" and line["unit"] == "tokens/s"
    assert line["higher_is_better"] is True and line["value"] > 0 and line["steps"] == 2
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["cpu_baseline"]["value"] == line["value"] == line["e2e"]["value"]
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0
    assert "workload" in line["config"] and "model" not in line["config"]


def test_other_ranks_of_the_reference_arm_do_nothing():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--workload", "c1",
                          "--gpus", "2", "--steps", "1", "--warmup", "0"], capture_output=True, text=True, timeout=120,
                         cwd=ROOT, env=env)
    assert out.returncode == 0 and out.stdout.strip() == ""


def test_algorithmic_bytes_per_token_head():
    sys.path.insert(0, ROOT)
    import bench
    assert bench.bytes_per_token_head("int8_dyn", 0) == 272          # 2 x (128 B payload + 4 fp16 scales)
    assert bench.bytes_per_token_head("int4_asym", 0) == 160         # 2 x (64 B + 4 scales + 4 zero-points)
    assert bench.bytes_per_token_head("int4_outlier", 3) == 156      # 2 x (64 B + 4 scales + 3 fp16 side values)
    assert bench.bytes_per_token_head("int4_outlier", 1) == 148
    assert bench.bytes_per_token_head("fp16", 0) == 512
    for name, wl in bench.WORKLOADS.items():
        cfg = bench.workload_config(wl, name)
        assert cfg["name"] == name and "workload" in cfg
