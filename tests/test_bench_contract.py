"""The benchmark's output contract, checked on the CPU arm (no GPU needed): one JSON line with the agreed keys."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_bench(*args, env=None):
    e = dict(os.environ)
    e.update(env or {})
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], cwd=ROOT, env=e, capture_output=True,
                         text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    return [l for l in out.stdout.splitlines() if l.strip()]


def test_reference_arm_prints_one_line_with_the_contract_keys():
    lines = run_bench("--impl", "reference", "--steps", "1", "--warmup", "1", "--layers", "2", "--vocab", "2048")
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference"
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e", "gpu_launches"):
        assert key in line, key
    assert line["metric"] == "decode_tokens_per_s" and line["unit"] == "tokens/s" and line["higher_is_better"] is True
    assert line["vs_baseline"] is None and line["data"] == "synthetic" and line["value"] > 0
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1 and line["cpu_baseline"]["sample"]
    assert line["cpu_baseline"]["value"] == line["value"] == line["e2e"]["value"]
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0
    assert "workload" in line["config"] and "model" not in line["config"]


def test_reference_arm_only_rank_zero_works_under_a_multi_rank_launch():
    lines = run_bench("--impl", "reference", "--gpus", "2", "--steps", "1", "--warmup", "1", "--layers", "2", "--vocab", "2048",
                      env={"RANK": "1", "WORLD_SIZE": "2", "LOCAL_RANK": "1"})
    assert lines == []


def test_strong_scaling_is_the_default_and_shards_cover_every_session():
    sys.path.insert(0, ROOT)
    import bench
    old = sys.argv
    sys.argv = ["bench.py"]
    try:
        args = bench.parse_args()
    finally:
        sys.argv = old
    assert args.scaling == "strong" and args.sessions == 256 and args.repeats >= 10
    for n in (1, 2, 3, 4, 8):
        shards = bench.sessions_per_gpu(args, n)
        assert sum(shards) == 256 and max(shards) - min(shards) <= 1
        cfg = bench.workload_config(args, n)
        assert cfg["sessions_total"] == 256 and "strong" in cfg["parallelism"]
    args.scaling = "weak"
    assert bench.sessions_per_gpu(args, 4) == [256] * 4
