"""bench.py's reference arm (the reference's computation on the host cores) runs without a GPU and
prints the contract's JSON line."""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.parametrize("workload", ["bf16_rowsharded_131072x8192x8192", "mxfp8_rowsharded_131072x8192x8192"])
def test_reference_arm_prints_one_json_line(workload):
    env = dict(os.environ, GEMM_B200_REF_BUDGET_S="2")
    out = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "2", "--warmup", "1",
                          "--workload", workload], cwd=ROOT, env=env, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["metric"] == "tflops" and line["unit"] == "TFLOP/s"
    assert line["value"] > 0 and line["steps"] == 2 and line["warmup"] == 1 and line["higher_is_better"] is True
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"] == {"value": line["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert line["config"]["workload"] == workload


def test_other_ranks_of_the_reference_arm_do_nothing():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2")
    out = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--gpus", "2"], cwd=ROOT, env=env,
                         capture_output=True, text=True, timeout=120)
    assert out.returncode == 0 and out.stdout.strip() == ""


def test_reference_arm_uses_every_core_under_a_launcher_that_exports_one_thread():
    """torch.distributed.run gives its children OMP_NUM_THREADS=1; the reference arm must still run
    on every core it may use, or its rate at N >= 2 is not comparable with N = 1."""
    cores = len(os.sched_getaffinity(0))
    if cores < 2:
        pytest.skip("one core only")
    env = dict(os.environ, GEMM_B200_REF_BUDGET_S="2", OMP_NUM_THREADS="1", MKL_NUM_THREADS="1", RANK="0", WORLD_SIZE="2")
    out = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "2",
                          "--warmup", "1"], cwd=ROOT, env=env, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["cpu_baseline"]["cores"] == cores > 1
    assert set(line["cpu_baseline"]["variants"]) == {"bf16_matmul", "fp32_matmul_of_bf16"}
    assert line["value"] == max(line["cpu_baseline"]["variants"].values()) or line["cpu_baseline"]["variant"] in line["cpu_baseline"]["variants"]


def test_recorded_traffic_is_labelled_and_parsed():
    sys.path.insert(0, str(ROOT))
    import bench
    rec = bench.recorded_traffic()
    assert rec is not None and rec["bytes_per_launch_n1"] > 4.43e9 and rec["capture"].startswith("profiles/")
