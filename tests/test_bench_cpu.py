"""The benchmark's reference arm needs no GPU: it times the CPU oracle and prints the same JSON
line as the GPU arm.  Checked here on a small shape (the contract's keys, rank 0 only)."""

import json
import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def run_reference_arm(rank):
    env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2", LOCAL_RANK=str(rank))
    return subprocess.run(
        [sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1",
         "--warmup", "0", "--m", "64", "--n", "256", "--k", "1024"],
        capture_output=True, text=True, env=env, timeout=300, check=True)


def test_reference_arm_prints_the_contract_line_on_rank_zero_only():
    line = json.loads(run_reference_arm(0).stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["metric"] == "g256_gemm_effective_int8_tops"
    assert line["unit"] == "TOPS" and line["higher_is_better"] is True and line["value"] > 0
    assert line["config"]["workload"] == "gemm_g256_m64_n256_k1024_bf16"
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["cpu_baseline"]["value"] == line["value"] == line["e2e"]["value"]
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0
    assert line["gpu_launches"] == 0 and line["n_gpus"] == 2
    assert run_reference_arm(1).stdout.strip() == ""
