"""Host-side logic of bench.py on the CPU: the multi-rank aggregation with two gloo ranks, the FLOP
accounting, and the reference arm's rank-0-only contract."""

import json
import os
import subprocess
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import bench  # noqa: E402


def _rank_main(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    slowest = bench.max_over_ranks(10.0 + 5.0 * rank, world, torch.device("cpu"))
    out[rank] = (slowest, bench.whole_job_tokens_per_second(65536, world, slowest))
    dist.destroy_process_group()


def test_two_ranks_report_the_slowest_time_and_the_whole_job_rate():
    manager = mp.Manager()
    out = manager.dict()
    mp.spawn(_rank_main, args=(2, 29731, out), nprocs=2, join=True)
    for rank in (0, 1):
        slowest, value = out[rank]
        assert slowest == 15.0
        assert abs(value - 2 * 65536 / 15e-3) < 1e-6
    assert bench.max_over_ranks(7.0, 1, torch.device("cpu")) == 7.0


def test_algorithmic_flops_match_the_counted_figures():
    f = bench.algorithmic_flops(bench.WORKLOADS["c2"])
    p = 16384 * 16385 / 2
    assert abs(f["attention_only"] - 14 * 64 * p * 64) < 1
    assert abs(f["backward"] - (10 * 64 * 64 + 6 * 64 * 4) * p) < 1
    assert abs(f["forward"] - (4 * 64 * 64 + 4 * 64 * 4 + 2 * 128 * 4) * p) < 1
    assert 8.0e12 < f["forward"] + f["backward"] < 8.4e12
    c3 = bench.algorithmic_flops(bench.WORKLOADS["c3"])
    assert c3["backward"] > f["backward"] and bench.WORKLOADS["c4"]["backward"] is False


def test_reference_arm_prints_one_line_on_rank_zero_only():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    other = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2",
                            "--steps", "1", "--warmup", "0", "--seq", "256"], env=env, capture_output=True, text=True)
    assert other.returncode == 0 and other.stdout.strip() == ""
    env.update(RANK="0", LOCAL_RANK="0")
    first = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2",
                            "--steps", "1", "--warmup", "0", "--seq", "256"], env=env, capture_output=True, text=True)
    assert first.returncode == 0, first.stderr
    line = json.loads(first.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["unit"] == "tokens/s" and line["value"] > 0
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["cpu_baseline"]["kind"] == "port"
