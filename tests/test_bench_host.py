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
    plan = bench.shard_plan(bench.WORKLOADS["c2"], rank, world, replicas=False)
    out[rank] = (slowest, bench.whole_job_tokens_per_second(plan["tokens"], slowest), list(plan["seqs"]))
    dist.destroy_process_group()


def test_two_ranks_report_the_slowest_time_and_the_whole_job_rate():
    manager = mp.Manager()
    out = manager.dict()
    mp.spawn(_rank_main, args=(2, 29731, out), nprocs=2, join=True)
    for rank in (0, 1):
        slowest, value, seqs = out[rank]
        assert slowest == 15.0
        assert abs(value - 65536 / 15e-3) < 1e-6            # one batch over both ranks: strong scaling
        assert seqs == [2 * rank, 2 * rank + 1]
    assert bench.max_over_ranks(7.0, 1, torch.device("cpu")) == 7.0


def test_shard_plans_cover_the_batch_exactly_once():
    c2, c3, c4, wide = (bench.WORKLOADS[n] for n in ("c2", "c3", "c4", "c2d128"))
    assert bench.algorithmic_flops(wide)["attention_only"] == bench.algorithmic_flops(c2)["attention_only"]
    for w in (c2, c3, c4, wide):
        for world in (1, 2, 4, 8):
            if w is c4 and world == 1:
                continue
            seen = set()
            for rank in range(world):
                plan = bench.shard_plan(w, rank, world, replicas=False)
                assert plan["scaling"] == "strong" and plan["tokens"] == w["batch"] * w["seq"]
                assert rank in plan["group"]
                for b in plan["seqs"]:
                    for h in plan["heads"]:
                        assert (b, h) not in seen
                        seen.add((b, h))
            assert len(seen) == w["batch"] * w["heads"]
    eight = [bench.shard_plan(c2, r, 8, replicas=False) for r in range(8)]
    assert all(p["selector"] and len(p["heads"]) == 8 for p in eight)
    assert eight[5]["group"] == [4, 5] and list(eight[5]["seqs"]) == [2] and list(eight[5]["heads"]) == list(range(8, 16))
    assert not bench.shard_plan(c2, 3, 4, replicas=False)["selector"]
    assert bench.shard_plan(c4, 1, 2, replicas=False)["selector"]                  # B = 1: heads split from 2 GPUs on
    weak = bench.shard_plan(c2, 1, 4, replicas=True)
    assert weak["scaling"] == "weak" and weak["tokens"] == 4 * 65536


def _selector_rank(rank, world, port, out):
    """The reduction the head-sharded ranks run on their partial selector gradients, with gloo on the CPU."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    g = torch.Generator().manual_seed(5)
    parts = torch.randn(world, 2, 16, 8, generator=g)            # every rank knows all partial sums (for the check)
    flat = parts[rank].reshape(-1).clone()
    dist.all_reduce(flat)
    out[rank] = bool(torch.allclose(flat.view(2, 16, 8), parts.sum(0), atol=1e-6))
    dist.destroy_process_group()


def test_partial_selector_gradients_sum_across_two_ranks():
    manager = mp.Manager()
    out = manager.dict()
    mp.spawn(_selector_rank, args=(2, 29733, out), nprocs=2, join=True)
    assert out[0] and out[1]


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
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["cpu_baseline"]["kind"] in ("port", "reference")
